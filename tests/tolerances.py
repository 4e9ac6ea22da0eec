"""The one place tolerances live.

float32: the engine and the plain implementation differ only by the order of float32
additions.  bfloat16: the reference's own bound for bfloat16 logits against an independent
implementation (``tests/cpu/test_inference.py:123,126`` of harleyszhang/rapid_llm:
``atol=0.008, rtol=0.03``); the model folder is written in bfloat16 so both sides hold the
same weights.

That bound's absolute part was made for logits of the tiny models' size (root mean square 0.17
to 0.20 with the weights the tests draw).  The rounding error of bfloat16 is relative, so a
model whose logits are k times larger (the wide layers: hidden 5120, about 1.4) gets k times the
absolute part through :func:`at_scale`; the relative part is the same.
"""

import torch

F32 = {"rtol": 1e-4, "atol": 2e-5}
BF16 = {"rtol": 3e-2, "atol": 8e-3}


def for_dtype(dtype) -> dict:
    return F32 if dtype in (torch.float32, "float32") else BF16


TINY_LOGIT_RMS = 0.2


def at_scale(dtype, reference: torch.Tensor) -> dict:
    """The bound of ``for_dtype`` with its absolute part scaled to the size of ``reference``."""
    bound = dict(for_dtype(dtype))
    rms = float(reference.float().pow(2).mean().sqrt())
    bound["atol"] *= max(1.0, rms / TINY_LOGIT_RMS)
    return bound
