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

The bound was also made for rows of a few hundred logits.  An element's error is a sum of thousands of
independent roundings, close to normal, and the largest of N such errors grows like sqrt(2 ln N): a row of
the real vocabulary (151,936 logits, tens of rows a test) has a largest error about 1.4 times that of a
row of 400 at the very same error per element.  :func:`at_scale` therefore multiplies both parts of the
bfloat16 bound by ``sqrt(ln N / ln 400)`` for rows wider than 4,096 (a factor fixed by N alone), and
:func:`assert_rows_close` also holds the root-mean-square error of every such row to a quarter of the
unwidened absolute part, so the wider tail cannot hide a shift of the whole row.  float32 bounds do not
grow.
"""

import math

import torch

F32 = {"rtol": 1e-4, "atol": 2e-5}
BF16 = {"rtol": 3e-2, "atol": 8e-3}


def for_dtype(dtype) -> dict:
    return F32 if dtype in (torch.float32, "float32") else BF16


TINY_LOGIT_RMS = 0.2


TINY_ROW, WIDE_ROW = 400, 4096


def at_scale(dtype, reference: torch.Tensor) -> dict:
    """The bound of ``for_dtype`` with its absolute part scaled to the size of ``reference`` and, in
    bfloat16, both parts scaled to the width of its rows (see the module's text)."""
    bound = dict(for_dtype(dtype))
    rms = float(reference.float().pow(2).mean().sqrt())
    bound["atol"] *= max(1.0, rms / TINY_LOGIT_RMS)
    width = reference.shape[-1]
    if dtype not in (torch.float32, "float32") and width > WIDE_ROW:
        tail = math.sqrt(math.log(width) / math.log(TINY_ROW))
        bound = {name: value * tail for name, value in bound.items()}
    return bound


def assert_rows_close(got: torch.Tensor, want: torch.Tensor, dtype) -> None:
    """``got`` against ``want`` row by row within :func:`at_scale`; wide bfloat16 rows are also held to a
    root-mean-square error of a quarter of the absolute part that rows of any width get."""
    torch.testing.assert_close(got, want, **at_scale(dtype, want))
    if dtype not in (torch.float32, "float32") and want.shape[-1] > WIDE_ROW:
        rms = float(want.float().pow(2).mean().sqrt())
        limit = BF16["atol"] * max(1.0, rms / TINY_LOGIT_RMS) / 4
        error = (got.float() - want.float()).pow(2).mean(dim=-1).sqrt()
        assert float(error.max()) <= limit, f"root-mean-square error {float(error.max()):.4g} of a row exceeds {limit:.4g}"
