"""The one place tolerances live.

float32: the engine and the plain implementation differ only by the order of float32
additions.  bfloat16: the reference's own bound for bfloat16 logits against an independent
implementation (``tests/cpu/test_inference.py:123,126`` of harleyszhang/rapid_llm:
``atol=0.008, rtol=0.03``); the model folder is written in bfloat16 so both sides hold the
same weights.
"""

import torch

F32 = {"rtol": 1e-4, "atol": 2e-5}
BF16 = {"rtol": 3e-2, "atol": 8e-3}


def for_dtype(dtype) -> dict:
    return F32 if dtype in (torch.float32, "float32") else BF16
