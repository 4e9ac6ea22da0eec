"""Dense matrix products ``y = x @ W^T`` of the linear layers.

float32 runs the hand-written true 32-bit kernel.  bfloat16 calls the library product
(cuBLAS through ``torch.mm``), which is where the reference's engine uses a library as well
(``rapid_llm/kernels/ops/gemm/linear.py:17-40``).
"""

from __future__ import annotations

import torch

from . import kernels


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[T, N] = x[T, K] @ weight[N, K]^T``; all three on the GPU, same dtype."""
    if not x.is_cuda:
        raise kernels.KernelError("linear: tensors must live on a CUDA device; there is no CPU path")
    if x.dtype != weight.dtype or out.dtype != x.dtype:
        raise kernels.KernelError(f"linear: dtypes differ ({x.dtype}, {weight.dtype}, {out.dtype})")
    if x.dtype == torch.float32:
        return kernels.gemm_f32(x, weight, out)
    if x.shape[0] == 0:
        return out
    torch.mm(x, weight.t(), out=out)
    return out
