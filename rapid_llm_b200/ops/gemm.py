"""Dense matrix products ``y = x @ W^T`` of the linear layers.

float32 runs the hand-written true 32-bit kernel.  bfloat16 steps of up to
:data:`TENSOR_CORE_MAX_TOKENS` tokens (decoding, small portions) run the hand-written
tcgen05/TMA kernel, which streams the weight once at close to memory speed; larger steps call
the library product (cuBLAS through ``torch.mm``), which is where the reference's engine
uses a library as well (``rapid_llm/kernels/ops/gemm/linear.py:17-40``) and is still the
faster of the two at thousands of tokens.  ``FORCE`` pins one of the two for tests and
measurements.
"""

from __future__ import annotations

import torch

from . import kernels

TENSOR_CORE_MAX_TOKENS = 64
FORCE: str | None = None      # "tcgen05", "library" or None (choose by size)


def use_tensor_core_kernel(x: torch.Tensor, weight: torch.Tensor) -> bool:
    if x.dtype != torch.bfloat16 or not kernels.gemm_bf16_supports(x, weight):
        return False
    if FORCE is not None:
        return FORCE == "tcgen05"
    return x.shape[0] <= TENSOR_CORE_MAX_TOKENS


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, fault: torch.Tensor | None = None) -> torch.Tensor:
    """``out[T, N] = x[T, K] @ weight[N, K]^T``; all three on the GPU, same dtype."""
    if not x.is_cuda:
        raise kernels.KernelError("linear: tensors must live on a CUDA device; there is no CPU path")
    if x.dtype != weight.dtype or out.dtype != x.dtype:
        raise kernels.KernelError(f"linear: dtypes differ ({x.dtype}, {weight.dtype}, {out.dtype})")
    if x.dtype == torch.float32:
        return kernels.gemm_f32(x, weight, out)
    if x.shape[0] == 0:
        return out
    if fault is not None and use_tensor_core_kernel(x, weight):
        return kernels.gemm_bf16(x, weight, out, fault)
    torch.mm(x, weight.t(), out=out)
    return out


def gated_linear(x: torch.Tensor, gate_up: torch.Tensor, act: torch.Tensor, workspace, fault: torch.Tensor) -> torch.Tensor:
    """``act = silu(x @ gate^T) * (x @ up^T)`` for a ``[2 I, K]`` weight with the gate rows first.

    One fused tensor-core kernel where it applies; otherwise the product into a ``[T, 2 I]``
    buffer from ``workspace`` followed by the SiLU-multiply kernel.
    """
    if use_tensor_core_kernel(x, gate_up):
        return kernels.gemm_bf16(x, gate_up, act, fault, swiglu=True)
    wide = workspace.get("ffn_gate_up", x.shape[0], gate_up.shape[0], x.dtype)
    linear(x, gate_up, wide, fault)
    return kernels.silu_mul(wide, act)
