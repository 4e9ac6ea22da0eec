"""Dense matrix products ``y = x @ W^T`` of the linear layers.

float32 runs the hand-written true 32-bit kernel.  bfloat16 steps of up to
:data:`TENSOR_CORE_MAX_TOKENS` tokens (decoding, small portions) run the hand-written
tcgen05/TMA kernel, which streams the weight once at close to memory speed; larger steps call
the library product (cuBLAS through ``torch.mm``), which is where the reference's engine
uses a library as well (``rapid_llm/kernels/ops/gemm/linear.py:17-40``) and is still the
faster of the two at thousands of tokens.  The exception is the gate/up product of steps of
:data:`PAIR_GATED_MIN_TOKENS` tokens and more: the kernel that pairs two CTAs on 256 x 256 tiles
(``csrc/gemm_bf16_pair.cu``) applies SiLU(gate) * up in its epilogue, which saves the ``[T, 2 I]``
intermediate and the activation kernel and is faster than the library with that kernel from there on.
``FORCE`` pins one for tests and measurements: ``"tcgen05"`` (the streaming kernel at any size),
``"pair"`` (the pair kernel for every product above 64 tokens: 0.85 to 1.0 of the library's pace at
2,048 tokens and more, about half of it at a few hundred) or ``"library"``.

A weight-only RMS norm between two tensor-core products rides on them instead of running as a
kernel of its own (:class:`FollowingNorm` into the product before it, :class:`ScaledRows` out
of it and into the product after it); ``FUSE_NORMS`` switches that off.

Products of a small step that follow one another (a layer's output projection, gate/up, down, the
next layer's q/k/v) run as ONE persistent kernel whose weight stream does not stop at their
boundaries (``csrc/gemm_chain.cu``).  A caller that passes ``defer=True`` lets its product wait
in a queue; the queue runs when it is full, when a product that cannot join it comes, or before
any other kernel of :mod:`ops.kernels` is launched (so a deferred result may only be handed to
such a kernel or to another product, never to a library call).  ``CHAIN`` switches it on; it is
off by default: measured on the 8B layer shapes the persistent kernel loses more at each phase's end
(partial tiles and the barrier go through global memory, about 8 us a phase) than its continuous
weight stream gains over kernels chained by programmatic dependent launch.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from . import kernels

TENSOR_CORE_MAX_TOKENS = 64
PAIR_GATED_MIN_TOKENS = 1024  # gate/up with the activation fused, on pairs of CTAs, from this many tokens on
FORCE: str | None = None      # "tcgen05", "pair", "library" or None (choose by size)
FUSE_NORMS = True             # let a norm between two tensor-core products ride on them
CHAIN = False                 # run deferred products of a small step as one persistent kernel

_PENDING: list[dict] = []     # deferred products, in order
_PENDING_FAULT: list[torch.Tensor] = []


def flush() -> None:
    """Run the deferred products now (one persistent kernel, or the single-product kernel for one)."""
    if not _PENDING:
        return
    products, fault = list(_PENDING), _PENDING_FAULT[0]
    _PENDING.clear()
    _PENDING_FAULT.clear()
    if len(products) == 1:
        product = products[0]
        kernels.gemm_bf16(product.pop("x"), product.pop("w"), product.pop("out"), fault, **product)
    else:
        kernels.gemm_chain(products, fault)


kernels.BEFORE_LAUNCH = flush


def _product(x, weight, out, fault, defer: bool, **options) -> None:
    """One tensor-core product: queued if the caller allows it, else run at once (after the queue)."""
    options = {name: value for name, value in options.items() if value is not None and value is not False}
    if defer and CHAIN and x.shape[0] <= kernels.GEMM_CHAIN_MAX_TOKENS:
        if _PENDING and (len(_PENDING) == kernels.GEMM_CHAIN_MAX_PHASES or _PENDING[0]["x"].shape[0] != x.shape[0]
                         or _PENDING_FAULT[0] is not fault):
            flush()
        _PENDING.append({"x": x, "w": weight, "out": out, **options})
        if not _PENDING_FAULT:
            _PENDING_FAULT.append(fault)
        return
    kernels.gemm_bf16(x, weight, out, fault, **options)


@dataclass
class FollowingNorm:
    """A norm ``y = r * rsqrt(mean(r^2) + eps) * weight`` of ``r = residual + (a product's result)``,
    offered to that product: ``residual`` (float32, updated in place) and the norm's float32 ``weight``;
    ``workspace`` lends the buffers of the result."""

    residual: torch.Tensor
    weight: torch.Tensor
    eps: float
    workspace: Any


@dataclass
class ScaledRows:
    """Rows of a norm's result that still lack their scale: ``rows[t] = r[t] * weight`` and the true
    row is ``rows[t] * rsqrt(sum(sumsq[t]) / size + eps)``.  A product of these rows multiplies its
    own result by the scale instead (float32), which is the same up to rounding."""

    rows: torch.Tensor
    sumsq: torch.Tensor
    eps: float
    size: int

    @property
    def shape(self):
        return self.rows.shape

    @property
    def dtype(self):
        return self.rows.dtype


def _open_scale(x) -> tuple[torch.Tensor, dict]:
    if isinstance(x, ScaledRows):
        return x.rows, {"sumsq_in": x.sumsq, "norm_eps": x.eps, "norm_size": x.size}
    return x, {}


def use_tensor_core_kernel(x: torch.Tensor, weight: torch.Tensor) -> bool:
    if x.dtype != torch.bfloat16 or not kernels.gemm_bf16_supports(x, weight):
        return False
    if FORCE is not None and FORCE != "pair":
        return FORCE == "tcgen05"
    return x.shape[0] <= TENSOR_CORE_MAX_TOKENS


_BIAS_IN_DTYPE: dict[tuple[int, torch.dtype], torch.Tensor] = {}


def _bias_as(bias: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The float32 bias in the product's dtype for the library call (made once per vector)."""
    key = (bias.data_ptr(), dtype)
    if key not in _BIAS_IN_DTYPE:
        _BIAS_IN_DTYPE[key] = bias.to(dtype)
    return _BIAS_IN_DTYPE[key]


def linear(x, weight: torch.Tensor, out: torch.Tensor, fault: torch.Tensor | None = None, *,
           then_norm: FollowingNorm | None = None, bias: torch.Tensor | None = None, defer: bool = False):
    """``out[T, N] = x[T, K] @ weight[N, K]^T (+ bias[N], float32)``; all on the GPU, same dtype.

    ``x`` may be :class:`ScaledRows`.  With ``then_norm`` the product may take the norm along:
    it then returns :class:`ScaledRows` (the residual is updated, ``out`` is not written);
    otherwise it returns ``out`` and the caller runs the norm.  With ``defer`` the product may be
    queued (see the module's text): its result exists once :func:`flush` has run.
    """
    x, scale = _open_scale(x)
    if not x.is_cuda:
        raise kernels.KernelError("linear: tensors must live on a CUDA device; there is no CPU path")
    if x.dtype != weight.dtype or out.dtype != x.dtype:
        raise kernels.KernelError(f"linear: dtypes differ ({x.dtype}, {weight.dtype}, {out.dtype})")
    if x.dtype == torch.float32:
        return kernels.gemm_f32(x, weight, out, bias)
    if x.shape[0] == 0:
        return out
    if fault is not None and use_tensor_core_kernel(x, weight):
        rows, width = out.shape
        if (then_norm is not None and FUSE_NORMS and rows <= kernels.GEMM_NORM_MAX_TOKENS and width % 8 == 0
                and rows <= TENSOR_CORE_MAX_TOKENS):
            normed = then_norm.workspace.get("normed", rows, width, x.dtype)
            sumsq = then_norm.workspace.get("normed_sumsq", rows, kernels.gemm_bf16_sumsq_count(width), torch.float32)
            _product(x, weight, normed, fault, defer, residual=then_norm.residual, norm_weight=then_norm.weight,
                     sumsq_out=sumsq, bias=bias, **scale)
            return ScaledRows(normed, sumsq, then_norm.eps, width)
        _product(x, weight, out, fault, defer, bias=bias, **scale)
        return out
    flush()
    if scale:
        raise kernels.KernelError("linear: rows with an open scale need the tensor-core product")
    if (FORCE == "pair" and fault is not None and kernels.gemm_bf16_supports(x, weight)
            and kernels.gemm_bf16_pair_takes(x.shape[0], out.shape[1], False)):
        return kernels.gemm_bf16_pair(x, weight, out, fault, bias=bias)
    if bias is None:
        torch.mm(x, weight.t(), out=out)
    else:
        torch.addmm(_bias_as(bias, x.dtype), x, weight.t(), out=out)
    return out


def gated_linear(x, gate_up: torch.Tensor, act: torch.Tensor, workspace, fault: torch.Tensor, *,
                 defer: bool = False) -> torch.Tensor:
    """``act = silu(x @ gate^T) * (x @ up^T)`` for a ``[2 I, K]`` weight with the gate rows first.

    One fused tensor-core kernel where it applies; otherwise the product into a ``[T, 2 I]``
    buffer from ``workspace`` followed by the SiLU-multiply kernel.  ``x`` may be :class:`ScaledRows`.
    """
    x, scale = _open_scale(x)
    if use_tensor_core_kernel(x, gate_up):
        _product(x, gate_up, act, fault, defer, swiglu=True, **scale)
        return act
    if scale:
        raise kernels.KernelError("gated_linear: rows with an open scale need the tensor-core product")
    if (x.dtype == torch.bfloat16 and x.shape[0] >= PAIR_GATED_MIN_TOKENS and FORCE in (None, "pair")
            and kernels.gemm_bf16_supports(x, gate_up) and kernels.gemm_bf16_pair_takes(x.shape[0], act.shape[1], True)):
        flush()
        return kernels.gemm_bf16_pair(x, gate_up, act, fault, swiglu=True)      # no [T, 2 I] intermediate
    wide = workspace.get("ffn_gate_up", x.shape[0], gate_up.shape[0], x.dtype)
    linear(x, gate_up, wide, fault)
    return kernels.silu_mul(wide, act)
