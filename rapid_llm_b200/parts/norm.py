"""RMSNorm with the residual add folded in.

``y = r * rsqrt(mean(r^2) + eps) * w`` with ``r = x`` or ``r = x + residual``; the weight
multiplies as ``w`` (not ``1 + w``).  Formula and the fused residual are the reference's
(``rapid_llm/kernels/ops/layernorm/skip_rmsnorm.py:41-48,51-85``; CPU twin
``rapid_llm/kernels/backend/cpu.py:18-29``); here the residual stream stays float32.
"""

from __future__ import annotations

import torch

from ..ops import gemm, kernels
from .base import NORMS, VECTOR, Norm, TensorSpec

FIRST, ADD, PLAIN = 0, 1, 2


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    reads_deferred = True       # it launches through ops.kernels, which runs queued products first

    def __init__(self, *, size: int, eps: float, dtype, device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.size = int(size)
        self.eps = float(eps)
        self.weight = self.new_storage((self.size,), VECTOR)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.size,), VECTOR, init="ones_normal")}

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        if name != "weight":
            raise KeyError(name)
        self.weight.copy_(tensor.to(torch.float32))

    def parameter_bytes(self) -> int:
        return self.weight.numel() * 4

    def workspace_elements_per_token(self) -> int:
        return self.size

    def following(self, residual: torch.Tensor, batch) -> gemm.FollowingNorm | None:
        """This norm of ``residual + (a product's result)``, as an offer to that product."""
        if self.dtype != torch.bfloat16 or residual is None:
            return None
        return gemm.FollowingNorm(residual, self.weight, self.eps, batch.workspace)

    def forward(self, x, residual, batch, *, mode, write_residual, row_index=None, name="normed"):
        """Norm of ``x`` (``FIRST``/``PLAIN``) or of ``x + residual`` (``ADD``).

        With ``write_residual`` the float32 sum is stored into ``residual``.  ``row_index``
        selects input rows (the rows whose logits are wanted, for the final norm).
        """
        rows = x.shape[0] if row_index is None else row_index.numel()
        out = batch.workspace.get(name, rows, self.size, x.dtype, min_rows=None if row_index is None else 64)
        return kernels.add_rmsnorm(
            x, residual, self.weight, out, self.eps,
            mode=mode, write_residual=write_residual, row_index=row_index,
        )
