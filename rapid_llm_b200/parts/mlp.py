"""Dense SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))``.

Gate and up share one product over a fused ``[2I, H]`` weight, gate rows first
(``rapid_llm/modules/mlp.py:52-68``, ``rapid_llm/modules/linear.py:157-172``);
``silu(z) = z * sigmoid(z)`` in float32 (``rapid_llm/kernels/ops/activation/swiglu.py:91-121``).
No biases.
"""

from __future__ import annotations

import torch

from ..ops import gemm
from .base import FEED_FORWARDS, MATRIX, FeedForward, TensorSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    rides_norms = True

    def __init__(self, *, hidden_size: int, intermediate_size: int, dtype, device,
                 gate_name: str = "gate_proj", up_name: str = "up_proj", down_name: str = "down_proj") -> None:
        super().__init__(dtype=dtype, device=device)
        self.hidden, self.inter = int(hidden_size), int(intermediate_size)
        self.names = (gate_name, up_name, down_name)
        self.gate_up = self.new_storage((2 * self.inter, self.hidden), MATRIX)
        self.down = self.new_storage((self.hidden, self.inter), MATRIX)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        gate, up, down = self.names
        return {
            f"{gate}.weight": TensorSpec((self.inter, self.hidden)),
            f"{up}.weight": TensorSpec((self.inter, self.hidden)),
            f"{down}.weight": TensorSpec((self.hidden, self.inter)),
        }

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        gate, up, down = self.names
        if name == f"{gate}.weight":
            self.gate_up[: self.inter].copy_(tensor)
        elif name == f"{up}.weight":
            self.gate_up[self.inter :].copy_(tensor)
        elif name == f"{down}.weight":
            self.down.copy_(tensor)
        else:
            raise KeyError(name)

    def parameter_bytes(self) -> int:
        return (self.gate_up.numel() + self.down.numel()) * self.gate_up.element_size()

    def workspace_elements_per_token(self) -> int:
        return 3 * self.inter + self.hidden          # gate and up of a library-product step, act, out

    def forward(self, x, batch, then_norm=None):
        rows = x.shape[0]
        act = batch.workspace.get("ffn_act", rows, self.inter, x.dtype)
        gemm.gated_linear(x, self.gate_up, act, batch.workspace, batch.fault, defer=batch.defer_products)
        out = batch.workspace.get("ffn_out", rows, self.hidden, x.dtype)
        return gemm.linear(act, self.down, out, batch.fault, then_norm=then_norm, defer=batch.defer_products)
