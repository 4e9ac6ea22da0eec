"""Rotary position encoding: float32 cos/sin tables indexed by absolute position.

``inv_freq_i = theta^(-2i / R)`` for ``i < R/2`` in float32, ``angle = p * inv_freq``, one
table row per position (``rapid_llm/modules/rotary_embedding.py:30-37,194-202``).  The
rotation itself (half-split pairs ``(i, i + R/2)``) happens inside the fused
q/k-norm + rotation + cache-write kernel, in float32 in both engine precisions.
Identical tables are shared between the layers that ask for them.
"""

from __future__ import annotations

import torch

from .base import POSITION_ENCODINGS, PositionEncoding

_SHARED: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


def rope_tables(rotary_dim: int, theta: float, max_positions: int) -> tuple[torch.Tensor, torch.Tensor]:
    """cos and sin, float32 ``[max_positions, rotary_dim / 2]``, computed on the host."""
    exponents = torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim
    inv_freq = 1.0 / (torch.tensor(float(theta), dtype=torch.float32) ** exponents)
    angles = torch.outer(torch.arange(max_positions, dtype=torch.float32), inv_freq)
    return torch.cos(angles), torch.sin(angles)


@POSITION_ENCODINGS.register("rope")
class RotaryEmbedding(PositionEncoding):
    def __init__(self, *, head_dim: int, rotary_dim: int, theta: float, max_positions: int, dtype, device) -> None:
        super().__init__(dtype=dtype, device=device)
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and within head_dim {head_dim}")
        self.head_dim, self.rotary_dim = int(head_dim), int(rotary_dim)
        self.theta, self.max_positions = float(theta), int(max_positions)
        key = (self.rotary_dim, self.theta, self.max_positions, str(self.device))
        if key not in _SHARED:
            cos, sin = rope_tables(self.rotary_dim, self.theta, self.max_positions)
            _SHARED[key] = (cos.to(self.device).contiguous(), sin.to(self.device).contiguous())
        self.cos, self.sin = _SHARED[key]

    def tables(self) -> tuple[torch.Tensor, torch.Tensor]:
        return self.cos, self.sin
