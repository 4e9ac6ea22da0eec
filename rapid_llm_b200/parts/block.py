"""Arrangement of a layer's parts: the pre-norm residual block.

``h' = h + Mixer(Norm(h)); h'' = h' + FeedForward(Norm(h'))`` with each add deferred into
the next norm, so a pair ``(x, residual)`` is threaded through the stack
(``rapid_llm/models/base.py:231-266,372-375``): ``residual`` is ``None`` entering the first
layer; the norm kernel forms ``x + residual`` in float32, stores it back and norms it.

Where the parts on both sides of a norm can take it along (``rides_norms``: the product before
it adds to the residual and applies the norm's weight, the product after it applies the row's
scale), the norm is offered to them and no norm kernel runs; the parts decide step by step
whether they accept (small steps in bfloat16 do).
"""

from __future__ import annotations

import torch

from ..config.model_spec import LayerSpec
from ..ops import gemm
from ..ops.gemm import ScaledRows
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, TensorSpec
from .norm import ADD, FIRST


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    """``names`` maps the roles to their checkpoint sub-prefixes."""

    NAMES = {
        "mixer_norm": "input_layernorm.",
        "mixer": "self_attn.",
        "feed_forward_norm": "post_attention_layernorm.",
        "feed_forward": "mlp.",
    }

    def __init__(self, *, layer: LayerSpec, dtype, device, names: dict[str, str] | None = None) -> None:
        super().__init__(dtype=dtype, device=device)
        self.names = dict(self.NAMES)
        self.names.update(names or {})
        self.mixer_norm = NORMS.build(layer.norm, dtype=dtype, device=device)
        self.mixer = MIXERS.build(layer.mixer, dtype=dtype, device=device)
        self.feed_forward_norm = NORMS.build(layer.norm, dtype=dtype, device=device)
        self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, dtype=dtype, device=device)

    def _children(self):
        return (
            (self.names["mixer_norm"], self.mixer_norm),
            (self.names["mixer"], self.mixer),
            (self.names["feed_forward_norm"], self.feed_forward_norm),
            (self.names["feed_forward"], self.feed_forward),
        )

    def cache_need(self):
        return self.mixer.cache_need()

    def state_need(self):
        return self.mixer.state_need()

    def step_planners(self):
        planner = self.mixer.step_planner()
        return [] if planner is None else [planner]

    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs = {}
        for prefix, part in self._children():
            for name, spec in part.tensor_specs().items():
                specs[prefix + name] = spec
        return specs

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        for prefix, part in self._children():
            if name.startswith(prefix):
                part.load_tensor(name[len(prefix):], tensor)
                return
        raise KeyError(name)

    def finalize(self, loaded: set[str]) -> None:
        for prefix, part in self._children():
            part.finalize({name[len(prefix):] for name in loaded if name.startswith(prefix)})

    def parameter_bytes(self) -> int:
        return sum(part.parameter_bytes() for _, part in self._children())

    def workspace_elements_per_token(self) -> int:
        return sum(part.workspace_elements_per_token() for _, part in self._children())

    def leading_norm(self):
        return self.mixer_norm if self.mixer.rides_norms else None

    def forward(self, x, residual, batch, cache, then_norm=None):
        """``(x, residual)`` in, ``(x, residual)`` out; ``residual`` is ``None`` for the first layer."""
        if not self.mixer_norm.reads_deferred:
            gemm.flush()        # a norm that is no kernel of ops.kernels reads finished results only
        if isinstance(x, ScaledRows):
            normed = x          # the block before took this block's first norm along
        elif residual is None:
            residual = batch.workspace.get("residual", x.shape[0], x.shape[1], torch.float32)
            normed = self.mixer_norm.forward(x, residual, batch, mode=FIRST, write_residual=True)
        else:
            normed = self.mixer_norm.forward(x, residual, batch, mode=ADD, write_residual=True)
        if self.mixer.rides_norms:
            offer = self.feed_forward_norm.following(residual, batch) if self.feed_forward.rides_norms else None
            mixed = self.mixer.forward(normed, batch, cache, then_norm=offer)
        else:
            mixed = self.mixer.forward(normed, batch, cache)
        if isinstance(mixed, ScaledRows):
            normed = mixed
        else:
            if not self.feed_forward_norm.reads_deferred:
                gemm.flush()
            normed = self.feed_forward_norm.forward(mixed, residual, batch, mode=ADD, write_residual=True)
        if self.feed_forward.rides_norms:
            offer = then_norm.following(residual, batch) if then_norm is not None else None
            return self.feed_forward.forward(normed, batch, then_norm=offer), residual
        return self.feed_forward.forward(normed, batch), residual
