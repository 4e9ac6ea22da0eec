"""The one model class: a decoder built from a :class:`ModelSpec` and run in its order.

embed -> the layers named by the run order -> final norm over the wanted rows -> output
head, as the reference's skeleton does (``rapid_llm/models/base.py:556-631``), except that
which layer runs when, and whose cache it uses, is read from ``spec.schedule``.
"""

from __future__ import annotations

import torch

from ..config.model_spec import ModelSpec
from ..engine.batch import LayerCache, StepBatch
from ..ops import gemm
from ..parts.base import BLOCKS, EMBEDDINGS, HEADS, NORMS, CacheNeed, StateNeed, TensorSpec
from ..parts.norm import ADD, PLAIN


class CausalLM:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device | str) -> None:
        spec.validate()
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        context = {"dtype": dtype, "device": self.device}
        self.embedding = EMBEDDINGS.build(spec.embedding, **context)
        self.layers = [
            BLOCKS.get(layer.arrangement)(layer=layer, **context) for layer in spec.layers
        ]
        self.final_norm = NORMS.build(spec.final_norm, **context)
        self.head = HEADS.build(spec.head, **context)
        if hasattr(self.head, "tie_to"):
            self.head.tie_to(self.embedding)

    # -- weights ----------------------------------------------------------------- #
    def _owners(self):
        """``(prefix, part)`` for every part that owns checkpoint tensors."""
        yield self.spec.embedding_prefix, self.embedding
        for layer_spec, layer in zip(self.spec.layers, self.layers):
            yield layer_spec.prefix, layer
        yield self.spec.final_norm_prefix, self.final_norm
        yield self.spec.head_prefix, self.head

    def tensor_specs(self) -> dict[str, TensorSpec]:
        """Every checkpoint tensor by full name, in a fixed order."""
        specs: dict[str, TensorSpec] = {}
        for prefix, part in self._owners():
            for name, spec in part.tensor_specs().items():
                specs[prefix + name] = spec
        return specs

    def load_tensor(self, full_name: str, tensor: torch.Tensor) -> None:
        for prefix, part in self._owners():
            if full_name.startswith(prefix):
                part.load_tensor(full_name[len(prefix):], tensor)
                return
        raise KeyError(full_name)

    def finalize(self, loaded: set[str]) -> None:
        for prefix, part in self._owners():
            part.finalize({name[len(prefix):] for name in loaded if name.startswith(prefix)})

    def parameter_bytes(self) -> int:
        return sum(part.parameter_bytes() for _, part in self._owners())

    def activation_bytes_per_token(self) -> int:
        """Bytes of activation buffers one token of a step needs: the widest layer's buffers (the layers
        share them), the embedding's output and the float32 residual stream."""
        element = torch.empty((), dtype=self.dtype).element_size()
        widest = max(layer.workspace_elements_per_token() for layer in self.layers)
        return (widest + 2 * self.spec.hidden_size) * element + 4 * self.spec.hidden_size

    # -- what the cache manager has to provide -------------------------------------- #
    def cache_needs(self) -> list[CacheNeed | None]:
        """One entry per position of the run order; ``None`` = no pages of its own."""
        needs: list[CacheNeed | None] = []
        for entry in self.spec.schedule:
            need = self.layers[entry.layer].cache_need()
            needs.append(None if entry.cache_from is not None else need)
        return needs

    def state_needs(self) -> list[StateNeed | None]:
        return [self.layers[entry.layer].state_need() for entry in self.spec.schedule]

    def step_planners(self) -> list:
        """The distinct host-side planners of the layers (one per key)."""
        planners: dict[tuple, object] = {}
        for layer in self.layers:
            for planner in layer.step_planners():
                planners.setdefault(planner.key, planner)
        return list(planners.values())

    # -- forward ------------------------------------------------------------------- #
    def forward(self, batch: StepBatch, caches: list[LayerCache]) -> torch.Tensor:
        """Logits ``[R, vocab]`` at ``batch.logit_rows``; runs only the tokens of the step."""
        batch.defer_products = True      # the queue is run below, before anything but a kernel reads a result
        x = self.embedding.forward(batch)
        residual = None
        schedule = self.spec.schedule
        for position, entry in enumerate(schedule):
            # the norm that the next layer starts with may ride on this layer's last product
            after = self.layers[schedule[position + 1].layer].leading_norm() if position + 1 < len(schedule) else None
            x, residual = self.layers[entry.layer].forward(x, residual, batch, caches[position], then_norm=after)
        if batch.num_logit_rows == 0 or not self.final_norm.reads_deferred:
            gemm.flush()
        if batch.num_logit_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=self.dtype, device=self.device)
        if residual is None:
            hidden = self.final_norm.forward(
                x, None, batch, mode=PLAIN, write_residual=False,
                row_index=batch.logit_rows, name="final_normed",
            )
        else:
            hidden = self.final_norm.forward(
                x, residual, batch, mode=ADD, write_residual=False,
                row_index=batch.logit_rows, name="final_normed",
            )
        logits = self.head.forward(hidden, batch)
        gemm.flush()
        return logits
