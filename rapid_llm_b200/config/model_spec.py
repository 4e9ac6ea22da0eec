"""Architecture-neutral description of a decoder, as data.

An architecture's own configuration class (for instance
:class:`rapid_llm_b200.config.qwen3.Qwen3Config`) turns the keys of its
``config.json`` into a :class:`ModelSpec`.  Nothing below the specification
knows which architecture it serves: the engine builds every layer by looking
the part kinds up in the part registries (:mod:`rapid_llm_b200.parts.base`) and
runs the layers in the order of :attr:`ModelSpec.schedule`.

The reference threads the same information through class flags and factory
methods on its model skeleton (``rapid_llm/models/base.py:393-404,449-478``);
here it is a value that can be printed, compared and written by a test.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registry key of its class and its parameters.

    Every size and constant the part needs is in ``params``; a part never reads
    a model-wide configuration object.
    """

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def with_params(self, **updates: Any) -> "PartSpec":
        merged = dict(self.params)
        merged.update(updates)
        return PartSpec(self.kind, merged)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: its parts, how they are arranged, and where its weights live.

    Attributes:
        arrangement: Registry key of the block class that wires mixer,
            feed-forward and norms together (``"prenorm"`` for the usual
            pre-norm residual block).
        mixer: The token mixer (attention here).
        feed_forward: The feed-forward (dense here, experts elsewhere).
        norm: The norm kind the arrangement instantiates where it needs one.
        prefix: Checkpoint prefix of the layer's tensors, e.g.
            ``"model.layers.3."``.
    """

    arrangement: str
    mixer: PartSpec
    feed_forward: PartSpec
    norm: PartSpec
    prefix: str


@dataclass(frozen=True)
class ScheduleEntry:
    """One position in the run order.

    ``layer`` indexes :attr:`ModelSpec.layers`; the same layer may be named by
    several entries (its weights are then shared, each entry still owns a cache
    of its own).  ``cache_from`` names an *earlier entry* whose cache this entry
    reads instead of writing one.
    """

    layer: int
    cache_from: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    """Everything the engine needs to build and run a decoder."""

    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    final_norm_prefix: str = "model.norm."
    embedding_prefix: str = "model.embed_tokens."
    head_prefix: str = "lm_head."

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if not self.schedule:
            raise ValueError("the run order is empty")
        for index, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(
                    f"schedule entry {index} names layer {entry.layer}, "
                    f"but the model has {len(self.layers)} layers"
                )
            if entry.cache_from is not None:
                if not 0 <= entry.cache_from < index:
                    raise ValueError(
                        f"schedule entry {index} reads the cache of entry "
                        f"{entry.cache_from}, which does not run before it"
                    )
                if self.schedule[entry.cache_from].cache_from is not None:
                    raise ValueError(
                        f"schedule entry {index} reads the cache of entry "
                        f"{entry.cache_from}, which has no cache of its own"
                    )
