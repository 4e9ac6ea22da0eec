"""Interfaces and registries of the parts a layer is put together from.

A part is built from a :class:`~rapid_llm_b200.config.model_spec.PartSpec`: its class is
looked up by kind in the registry of its role and constructed with the spec's parameters
plus ``dtype`` and ``device``.  A part owns its weights, names them relative to its own
checkpoint prefix, and never learns which model it is in.  The reference reaches the same
seam through factory methods and class flags on the model skeleton
(``rapid_llm/models/base.py:393-404,449-478``).

Roles and what each must provide:

* **Mixer** — ``forward(x, batch, cache) -> y`` over the packed tokens of a step;
  ``cache_need()`` says which pages it wants (all keys, a window of them, none),
  ``state_need()`` which per-request state of fixed size, and ``step_planner()`` may name
  host-side planning it wants done once per step (work lists for its kernels).
* **FeedForward** — ``forward(x, batch) -> y``.
* **Norm** — ``forward(x, residual, batch, mode, ...) -> normed``; the residual stream is a
  float32 buffer the norm adds into.
* **PositionEncoding** — ``tables() -> (cos, sin)`` float32 ``[positions, rotary_dim / 2]``.
* **Block** (arrangement) — ``forward(x, residual, batch, cache) -> (x, residual)``; builds
  its mixer, feed-forward and norms from the layer's specification.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch

from ..config.model_spec import PartSpec

MATRIX = "matrix"   # operand of a matrix product: kept in the engine dtype
VECTOR = "vector"   # scale or bias vector: kept in float32 (a 16-bit value widens exactly)
TABLE = "table"     # integer table: kept in int32


@dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor a part expects.

    Attributes:
        shape: Shape in the checkpoint.
        kind: :data:`MATRIX`, :data:`VECTOR` or :data:`TABLE`; decides the dtype it is kept in.
        init: How the random-weights mode draws it: ``"normal"`` is N(0, std),
            ``"ones_normal"`` is 1 + N(0, std), ``"zeros"``.
        optional: May be absent from the checkpoint (the part then has a rule for it).
    """

    shape: tuple[int, ...]
    kind: str = MATRIX
    init: str = "normal"
    optional: bool = False


@dataclass(frozen=True)
class CacheNeed:
    """Pages a mixer wants.

    ``kind`` says which positions are kept: ``"full"`` (all of them) or ``"window"`` (the last
    ``window``).  What a page holds is the mixer's business: by default a key and a value per kv
    head, ``[2, num_kv_heads, page_size, head_dim]``; a mixer that caches something else (one
    latent row per token, keys without values) names the shape of one token's row in
    ``token_shape`` and gets pages ``[page_size, *token_shape]``.
    """

    kind: str
    num_kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    token_shape: tuple[int, ...] | None = None

    def group_key(self) -> tuple:
        return (self.kind, self.window, self.num_kv_heads, self.head_dim, self.token_shape)

    def page_shape(self, page_size: int) -> tuple[int, ...]:
        if self.token_shape is not None:
            return (page_size, *self.token_shape)
        return (2, self.num_kv_heads, page_size, self.head_dim)

    def elements_per_token(self) -> int:
        if self.token_shape is not None:
            count = 1
            for extent in self.token_shape:
                count *= int(extent)
            return count
        return 2 * self.num_kv_heads * self.head_dim


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size: one ``shape`` tensor of ``dtype`` per slot."""

    shape: tuple[int, ...]
    dtype: torch.dtype


@dataclass(frozen=True)
class StepShape:
    """What the host knows about a step before it runs, for parts that plan work on the host.

    ``lengths[i]`` tokens of entry ``i`` start at position ``starts[i]`` of its request;
    padding rows of a captured decode batch are entries of one token at position 0.
    """

    lengths: Any          # numpy int32 [entries]
    starts: Any           # numpy int32 [entries]
    decode_only: bool
    page_size: int = 0    # tokens per cache page (0 = not said)
    padding: int = 0      # how many of the entries, at the end, are padding rows


class StepPlanner:
    """Host-side work planning a part wants done once per step, before the metadata upload.

    Parts that return planners with equal ``key`` share one plan.  ``plan`` returns int32
    arrays (uploaded with the step's metadata and handed to the part as device tensors in
    ``batch.extras[key]``) and plain Python values (handed over as they are).
    """

    key: tuple = ()

    def capacity(self, max_tokens: int, max_entries: int) -> int:
        """Most int32 words the arrays of one step can take."""
        return 0

    def plan(self, shape: StepShape) -> dict[str, Any]:
        return {}


class Part:
    """Base of every part: construction parameters and weights by checkpoint name."""

    def __init__(self, *, dtype: torch.dtype, device: torch.device | str) -> None:
        self.dtype = dtype
        self.device = torch.device(device)

    # -- weights ------------------------------------------------------------ #
    def tensor_specs(self) -> dict[str, TensorSpec]:
        """Checkpoint tensors of this part, named relative to its prefix."""
        return {}

    def load_tensor(self, name: str, tensor: torch.Tensor) -> None:
        """Place one checkpoint tensor (already shape-checked) into device storage."""
        raise KeyError(name)

    def finalize(self, loaded: set[str]) -> None:
        """Called once after loading, with the names that were present."""

    def parameter_bytes(self) -> int:
        return 0

    def workspace_elements_per_token(self) -> int:
        """Elements of the engine dtype this part's activation buffers hold per token of a step
        (for sizing the cache pool from free memory; 0 = negligible or unknown)."""
        return 0

    # -- helpers ------------------------------------------------------------ #
    def storage_dtype(self, kind: str) -> torch.dtype:
        if kind == MATRIX:
            return self.dtype
        if kind == VECTOR:
            return torch.float32
        if kind == TABLE:
            return torch.int32
        raise ValueError(f"unknown tensor kind {kind!r}")

    def new_storage(self, shape: tuple[int, ...], kind: str) -> torch.Tensor:
        return torch.zeros(shape, dtype=self.storage_dtype(kind), device=self.device)


class Mixer(Part):
    # A mixer or feed-forward with ``rides_norms`` takes the norm's unscaled result as ``x``
    # (``ops.gemm.ScaledRows``, which its first product resolves) and an extra keyword
    # ``then_norm`` (``ops.gemm.FollowingNorm`` or ``None``): the norm after it, which its last
    # product may take along, returning ``ScaledRows`` instead of a tensor.  Without the flag a
    # part sees plain tensors only.
    rides_norms = False

    def cache_need(self) -> CacheNeed | None:
        return None

    def state_need(self) -> StateNeed | None:
        return None

    def step_planner(self) -> StepPlanner | None:
        return None

    def forward(self, x: torch.Tensor, batch, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    rides_norms = False      # as for a mixer

    def forward(self, x: torch.Tensor, batch) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    # Whether ``forward`` may be handed the result of a product that is still queued (``ops.gemm`` with
    # ``defer``): true only for a norm that launches through ``ops.kernels``, which runs the queue first.
    # For any other norm the caller runs the queue before it calls.
    reads_deferred = False

    def forward(self, x, residual, batch, *, mode: int, write_residual: bool, row_index=None, name="normed"):
        raise NotImplementedError

    def following(self, residual, batch):
        """This norm of ``residual + (a product's result)`` as an offer to that product
        (``ops.gemm.FollowingNorm``), or ``None`` if it only runs as a kernel of its own."""
        return None


class PositionEncoding(Part):
    def tables(self) -> tuple[torch.Tensor, torch.Tensor]:
        raise NotImplementedError


class Block(Part):
    def cache_need(self) -> CacheNeed | None:
        return None

    def state_need(self) -> StateNeed | None:
        return None

    def step_planners(self) -> list[StepPlanner]:
        return []

    def leading_norm(self) -> "Norm | None":
        """The norm this block starts with, if the block takes its unscaled result
        (``ops.gemm.ScaledRows``) as ``x`` from the block before it."""
        return None

    def forward(self, x, residual, batch, cache, then_norm=None):
        """``then_norm``: the next block's :meth:`leading_norm`, which this block's last product may
        take along (it then returns ``ScaledRows`` as ``x`` and the residual already holds the sum)."""
        raise NotImplementedError


class Registry:
    """Kind name -> class, for one role."""

    def __init__(self, role: str) -> None:
        self.role = role
        self._classes: dict[str, type] = {}

    def register(self, kind: str) -> Callable[[type], type]:
        def decorator(cls: type) -> type:
            self._classes[kind] = cls
            return cls

        return decorator

    def get(self, kind: str) -> type:
        try:
            return self._classes[kind]
        except KeyError:
            raise ValueError(
                f"no {self.role} registered as {kind!r}; known: {sorted(self._classes)}"
            ) from None

    def build(self, spec: PartSpec, **context: Any):
        return self.get(spec.kind)(**dict(spec.params), **context)

    def kinds(self) -> list[str]:
        return sorted(self._classes)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block arrangement")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("output head")
