"""Parts a layer is put together from; importing the package registers the built-in ones."""

from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (registration)
from .base import (
    BLOCKS,
    EMBEDDINGS,
    FEED_FORWARDS,
    HEADS,
    MIXERS,
    NORMS,
    POSITION_ENCODINGS,
    Block,
    CacheNeed,
    FeedForward,
    Mixer,
    Norm,
    Part,
    PositionEncoding,
    StateNeed,
    StepPlanner,
    StepShape,
    TensorSpec,
)

__all__ = [
    "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS",
    "Block", "CacheNeed", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding",
    "StateNeed", "StepPlanner", "StepShape", "TensorSpec",
]
