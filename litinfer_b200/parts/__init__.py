from .base import (
    BLOCKS,
    FEED_FORWARDS,
    MIXERS,
    NORMS,
    POSITIONS,
    Block,
    FeedForward,
    FixedState,
    Mixer,
    Norm,
    PagedKV,
    Part,
    Position,
)
from . import norm, rope, attention, mlp, block  # noqa: F401  (registers the built-in kinds)
from .linear import FusedLinear

__all__ = [
    "BLOCKS",
    "FEED_FORWARDS",
    "MIXERS",
    "NORMS",
    "POSITIONS",
    "Block",
    "FeedForward",
    "FixedState",
    "FusedLinear",
    "Mixer",
    "Norm",
    "PagedKV",
    "Part",
    "Position",
]
