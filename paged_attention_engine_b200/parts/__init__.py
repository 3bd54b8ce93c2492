from .base import (
    BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS,
    CacheNeed, EntryCache, Part, Registry, Runtime, StateNeed, TensorSpec,
)
from . import attention, blocks, feed_forward, heads, norms, rotary  # noqa: F401  (registration)

__all__ = [
    "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS",
    "CacheNeed", "EntryCache", "Part", "Registry", "Runtime", "StateNeed", "TensorSpec",
]
