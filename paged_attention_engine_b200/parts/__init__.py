from .base import (
    BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS,
    REGISTRIES, Block, CacheNeed, EntryCache, Part, Registry, Runtime, StateNeed, TensorSpec,
    layer_part_specs, with_sub_parts,
)
from . import attention, blocks, feed_forward, heads, norms, rotary  # noqa: F401  (registration)

__all__ = [
    "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS",
    "REGISTRIES", "Block", "CacheNeed", "EntryCache", "Part", "Registry", "Runtime", "StateNeed", "TensorSpec",
    "layer_part_specs", "with_sub_parts",
]
