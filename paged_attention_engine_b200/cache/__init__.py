from .allocator import HOLE, AllocResult, AllocStatus, BlockAllocator
from .manager import CacheManager, CachePlan, KVGroupSpec, StateSlotPool, plan_cache
from .storage import PagedKVCache

__all__ = [
    "HOLE", "AllocResult", "AllocStatus", "BlockAllocator", "CacheManager", "CachePlan", "KVGroupSpec",
    "PagedKVCache", "StateSlotPool", "plan_cache",
]
