"""Device memory of the cache: the pages of every group and the per-request state.

Per group one tensor [entries, 2, pages, kv_heads, page_size, head_dim] in the engine's
dtype: the keys (index 0) and values (index 1) of one kv head of one page are
page_size x head_dim contiguous elements, which a kernel reads as one run. (The
reference keeps one K and one V tensor per layer of [blocks, block_size, kv_heads,
head_dim], engine/cache.py:305-334, and gathers whole sequences out of them.)
"""

from __future__ import annotations

import torch

from ..parts.base import EntryCache
from .manager import CacheManager, CachePlan


class PagedKVCache:
    def __init__(self, plan: CachePlan, manager: CacheManager, dtype: torch.dtype, device) -> None:
        self.plan = plan
        self.manager = manager
        self.dtype = dtype
        self.device = torch.device(device)
        self.page_size = manager.block_size
        self.pools: list[torch.Tensor] = []
        for group, allocator in zip(plan.groups, manager.allocators):
            shape = (len(group.entries), 2, allocator.num_blocks, group.num_kv_heads, self.page_size, group.head_dim)
            self.pools.append(torch.zeros(shape, dtype=dtype, device=self.device))
        self.states: dict[int, torch.Tensor] = {
            # one spare slot behind the real ones, for the padding rows of a captured step
            pos: torch.zeros((manager.slots.num_slots + 1, *need.shape), dtype=need.dtype, device=self.device)
            for pos, need in plan.state_needs.items()
        }

    def entry_cache(self, position: int) -> EntryCache:
        """What the schedule entry at `position` sees."""
        view = EntryCache(page_size=self.page_size, state=self.states.get(position))
        if position in self.plan.entry_group:
            g, i = self.plan.entry_group[position]
            view.group = g
            view.keys = self.pools[g][i, 0]
            view.values = self.pools[g][i, 1]
            view.writes = self.plan.entry_writes[position]
        return view

    def reset_state(self, slot: int) -> None:
        """A newly admitted request starts from zero state."""
        for tensor in self.states.values():
            tensor[slot].zero_()

    def storage_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.pools) + sum(
            t.numel() * t.element_size() for t in self.states.values()
        )

    def bytes_per_token(self) -> int:
        """Key and value bytes that one token adds over all entries of all groups."""
        size = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * len(g.entries) * g.num_kv_heads * g.head_dim * size for g in self.plan.groups)
