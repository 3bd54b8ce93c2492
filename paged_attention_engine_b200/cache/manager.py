"""The cache manager: pages for groups of layers, block tables per request, state slots.

Schedule entries whose mixers have the same need (kv heads, head size, window) form
one group. Each group has a page pool of its own, a `BlockAllocator` of its own and a
block table per request; a page id is valid for every entry of its group. Pages go
back when a request ends (or is preempted: its keys are recomputed later, as in
engine/scheduler.py:624-645) and, in a group with a window, as soon as the window
has passed them. Beside the pages, every live request owns one slot of fixed-size
state for the mixers that declare some (none in Qwen2; the reference has no such
thing: a sequence id there is a counter that is never reused, engine/scheduler.py:523).

This class is host-only bookkeeping (no tensors), so it is tested without a GPU.
The device memory that the ids point into is `storage.PagedKVCache`.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Hashable, Sequence

import numpy as np

from ..config.model_spec import ModelSpec
from ..parts.base import REGISTRIES, CacheNeed, StateNeed, layer_part_specs
from .allocator import HOLE, AllocResult, AllocStatus, BlockAllocator


@dataclass(frozen=True)
class KVGroupSpec:
    """A group of schedule entries that share page ids."""

    num_kv_heads: int
    head_dim: int
    window: int                    # 0: every key is kept
    entries: tuple[int, ...]       # schedule positions that own keys and values here


@dataclass(frozen=True)
class CachePlan:
    groups: tuple[KVGroupSpec, ...]
    entry_group: dict              # schedule position -> (group index, index within group); readers map to their source
    entry_writes: dict             # schedule position -> bool
    state_needs: dict              # schedule position -> StateNeed

    def bytes_per_block(self, block_size: int, element_size: int) -> int:
        """Bytes of one page id: its keys and values in every entry of every group (each group
        has a pool of its own with the same number of pages)."""
        return sum(2 * len(g.entries) * g.num_kv_heads * g.head_dim * block_size * element_size for g in self.groups)


def layer_needs(layer) -> tuple[CacheNeed | None, StateNeed | None]:
    """What a layer's parts need of the cache: pages (keys and values) and per-request state.
    Whichever part declares a need gets the schedule entry's `EntryCache` from its block; one
    part per layer may need pages and one may need state (a layer with two such mixers is two
    layers in the schedule)."""
    pages, states = [], []
    for role, registry, part in layer_part_specs(layer):
        cls = REGISTRIES[registry].get(part.kind)
        need = getattr(cls, "cache_need", lambda _spec: None)(part)
        state = getattr(cls, "state_need", lambda _spec: None)(part)
        if need is not None:
            pages.append((role, need))
        if state is not None:
            states.append((role, state))
    for what, found in (("pages", pages), ("per-request state", states)):
        if len(found) > 1:
            raise ValueError(
                f"a '{layer.block}' layer has {len(found)} parts that need {what} ({', '.join(r for r, _ in found)}); "
                "one schedule entry has one cache: put them in layers of their own"
            )
    return (pages[0][1] if pages else None), (states[0][1] if states else None)


def plan_cache(spec: ModelSpec) -> CachePlan:
    """Groups the schedule's entries by what their mixers need of the cache."""
    by_need: dict[CacheNeed, list[int]] = {}
    state_needs: dict[int, StateNeed] = {}
    needs: dict[int, CacheNeed | None] = {}
    for pos, entry in enumerate(spec.schedule):
        need, state = layer_needs(spec.layers[entry.layer])
        needs[pos] = need
        if state is not None:
            state_needs[pos] = state
        if entry.cache_from is None and need is not None:
            by_need.setdefault(need, []).append(pos)
    groups = tuple(
        KVGroupSpec(need.num_kv_heads, need.head_dim, need.window, tuple(entries))
        for need, entries in by_need.items()
    )
    entry_group: dict[int, tuple[int, int]] = {}
    entry_writes: dict[int, bool] = {}
    for g, group in enumerate(groups):
        for i, pos in enumerate(group.entries):
            entry_group[pos] = (g, i)
            entry_writes[pos] = True
    for pos, entry in enumerate(spec.schedule):
        if entry.cache_from is not None and needs[pos] is not None:
            src = needs[entry.cache_from]
            if src is None or (src.num_kv_heads, src.head_dim) != (needs[pos].num_kv_heads, needs[pos].head_dim):
                raise ValueError(
                    f"schedule[{pos}] reads the cache of entry {entry.cache_from}, whose keys have another shape"
                )
            entry_group[pos] = entry_group[entry.cache_from]
            entry_writes[pos] = False
    return CachePlan(groups, entry_group, entry_writes, state_needs)


class StateSlotPool:
    """Slots 0..n-1 for per-request state; a live request owns exactly one."""

    def __init__(self, num_slots: int) -> None:
        if num_slots < 1:
            raise ValueError(f"num_slots must be at least 1, got {num_slots}")
        self.num_slots = num_slots
        self._free: deque[int] = deque(range(num_slots))
        self._owner: dict[Hashable, int] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    def acquire(self, key: Hashable) -> int | None:
        """The slot now owned by `key`, or None when all are taken."""
        if key in self._owner:
            raise KeyError(f"request {key!r} already owns slot {self._owner[key]}")
        if not self._free:
            return None
        slot = self._free.popleft()
        self._owner[key] = slot
        return slot

    def release(self, key: Hashable) -> int:
        slot = self._owner.pop(key)
        self._free.appendleft(slot)      # the next request takes it: steps of the same shape then meet the same slots again
        return slot

    def slot_of(self, key: Hashable) -> int:
        return self._owner[key]

    def owners(self) -> dict:
        return dict(self._owner)


class _Live:
    __slots__ = ("slot", "computed")

    def __init__(self, slot: int) -> None:
        self.slot = slot
        self.computed = 0     # tokens whose keys and values are in the pages


class CacheManager:
    """Pages of every group and state slots, for the requests that are live."""

    def __init__(
        self,
        groups: Sequence[KVGroupSpec],
        num_blocks: int | Sequence[int],
        block_size: int,
        max_requests: int = 256,
    ) -> None:
        self.groups = tuple(groups)
        counts = [num_blocks] * len(self.groups) if isinstance(num_blocks, int) else list(num_blocks)
        if len(counts) != len(self.groups):
            raise ValueError(f"{len(counts)} block counts for {len(self.groups)} groups")
        self.block_size = block_size
        self.allocators = [BlockAllocator(n, block_size) for n in counts]
        self.slots = StateSlotPool(max_requests)
        self._live: dict[Hashable, _Live] = {}
        # Mirror of the block tables by state slot, ready to be copied to the device.
        self._tables = [np.full((max_requests, 8), HOLE, dtype=np.int32) for _ in self.groups]

    # -- sizes ------------------------------------------------------------ #

    @property
    def num_blocks(self) -> int:
        """Blocks of the smallest pool (the one that binds first)."""
        return min((a.num_blocks for a in self.allocators), default=0)

    @property
    def num_free(self) -> int:
        return min((a.num_free for a in self.allocators), default=0)

    def blocks_needed(self, num_tokens: int) -> int:
        return (num_tokens + self.block_size - 1) // self.block_size

    def live_requests(self) -> tuple:
        return tuple(self._live)

    def is_live(self, key: Hashable) -> bool:
        return key in self._live

    # -- capacity questions (the scheduler's predicates) ------------------ #

    def fits_alone(self, max_total_len: int, margin_blocks: int = 0) -> bool:
        """Could a request that grows to `max_total_len` tokens ever be held, keeping the
        margin free in every pool (the admission guard of engine/scheduler.py:78-91)?"""
        need = self.blocks_needed(max_total_len)
        return all(need <= a.num_blocks - margin_blocks for a in self.allocators)

    def can_append(self, key: Hashable | None, count: int, margin_blocks: int = 0) -> bool:
        """Would reserving `count` more tokens for `key` (None: a new request) leave
        `margin_blocks` free in every pool?"""
        if key is None and self.slots.num_free == 0:
            return False
        for a in self.allocators:
            if a.blocks_to_append(key, count) + margin_blocks > a.num_free:
                return False
        return True

    # -- lifecycle -------------------------------------------------------- #

    def create_request(self, key: Hashable) -> int | None:
        """Registers a request and returns its state slot; None if no slot is free."""
        if key in self._live:
            raise KeyError(f"request {key!r} is already live")
        slot = self.slots.acquire(key)
        if slot is None:
            return None
        self._live[key] = _Live(slot)
        for a, table in zip(self.allocators, self._tables):
            a.create_sequence(key)
            table[slot, :] = HOLE
        return slot

    def reserve(self, key: Hashable, count: int) -> AllocResult:
        """Room for `count` more tokens in every group, or in none."""
        live = self._live[key]
        # One pool takes all of the blocks or none by itself; several are asked first.
        if len(self.allocators) != 1 and not self.can_append(key, count, 0):
            return AllocResult(AllocStatus.OUT_OF_BLOCKS)
        first = AllocResult(AllocStatus.OK)
        for g, a in enumerate(self.allocators):
            before = a.table_len(key)
            result = a.append_tokens(key, count)
            if not result.ok:
                assert len(self.allocators) == 1
                return result
            self._write_table(g, live.slot, before, result.new_block_ids)
            if g == 0:
                first = result
        return first

    def _write_table(self, g: int, slot: int, start: int, ids: Sequence[int]) -> None:
        if not ids:
            return
        table = self._tables[g]
        end = start + len(ids)
        if end > table.shape[1]:
            grown = np.full((table.shape[0], max(end, 2 * table.shape[1])), HOLE, dtype=np.int32)
            grown[:, : table.shape[1]] = table
            self._tables[g] = table = grown
        table[slot, start:end] = ids

    def num_reserved(self, key: Hashable) -> int:
        if not self.allocators:
            return 1 << 60
        return self.allocators[0].num_tokens(key)

    def num_computed(self, key: Hashable) -> int:
        return self._live[key].computed

    def slot_of(self, key: Hashable) -> int:
        return self._live[key].slot

    def advance(self, key: Hashable, count: int) -> None:
        """Records that `count` more tokens were written, and gives back the pages that
        every window has passed: the next query, at position n, reads keys j > n - window."""
        live = self._live[key]
        if live.computed + count > self.num_reserved(key):
            raise ValueError(
                f"request {key!r}: {live.computed} + {count} tokens written, {self.num_reserved(key)} reserved"
            )
        live.computed += count
        for g, (group, a) in enumerate(zip(self.groups, self.allocators)):
            if group.window > 0:
                first_needed = live.computed - group.window + 1
                freed = a.release_before(key, first_needed)
                if freed:
                    upto = max(first_needed, 0) // self.block_size
                    self._tables[g][live.slot, :upto] = HOLE

    def free_request(self, key: Hashable) -> int:
        """Gives back every page and the state slot; returns how many pages of the first group."""
        live = self._live.pop(key)
        count = 0
        for g, a in enumerate(self.allocators):
            freed = a.free_sequence(key)
            if g == 0:
                count = len(freed)
        self.slots.release(key)
        for table in self._tables:
            table[live.slot, :] = HOLE
        return count

    # -- what a step needs ------------------------------------------------ #

    def block_table(self, key: Hashable, group: int = 0) -> tuple[int, ...]:
        return self.allocators[group].block_table(key)

    def table_rows(self, group: int, slots: Sequence[int], width: int) -> np.ndarray:
        """[len(slots), width] int32 block tables of the given state slots."""
        table = self._tables[group]
        if width > table.shape[1]:
            out = np.full((len(slots), width), HOLE, dtype=np.int32)
            out[:, : table.shape[1]] = table[list(slots)]
            return out
        return table[list(slots), :width]

    def tokens_held(self) -> int:
        """Tokens that the live requests have reserved room for (engine/scheduler.py:389-401)."""
        return sum(self.num_reserved(key) for key in self._live) if self.allocators else 0
