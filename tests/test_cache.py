"""The cache manager without a model and without floats: after every operation, under
random orders of requests, every page is in exactly one place (the free list or one
table), nothing is lost, held twice or freed twice; exhaustion is a value and changes
nothing; windows give pages back; state slots have one owner."""

import random

import pytest

from paged_attention_engine_b200.cache import (
    HOLE, AllocStatus, BlockAllocator, CacheManager, KVGroupSpec, StateSlotPool, plan_cache,
)
from paged_attention_engine_b200.config import resolve
import helpers


def check_allocator(a: BlockAllocator):
    held = [b for s in a.sequence_ids() for b in a.block_table(s) if b != HOLE]
    free = list(a.free_block_ids())
    assert len(held) == len(set(held)), "a page is held twice"
    assert len(free) == len(set(free)), "a page is free twice"
    assert not set(held) & set(free), "a page is both held and free"
    assert sorted(held + free) == list(range(a.num_blocks)), "a page is lost"
    assert a.num_allocated == len(held) and a.num_free == len(free)


def test_random_operations_keep_every_page_in_one_place():
    rng = random.Random(0)
    a = BlockAllocator(37, 4)
    live, next_id = {}, 0
    for _ in range(4000):
        op = rng.random()
        if op < 0.25 and len(live) < 12:
            a.create_sequence(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.75 and live:
            s = rng.choice(list(live))
            n = rng.randint(0, 9)
            free_before, table_before = a.free_block_ids(), a.block_table(s)
            result = a.append_tokens(s, n)
            if result.ok:
                live[s] += n
                assert a.num_tokens(s) == live[s]
                assert len(a.block_table(s)) == a.blocks_needed(live[s])
                assert tuple(free_before[: len(result.new_block_ids)]) == result.new_block_ids, "pages leave the front"
            else:
                assert result.status is AllocStatus.OUT_OF_BLOCKS and result.new_block_ids == ()
                assert a.free_block_ids() == free_before and a.block_table(s) == table_before, "a failure changes nothing"
        elif op < 0.85 and live:
            s = rng.choice(list(live))
            freed = a.release_before(s, rng.randint(0, live[s] + 3))
            assert a.free_block_ids()[len(a.free_block_ids()) - len(freed):] == freed, "freed pages go to the back"
        elif live:
            s = rng.choice(list(live))
            held = tuple(b for b in a.block_table(s) if b != HOLE)
            assert a.free_sequence(s) == held
            del live[s]
        check_allocator(a)


def test_misuse_raises():
    a = BlockAllocator(4, 2)
    a.create_sequence("x")
    with pytest.raises(KeyError):
        a.create_sequence("x")
    with pytest.raises(KeyError):
        a.append_tokens("nobody", 1)
    a.append_tokens("x", 3)
    assert a.physical_slot("x", 2) == (1, 0)
    with pytest.raises(IndexError):
        a.physical_slot("x", 3)
    a.free_sequence("x")
    with pytest.raises(KeyError):
        a.free_sequence("x")
    with pytest.raises(ValueError):
        BlockAllocator(0, 4)
    with pytest.raises(ValueError):
        a.blocks_needed(-1)


def test_freed_pages_are_reused_last():
    a = BlockAllocator(6, 2)
    a.create_sequence(0)
    a.append_tokens(0, 4)            # pages 0, 1
    a.free_sequence(0)
    a.create_sequence(1)
    assert a.append_tokens(1, 8).new_block_ids == (2, 3, 4, 5)
    assert a.append_tokens(1, 2).new_block_ids == (0,)


def test_state_slots_have_one_owner():
    pool = StateSlotPool(2)
    assert pool.acquire("a") == 0 and pool.acquire("b") == 1
    assert pool.acquire("c") is None
    with pytest.raises(KeyError):
        pool.acquire("a")
    assert pool.release("a") == 0
    with pytest.raises(KeyError):
        pool.release("a")
    assert pool.acquire("c") == 0 and pool.num_free == 0


def manager_invariants(m: CacheManager):
    for a in m.allocators:
        check_allocator(a)
        assert set(a.sequence_ids()) == set(m.live_requests())
    owners = m.slots.owners()
    assert set(owners) == set(m.live_requests())
    assert len(set(owners.values())) == len(owners)
    for key in m.live_requests():
        slot = m.slot_of(key)
        for g, a in enumerate(m.allocators):
            table = a.block_table(key)
            row = m.table_rows(g, [slot], max(1, len(table)))[0]
            assert tuple(row[: len(table)]) == table, "the device mirror of a block table is stale"


def test_manager_random_requests_two_groups_one_windowed():
    rng = random.Random(3)
    groups = [KVGroupSpec(2, 16, 0, (0, 1)), KVGroupSpec(2, 16, 10, (2, 3))]
    m = CacheManager(groups, [24, 9], 4, max_requests=5)
    live = {}
    n = 0
    for _ in range(3000):
        op = rng.random()
        if op < 0.2:
            key = f"k{n}"
            n += 1
            slot = m.create_request(key)
            if slot is None:
                assert len(live) == 5
            else:
                live[key] = [0, 0]           # reserved, computed
        elif op < 0.6 and live:
            key = rng.choice(list(live))
            count = rng.randint(1, 7)
            could = m.can_append(key, count)
            result = m.reserve(key, count)
            assert result.ok == could
            if result.ok:
                live[key][0] += count
        elif op < 0.85 and live:
            key = rng.choice(list(live))
            reserved, computed = live[key]
            if reserved > computed:
                step = rng.randint(1, reserved - computed)
                m.advance(key, step)
                live[key][1] += step
                # A windowed group keeps only the pages that the next query can still see.
                first_needed = max(0, live[key][1] - 10 + 1)
                table = m.block_table(key, 1)
                for i, page in enumerate(table):
                    assert (page == HOLE) == ((i + 1) * 4 <= first_needed)
                assert HOLE not in m.block_table(key, 0)
        elif live:
            key = rng.choice(list(live))
            m.free_request(key)
            del live[key]
        manager_invariants(m)
    for key in list(live):
        m.free_request(key)
    manager_invariants(m)
    assert all(a.num_free == a.num_blocks for a in m.allocators)


def test_reserve_is_all_groups_or_none():
    groups = [KVGroupSpec(1, 8, 0, (0,)), KVGroupSpec(1, 8, 0, (1,))]
    m = CacheManager(groups, [10, 2], 4, max_requests=2)
    m.create_request("a")
    assert m.reserve("a", 8).ok
    before = [a.free_block_ids() for a in m.allocators]
    assert not m.reserve("a", 1).ok
    assert [a.free_block_ids() for a in m.allocators] == before
    assert m.num_reserved("a") == 8
    with pytest.raises(ValueError):
        m.advance("a", 9)


def test_plan_groups_layers_by_need():
    _, spec = resolve(helpers.TINY_C)
    plan = plan_cache(spec)
    assert [(g.window, g.entries) for g in plan.groups] == [(0, (0, 1)), (24, (2, 3))]
    assert plan.entry_group[3] == (1, 1) and all(plan.entry_writes.values())
    _, spec_a = resolve(helpers.TINY_A)
    assert len(plan_cache(spec_a).groups) == 1
