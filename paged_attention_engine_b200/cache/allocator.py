"""Pages of one group: a free list and the block table of every request that holds some.

The behaviour is the reference's `BlockAllocator` (engine/cache.py:173-277), whose
public names are kept: blocks are handed out from the front of a FIFO and freed
blocks go to its back, so that reuse is as late as possible and a stale read shows
up as wrong data (engine/cache.py:180-184); `append_tokens` takes everything it needs
or nothing and reports exhaustion as a value, not an exception
(engine/cache.py:132-155,238-257); an unknown id, a second create and a second free are
caller faults and raise (engine/cache.py:221-264).

One thing is added for layers that see a window of keys only: `release_before` gives
back the blocks that lie wholly before a position, leaving holes (-1) at the front of
the table.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from enum import Enum

HOLE = -1


class AllocStatus(Enum):
    OK = "ok"
    OUT_OF_BLOCKS = "out_of_blocks"


@dataclass(frozen=True)
class AllocResult:
    """Outcome of a reservation; `new_block_ids` is empty when no new block was needed."""

    status: AllocStatus
    new_block_ids: tuple[int, ...] = ()

    @property
    def ok(self) -> bool:
        return self.status is AllocStatus.OK


class _Table:
    __slots__ = ("blocks", "tokens", "released")

    def __init__(self) -> None:
        self.blocks: list[int] = []   # logical block index -> physical id, HOLE once released
        self.tokens = 0               # tokens reserved so far
        self.released = 0             # leading logical blocks already given back


class BlockAllocator:
    """Every physical block is either in the free list or in exactly one table."""

    def __init__(self, num_blocks: int, block_size: int) -> None:
        if num_blocks < 1:
            raise ValueError(f"num_blocks must be at least 1, got {num_blocks}")
        if block_size < 1:
            raise ValueError(f"block_size must be at least 1, got {block_size}")
        self.num_blocks = num_blocks
        self.block_size = block_size
        self._free: deque[int] = deque(range(num_blocks))
        self._tables: dict[object, _Table] = {}

    # -- pool ------------------------------------------------------------- #

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_allocated(self) -> int:
        return sum(len(t.blocks) - t.released for t in self._tables.values())

    def free_block_ids(self) -> tuple[int, ...]:
        """The free list in the order in which blocks will be handed out."""
        return tuple(self._free)

    def sequence_ids(self) -> tuple:
        return tuple(self._tables)

    def blocks_needed(self, num_tokens: int) -> int:
        if num_tokens < 0:
            raise ValueError(f"num_tokens must not be negative, got {num_tokens}")
        return (num_tokens + self.block_size - 1) // self.block_size

    # -- one request ------------------------------------------------------ #

    def create_sequence(self, seq_id) -> None:
        if seq_id in self._tables:
            raise KeyError(f"sequence {seq_id!r} already exists")
        self._tables[seq_id] = _Table()

    def has_sequence(self, seq_id) -> bool:
        return seq_id in self._tables

    def block_table(self, seq_id) -> tuple[int, ...]:
        """A copy of the table; released leading blocks read HOLE (-1)."""
        return tuple(self._tables[seq_id].blocks)

    def table_len(self, seq_id) -> int:
        """Entries of the table, released leading ones included."""
        return len(self._tables[seq_id].blocks)

    def num_tokens(self, seq_id) -> int:
        return self._tables[seq_id].tokens

    def num_held(self, seq_id) -> int:
        t = self._tables[seq_id]
        return len(t.blocks) - t.released

    def blocks_to_append(self, seq_id, count: int) -> int:
        """New blocks that `append_tokens(seq_id, count)` would take (seq_id None: a new request)."""
        if count < 0:
            raise ValueError(f"count must not be negative, got {count}")
        if seq_id is None:
            return self.blocks_needed(count)
        t = self._tables[seq_id]
        return self.blocks_needed(t.tokens + count) - len(t.blocks)

    def append_token(self, seq_id) -> AllocResult:
        return self.append_tokens(seq_id, 1)

    def append_tokens(self, seq_id, count: int) -> AllocResult:
        """Reserves room for `count` more tokens: all of the blocks or none."""
        needed = self.blocks_to_append(seq_id, count)
        if needed > len(self._free):
            return AllocResult(AllocStatus.OUT_OF_BLOCKS)
        t = self._tables[seq_id]
        taken = tuple(self._free.popleft() for _ in range(needed))
        t.blocks.extend(taken)
        t.tokens += count
        return AllocResult(AllocStatus.OK, taken)

    def release_before(self, seq_id, position: int) -> tuple[int, ...]:
        """Gives back the blocks whose tokens all lie before `position`."""
        t = self._tables[seq_id]
        upto = min(max(position, 0) // self.block_size, len(t.blocks))
        freed = []
        for i in range(t.released, upto):
            freed.append(t.blocks[i])
            t.blocks[i] = HOLE
        if upto > t.released:
            t.released = upto
        self._free.extend(freed)
        return tuple(freed)

    def free_sequence(self, seq_id) -> tuple[int, ...]:
        """Drops the table and gives back every block it still held, in table order."""
        t = self._tables.pop(seq_id)
        freed = tuple(b for b in t.blocks if b != HOLE)
        self._free.extend(freed)
        return freed

    def physical_slot(self, seq_id, position: int) -> tuple[int, int]:
        """(physical block id, offset in the block) of one reserved token position."""
        t = self._tables[seq_id]
        if not 0 <= position < t.tokens:
            raise IndexError(f"position {position} out of range for sequence {seq_id!r} of {t.tokens} tokens")
        block, offset = divmod(position, self.block_size)
        if t.blocks[block] == HOLE:
            raise IndexError(f"position {position} of sequence {seq_id!r} lies in a released block")
        return t.blocks[block], offset
