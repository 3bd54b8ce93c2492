"""One step's batch, flattened: the tokens of all entries in a row, and beside them
everything a kernel needs to know where a token stands.

The reference pads a step to a rectangle [rows, longest] with a boolean mask and
rebuilds slot index tensors row by row (engine/model.py:435-446,
engine/attention.py:556-586). Here nothing is padded: an entry is (request, its next
tokens, the places whose logits are wanted); tokens of all entries are laid end to end,
and the causal rule j <= position is evaluated inside the attention kernel from
`q_pos0` and `kv_len`. All integer arrays of a step travel to the device in one copy.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Hashable, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager


@dataclass(frozen=True)
class StepEntry:
    """One request's share of a step: its next tokens (a portion of its prompt, or one
    decoded token) and the offsets among them whose logits are wanted."""

    key: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class GroupStep:
    """Per page group: the block tables of the step's entries and every token's slot."""

    block_table: torch.Tensor     # int32 [entries, pages]
    slots: torch.Tensor           # int32 [tokens]: page id * page_size + offset


@dataclass
class StepContext:
    ops: Any
    dtype: torch.dtype
    device: torch.device
    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor       # int32 [tokens]
    positions: torch.Tensor       # int32 [tokens]
    seq_index: torch.Tensor       # int32 [tokens]: which entry a token belongs to
    q_start: torch.Tensor         # int32 [entries + 1]: first token of each entry
    q_pos0: torch.Tensor          # int32 [entries]: position of an entry's first token
    kv_len: torch.Tensor          # int32 [entries]: tokens of the request after this step
    state_slot: torch.Tensor      # int32 [entries]
    logit_rows: torch.Tensor      # int32 [wanted]: token rows whose logits are wanted
    max_q_len: int
    max_kv_len: int
    num_single: int               # entries that bring exactly one token
    # int32 [entries - num_single]: the entries that bring more than one token, in their order; None
    # when all or none do. Attention's portion kernels then launch blocks for these entries only.
    multi_index: torch.Tensor | None
    wants_every_token: bool       # logit_rows is 0, 1, ..., tokens - 1: no gather is needed
    groups: list[GroupStep]
    # Host copies, for parts (and tests) that plan on the host.
    host_q_lens: list[int] = field(default_factory=list)
    host_q_pos0: list[int] = field(default_factory=list)
    host_state_slots: list[int] = field(default_factory=list)
    # (temperature, seed_lo, seed_hi, request_key, output_index), one element per wanted place
    sampling: tuple | None = None
    buffer: torch.Tensor | None = None    # the one device tensor that all integer arrays above are views of
    # (last_token [slots], state_slot, seq_index): where a token id of -1 is looked up on the device
    feedback: tuple | None = None
    memo: dict = field(default_factory=dict)


class _Staging:
    """Pinned host buffers that take turns, so that a buffer is not refilled while the
    copy out of it may still be in flight. The step's integers are written straight into
    the pinned buffer and leave it in one copy."""

    def __init__(self, device: torch.device, turns: int = 4) -> None:
        self.device = device
        self.pinned = device.type == "cuda"
        self.buffers: list[torch.Tensor | None] = [None] * turns
        self.views: list[np.ndarray | None] = [None] * turns
        self.events: list[Any] = [None] * turns
        self.turn = 0

    def acquire(self, size: int) -> tuple[int, np.ndarray]:
        """(turn, int32 host array of at least `size` elements) to be filled, then `commit`ted."""
        i = self.turn
        self.turn = (self.turn + 1) % len(self.buffers)
        if self.events[i] is not None:
            self.events[i].synchronize()
            self.events[i] = None
        buf = self.buffers[i]
        if buf is None or buf.numel() < size:
            buf = torch.empty(max(size, 4096), dtype=torch.int32)
            if self.pinned:
                buf = buf.pin_memory()
            self.buffers[i] = buf
            self.views[i] = buf.numpy()
        return i, self.views[i]

    def commit(self, turn: int, size: int, into: torch.Tensor | None = None) -> torch.Tensor:
        """Copies the first `size` elements to the device: into `into` (a buffer that the kernels
        of a captured graph read) when given, else into a fresh tensor."""
        buf = self.buffers[turn]
        if not self.pinned:
            if into is None:
                return buf[:size].clone()
            into[:size].copy_(buf[:size])
            return into
        out = into if into is not None else torch.empty(size, dtype=torch.int32, device=self.device)
        out[:size].copy_(buf[:size], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self.events[turn] = event
        return out


def _layout(sizes: list[int]) -> tuple[list[int], int]:
    """Start of each section (each on a 16-byte boundary) and the total, in int32 elements."""
    starts, total = [], 0
    for n in sizes:
        starts.append(total)
        total += (n + 3) // 4 * 4
    return starts, max(total, 4)


def _signed32(value: int) -> int:
    value &= 0xFFFFFFFF
    return value - (1 << 32) if value >= (1 << 31) else value


class BatchBuilder:
    def __init__(self, manager: CacheManager, ops: Any, dtype: torch.dtype, device, vocab_size: int | None = None) -> None:
        self.manager = manager
        self.ops = ops
        self.dtype = dtype
        self.device = torch.device(device)
        self.vocab_size = vocab_size
        self.staging = _Staging(self.device)
        self.bytes_uploaded = 0

    def build(
        self,
        entries: Sequence[StepEntry],
        sampling: Sequence[Any] | None = None,
        table_width: int | None = None,
        into: torch.Tensor | None = None,
        pad_to: int | None = None,
        max_kv_len: int | None = None,
    ) -> StepContext:
        """Flattens the entries. `sampling` (one row per wanted place: temperature, seed,
        request key, output index) travels in the same copy. `table_width` fixes the width of
        the block tables (a captured graph needs the same layout every step) and `into` is
        the device buffer that such a graph reads. `pad_to` (a step of single tokens that wants
        all their logits only) adds rows up to that many entries: each is a token at position 0
        of nobody's request, which writes no page (slot -1), reads page 0 and owns the spare
        state slot behind the real ones; its logits and its token are computed and ignored, so
        that steps of neighbouring batch sizes can share one captured graph. `max_kv_len` is the
        longest context that the step's kernels are to plan for (at least the true one; a captured
        graph fixes it); without it, the table's width when that is fixed, else the true one."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        manager = self.manager
        page = manager.block_size
        seen = set()
        q_lens, pos0, slots_of = [], [], []
        for e in entries:
            if e.key in seen:
                raise ValueError(f"request {e.key!r} appears twice in one step")
            seen.add(e.key)
            n = len(e.tokens)
            if n < 1:
                raise ValueError(f"request {e.key!r}: an entry needs at least one token")
            start = manager.num_computed(e.key)
            if start + n > manager.num_reserved(e.key):
                raise ValueError(
                    f"request {e.key!r}: tokens {start}..{start + n - 1} run, "
                    f"room is reserved for {manager.num_reserved(e.key)}"
                )
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {e.key!r}: wanted place {w} is outside its {n} tokens")
            q_lens.append(n)
            pos0.append(start)
            slots_of.append(manager.slot_of(e.key))

        real = len(entries)
        decode_only = all(n == 1 for n in q_lens)
        pads = 0
        if pad_to is not None and pad_to > real:
            if not decode_only or any(tuple(e.want) != (0,) for e in entries):
                raise ValueError("only a step of single tokens that wants all their logits can be padded")
            pads = pad_to - real
            q_lens = q_lens + [1] * pads
            pos0 = pos0 + [0] * pads
            slots_of = slots_of + [manager.slots.num_slots] * pads      # the spare slot behind the real ones
        b = real + pads
        total = b if decode_only else sum(q_lens)
        pos0_arr = np.asarray(pos0, dtype=np.int32)
        if decode_only:
            token_ids = np.zeros(b, dtype=np.int32)
            token_ids[:real] = np.fromiter((e.tokens[0] for e in entries), dtype=np.int32, count=real)
            seq_index = np.arange(b, dtype=np.int32)
            positions = pos0_arr
            q_start = np.arange(b + 1, dtype=np.int32)
            kv_len = pos0_arr + 1
        else:
            q_start = np.zeros(b + 1, dtype=np.int32)
            np.cumsum(q_lens, out=q_start[1:])
            token_ids = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
            seq_index = np.repeat(np.arange(b, dtype=np.int32), q_lens)
            positions = np.concatenate([np.arange(p, p + n, dtype=np.int32) for p, n in zip(pos0, q_lens)])
            kv_len = pos0_arr + np.asarray(q_lens, dtype=np.int32)
        # -1 is not a token: it asks for the token the request sampled in the step before.
        if self.vocab_size is not None and (int(token_ids.min()) < -1 or int(token_ids.max()) >= self.vocab_size):
            bad = int(token_ids[(token_ids < -1) | (token_ids >= self.vocab_size)][0])
            raise ValueError(f"token id {bad} is outside the vocabulary of {self.vocab_size}")
        rows = [int(q_start[i]) + int(w) for i, e in enumerate(entries) for w in e.want] + list(range(real, b))

        max_kv = int(kv_len.max())
        width = (max_kv + page - 1) // page
        if table_width is not None:
            if table_width < width:
                raise ValueError(f"block tables of {width} pages do not fit the fixed width {table_width}")
            width = table_width
        planned_kv = max_kv_len if max_kv_len is not None else (width * page if table_width is not None else max_kv)
        if planned_kv < max_kv:
            raise ValueError(f"a context of {max_kv} keys does not fit the {planned_kv} that the step plans for")
        num_groups = len(manager.groups)
        if sampling is not None and len(sampling) != len(rows) - pads:
            raise ValueError(f"{len(sampling)} sampling rows for {len(rows) - pads} wanted places")
        multi = [i for i, n in enumerate(q_lens) if n > 1]
        if len(multi) in (0, b):
            multi = []
        sizes = [total, total, total, b + 1, b, b, b, len(rows)] + [b * width, total] * num_groups
        multi_at = len(sizes)
        sizes.append(len(multi))
        first_sampling = len(sizes)
        if sampling is not None:
            sizes += [len(rows)] * 5
        starts, size = _layout(sizes)
        turn, host = self.staging.acquire(size)

        def put(i: int, values) -> None:
            host[starts[i] : starts[i] + sizes[i]] = values

        put(0, token_ids)
        put(1, positions)
        put(2, seq_index)
        put(3, q_start)
        put(4, pos0_arr)
        put(5, kv_len)
        put(6, slots_of)
        put(7, rows)
        put(multi_at, multi)
        page_index = positions // page
        offset = positions - page_index * page
        for g in range(num_groups):
            table = manager.table_rows(g, slots_of[:real], width)
            page_of_token = table[seq_index[: total - pads], page_index[: total - pads]]
            if int(page_of_token.min()) < 0:
                bad = int(np.argmax(page_of_token < 0))
                raise ValueError(
                    f"request {entries[int(seq_index[bad])].key!r}: position {int(positions[bad])} has no page in group {g}"
                )
            tables = host[starts[8 + 2 * g] : starts[8 + 2 * g] + b * width].reshape(b, width)
            tables[:real] = table
            tables[real:] = 0                        # a padding row reads page 0
            token_slots = host[starts[9 + 2 * g] : starts[9 + 2 * g] + total]
            token_slots[: total - pads] = page_of_token * page + offset[: total - pads]
            token_slots[total - pads :] = -1         # and writes nothing
        if sampling is not None:
            f = first_sampling
            zeros = [0] * pads
            host[starts[f] : starts[f] + len(rows)].view(np.float32)[:] = [r.temperature for r in sampling] + [0.0] * pads
            put(f + 1, [_signed32(r.seed) for r in sampling] + zeros)
            put(f + 2, [_signed32(r.seed >> 32) for r in sampling] + zeros)
            put(f + 3, [_signed32(r.request_key) for r in sampling] + zeros)
            put(f + 4, [_signed32(r.output_index) for r in sampling] + zeros)
        dev = self.staging.commit(turn, size, into)
        self.bytes_uploaded = 4 * size
        spans = list(zip(starts, sizes))

        def part(i: int) -> torch.Tensor:
            start, size = spans[i]
            return dev[start : start + size]

        groups = []
        for g in range(len(manager.groups)):
            groups.append(GroupStep(part(8 + 2 * g).view(b, width), part(9 + 2 * g)))
        sampling_parts = None
        if sampling is not None:
            f = first_sampling
            sampling_parts = (part(f).view(torch.float32), part(f + 1), part(f + 2), part(f + 3), part(f + 4))
        return StepContext(
            ops=self.ops, dtype=self.dtype, device=self.device, num_tokens=total, num_seqs=b,
            token_ids=part(0), positions=part(1), seq_index=part(2), q_start=part(3), q_pos0=part(4),
            kv_len=part(5), state_slot=part(6), logit_rows=part(7),
            max_q_len=max(q_lens), max_kv_len=planned_kv,
            num_single=sum(1 for n in q_lens if n == 1), multi_index=part(multi_at) if multi else None, wants_every_token=len(rows) == total and rows == list(range(total)), groups=groups,
            host_q_lens=list(q_lens), host_q_pos0=list(pos0), host_state_slots=list(slots_of),
            sampling=sampling_parts, buffer=dev,
        )
