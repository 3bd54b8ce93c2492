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
    groups: list[GroupStep]
    # Host copies, for parts (and tests) that plan on the host.
    host_q_lens: list[int] = field(default_factory=list)
    host_q_pos0: list[int] = field(default_factory=list)
    host_state_slots: list[int] = field(default_factory=list)
    # (temperature, seed_lo, seed_hi, request_key, output_index), one element per wanted place
    sampling: tuple | None = None
    buffer: torch.Tensor | None = None    # the one device tensor that all integer arrays above are views of
    memo: dict = field(default_factory=dict)


class _Staging:
    """Pinned host buffers that take turns, so that a buffer is not refilled while the
    copy out of it may still be in flight."""

    def __init__(self, device: torch.device, turns: int = 4) -> None:
        self.device = device
        self.pinned = device.type == "cuda"
        self.buffers: list[torch.Tensor | None] = [None] * turns
        self.events: list[Any] = [None] * turns
        self.turn = 0

    def upload(self, flat: np.ndarray, into: torch.Tensor | None = None) -> torch.Tensor:
        """Copies `flat` to the device: into `into` (a buffer that kernels of a captured
        graph read) when given, else into a fresh tensor."""
        if not self.pinned:
            fresh = torch.from_numpy(flat.copy())
            if into is None:
                return fresh
            into[: flat.size].copy_(fresh)
            return into
        i = self.turn
        self.turn = (self.turn + 1) % len(self.buffers)
        if self.events[i] is not None:
            self.events[i].synchronize()
        buf = self.buffers[i]
        if buf is None or buf.numel() < flat.size:
            buf = torch.empty(max(flat.size, 4096), dtype=torch.int32).pin_memory()
            self.buffers[i] = buf
        buf[: flat.size].copy_(torch.from_numpy(flat))
        out = into if into is not None else torch.empty(flat.size, dtype=torch.int32, device=self.device)
        out[: flat.size].copy_(buf[: flat.size], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self.events[i] = event
        return out


def _pack(sections: list[np.ndarray]) -> tuple[np.ndarray, list[tuple[int, int]]]:
    """Concatenates int32 arrays, each starting on a 16-byte boundary."""
    spans = []
    total = 0
    for s in sections:
        spans.append((total, s.size))
        total += (s.size + 3) // 4 * 4
    flat = np.zeros(max(total, 4), dtype=np.int32)
    for (start, size), s in zip(spans, sections):
        flat[start : start + size] = s.reshape(-1)
    return flat, spans


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
    ) -> StepContext:
        """Flattens the entries. `sampling` (one row per wanted place: temperature, seed,
        request key, output index) travels in the same copy. `table_width` fixes the width of
        the block tables (a captured graph needs the same layout every step) and `into` is
        the device buffer that such a graph reads."""
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

        b = len(entries)
        q_start = np.zeros(b + 1, dtype=np.int32)
        np.cumsum(q_lens, out=q_start[1:])
        total = int(q_start[-1])
        token_ids = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
        if self.vocab_size is not None and ((token_ids < 0) | (token_ids >= self.vocab_size)).any():
            bad = int(token_ids[(token_ids < 0) | (token_ids >= self.vocab_size)][0])
            raise ValueError(f"token id {bad} is outside the vocabulary of {self.vocab_size}")
        seq_index = np.repeat(np.arange(b, dtype=np.int32), q_lens)
        positions = np.concatenate([np.arange(p, p + n, dtype=np.int32) for p, n in zip(pos0, q_lens)])
        kv_len = np.asarray(pos0, dtype=np.int32) + np.asarray(q_lens, dtype=np.int32)
        rows = [int(q_start[i]) + int(w) for i, e in enumerate(entries) for w in e.want]
        logit_rows = np.asarray(rows, dtype=np.int32)

        sections = [
            token_ids, positions, seq_index, q_start, np.asarray(pos0, dtype=np.int32), kv_len,
            np.asarray(slots_of, dtype=np.int32), logit_rows,
        ]
        max_kv = int(kv_len.max())
        width = (max_kv + page - 1) // page
        if table_width is not None:
            if table_width < width:
                raise ValueError(f"block tables of {width} pages do not fit the fixed width {table_width}")
            width = table_width
        for g in range(len(manager.groups)):
            table = manager.table_rows(g, slots_of, width)
            page_of_token = table[seq_index, positions // page]
            if (page_of_token < 0).any():
                bad = int(np.argmax(page_of_token < 0))
                raise ValueError(
                    f"request {entries[int(seq_index[bad])].key!r}: position {int(positions[bad])} has no page in group {g}"
                )
            sections += [np.ascontiguousarray(table), page_of_token * page + positions % page]
        first_sampling = len(sections)
        if sampling is not None:
            if len(sampling) != len(rows):
                raise ValueError(f"{len(sampling)} sampling rows for {len(rows)} wanted places")
            sections += [
                np.asarray([r.temperature for r in sampling], dtype=np.float32).view(np.int32),
                np.asarray([_signed32(r.seed) for r in sampling], dtype=np.int32),
                np.asarray([_signed32(r.seed >> 32) for r in sampling], dtype=np.int32),
                np.asarray([_signed32(r.request_key) for r in sampling], dtype=np.int32),
                np.asarray([_signed32(r.output_index) for r in sampling], dtype=np.int32),
            ]

        flat, spans = _pack(sections)
        dev = self.staging.upload(flat, into)
        self.bytes_uploaded = 4 * flat.size

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
            max_q_len=max(q_lens), max_kv_len=width * page if table_width is not None else max_kv,
            num_single=sum(1 for n in q_lens if n == 1), groups=groups,
            host_q_lens=list(q_lens), host_q_pos0=list(pos0), host_state_slots=list(slots_of),
            sampling=sampling_parts, buffer=dev,
        )
