"""The step function: a batch of (request, its next tokens) in, logits at the wanted
places out.

It runs only the tokens it is given, as one batch, against the cache that earlier
steps left, whatever the mix: portions of prompts beside single decoded tokens, cut
anywhere. Room for the tokens must have been reserved before (capacity is the
caller's decision, as in engine/scheduler.py:255-266 and engine/model.py:386-397);
the step never allocates pages.

A step that only decodes (every entry brings one token and wants its logits) is
launch-bound: some hundreds of small kernels. Such a step is captured once per (batch
size, block-table width) into a CUDA graph whose kernels read the step's integers from a
fixed device buffer, and replayed afterwards. The graph holds the same kernels as the
eager step; what it computes does not differ.

Any other step costs its launches' host time (some 200 launches of 14 microseconds), which is
more than the GPU needs for a portion of a few hundred tokens. A step whose SHAPE comes again
(the same number of tokens, start, wanted places and state slot for every entry, in order: the
first portion of a long prompt under a token budget, a prompt length that repeats) is recorded
at its second appearance and replayed from then on; a few such recordings are kept, the least
recently used one goes first. Everything that the host knows of such a step (`host_q_lens`,
`host_q_pos0`, `host_state_slots`, what the kernels' wrappers plan from them) follows from its
shape, so the recording holds exactly the eager step's launches; token ids, pages and slots in
the pages are read from the step's device buffer, which every replay refills.
"""

from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass
from typing import Any, Hashable, Sequence

import torch

from ..cache.storage import PagedKVCache
from .batch import BatchBuilder, StepEntry
from .model import DecoderModel


@dataclass
class StepOutput:
    """`logits[i]` belongs to `wanted[i]` = (request key, offset among the entry's tokens);
    `tokens[i]` is the token sampled from it when sampling rows were given. Both live on the
    device and are valid until the next step."""

    logits: torch.Tensor | None
    wanted: list[tuple[Hashable, int]]
    num_tokens: int
    tokens: torch.Tensor | None = None


class _DecodeGraph:
    def __init__(self, buffer: torch.Tensor) -> None:
        self.buffer = buffer
        self.graph: Any = None
        self.logits: torch.Tensor | None = None
        self.tokens: torch.Tensor | None = None
        self.launches = 0
        self.num_tokens = 0


class ModelRunner:
    # A graph per (batch size, block-table width, longest context rounded up, sampling). They share
    # one memory pool (they never run at the same time), so a graph costs its launches and little else.
    MAX_GRAPHS = 512
    # A recorded step plans its attention (how the keys are sliced) for a longest context that is
    # fixed in the recording: the true longest context rounded up to a multiple of this many
    # keys, not to the block table's width, which is a power of two (at context 4,097 the table
    # is 8,192 keys wide, and slices planned for 8,192 keys would be twice as long as needed).
    KV_BUCKET = 512
    # Recordings of steps that are not decode-only, by exact shape: how many are kept, how many
    # shapes are remembered as seen once, and the largest step (tokens, entries) that is recorded.
    SHAPE_GRAPHS = 8
    SHAPES_REMEMBERED = 256
    SHAPE_GRAPH_MAX_TOKENS = 8192
    SHAPE_GRAPH_MAX_ENTRIES = 16

    def __init__(self, model: DecoderModel, cache: PagedKVCache, use_graphs: bool = True) -> None:
        self.model = model
        self.cache = cache
        self.manager = cache.manager
        self.runtime = model.runtime
        self.builder = BatchBuilder(
            self.manager, self.runtime.ops, self.runtime.dtype, self.runtime.device, model.spec.vocab_size
        )
        self.entry_caches = [cache.entry_cache(p) for p in range(len(model.spec.schedule))]
        # The checked build hands its limits to the libraries between launches: it records no graphs.
        self.use_graphs = (use_graphs and self.runtime.device.type == "cuda" and model.graph_safe
                           and not getattr(self.runtime.ops, "bounds_checked", False))
        self.graphs: dict[tuple[int, int, int, bool], _DecodeGraph] = {}
        self.graph_pool = None
        self.capture_stream = None
        self.graph_replays = 0
        self.shape_graphs: OrderedDict[tuple, _DecodeGraph] = OrderedDict()
        self.shapes_seen: OrderedDict[tuple, int] = OrderedDict()
        self.shape_graph_replays = 0
        # The token last sampled for the request in each state slot; a step's token id of -1
        # reads it, so a sampled token can feed the next step without a trip to the host.
        self.last_token = torch.zeros(self.manager.slots.num_slots + 1, dtype=torch.int32, device=self.runtime.device)
        # The device's error word exists before any step is recorded: made inside a recording, its
        # zero-fill would be part of the graph and clear the word at every replay.
        if self.runtime.device.type == "cuda" and hasattr(self.runtime.ops, "error_flag"):
            self.runtime.ops.error_flag(self.runtime.device)

    def begin_request(self, key: Hashable) -> bool:
        """Registers a request (state slot, empty block tables); False when no slot is free."""
        slot = self.manager.create_request(key)
        if slot is None:
            return False
        self.cache.reset_state(slot)
        return True

    def end_request(self, key: Hashable) -> int:
        return self.manager.free_request(key)

    # ------------------------------------------------------------------ #

    def _run(self, ctx):
        ctx.feedback = (self.last_token, ctx.state_slot, ctx.seq_index)
        logits = self.model.forward(ctx, self.entry_caches)
        tokens = None
        if ctx.sampling is not None and logits is not None:
            ops = self.runtime.ops
            tokens = ops.sample(logits, *ctx.sampling, keep=(self.last_token, ctx.logit_rows, ctx.seq_index, ctx.state_slot))
        return logits, tokens

    def _graph_key(self, entries, sampling) -> tuple[int, int, int, bool] | None:
        if not self.use_graphs or len(entries) > 256:
            return None
        for e in entries:
            if len(e.tokens) != 1 or tuple(e.want) != (0,):
                return None
        page = self.manager.block_size
        longest = max(self.manager.num_computed(e.key) + 1 for e in entries)
        width = 16
        while width * page < longest:
            width *= 2
        bucket = min(width * page, -(-longest // self.KV_BUCKET) * self.KV_BUCKET)
        return (self.graph_batch(len(entries)), width, bucket, sampling is not None)

    def _shape_key(self, entries, sampling) -> tuple | None:
        """The exact shape of a step that is not decode-only (per entry: tokens, start, wanted places,
        state slot), or None when such steps are not recorded."""
        if not self.use_graphs or self.SHAPE_GRAPHS < 1 or len(entries) > self.SHAPE_GRAPH_MAX_ENTRIES:
            return None
        if sum(len(e.tokens) for e in entries) > self.SHAPE_GRAPH_MAX_TOKENS:
            return None
        return (tuple((len(e.tokens), self.manager.num_computed(e.key), tuple(e.want), self.manager.slot_of(e.key)) for e in entries),
                sampling is not None)

    @staticmethod
    def graph_batch(count: int) -> int:
        """The batch size whose graph a decode step of `count` requests replays: itself up to 8,
        then the next multiple of 2 up to 16, of 4 up to 32, of 8 beyond (padding rows fill the
        rest), so that a batch that shrinks and grows by ones records a few graphs, not one per size."""
        if count <= 8:
            return count
        step = 2 if count <= 16 else (4 if count <= 32 else 8)
        return -(-count // step) * step

    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry], sampling: Sequence[Any] | None = None) -> StepOutput:
        key = self._graph_key(entries, sampling)
        slot = self.graphs.get(key) if key is not None else None
        if slot is not None and slot.graph is not None:
            self.builder.build(entries, sampling, table_width=key[1], into=slot.buffer, pad_to=key[0], max_kv_len=key[2])
            slot.graph.replay()
            self.model.forward_pass_count += 1
            self.graph_replays += 1
            ops = self.runtime.ops
            if hasattr(ops, "launches"):
                ops.launches += slot.launches
            logits, tokens = slot.logits[: len(entries)], None if slot.tokens is None else slot.tokens[: len(entries)]
            num_tokens = len(entries)
        elif key is not None and len(self.graphs) < self.MAX_GRAPHS:
            # First time for this shape: its launches are recorded (nothing runs), then the
            # recording is replayed, which is this step's real work.
            ctx = self.builder.build(entries, sampling, table_width=key[1], pad_to=key[0], max_kv_len=key[2])
            slot = _DecodeGraph(ctx.buffer)
            self._capture(slot, ctx)
            self.graphs[key] = slot
            slot.graph.replay()
            self.model.forward_pass_count += 1
            ops = self.runtime.ops
            if hasattr(ops, "launches"):
                ops.launches += slot.launches
            logits, tokens = slot.logits[: len(entries)], None if slot.tokens is None else slot.tokens[: len(entries)]
            num_tokens = len(entries)
        else:
            logits, tokens, num_tokens = self._step_by_shape(entries, sampling) if key is None else self._eager(entries, sampling)
        for e in entries:
            self.manager.advance(e.key, len(e.tokens))
        wanted = [(e.key, int(w)) for e in entries for w in e.want]
        return StepOutput(logits, wanted, num_tokens, tokens)

    def _eager(self, entries, sampling):
        ctx = self.builder.build(entries, sampling)
        logits, tokens = self._run(ctx)
        return logits, tokens, ctx.num_tokens

    def _step_by_shape(self, entries, sampling):
        """A step that is not decode-only: eager the first time its shape is seen, recorded the
        second time, replayed afterwards."""
        key = self._shape_key(entries, sampling)
        if key is None:
            return self._eager(entries, sampling)
        slot = self.shape_graphs.get(key)
        if slot is None:
            seen = self.shapes_seen.pop(key, 0)
            if seen == 0:
                self.shapes_seen[key] = 1
                while len(self.shapes_seen) > self.SHAPES_REMEMBERED:
                    self.shapes_seen.popitem(last=False)
                return self._eager(entries, sampling)
            ctx = self.builder.build(entries, sampling)
            slot = _DecodeGraph(ctx.buffer)
            try:
                self._capture(slot, ctx)
            except torch.OutOfMemoryError:
                # No room for the recording's buffers beside the eager step's: such steps stay eager from here on.
                self.SHAPE_GRAPHS = 0
                self.shape_graphs.clear()
                torch.cuda.empty_cache()
                logits, tokens = self._run(ctx)
                return logits, tokens, ctx.num_tokens
            slot.num_tokens = ctx.num_tokens
            self.shape_graphs[key] = slot
            while len(self.shape_graphs) > self.SHAPE_GRAPHS:
                self.shape_graphs.popitem(last=False)       # its memory goes back to the graphs' pool
        else:
            self.shape_graphs.move_to_end(key)
            self.builder.build(entries, sampling, into=slot.buffer)
            self.shape_graph_replays += 1
        slot.graph.replay()
        self.model.forward_pass_count += 1
        ops = self.runtime.ops
        if hasattr(ops, "launches"):
            ops.launches += slot.launches
        return slot.logits, slot.tokens, slot.num_tokens

    def _capture(self, slot: _DecodeGraph, ctx) -> None:
        """Records the step of `ctx` (whose integers lie in the buffer that replays will refill).
        The recording runs on a stream of its own, as capture needs, with the graphs' shared pool;
        torch's context manager is not used because it collects garbage and empties the
        allocator's cache at every entry, which costs more than the recording."""
        ops = self.runtime.ops
        before = getattr(ops, "launches", 0)
        count = self.model.forward_pass_count
        graph = torch.cuda.CUDAGraph()
        if self.capture_stream is None:
            self.capture_stream = torch.cuda.Stream(device=self.runtime.device)
        current = torch.cuda.current_stream(self.runtime.device)
        self.capture_stream.wait_stream(current)
        with torch.cuda.stream(self.capture_stream):
            graph.capture_begin(pool=self.graph_pool)
            try:
                slot.logits, slot.tokens = self._run(ctx)
            finally:
                graph.capture_end()
        current.wait_stream(self.capture_stream)
        if self.graph_pool is None:
            self.graph_pool = graph.pool()
        self.model.forward_pass_count = count       # recording is not a traversal
        slot.launches = getattr(ops, "launches", 0) - before
        if hasattr(ops, "launches"):
            ops.launches = before
        slot.graph = graph
