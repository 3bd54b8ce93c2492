"""The scheduler's executor over the real model: reservation through the cache manager,
one step function call per step, sampling on the device, one read of the sampled tokens
back to the host (the reference reads one scalar per row, engine/scheduler.py:610)."""

from __future__ import annotations

from typing import Hashable, Sequence

import torch

from ..cache.allocator import AllocResult
from ..sampling import SamplingRow
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import ScheduledWork, WorkResult


class _TokenFuture:
    """Sampled tokens on their way to the host: a copy into pinned memory and an event. The
    device's error word travels in the same buffer, behind the tokens, and is looked at when
    the tokens are: a step in which a kernel gave up on a wait raises instead of handing out
    tokens."""

    def __init__(self, tokens: torch.Tensor, host: torch.Tensor, ops=None) -> None:
        count = tokens.numel()
        self.host = host[: count + 1]
        self.host[:count].copy_(tokens, non_blocking=True)
        self.ops = ops if hasattr(ops, "error_flag") else None
        self.device = tokens.device
        if self.ops is not None:
            self.host[count:].copy_(self.ops.error_flag(self.device), non_blocking=True)
        self.event = torch.cuda.Event()
        self.event.record()
        self.values: list[int] | None = None

    def result(self) -> list[int]:
        if self.values is None:
            self.event.synchronize()
            values = self.host.tolist()
            if self.ops is not None:
                self.ops.raise_for_error_word(values[-1], self.device)
            self.values = values[:-1]
        return self.values


class ModelExecutor:
    """`asynchronous` (the default on a GPU): `execute` returns as soon as the step is queued;
    sampled tokens stay on the device, feed the next step there, and reach the host a step
    later through a `_TokenFuture`. With `record_logits` the step is read back at once."""

    def __init__(self, runner: ModelRunner, asynchronous: bool | None = None, default_seed: int = 0) -> None:
        self.runner = runner
        self.default_seed = int(default_seed)
        self.manager = runner.manager
        on_gpu = runner.runtime.device.type == "cuda"
        self.asynchronous = on_gpu if asynchronous is None else (asynchronous and on_gpu)
        self._host_tokens = [torch.empty(1025, dtype=torch.int32).pin_memory() for _ in range(4)] if on_gpu else []
        self._turn = 0

    def begin(self, key: Hashable) -> bool:
        return self.runner.begin_request(key)

    def reserve(self, key: Hashable, num_tokens: int) -> AllocResult:
        return self.manager.reserve(key, num_tokens)

    def release(self, key: Hashable) -> int:
        return self.runner.end_request(key)

    def execute(self, work: Sequence[ScheduledWork], record_logits: bool) -> list[WorkResult]:
        entries, rows = [], []
        for w in work:
            if w.start != self.manager.num_computed(w.seq.request_id):
                raise AssertionError(
                    f"{w.seq.request_id}: portion starts at {w.start}, the cache holds "
                    f"{self.manager.num_computed(w.seq.request_id)} tokens"
                )
            entries.append(StepEntry(w.seq.request_id, w.token_ids, (len(w.token_ids) - 1,) if w.wants_token else ()))
            if w.wants_token:
                request = w.seq.request
                rows.append(
                    SamplingRow(request.temperature, self.default_seed if request.seed is None else request.seed,
                                request.sampling_key, len(w.seq.generated))
                )
        output = self.runner.step(entries, rows if rows else None)
        results = [WorkResult(None) for _ in work]
        if rows and self.asynchronous and not record_logits and len(rows) <= 1024:
            future = _TokenFuture(output.tokens, self._host_tokens[self._turn], self.runner.runtime.ops)
            self._turn = (self._turn + 1) % len(self._host_tokens)
            at = 0
            for i, w in enumerate(work):
                if w.wants_token:
                    results[i] = WorkResult(None, None, future, at)
                    at += 1
        elif rows:
            tokens = output.tokens.cpu().tolist()
            logits = output.logits.float().cpu() if record_logits else None
            check = getattr(self.runner.runtime.ops, "check_device_errors", None)
            if check is not None:
                check()         # a kernel that gave up on a wait left tokens that mean nothing
            at = 0
            for i, w in enumerate(work):
                if w.wants_token:
                    results[i] = WorkResult(int(tokens[at]), logits[at].clone() if logits is not None else None)
                    at += 1
        return results
