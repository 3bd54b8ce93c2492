"""The scheduler's executor over the real model: reservation through the cache manager,
one step function call per step, sampling on the device, one read of the sampled tokens
back to the host (the reference reads one scalar per row, engine/scheduler.py:610)."""

from __future__ import annotations

from typing import Hashable, Sequence

import torch

from ..cache.allocator import AllocResult
from ..sampling import Sampler, SamplingRow
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import ScheduledWork, WorkResult


class ModelExecutor:
    def __init__(self, runner: ModelRunner) -> None:
        self.runner = runner
        self.manager = runner.manager
        self.sampler = Sampler(runner.runtime.ops, runner.runtime.device)

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
                    SamplingRow(request.temperature, request.seed or 0, request.sampling_key, len(w.seq.generated))
                )
        output = self.runner.step(entries, rows if rows else None)
        results = [WorkResult(None) for _ in work]
        if rows:
            tokens = output.tokens.cpu().tolist()
            logits = output.logits.float().cpu() if record_logits else None
            at = 0
            for i, w in enumerate(work):
                if w.wants_token:
                    results[i] = WorkResult(int(tokens[at]), logits[at].clone() if logits is not None else None)
                    at += 1
        return results
