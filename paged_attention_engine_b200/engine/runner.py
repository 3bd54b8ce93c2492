"""The step function: a batch of (request, its next tokens) in, logits at the wanted
places out.

It runs only the tokens it is given, as one batch, against the cache that earlier
steps left, whatever the mix: portions of prompts beside single decoded tokens, cut
anywhere. Room for the tokens must have been reserved before (capacity is the
caller's decision, as in engine/scheduler.py:255-266 and engine/model.py:386-397);
the step never allocates pages.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Hashable, Sequence

import torch

from ..cache.storage import PagedKVCache
from .batch import BatchBuilder, StepEntry
from .model import DecoderModel


@dataclass
class StepOutput:
    """`logits[i]` belongs to `wanted[i]` = (request key, offset among the entry's tokens)."""

    logits: torch.Tensor | None
    wanted: list[tuple[Hashable, int]]
    num_tokens: int


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: PagedKVCache) -> None:
        self.model = model
        self.cache = cache
        self.manager = cache.manager
        self.runtime = model.runtime
        self.builder = BatchBuilder(self.manager, self.runtime.ops, self.runtime.dtype, self.runtime.device)
        self.entry_caches = [cache.entry_cache(p) for p in range(len(model.spec.schedule))]

    def begin_request(self, key: Hashable) -> bool:
        """Registers a request (state slot, empty block tables); False when no slot is free."""
        slot = self.manager.create_request(key)
        if slot is None:
            return False
        self.cache.reset_state(slot)
        return True

    def end_request(self, key: Hashable) -> int:
        return self.manager.free_request(key)

    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry]) -> StepOutput:
        ctx = self.builder.build(entries)
        logits = self.model.forward(ctx, self.entry_caches)
        for e in entries:
            self.manager.advance(e.key, len(e.tokens))
        wanted = [(e.key, int(w)) for e in entries for w in e.want]
        return StepOutput(logits, wanted, ctx.num_tokens)
