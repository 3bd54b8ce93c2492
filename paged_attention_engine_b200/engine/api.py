"""The Python entry point: requests in, generated tokens out.

The reference's usage (README.md:27-44) builds an engine from a loaded model, a
`BlockAllocator`, a paged cache, an executor and a `Scheduler`, then calls
`add_request(Request(...))` and `run_to_completion()`. The same names and meanings are
kept (`Request`, `Scheduler`, `add_request`, `step`, `run_to_completion`, `num_blocks`,
`block_size`, `max_num_seqs`, `max_num_batched_tokens`, `admission_margin_blocks`,
`record_logits`); `LLM` wires the pieces together for the common case.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any, Mapping, Sequence

from .executor import ModelExecutor
from .llm import Engine
from .scheduler import ADMISSION_MARGIN_BLOCKS, Request, Scheduler, StepResult

# The reference's pool: 3584 blocks of 16 tokens (engine/cache.py:29-30).
BLOCK_SIZE = 16
NUM_GPU_BLOCKS = 3584


class LLM:
    def __init__(
        self,
        engine: Engine,
        num_blocks: int = NUM_GPU_BLOCKS,
        block_size: int = BLOCK_SIZE,
        max_num_seqs: int | None = 64,
        max_num_batched_tokens: int | None = 8192,
        admission_margin_blocks: int = ADMISSION_MARGIN_BLOCKS,
        record_logits: bool = False,
        use_graphs: bool = True,
        asynchronous: bool | None = None,
    ) -> None:
        self.engine = engine
        slots = max_num_seqs if max_num_seqs is not None else 256
        self.cache = engine.new_paged_cache(num_blocks, block_size, slots)
        self.runner = engine.new_runner(self.cache, use_graphs)
        self.executor = ModelExecutor(self.runner, asynchronous)
        self.scheduler = Scheduler(
            self.executor, self.cache.manager, admission_margin_blocks=admission_margin_blocks,
            record_logits=record_logits, max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens,
            max_model_len=engine.spec.max_positions,
        )

    @classmethod
    def from_pretrained(cls, folder: str | Path, dtype="bfloat16", device="cuda:0", **options) -> "LLM":
        return cls(Engine.from_pretrained(folder, dtype, device), **options)

    @classmethod
    def from_random(cls, raw_config: Mapping[str, Any], seed: int = 0, dtype="bfloat16", device="cuda:0",
                    as_written: bool = False, **options) -> "LLM":
        return cls(Engine.from_random(raw_config, seed, dtype, device, as_written=as_written), **options)

    def add_request(self, request: Request) -> bool:
        return self.scheduler.add_request(request)

    def step(self) -> StepResult:
        return self.scheduler.step()

    def run_to_completion(self, max_steps: int = 100_000) -> dict[str, tuple[int, ...]]:
        return self.scheduler.run_to_completion(max_steps)

    def generate(
        self, prompts: Sequence[Sequence[int]], max_new_tokens: int, temperature: float = 0.0, seed: int | None = None
    ) -> list[tuple[int, ...]]:
        """Generated tokens of every prompt, in the prompts' order. A prompt that the
        admission guard rejects raises."""
        first = self.scheduler._next_arrival
        ids = [f"generate-{first + i}" for i in range(len(prompts))]
        for rid, prompt in zip(ids, prompts):
            if not self.add_request(Request(rid, tuple(prompt), max_new_tokens, temperature, seed)):
                raise ValueError(f"prompt of {len(prompt)} tokens + {max_new_tokens} new ones cannot fit the cache pool")
        done = self.run_to_completion()
        return [done[rid] for rid in ids]
