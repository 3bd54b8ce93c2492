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

from ..config.engine_config import ADMISSION_MARGIN_BLOCKS, BLOCK_SIZE, NUM_GPU_BLOCKS, EngineConfig
from .executor import ModelExecutor
from .llm import Engine
from .scheduler import Request, Scheduler, StepResult

__all__ = ["ADMISSION_MARGIN_BLOCKS", "BLOCK_SIZE", "NUM_GPU_BLOCKS", "EngineConfig", "LLM"]


class LLM:
    """`LLM(engine, EngineConfig(...))`, or the same options as keywords
    (`LLM(engine, num_blocks=..., max_num_seqs=...)`)."""

    def __init__(self, engine: Engine, config: EngineConfig | None = None, **options: Any) -> None:
        if config is not None and options:
            raise TypeError("give an EngineConfig or keyword options, not both")
        if config is None:
            options.setdefault("dtype", str(engine.dtype).replace("torch.", ""))
            config = EngineConfig.from_options(options)
        self.config = config
        self.engine = engine
        self.num_blocks = config.pool_blocks(engine.bytes_per_block(config.block_size))
        slots = config.max_num_seqs if config.max_num_seqs is not None else 256
        self.cache = engine.new_paged_cache(self.num_blocks, config.block_size, slots)
        self.runner = engine.new_runner(self.cache, config.use_graphs)
        self.executor = ModelExecutor(self.runner, config.asynchronous, default_seed=config.seed)
        self.scheduler = Scheduler(
            self.executor, self.cache.manager, admission_margin_blocks=config.admission_margin_blocks,
            record_logits=config.record_logits, max_num_seqs=config.max_num_seqs,
            max_num_batched_tokens=config.max_num_batched_tokens, max_model_len=engine.spec.max_positions,
        )

    @classmethod
    def from_pretrained(cls, folder: str | Path, dtype=None, device="cuda:0", config: EngineConfig | None = None,
                        **options) -> "LLM":
        dtype = dtype or (config.dtype if config is not None else options.get("dtype", "bfloat16"))
        options.pop("dtype", None)
        return cls(Engine.from_pretrained(folder, dtype, device), config, **options)

    @classmethod
    def from_random(cls, raw_config: Mapping[str, Any], seed: int = 0, dtype=None, device="cuda:0",
                    as_written: bool = False, config: EngineConfig | None = None, **options) -> "LLM":
        dtype = dtype or (config.dtype if config is not None else options.get("dtype", "bfloat16"))
        options.pop("dtype", None)
        return cls(Engine.from_random(raw_config, seed, dtype, device, as_written=as_written), config, **options)

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
