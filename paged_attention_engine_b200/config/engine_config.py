"""The engine's own options as one typed object.

The reference states them as module constants with the bytes behind them
(engine/cache.py:29-35: 16-token blocks, 3584 blocks, a margin of one block;
bench/baseline.py:78-90 works out the pool's bytes) and as constructor arguments of its
scheduler (engine/scheduler.py:317-327). Here they are one record that the entry point
and the command line build; the pool's size is given either as a number of pages or as
a byte budget from which the number of pages follows.
"""

from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Any, Mapping

from .errors import ConfigError

# The reference's pool (engine/cache.py:29-35).
BLOCK_SIZE = 16
NUM_GPU_BLOCKS = 3584
ADMISSION_MARGIN_BLOCKS = 1


@dataclass(frozen=True)
class EngineConfig:
    """`num_blocks` pages of `block_size` tokens in every page group, or as many as `kv_bytes`
    pay for (give one of the two; neither means the reference's 3584). `max_num_seqs` requests
    run at a time, a step carries at most `max_num_batched_tokens` tokens; `None` lifts either
    cap. `seed` is the sampling seed of requests that name none."""

    block_size: int = BLOCK_SIZE
    num_blocks: int | None = None
    kv_bytes: int | None = None
    admission_margin_blocks: int = ADMISSION_MARGIN_BLOCKS
    max_num_seqs: int | None = 64
    max_num_batched_tokens: int | None = 8192
    dtype: str = "bfloat16"
    seed: int = 0
    record_logits: bool = False
    use_graphs: bool = True
    asynchronous: bool | None = None

    def __post_init__(self) -> None:
        if self.block_size < 1:
            raise ConfigError(f"engine option 'block_size' must be at least 1, got {self.block_size}")
        if self.num_blocks is not None and self.kv_bytes is not None:
            raise ConfigError("engine options 'num_blocks' and 'kv_bytes' both size the pool: give one of them")
        if self.num_blocks is not None and self.num_blocks < 1:
            raise ConfigError(f"engine option 'num_blocks' must be at least 1, got {self.num_blocks}")
        if self.kv_bytes is not None and self.kv_bytes < 1:
            raise ConfigError(f"engine option 'kv_bytes' must be positive, got {self.kv_bytes}")
        if self.admission_margin_blocks < 0:
            raise ConfigError(f"engine option 'admission_margin_blocks' must not be negative, got {self.admission_margin_blocks}")
        for name in ("max_num_seqs", "max_num_batched_tokens"):
            value = getattr(self, name)
            if value is not None and value < 1:
                raise ConfigError(f"engine option '{name}' must be at least 1 (or None), got {value}")
        if str(self.dtype).replace("torch.", "") not in ("bfloat16", "bf16", "float32", "fp32", "f32"):
            raise ConfigError(f"engine option 'dtype' = {self.dtype!r}: bfloat16 or float32")

    @classmethod
    def from_options(cls, options: Mapping[str, Any]) -> "EngineConfig":
        known = {f.name for f in fields(cls)}
        unknown = [k for k in options if k not in known]
        if unknown:
            raise ConfigError(f"unknown engine option(s): {', '.join(unknown)}; known: {', '.join(sorted(known))}")
        return cls(**options)

    def pool_blocks(self, bytes_per_block: int) -> int:
        """Pages per group: the number given, or what `kv_bytes` pays for at `bytes_per_block`
        (one page of every group's every entry, keys and values)."""
        if self.kv_bytes is not None:
            blocks = self.kv_bytes // max(1, bytes_per_block)
            if blocks < 1:
                raise ConfigError(
                    f"engine option 'kv_bytes' = {self.kv_bytes} does not pay for one page of {bytes_per_block} bytes"
                )
            return int(blocks)
        return self.num_blocks if self.num_blocks is not None else NUM_GPU_BLOCKS
