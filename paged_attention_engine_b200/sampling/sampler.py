"""Sampling of a step's logits on the device: greedy (temperature 0, what the reference
does on the host row by row, engine/scheduler.py:610) and temperature sampling by
Gumbel-max with a counter-based generator. One launch serves all rows; each row has its
own temperature and its own counters (seed, request key, index of the output token), so
the token drawn for a request does not depend on the batch it is drawn in."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch


@dataclass(frozen=True)
class SamplingRow:
    temperature: float = 0.0
    seed: int = 0
    request_key: int = 0
    output_index: int = 0


def _signed32(value: int) -> int:
    value &= 0xFFFFFFFF
    return value - (1 << 32) if value >= (1 << 31) else value


class Sampler:
    def __init__(self, ops, device) -> None:
        self.ops = ops
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, rows: Sequence[SamplingRow]) -> torch.Tensor:
        """int32 [rows] on the device."""
        if logits.shape[0] != len(rows):
            raise ValueError(f"{logits.shape[0]} rows of logits for {len(rows)} sampling rows")
        packed = torch.tensor(
            [
                [_signed32(r.seed), _signed32(r.seed >> 32), _signed32(r.request_key), _signed32(r.output_index)]
                for r in rows
            ],
            dtype=torch.int32,
        ).t().contiguous()
        temperature = torch.tensor([float(r.temperature) for r in rows], dtype=torch.float32)
        if self.device.type == "cuda":
            packed = packed.pin_memory().to(self.device, non_blocking=True)
            temperature = temperature.pin_memory().to(self.device, non_blocking=True)
        return self.ops.sample(logits, temperature, packed[0], packed[1], packed[2], packed[3])
