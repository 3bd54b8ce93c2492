"""Sampling of a step's logits on the device: greedy (temperature 0, what the reference
does on the host row by row, engine/scheduler.py:610) and temperature sampling by
Gumbel-max with a counter-based generator. One launch serves all rows; each row has its
own temperature and its own counters (seed, request key, index of the output token), so
the token drawn for a request does not depend on the batch it is drawn in. The rows travel
to the device inside the step's one integer buffer (engine/batch.py) and the kernel
(csrc/sampling.cu) runs at the end of the step's launches (engine/runner.py)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingRow:
    temperature: float = 0.0
    seed: int = 0
    request_key: int = 0
    output_index: int = 0
