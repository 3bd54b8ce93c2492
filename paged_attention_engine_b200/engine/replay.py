"""Trace replay: feeds given token ids through the model step by step and writes logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

It samples nothing and has nothing of its own: the model, the step function, the cache
manager and the kernels are the ones generation uses. Steps come on standard input,
one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as one batch (portions of prompts beside single decoded
tokens, cut anywhere). For a step that wants logits the file OUT/<step>.f32 holds them
as little-endian float32 [wanted, vocab], in the order of the entries and of `want`.
After every step a line `done <step>` is printed and flushed. Requests named in `end`
give back what they hold after the step. The pool holds --max-tokens tokens, so pages
are used again. (The reference has no such program; its nearest pieces are the recorded
logits of engine/scheduler.py:192-197,607-609.)
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch

from .batch import StepEntry
from .llm import Engine


class ReplayError(RuntimeError):
    pass


class Replayer:
    """Runs trace records against one engine, cache and runner."""

    def __init__(self, engine: Engine, max_tokens: int, block_size: int = 16, max_live: int = 8) -> None:
        self.engine = engine
        self.block_size = block_size
        self.max_live = max_live
        num_blocks = max(1, -(-max_tokens // block_size))
        self.cache = engine.new_paged_cache(num_blocks, block_size, max_live)
        self.runner = engine.new_runner(self.cache)
        self.manager = self.cache.manager

    def run(self, record: dict) -> torch.Tensor | None:
        """One step: float32 logits [wanted, vocab] on the device, or None when none are wanted."""
        step = record["step"]
        manager = self.manager
        entries = []
        for item in record.get("entries", []):
            key = item["id"]
            tokens = [int(t) for t in item["tokens"]]
            if not manager.is_live(key) and not self.runner.begin_request(key):
                raise ReplayError(f"step {step}: request {key!r} cannot start, {self.max_live} are live")
            if not manager.reserve(key, len(tokens)).ok:
                raise ReplayError(
                    f"step {step}: no room for {len(tokens)} more tokens of request {key!r} "
                    f"({manager.num_free} of {manager.num_blocks} pages of {self.block_size} free)"
                )
            entries.append(StepEntry(key, tokens, [int(w) for w in item.get("want", [])]))
        logits = self.runner.step(entries).logits if entries else None
        for key in record.get("end", []):
            if manager.is_live(key):
                self.runner.end_request(key)
        return logits


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    parser.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="tokens that live requests hold at most, each rounded up to whole pages")
    parser.add_argument("--block-size", type=int, default=16, help="tokens per page")
    parser.add_argument("--max-live", type=int, default=8, help="requests that may be live at a time")
    args = parser.parse_args(argv)

    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)

    engine = Engine.from_pretrained(args.model, args.dtype)
    replayer = Replayer(engine, args.max_tokens, args.block_size, args.max_live)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        try:
            logits = replayer.run(record)
        except ReplayError as exc:
            print(str(exc), file=sys.stderr)
            return 3
        if logits is not None:
            host = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
            check = getattr(engine.runtime.ops, "check_device_errors", None)
            if check is not None:
                check()         # a kernel that gave up on a wait: no logits are written, the program fails
            np.ascontiguousarray(host).tofile(str(out_dir / f"{record['step']}.f32"))
        print(f"done {record['step']}", flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
