"""Measurement: decoded tokens a second at batch 8 (and 1, 64), prefill of 2,048 tokens,
and the fraction of the roofline, for the Qwen2.5-1.5B shape with random weights in
bfloat16 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

It prints ONE JSON line. `value` is decoded tokens a second of K decode steps timed on
the device (CUDA events) through the engine's step function and device sampler, the
requests standing at the context length of the configuration; `e2e` is the same through
the Python entry point (`LLM.add_request` / `step`), host tokens in and out.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Layer sizes of the Qwen2.5-1.5B shape; context 4,096 (2,048-token prompts plus up to
# 2,048 decoded tokens), pages of 16 tokens.
MODEL = dict(
    architectures=["Qwen2ForCausalLM"], num_hidden_layers=28, hidden_size=1536, num_attention_heads=12,
    num_key_value_heads=2, head_dim=128, intermediate_size=8960, vocab_size=151936, rope_theta=1e6,
    rms_norm_eps=1e-6, max_position_embeddings=32768, tie_word_embeddings=True, use_sliding_window=False,
)
CONTEXT = 4096
BLOCK_SIZE = 16
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]), "source": "measured"}
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while a region is timed."""

    QUERY = (
        "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self) -> None:
        self.process = None

    def start(self) -> None:
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
        except OSError:
            self.process = None

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            out, _ = self.process.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
            out, _ = self.process.communicate()
        clocks, top, reasons = [], None, set()
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                top = float(parts[1])
            except ValueError:
                continue
            for name, flag in zip(self.NAMES, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": top,
            "reasons": sorted(reasons),
            "samples": len(clocks),
        }


def layer_linear_params(m: dict) -> int:
    h, d = m["hidden_size"], m["head_dim"]
    qkv = (m["num_attention_heads"] + 2 * m["num_key_value_heads"]) * d
    return h * qkv + m["num_attention_heads"] * d * h + 3 * h * m["intermediate_size"]


def prefill_flops(m: dict, tokens: int, wanted: int = 1) -> float:
    linear = 2.0 * tokens * layer_linear_params(m) * m["num_hidden_layers"]
    attention = 4.0 * m["head_dim"] * m["num_attention_heads"] * (tokens * (tokens + 1) / 2) * m["num_hidden_layers"]
    head = 2.0 * wanted * m["vocab_size"] * m["hidden_size"]
    return linear + attention + head


def decode_bytes(engine, cache, contexts) -> float:
    """What a decode step has to read: every weight once, and the cache of the live requests."""
    weights = engine.weight_bytes()
    if engine.config.tie_word_embeddings:
        pass  # the tied table is counted once by weight_bytes (one tensor)
    return float(weights + cache.bytes_per_token() * sum(contexts))


def standing_requests(runner, cache, batch: int, context: int, vocab: int, torch):
    """`batch` live requests that hold `context` tokens each. Their pages hold random keys and
    values (what they hold does not change a decode step's cost); returns their keys."""
    manager = cache.manager
    keys = [f"bench-{i}" for i in range(batch)]
    for key in keys:
        assert runner.begin_request(key)
        assert manager.reserve(key, context).ok
        manager.advance(key, context)
    return keys


def time_decode(engine, batch: int, steps: int, warmup: int, torch, sampling_row):
    """Device-timed decode: `warmup` + `steps` steps of `batch` single tokens ending at CONTEXT."""
    from paged_attention_engine_b200.engine.batch import StepEntry
    from paged_attention_engine_b200.kernels import ops

    start_context = CONTEXT - (warmup + steps)
    blocks = batch * (CONTEXT // BLOCK_SIZE + 1) + 8
    cache = engine.new_paged_cache(blocks, BLOCK_SIZE, max(batch, 1))
    for pool in cache.pools:
        pool.normal_(0.0, 0.5)
    runner = engine.new_runner(cache)
    keys = standing_requests(runner, cache, batch, start_context, engine.vocab_size, torch)
    gen = torch.Generator().manual_seed(batch)
    rows = [sampling_row(0.0, 0, i, 0) for i in range(batch)]
    tokens = torch.randint(0, engine.vocab_size, (warmup + steps, batch), generator=gen).tolist()

    def one(i):
        for key in keys:
            assert cache.manager.reserve(key, 1).ok
        return runner.step([StepEntry(key, (tokens[i][b],), (0,)) for b, key in enumerate(keys)], rows).tokens

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    launches_before = ops.launches
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for i in range(warmup, warmup + steps):
        one(i)
    end.record()
    torch.cuda.synchronize()
    ms = begin.elapsed_time(end) / steps
    contexts = [CONTEXT - steps // 2] * batch
    info = {
        "ms_per_step": ms,
        "tokens_per_s": batch / (ms / 1e3),
        "bytes": decode_bytes(engine, cache, contexts),
        "launches": ops.launches - launches_before,
    }
    for key in keys:
        runner.end_request(key)
    del cache, runner
    torch.cuda.empty_cache()
    return info


def time_prefill(engine, torch, repeats: int = 3):
    from paged_attention_engine_b200.engine.batch import StepEntry

    cache = engine.new_paged_cache(PREFILL_TOKENS // BLOCK_SIZE + 2, BLOCK_SIZE, 2)
    runner = engine.new_runner(cache)
    gen = torch.Generator().manual_seed(99)
    times = []
    for r in range(repeats + 1):
        ids = torch.randint(0, engine.vocab_size, (PREFILL_TOKENS,), generator=gen).tolist()
        runner.begin_request("prefill")
        assert cache.manager.reserve("prefill", PREFILL_TOKENS).ok
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        runner.step([StepEntry("prefill", ids, (PREFILL_TOKENS - 1,))])
        end.record()
        torch.cuda.synchronize()
        if r:
            times.append(begin.elapsed_time(end))
        runner.end_request("prefill")
    del cache, runner
    torch.cuda.empty_cache()
    return statistics.median(times)


def time_end_to_end(engine, batch: int, steps: int, warmup: int, torch):
    """The same decode steps through the Python entry point: requests are added with host
    token ids, prefilled by the scheduler, and every timed `step()` copies its inputs to the
    device and reads the sampled tokens back."""
    from paged_attention_engine_b200 import LLM, Request
    from paged_attention_engine_b200.kernels import ops

    # Prompts are cut into portions under the token budget, so requests start to decode a few
    # steps apart; SLACK extra tokens keep every request alive through the timed steps.
    # The prefill of 8 x 4,000 tokens runs at the power cap, and the decode steps right after it
    # are 3 to 6 % slower than steady ones for about 60 ms (measured: windows of 64 steps after
    # 8, 16 and 48 warm-up steps take 1.42, 1.38 and 1.35 ms a step, later windows 1.35): the
    # warm-up is at least 48 steps.
    SLACK = 8
    warmup = max(warmup, 48)
    prompt_len = CONTEXT - (warmup + steps) - SLACK - 1
    llm = LLM(
        engine, num_blocks=batch * (CONTEXT // BLOCK_SIZE + 1) + 8, block_size=BLOCK_SIZE,
        max_num_seqs=batch, max_num_batched_tokens=8192,
    )
    gen = torch.Generator().manual_seed(7)
    for b in range(batch):
        prompt = torch.randint(0, engine.vocab_size, (prompt_len,), generator=gen).tolist()
        assert llm.add_request(Request(f"e2e-{b}", tuple(prompt), warmup + steps + SLACK + 1))
    while llm.scheduler.waiting or any(s.num_computed < s.request.prompt_len for s in llm.scheduler.running):
        llm.step()
    for _ in range(warmup):
        llm.step()
    torch.cuda.synchronize()
    launches_before = ops.launches
    t0 = time.perf_counter()
    produced = 0
    for _ in range(steps):
        result = llm.step()
        produced += len(result.decoded)
    llm.scheduler.resolve()            # the last steps' tokens reach the host inside the timed region
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert all(min(s.generated) >= 0 for s in llm.scheduler.running)
    # Per step: the packed integer arrays of the batch (tokens, positions, starts, lengths,
    # slots, block tables) and the sampler's rows go to the device; the tokens come back.
    h2d = llm.runner.builder.bytes_uploaded      # the last step's copy: all steps of the region have this size
    d2h = 4 * batch
    return {
        "value": produced / elapsed, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
        "launches": ops.launches - launches_before,
    }


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=MODEL["num_hidden_layers"],
                        help="fewer layers than the configuration has (both numbers are reported)")
    parser.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64")
    parser.add_argument("--only", choices=("all", "decode", "prefill"), default="all",
                        help="time one part only (for profiling); the JSON line then holds that part alone")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({
            "impl": "reference",
            "unavailable": "the reference is a source tree without setup.py or pyproject.toml: "
                           "pip install --no-index --target baseline/_ref fails with 'not installable'",
        }))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(3, args.warmup)

    import torch

    from paged_attention_engine_b200.engine.llm import Engine
    from paged_attention_engine_b200.sampling import SamplingRow

    torch.cuda.set_device(0)
    model = dict(MODEL)
    model["num_hidden_layers"] = args.layers
    engine = Engine.from_random(model, seed=0, dtype="bfloat16", device="cuda:0")
    peak = peaks()

    if args.only == "prefill":
        prefill_ms = time_prefill(engine, torch)
        flops = prefill_flops(model, PREFILL_TOKENS)
        print(json.dumps({"only": "prefill", "ms": round(prefill_ms, 3), "tokens": PREFILL_TOKENS,
                          "frac": round(flops / (prefill_ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4)}))
        return 0
    if args.only == "decode":
        decode = time_decode(engine, args.batch, args.steps, warmup, torch, SamplingRow)
        print(json.dumps({"only": "decode", "batch": args.batch, "ms_per_step": round(decode["ms_per_step"], 4),
                          "tokens_per_s": round(decode["tokens_per_s"], 1), "launches": decode["launches"]}))
        return 0

    sampler = ClockSampler()
    sampler.start()
    decode = time_decode(engine, args.batch, args.steps, warmup, torch, SamplingRow)

    points = {}
    if not args.skip_points:
        for name, b in (("decode_b1", 1), ("decode_b64", 64)):
            points[name] = round(time_decode(engine, b, max(8, args.steps // 2), 3, torch, SamplingRow)["tokens_per_s"], 1)
    prefill_ms = time_prefill(engine, torch)
    e2e = time_end_to_end(engine, args.batch, args.steps, warmup, torch)
    clocks = sampler.stop()      # sampled through every timed region of this run

    flops = prefill_flops(model, PREFILL_TOKENS)
    achieved = decode["bytes"] / (decode["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": "decode tok/s at batch 8, context 4096 (Qwen2.5-1.5B shape, bf16, random weights)",
        "value": round(decode["tokens_per_s"], 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": warmup,
        "ms_per_step": round(decode["ms_per_step"], 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: random token ids, random-init weights",
        "impl": "ours",
        "config": {
            "model": "Qwen2.5-1.5B shape", "layers": args.layers, "layers_of_config": MODEL["num_hidden_layers"],
            "hidden": model["hidden_size"], "heads": model["num_attention_heads"],
            "kv_heads": model["num_key_value_heads"], "head_dim": model["head_dim"],
            "intermediate": model["intermediate_size"], "vocab": model["vocab_size"], "tied": True,
            "global_batch": args.batch, "seq_len": CONTEXT, "block_size": BLOCK_SIZE,
            "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU", "l2": "inputs larger than L2",
            "peaks": peak["source"],
        },
        "clocks": clocks,
        "e2e": {
            "value": round(e2e["value"], 1), "unit": "tokens/s",
            "h2d_bytes_per_step": e2e["h2d_bytes_per_step"], "d2h_bytes_per_step": e2e["d2h_bytes_per_step"],
        },
        "gpu_launches": decode["launches"],
        "prefill": {
            "value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
            "ms": round(prefill_ms, 3), "frac": round(flops / (prefill_ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4),
        },
        "roofline": {
            "bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
            "frac": round(achieved / peak["hbm_gbs"], 4),
        },
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
