"""Measurement: decoded tokens a second at batch 8 (and 1, 64), prefill of 2,048 tokens,
and the fraction of the roofline, for the Qwen2.5-1.5B shape with random weights in
bfloat16 on one B200; plus the two request streams at the 7B and the 32B shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

It prints ONE JSON line. `value` is decoded tokens a second of K decode steps timed on
the device (CUDA events) through the engine's step function and device sampler, the
requests standing at the context length of the configuration: the median of three
passes of K steps, with the passes' range beside it. `e2e` is the same through the
Python entry point (`LLM.add_request` / `step`), host tokens in and out.

The method follows the reference's harness (bench/run.py:68-73,628-702): warm-up
discarded, three timed passes, median and range, a flag when the range exceeds 20 % of
the median, and the provenance (GPU, driver, torch) in the line.

`--impl reference` runs the reference's own engine (its unmodified `engine/` package,
from `baseline/_ref/`) through its own scheduler in its fused mode, at the same batch
and context, and prints the same line with `"impl": "reference"`.
"""

from __future__ import annotations

import argparse
import json
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
# The shapes of the two request streams (the reference's `mixed` and `control` streams,
# bench/workload.py:241-272, at the sizes of Qwen2.5-7B and Qwen2.5-32B).
MODEL_7B = dict(
    architectures=["Qwen2ForCausalLM"], num_hidden_layers=28, hidden_size=3584, num_attention_heads=28,
    num_key_value_heads=4, head_dim=128, intermediate_size=18944, vocab_size=152064, rope_theta=1e6,
    rms_norm_eps=1e-6, max_position_embeddings=32768, tie_word_embeddings=False, use_sliding_window=False,
)
MODEL_32B = dict(
    architectures=["Qwen2ForCausalLM"], num_hidden_layers=64, hidden_size=5120, num_attention_heads=40,
    num_key_value_heads=8, head_dim=128, intermediate_size=27648, vocab_size=152064, rope_theta=1e6,
    rms_norm_eps=1e-5, max_position_embeddings=32768, tie_word_embeddings=False, use_sliding_window=False,
)
CONTEXT = 4096
BLOCK_SIZE = 16
PREFILL_TOKENS = 2048
PASSES = 3
SPREAD_LIMIT = 0.20            # bench/run.py:68-73 of the reference
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


def provenance(torch) -> dict:
    """GPU, driver and torch, as the reference's `Provenance` records them (bench/run.py:231-317)."""
    driver = None
    try:
        out = subprocess.run(["nvidia-smi", "-i", "0", "--query-gpu=driver_version", "--format=csv,noheader"],
                             capture_output=True, text=True, timeout=20)
        driver = out.stdout.strip().splitlines()[0] if out.stdout.strip() else None
    except (OSError, subprocess.SubprocessError):
        pass
    return {"gpu": torch.cuda.get_device_name(0), "driver": driver, "torch": torch.__version__,
            "cuda": torch.version.cuda}


def summary(values: list[float]) -> dict:
    """Median and range of the passes; `spread_flag` when the range exceeds 20 % of the median."""
    mid = statistics.median(values)
    return {"median": mid, "min": min(values), "max": max(values),
            "spread_flag": bool(mid > 0 and (max(values) - min(values)) / mid > SPREAD_LIMIT)}


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
    """What a decode step has to read: every weight once (a tied table is one tensor and is
    counted once), and the cache of the live requests."""
    return float(engine.weight_bytes(len(contexts)) + cache.bytes_per_token() * sum(contexts))


def time_decode(engine, batch: int, steps: int, warmup: int, torch, sampling_row, passes: int = PASSES, context: int = CONTEXT):
    """Device-timed decode: `warmup` steps, then `passes` passes of `steps` steps of `batch`
    single tokens, the last pass ending at `context`. Returns the passes' ms per step and what
    the median pass read."""
    from paged_attention_engine_b200.engine.batch import StepEntry
    from paged_attention_engine_b200.kernels import ops

    total = warmup + passes * steps
    start_context = context - total
    blocks = batch * (context // BLOCK_SIZE + 1) + 8
    cache = engine.new_paged_cache(blocks, BLOCK_SIZE, max(batch, 1))
    for pool in cache.pools:
        pool.normal_(0.0, 0.5)       # what the pages hold does not change a decode step's cost
    runner = engine.new_runner(cache)
    manager = cache.manager
    keys = [f"bench-{i}" for i in range(batch)]
    for key in keys:
        assert runner.begin_request(key)
        assert manager.reserve(key, start_context).ok
        manager.advance(key, start_context)
    gen = torch.Generator().manual_seed(batch)
    rows = [sampling_row(0.0, 0, i, 0) for i in range(batch)]
    tokens = torch.randint(0, engine.vocab_size, (total, batch), generator=gen).tolist()

    def one(i):
        for key in keys:
            assert manager.reserve(key, 1).ok
        return runner.step([StepEntry(key, (tokens[i][b],), (0,)) for b, key in enumerate(keys)], rows).tokens

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    per_pass, launches = [], 0
    for p in range(passes):
        launches_before = ops.launches
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for i in range(warmup + p * steps, warmup + (p + 1) * steps):
            one(i)
        end.record()
        torch.cuda.synchronize()
        per_pass.append(begin.elapsed_time(end) / steps)
        launches = ops.launches - launches_before
    ops.check_device_errors()
    stats = summary(per_pass)
    middle = sorted(range(passes), key=lambda p: per_pass[p])[passes // 2]
    context = start_context + warmup + middle * steps + steps // 2
    info = {
        "ms_per_step": stats["median"], "ms_min": stats["min"], "ms_max": stats["max"],
        "spread_flag": stats["spread_flag"],
        "tokens_per_s": batch / (stats["median"] / 1e3),
        "bytes": decode_bytes(engine, cache, [context] * batch),
        "launches": launches,
    }
    for key in keys:
        runner.end_request(key)
    del cache, runner
    torch.cuda.empty_cache()
    return info


def time_prefill(engine, torch, repeats: int = PASSES, tokens: int = PREFILL_TOKENS):
    from paged_attention_engine_b200.engine.batch import StepEntry

    cache = engine.new_paged_cache(tokens // BLOCK_SIZE + 2, BLOCK_SIZE, 2)
    runner = engine.new_runner(cache)
    gen = torch.Generator().manual_seed(99)
    times = []
    for r in range(repeats + 2):
        ids = torch.randint(0, engine.vocab_size, (tokens,), generator=gen).tolist()
        runner.begin_request("prefill")
        assert cache.manager.reserve("prefill", tokens).ok
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        runner.step([StepEntry("prefill", ids, (tokens - 1,))])
        end.record()
        torch.cuda.synchronize()
        if r >= 2:
            times.append(begin.elapsed_time(end))
        runner.end_request("prefill")
    del cache, runner
    torch.cuda.empty_cache()
    return summary(times)


def time_products(model: dict, tokens: int, torch, peak: dict, copies: int = 28) -> list[dict]:
    """The four matrix products of a decoder layer for a step of `tokens` tokens, with what a step
    runs around them (norm before, rotation and page write, SiLU x up, residual after), each
    `copies` times in a row on weights of their own (nothing is found in L2), recorded into a
    CUDA graph and replayed: microseconds per product, for the kernels the engine picks and for
    the tcgen05 products with their summing kernels alone."""
    from paged_attention_engine_b200.kernels import ops

    dev = "cuda:0"
    hidden, inter = model["hidden_size"], model["intermediate_size"]
    heads, kv_heads, d = model["num_attention_heads"], model["num_key_value_heads"], model["head_dim"]
    gen = torch.Generator(device=dev).manual_seed(0)

    def bf(*shape, std=1.0):
        return (torch.randn(*shape, device=dev, generator=gen) * std).to(torch.bfloat16)

    x, xi, res, attn = bf(tokens, hidden), bf(tokens, inter, std=0.3), bf(tokens, hidden), bf(tokens, heads * d)
    gamma = torch.rand(hidden, device=dev, generator=gen) + 0.5
    nq = (heads + 2 * kv_heads) * d
    wq = [bf(nq, hidden, std=0.02) for _ in range(copies)]
    bq = torch.randn(nq, device=dev, generator=gen)
    wo = [bf(hidden, heads * d, std=0.02) for _ in range(copies)]
    wgu = [ops.interleave_gate_up(bf(inter, hidden, std=0.02), bf(inter, hidden, std=0.02)) for _ in range(copies)]
    wd = [bf(hidden, inter, std=0.02) for _ in range(copies)]
    table = torch.randn(tokens, d, device=dev, generator=gen)
    page = BLOCK_SIZE
    keys = torch.zeros(tokens // page + 2, kv_heads, page, d, dtype=torch.bfloat16, device=dev)
    values = torch.zeros_like(keys)
    slots = torch.arange(tokens, dtype=torch.int32, device=dev)
    flush = torch.empty(512 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def qkv():
        for w in wq:
            ops.materialized(ops.qkv_projection(ops.rms_norm(x, gamma, 1e-6), w, bq, table, slots, keys, values, heads, kv_heads, d, page))

    def o():
        for w in wo:      # the sum of a split product is part of the norm that follows it: run that norm, too
            ops.materialized(ops.rms_norm(ops.linear(attn, w, residual=res), gamma, 1e-6))

    def gate_up():
        for w in wgu:
            ops.materialized(ops.linear_swiglu(ops.rms_norm(x, gamma, 1e-6), w))

    def down():
        for w in wd:
            ops.materialized(ops.linear(xi, w, residual=res))

    def layer():
        for i in range(copies):
            ops.qkv_projection(ops.rms_norm(x, gamma, 1e-6), wq[i], bq, table, slots, keys, values, heads, kv_heads, d, page)
            r = ops.linear(attn, wo[i], residual=res)
            a = ops.linear_swiglu(ops.rms_norm(r, gamma, 1e-6), wgu[i])
            ops.materialized(ops.linear(a, wd[i], residual=r))

    def replayed(fn) -> float:
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            fn()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(7):
            flush.zero_()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            graph.replay()
            end.record()
            torch.cuda.synchronize()
            times.append(begin.elapsed_time(end) * 1e3 / copies)
        return statistics.median(times)

    groups = (("q|k|v", qkv, nq * hidden), ("o", o, hidden * heads * d), ("gate|up", gate_up, 2 * inter * hidden), ("down", down, hidden * inter),
              ("the four in a row", layer, nq * hidden + hidden * heads * d + 3 * inter * hidden))
    rows = []
    for name, fn, weights in groups:
        row = {"only": "products", "product": name, "tokens": tokens, "weight_mb": round(weights * 2 / 1e6, 1),
               "us_at_hbm_peak": round(weights * 2 / peak["hbm_gbs"] / 1e3, 2)}
        for label, few in (("us", True), ("us_tcgen05_chain", False)):
            ops.use_few_token_products = few
            try:
                row[label] = round(replayed(fn), 2)
            finally:
                ops.use_few_token_products = True
        rows.append(row)
    return rows


def time_end_to_end(engine, batch: int, steps: int, warmup: int, torch):
    """The same decode steps through the Python entry point: requests are added with host
    token ids, prefilled by the scheduler, and every timed `step()` copies its inputs to the
    device and reads the sampled tokens back. Three passes of `steps` steps; the median."""
    from paged_attention_engine_b200 import LLM, Request
    from paged_attention_engine_b200.kernels import ops

    # Prompts are cut into portions under the token budget, so requests start to decode a few
    # steps apart; SLACK extra tokens keep every request alive through the timed steps.
    # The prefill of 8 x 4,000 tokens runs at the power cap, and the decode steps right after it
    # are 3 to 6 % slower than steady ones for about 60 ms: the warm-up is at least 48 steps.
    SLACK = 8
    warmup = max(warmup, 48)
    total = warmup + PASSES * steps
    prompt_len = CONTEXT - total - SLACK - 1
    llm = LLM(
        engine, num_blocks=batch * (CONTEXT // BLOCK_SIZE + 1) + 8, block_size=BLOCK_SIZE,
        max_num_seqs=batch, max_num_batched_tokens=8192,
    )
    gen = torch.Generator().manual_seed(7)
    for b in range(batch):
        prompt = torch.randint(0, engine.vocab_size, (prompt_len,), generator=gen).tolist()
        assert llm.add_request(Request(f"e2e-{b}", tuple(prompt), total + SLACK + 1))
    while llm.scheduler.waiting or any(s.num_computed < s.request.prompt_len for s in llm.scheduler.running):
        llm.step()
    for _ in range(warmup):
        llm.step()
    llm.scheduler.resolve()
    torch.cuda.synchronize()
    rates, launches = [], 0
    for _ in range(PASSES):
        launches_before = ops.launches
        t0 = time.perf_counter()
        produced = 0
        for _ in range(steps):
            result = llm.step()
            produced += len(result.decoded)
        llm.scheduler.resolve()            # the last steps' tokens reach the host inside the timed region
        torch.cuda.synchronize()
        rates.append(produced / (time.perf_counter() - t0))
        launches = ops.launches - launches_before
    assert all(min(s.generated) >= 0 for s in llm.scheduler.running)
    stats = summary(rates)
    # Per step: the packed integer arrays of the batch (tokens, positions, starts, lengths,
    # slots, block tables) and the sampler's rows go to the device; the tokens come back.
    h2d = llm.runner.builder.bytes_uploaded      # the last step's copy: all steps of the region have this size
    return {"value": stats["median"], "min": stats["min"], "max": stats["max"], "spread_flag": stats["spread_flag"],
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * batch, "launches": launches}


# --------------------------------------------------------------------------------------- #
# Request streams through the scheduler (the reference's driver loop: bench/run.py:463-528)
# --------------------------------------------------------------------------------------- #

def run_stream(engine, stream, num_blocks: int, max_num_seqs: int, budget: int, torch):
    """Adds every request, runs the scheduler dry, and reports what the reference's harness
    reports for a level: generated tokens a second over the whole stream (prefill included),
    steps, preemptions; and the tokens, for comparing two runs."""
    from paged_attention_engine_b200 import LLM, Request
    from paged_attention_engine_b200.engine.scheduler import EventKind
    from paged_attention_engine_b200.kernels import ops

    llm = LLM(engine, num_blocks=num_blocks, block_size=BLOCK_SIZE, max_num_seqs=max_num_seqs,
              max_num_batched_tokens=budget)
    accepted = 0
    for i, (prompt, decode) in enumerate(stream):
        accepted += bool(llm.add_request(Request(f"req-{i}", tuple(prompt), decode)))
    torch.cuda.synchronize()
    started = time.perf_counter()
    out = llm.run_to_completion()
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - started
    ops.check_device_errors()
    generated = sum(len(v) for v in out.values())
    info = {
        "tokens_per_s": generated / elapsed, "seconds": elapsed, "generated": generated, "accepted": accepted,
        "steps": llm.scheduler._step, "preemptions": len(llm.scheduler.events_of(EventKind.PREEMPT)),
        "tokens": out,
    }
    del llm
    torch.cuda.empty_cache()
    return info


def near_tie(engine, prompt, first, second, at: int, torch) -> bool:
    """Whether two greedy runs that part at output `at` part at a near tie: both tokens' logits,
    for the common history, within twice the bfloat16 budget of the tests (2^-5 of the largest
    logit's magnitude) of each other."""
    from paged_attention_engine_b200.engine.batch import StepEntry

    history = list(prompt) + list(first[:at])
    cache = engine.new_paged_cache(len(history) // BLOCK_SIZE + 2, BLOCK_SIZE, 2)
    runner = engine.new_runner(cache, use_graphs=False)
    assert runner.begin_request("tie") and cache.manager.reserve("tie", len(history)).ok
    logits = runner.step([StepEntry("tie", history, (len(history) - 1,))]).logits[0].float()
    gap = abs(float(logits[first[at]]) - float(logits[second[at]]))
    limit = 2.0 * 2.0 ** -5 * max(1.0, float(logits.abs().max()))
    runner.end_request("tie")
    return gap <= limit


def stream_7b(torch, layers: int) -> dict:
    """256 seeded requests, prompts U[16, 2048], decodes U[8, 1024], 64 at a time, 8,192 tokens a
    step (bench/workload.py:241-254). Twice: with a pool in which 64 requests of the longest kind
    fit (12,352 pages of 16 tokens, 11.3 GB at this shape), and with the reference's pool of 3,584
    pages (engine/cache.py:29-35), which 64 such requests overflow, so that many are preempted
    and recomputed."""
    from paged_attention_engine_b200.cli import synthetic_stream
    from paged_attention_engine_b200.engine.llm import Engine

    model = dict(MODEL_7B, num_hidden_layers=layers)
    engine = Engine.from_random(model, seed=0, dtype="bfloat16", device="cuda:0")
    stream = synthetic_stream("mixed", 0, 256, model["vocab_size"], smoke=False)
    roomy_pages = 64 * (3072 // BLOCK_SIZE + 1)
    info = run_stream(engine, stream, roomy_pages, 64, 8192, torch)
    tight = run_stream(engine, stream, 3584, 64, 8192, torch)
    from paged_attention_engine_b200.sampling import SamplingRow

    step = time_decode(engine, 64, 24, 8, torch, SamplingRow, passes=PASSES, context=1024)
    out = {
        "decode_7b_b64_ctx1024": round(step["tokens_per_s"], 1),
        "decode_7b_b64_ctx1024_hbm_frac": round(step["bytes"] / (step["ms_per_step"] / 1e3) / 1e9 / peaks()["hbm_gbs"], 4),
        "stream_7b_tok_s": round(info["tokens_per_s"], 1), "stream_7b_seconds": round(info["seconds"], 2),
        "stream_7b_generated": info["generated"], "stream_7b_steps": info["steps"],
        "stream_7b_preemptions": info["preemptions"], "stream_7b_pages": roomy_pages,
        "stream_7b_pool3584_tok_s": round(tight["tokens_per_s"], 1), "stream_7b_pool3584_steps": tight["steps"],
        "stream_7b_pool3584_preemptions": tight["preemptions"],
        "stream_7b_weight_gb": round(engine.weight_bytes() / 1e9, 2),
        "stream_7b_layers": layers, "stream_7b_layers_of_config": MODEL_7B["num_hidden_layers"],
    }
    del engine
    torch.cuda.empty_cache()
    return out


def pressure_32b(torch, layers: int) -> dict:
    """64 requests of 512 + 512 tokens at once under a pool of 3,584 pages, which 64 x 1,024
    tokens (4,096 pages) do not fit into: requests are preempted and recomputed
    (bench/workload.py:256-272). The same stream then runs with a pool that never preempts, and
    the tokens of the two runs are compared request by request; where they part, the two
    tokens' logits are checked to be a near tie (a recomputed prefix is rounded otherwise than
    a decoded one, so greedy tokens may part where two logits nearly tie, and only there)."""
    from paged_attention_engine_b200.cli import synthetic_stream
    from paged_attention_engine_b200.engine.llm import Engine

    model = dict(MODEL_32B, num_hidden_layers=layers)
    engine = Engine.from_random(model, seed=0, dtype="bfloat16", device="cuda:0")
    stream = synthetic_stream("control", 0, 64, model["vocab_size"], smoke=False)
    tight = run_stream(engine, stream, 3584, 64, 8192, torch)
    roomy = run_stream(engine, stream, 64 * (1024 // BLOCK_SIZE + 1) + 8, 64, 8192, torch)
    equal, parted, ties = 0, [], 0
    for i, (prompt, _) in enumerate(stream):
        a, b = tight["tokens"][f"req-{i}"], roomy["tokens"][f"req-{i}"]
        if a == b:
            equal += 1
            continue
        at = next(k for k in range(min(len(a), len(b))) if a[k] != b[k])
        parted.append(at)
        ties += bool(near_tie(engine, prompt, b, a, at, torch))
    from paged_attention_engine_b200.sampling import SamplingRow

    step = time_decode(engine, 64, 16, 8, torch, SamplingRow, passes=PASSES, context=1024)
    out = {
        "decode_32b_b64_ctx1024": round(step["tokens_per_s"], 1),
        "decode_32b_b64_ctx1024_hbm_frac": round(step["bytes"] / (step["ms_per_step"] / 1e3) / 1e9 / peaks()["hbm_gbs"], 4),
        "pressure_32b_tok_s": round(tight["tokens_per_s"], 1), "pressure_32b_seconds": round(tight["seconds"], 2),
        "pressure_32b_steps": tight["steps"], "pressure_32b_preemptions": tight["preemptions"],
        "pressure_32b_unpressured_tok_s": round(roomy["tokens_per_s"], 1),
        "pressure_32b_unpressured_preemptions": roomy["preemptions"],
        "pressure_32b_requests_equal": equal, "pressure_32b_requests_parted": len(parted),
        "pressure_32b_parted_at_near_ties": ties,
        "pressure_32b_weight_gb": round(engine.weight_bytes() / 1e9, 2),
        "pressure_32b_layers": layers, "pressure_32b_layers_of_config": MODEL_32B["num_hidden_layers"],
    }
    del engine
    torch.cuda.empty_cache()
    return out


def config_record(model: dict, batch: int, peak_source: str) -> dict:
    """The sizes of the run, flat; the same record for both arms."""
    return {
        "model": "Qwen2.5-1.5B shape", "layers": model["num_hidden_layers"], "layers_of_config": MODEL["num_hidden_layers"],
        "hidden": model["hidden_size"], "heads": model["num_attention_heads"],
        "kv_heads": model["num_key_value_heads"], "head_dim": model["head_dim"],
        "intermediate": model["intermediate_size"], "vocab": model["vocab_size"], "tied": True,
        "global_batch": batch, "seq_len": CONTEXT, "block_size": BLOCK_SIZE,
        "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU", "l2": "inputs larger than L2",
        "peaks": peak_source, "passes": PASSES,
    }


# --------------------------------------------------------------------------------------- #
# The reference arm
# --------------------------------------------------------------------------------------- #

def reference_tree() -> Path | None:
    for candidate in (ROOT / "baseline" / "_ref", Path("/root/reference")):
        if (candidate / "engine" / "model.py").is_file() and (candidate / "engine" / "scheduler.py").is_file():
            return candidate
    return None


def run_reference(args) -> dict:
    """The unmodified reference: its `Qwen2Engine` over random bfloat16 weights of the same shape
    and init, its `BlockAllocator`, paged cache, `Qwen2Executor` and `Scheduler` in FUSED mode
    (README.md:27-44 of the reference), batch 8 prefilled so that the timed `step()` calls decode
    at context 4,096. Nothing of this repository's package is imported."""
    tree = reference_tree()
    if tree is None:
        return {"impl": "reference", "unavailable": "baseline/_ref/engine (a copy of the reference's engine package) is not there"}
    sys.path.insert(0, str(tree))
    import torch
    from engine.cache import BlockAllocator
    from engine.model import LayerWeights, ModelDims, Qwen2Engine, Qwen2Weights
    from engine.scheduler import ExecutionMode, Qwen2Executor, Request, Scheduler

    torch.cuda.set_device(0)
    device = torch.device("cuda:0")
    m = dict(MODEL)
    m["num_hidden_layers"] = args.layers
    batch, steps = args.batch, args.steps
    warmup = max(3, args.warmup, 48)
    gen = torch.Generator(device=device).manual_seed(0)

    def normal(*shape, mean=0.0):
        return (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * 0.02 + mean).to(torch.bfloat16)

    h, d, nh, nkv, inter = m["hidden_size"], m["head_dim"], m["num_attention_heads"], m["num_key_value_heads"], m["intermediate_size"]
    layers = tuple(
        LayerWeights(
            q_proj_weight=normal(nh * d, h), q_proj_bias=normal(nh * d),
            k_proj_weight=normal(nkv * d, h), k_proj_bias=normal(nkv * d),
            v_proj_weight=normal(nkv * d, h), v_proj_bias=normal(nkv * d),
            o_proj_weight=normal(h, nh * d),
            gate_proj_weight=normal(inter, h), up_proj_weight=normal(inter, h), down_proj_weight=normal(h, inter),
            input_layernorm_weight=normal(h, mean=1.0), post_attention_layernorm_weight=normal(h, mean=1.0),
        )
        for _ in range(m["num_hidden_layers"])
    )
    embed = normal(m["vocab_size"], h)
    dims = ModelDims(num_layers=m["num_hidden_layers"], num_heads=nh, num_kv_heads=nkv, head_dim=d, hidden_size=h,
                     rms_norm_eps=m["rms_norm_eps"], vocab_size=m["vocab_size"], rope_theta=m["rope_theta"])
    engine = Qwen2Engine(Qwen2Weights(embed, layers, normal(h, mean=1.0), embed), dims, device, torch.bfloat16)
    allocator = BlockAllocator(num_blocks=batch * (CONTEXT // BLOCK_SIZE + 1) + 8, block_size=BLOCK_SIZE)
    cache = engine.new_paged_cache(allocator.num_blocks, allocator.block_size)
    scheduler = Scheduler(Qwen2Executor(engine, cache, allocator), allocator, mode=ExecutionMode.FUSED,
                          max_num_seqs=batch, max_num_batched_tokens=8192)
    SLACK = 8
    total = warmup + PASSES * steps
    prompt_len = CONTEXT - total - SLACK - 1
    host = torch.Generator().manual_seed(7)
    for b in range(batch):
        prompt = torch.randint(0, m["vocab_size"], (prompt_len,), generator=host).tolist()
        assert scheduler.add_request(Request(f"ref-{b}", tuple(prompt), total + SLACK + 1))

    sampler = ClockSampler()
    sampler.start()
    with torch.inference_mode():
        while scheduler.waiting:
            scheduler.step()
        for _ in range(warmup):
            scheduler.step()
        torch.cuda.synchronize()
        device_ms, wall_rates = [], []
        for _ in range(PASSES):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            produced = 0
            t0 = time.perf_counter()
            begin.record()
            for _ in range(steps):
                produced += len(scheduler.step().decoded)
            end.record()
            torch.cuda.synchronize()
            wall_rates.append(produced / (time.perf_counter() - t0))
            device_ms.append(begin.elapsed_time(end) / steps)
            assert produced == batch * steps, f"{produced} tokens in {steps} steps of {batch}"
    clocks = sampler.stop()
    dev, wall = summary(device_ms), summary(wall_rates)
    pages = -(-CONTEXT // BLOCK_SIZE)
    return {
        "metric": "decode tok/s at batch 8, context 4096 (Qwen2.5-1.5B shape, bf16, random weights)",
        "value": round(batch / (dev["median"] / 1e3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(dev["median"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random token ids, random-init weights",
        "impl": "reference",
        "config": config_record(m, batch, peaks()["source"]),
        "path": "Scheduler(FUSED) + Qwen2Executor + BlockAllocator of the unmodified reference",
        "range_ms": [round(dev["min"], 4), round(dev["max"], 4)], "spread_flag": dev["spread_flag"],
        "clocks": clocks,
        "e2e": {
            "value": round(wall["median"], 1), "unit": "tokens/s", "min": round(wall["min"], 1), "max": round(wall["max"], 1),
            # per row and step: two block tables and the ids, positions and lengths as 64-bit
            # integers go up (engine/attention.py:374-385, engine/model.py:437-446 of the reference);
            # one 64-bit token comes back (engine/scheduler.py:610)
            "h2d_bytes_per_step": batch * (2 * pages * 8 + 32), "d2h_bytes_per_step": batch * 8,
        },
        "gpu_launches": 0,
        "provenance": provenance(torch),
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
    parser.add_argument("--skip-streams", action="store_true", help="leave out the 7B stream and the 32B pressure run")
    parser.add_argument("--layers-7b", type=int, default=MODEL_7B["num_hidden_layers"])
    parser.add_argument("--layers-32b", type=int, default=MODEL_32B["num_hidden_layers"])
    parser.add_argument("--shape", choices=("1.5b", "7b", "32b"), default="1.5b",
                        help="layer sizes for --only decode / prefill (the headline line is always the 1.5B shape)")
    parser.add_argument("--context", type=int, default=CONTEXT, help="context length for --only decode")
    parser.add_argument("--tokens", type=int, default=PREFILL_TOKENS, help="prompt length for --only prefill")
    parser.add_argument("--only", choices=("all", "decode", "prefill", "products", "stream7b", "pressure32b"), default="all",
                        help="time one part only (for profiling); the JSON line then holds that part alone")
    args = parser.parse_args()

    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        try:
            line = run_reference(args)
        except Exception as exc:  # noqa: BLE001  (the arm reports why it could not run)
            line = {"impl": "reference", "unavailable": f"{type(exc).__name__}: {exc}"[:400]}
        print(json.dumps(line))
        return 0
    warmup = max(3, args.warmup)

    import torch

    from paged_attention_engine_b200.engine.llm import Engine
    from paged_attention_engine_b200.sampling import SamplingRow

    torch.cuda.set_device(0)
    peak = peaks()
    if args.only == "stream7b":
        print(json.dumps(stream_7b(torch, args.layers_7b)))
        return 0
    if args.only == "pressure32b":
        print(json.dumps(pressure_32b(torch, args.layers_32b)))
        return 0
    if args.only == "products":
        for row in time_products({"1.5b": MODEL, "7b": MODEL_7B, "32b": MODEL_32B}[args.shape], args.batch, torch, peak):
            print(json.dumps(row))
        return 0

    model = dict({"1.5b": MODEL, "7b": MODEL_7B, "32b": MODEL_32B}[args.shape] if args.only != "all" else MODEL)
    if args.only != "all" and args.shape != "1.5b" and args.layers == MODEL["num_hidden_layers"]:
        args.layers = model["num_hidden_layers"]
    model["num_hidden_layers"] = args.layers
    engine = Engine.from_random(model, seed=0, dtype="bfloat16", device="cuda:0")

    if args.only == "prefill":
        prefill = time_prefill(engine, torch, tokens=args.tokens)
        flops = prefill_flops(model, args.tokens)
        print(json.dumps({"only": "prefill", "shape": args.shape, "layers": args.layers, "ms": round(prefill["median"], 3),
                          "tokens": args.tokens, "tflops": round(flops / (prefill["median"] / 1e3) / 1e12, 1),
                          "frac": round(flops / (prefill["median"] / 1e3) / (peak["bf16_tflops"] * 1e12), 4)}))
        return 0
    if args.only == "decode":
        decode = time_decode(engine, args.batch, args.steps, warmup, torch, SamplingRow, context=args.context)
        gbs = decode["bytes"] / (decode["ms_per_step"] / 1e3) / 1e9
        print(json.dumps({"only": "decode", "shape": args.shape, "layers": args.layers, "batch": args.batch,
                          "context": args.context, "ms_per_step": round(decode["ms_per_step"], 4),
                          "tokens_per_s": round(decode["tokens_per_s"], 1), "gb_per_step": round(decode["bytes"] / 1e9, 3),
                          "hbm_frac": round(gbs / peak["hbm_gbs"], 4), "launches": decode["launches"]}))
        return 0

    sampler = ClockSampler()
    sampler.start()
    decode = time_decode(engine, args.batch, args.steps, warmup, torch, SamplingRow)

    points: dict = {}
    flags = ["decode"] if decode["spread_flag"] else []
    if not args.skip_points:
        for name, b in (("decode_b1", 1), ("decode_b64", 64)):
            point = time_decode(engine, b, max(32, args.steps), max(8, warmup), torch, SamplingRow)
            points[name] = round(point["tokens_per_s"], 1)
            points[name + "_hbm_frac"] = round(point["bytes"] / (point["ms_per_step"] / 1e3) / 1e9 / peak["hbm_gbs"], 4)
            if point["spread_flag"]:
                flags.append(name)
    prefill = time_prefill(engine, torch)
    if prefill["spread_flag"]:
        flags.append("prefill")
    e2e = time_end_to_end(engine, args.batch, args.steps, warmup, torch)
    if e2e["spread_flag"]:
        flags.append("e2e")
    clocks = sampler.stop()      # sampled through every timed region of the headline numbers
    weight_bytes = engine.weight_bytes()
    del engine
    torch.cuda.empty_cache()

    if not args.skip_streams:
        for name, run, layers in (("stream_7b", stream_7b, args.layers_7b), ("pressure_32b", pressure_32b, args.layers_32b)):
            try:
                points.update(run(torch, layers))
            except Exception as exc:  # noqa: BLE001  (a failed stream must not lose the headline)
                points[name + "_error"] = f"{type(exc).__name__}: {exc}"[:300]
                torch.cuda.empty_cache()

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
        "config": config_record(model, args.batch, peak["source"]),
        "range_ms": [round(decode["ms_min"], 4), round(decode["ms_max"], 4)],
        "spread_flags": flags,
        "clocks": clocks,
        "e2e": {
            "value": round(e2e["value"], 1), "unit": "tokens/s", "min": round(e2e["min"], 1), "max": round(e2e["max"], 1),
            "h2d_bytes_per_step": e2e["h2d_bytes_per_step"], "d2h_bytes_per_step": e2e["d2h_bytes_per_step"],
        },
        "gpu_launches": decode["launches"],
        "prefill": {
            "value": round(PREFILL_TOKENS / (prefill["median"] / 1e3), 1), "tokens": PREFILL_TOKENS,
            "ms": round(prefill["median"], 3), "ms_min": round(prefill["min"], 3), "ms_max": round(prefill["max"], 3),
            "frac": round(flops / (prefill["median"] / 1e3) / (peak["bf16_tflops"] * 1e12), 4),
        },
        "roofline": {
            "bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
            "frac": round(achieved / peak["hbm_gbs"], 4), "weight_gb": round(weight_bytes / 1e9, 3),
        },
        "points": points,
        "provenance": provenance(torch),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
