"""Shared pieces of the tests: tiny configurations, model folders, traces, tolerances."""

from __future__ import annotations

import json
import random
from pathlib import Path

import torch

from plain import qwen2_plain as plain

# --------------------------------------------------------------------------- #
# Tolerances, fixed here and nowhere else.
#
# float32: engine and oracle compute the same float32 formulas in different orders
# of summation. The reference allows 1e-3 at |logit| ~ 22 and measures 3e-5
# (conftest.py:87-93 of the reference); these tiny models have logits of a few units,
# so 5e-5 relative to max(1, max |logit|) leaves about that margin.
#
# bfloat16: the engine rounds activations to bfloat16 where the reference's model
# dtype would (residual stream, projections, attention output, feed-forward); the
# reference's own half-precision budget is 4 ulp of the logit's magnitude
# (tests/test_parity_fp16.py:178 of the reference: 6.25e-2 at 22 in float16). 4 ulp
# of bfloat16 at magnitude m is m * 2**-5.
#
# Between two runs of the ENGINE that cut the same tokens differently only the order
# of float32 sums inside attention changes, then one rounding to the engine dtype:
# CUT_ATOL bounds that.
# --------------------------------------------------------------------------- #
FP32_RTOL = 5e-5
BF16_RTOL = 2.0 ** -5


def tolerance(dtype: torch.dtype, reference_logits: torch.Tensor) -> float:
    top = max(1.0, float(reference_logits.abs().max()))
    return (FP32_RTOL if dtype == torch.float32 else BF16_RTOL) * top


# --------------------------------------------------------------------------- #
# Tiny configurations. A and B are the two of the task's baseline; C adds a window
# on its later layers, so that it has two page groups. They differ in every size.
# --------------------------------------------------------------------------- #
TINY_A = dict(
    architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
    num_key_value_heads=2, head_dim=16, intermediate_size=176, vocab_size=256, rope_theta=10000.0,
    rms_norm_eps=1e-6, max_position_embeddings=128, tie_word_embeddings=True, use_sliding_window=False,
)
TINY_B = dict(
    architectures=["Qwen2ForCausalLM"], num_hidden_layers=3, hidden_size=96, num_attention_heads=3,
    num_key_value_heads=1, head_dim=32, intermediate_size=256, vocab_size=509, rope_theta=1e6,
    rms_norm_eps=1e-5, max_position_embeddings=256, tie_word_embeddings=False, use_sliding_window=False,
)
TINY_C = dict(
    architectures=["Qwen2ForCausalLM"], num_hidden_layers=4, hidden_size=80, num_attention_heads=5,
    num_key_value_heads=5, head_dim=48, intermediate_size=112, vocab_size=300, rope_theta=5e4,
    rms_norm_eps=3e-6, max_position_embeddings=512, tie_word_embeddings=False, use_sliding_window=True,
    sliding_window=24, max_window_layers=2,
)
# D is wide enough for the tensor-core kernels' other forms: head_dim 64 (tcgen05 attention for long
# portions), K of 256 and 512 (products whose K is split, the LM head among them).
TINY_D = dict(
    architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=256, num_attention_heads=4,
    num_key_value_heads=2, head_dim=64, intermediate_size=512, vocab_size=1000, rope_theta=1e6,
    rms_norm_eps=1e-6, max_position_embeddings=512, tie_word_embeddings=True, use_sliding_window=False,
)
TINY = {"tiny_a": (TINY_A, 4, 0), "tiny_b": (TINY_B, 16, 1), "tiny_c": (TINY_C, 8, 2), "tiny_d": (TINY_D, 16, 3)}  # config, page size, seed


def decoder_layer(mixer_norm, mixer, feed_forward_norm, feed_forward):
    """A `LayerSpec` of the usual arrangement: norm, mixer, add; norm, feed-forward, add."""
    from paged_attention_engine_b200.config import LayerSpec

    return LayerSpec("pre_norm_residual", dict(
        mixer_norm=mixer_norm, mixer=mixer, feed_forward_norm=feed_forward_norm, feed_forward=feed_forward))


def write_model(folder: Path, raw: dict, seed: int, dtype: torch.dtype, sharpen: float = 1.0) -> Path:
    """A random model folder; `sharpen` scales every q and k projection so that attention
    scores spread out and one wrong, missing or extra key changes the logits visibly."""
    from safetensors.torch import load_file, save_file

    from paged_attention_engine_b200.weights import write_random_model

    write_random_model(folder, raw, seed, dtype)
    if sharpen != 1.0:
        path = str(Path(folder) / "model.safetensors")
        tensors = load_file(path)
        for name in list(tensors):
            if ".q_proj." in name or ".k_proj." in name:
                tensors[name] = (tensors[name].float() * sharpen).to(tensors[name].dtype)
        save_file(tensors, path)
    return Path(folder)


def plain_logits(folder: Path, token_ids) -> torch.Tensor:
    """The oracle: float32 logits [tokens, vocab] of one whole sequence, weights as stored."""
    cfg = plain.read_config(folder)
    weights = {k: v.float() for k, v in plain.read_weights(folder).items()}
    return plain.forward_logits(list(token_ids), weights, cfg)


def teacher_forced_check(folder, dtype, prompt, tokens, step_logits):
    """Greedy tokens may differ between precisions where two logits nearly tie; what must hold is
    that every step's logits are those of the plain model for the engine's own token history."""
    oracle = plain_logits(folder, list(prompt) + list(tokens))[len(prompt) - 1 : -1]
    got = torch.stack(step_logits)
    gap = (got - oracle).abs().max().item()
    assert gap <= tolerance(dtype, oracle), f"max |dlogit| {gap}"
    margin = 2 * tolerance(dtype, oracle)
    for row, token in zip(oracle, tokens):
        assert row[token].item() >= row.max().item() - margin, "the sampled token is not the plain model's best"


def random_tokens(vocab: int, count: int, seed: int) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count,), generator=gen).tolist()


# --------------------------------------------------------------------------- #
# Traces. A trace is a list of step records as bin/trace_run reads them. Every
# builder wants the logits of EVERY token it feeds, so whole sequences are compared.
# --------------------------------------------------------------------------- #

def _entry(key, tokens, want_all=True):
    return {"id": key, "tokens": list(tokens), "want": list(range(len(tokens))) if want_all else []}


def trace_whole(requests: dict[str, list[int]], first_step: int = 0) -> list[dict]:
    """Each request alone and whole."""
    return [
        {"step": first_step + i, "entries": [_entry(key, ids)], "end": [key]}
        for i, (key, ids) in enumerate(requests.items())
    ]


def trace_tail(requests: dict[str, list[int]], tail: int = 32, first_step: int = 0) -> list[dict]:
    """Most of a request in one step, its last `tail` tokens one by one."""
    out, step = [], first_step
    for key, ids in requests.items():
        head = max(1, len(ids) - tail)
        out.append({"step": step, "entries": [_entry(key, ids[:head])], "end": []})
        step += 1
        for i in range(head, len(ids)):
            out.append({"step": step, "entries": [_entry(key, ids[i : i + 1])], "end": [key] if i == len(ids) - 1 else []})
            step += 1
        if head == len(ids):
            out[-1]["end"] = [key]
    return out


def trace_chunks(requests: dict[str, list[int]], seed: int, first_step: int = 0) -> list[dict]:
    """Portions of changing size, down to two tokens, one request at a time."""
    rng = random.Random(seed)
    out, step = [], first_step
    for key, ids in requests.items():
        at = 0
        sizes = [7, 2, 13, 2, 5, 3, 16, 1, 2, 31, 4, 17, 2, 9]
        rng.shuffle(sizes)
        i = 0
        while at < len(ids):
            n = min(sizes[i % len(sizes)], len(ids) - at)
            i += 1
            out.append({"step": step, "entries": [_entry(key, ids[at : at + n])], "end": [key] if at + n == len(ids) else []})
            at += n
            step += 1
    return out


def trace_mixed(requests: dict[str, list[int]], seed: int, live_limit: int = 4, decode_tail: int = 12,
                first_step: int = 0) -> list[dict]:
    """Up to `live_limit` live requests; portions of some beside single tokens of others; a
    request sits a step out now and then; a finished request makes room for the next."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: dict[str, int] = {}        # key -> tokens fed so far
    out, step = [], first_step
    while waiting or live:
        while waiting and len(live) < live_limit and (not live or rng.random() < 0.7):
            key, _ = waiting.pop(0)
            live[key] = 0
        entries, ended = [], []
        for key in list(live):
            ids = requests[key]
            fed = live[key]
            if len(live) > 1 and rng.random() < 0.15:
                continue            # left out of this step, goes on later
            left = len(ids) - fed
            if left <= decode_tail:
                n = 1
            else:
                n = min(left - decode_tail, rng.choice([2, 2, 3, 5, 8, 13, 21, 34]))
            entries.append(_entry(key, ids[fed : fed + n]))
            live[key] = fed + n
            if fed + n == len(ids):
                ended.append(key)
                del live[key]
        if entries:
            out.append({"step": step, "entries": entries, "end": ended})
            step += 1
    return out


def collect(trace: list[dict], outputs: dict[int, torch.Tensor], requests: dict[str, list[int]]) -> dict[str, torch.Tensor]:
    """Stitches the per-step logits back into one [tokens, vocab] tensor per request."""
    rows: dict[str, list[torch.Tensor]] = {k: [] for k in requests}
    for record in trace:
        if record["step"] not in outputs:
            continue
        block = outputs[record["step"]]
        at = 0
        for e in record["entries"]:
            n = len(e["want"])
            assert e["want"] == list(range(len(e["tokens"]))), "collect() expects every place to be wanted"
            rows[e["id"]].append(block[at : at + n])
            at += n
        assert at == block.shape[0]
    return {k: torch.cat(v) for k, v in rows.items() if v}


def max_live_tokens(trace: list[dict], page: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to `page`."""
    held: dict[str, int] = {}
    worst = 0
    for record in trace:
        for e in record["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-n // page) * page for n in held.values()))
        for key in record["end"]:
            held.pop(key, None)
    return worst


def fragment_pool(manager, seed: int) -> None:
    """Leaves every group's free list in a shuffled order (the reference's `_fragment_pool`,
    tests/test_parity.py:196-223): placeholder requests take every page, one page each round
    robin, and give them back in a seeded random order; freed pages queue up at the back, so
    the next requests get pages that are neither adjacent nor ascending."""
    rng = random.Random(seed)
    holders = [f"__fragment_{i}" for i in range(manager.slots.num_free)]
    for key in holders:
        assert manager.create_request(key) is not None
    taken = True
    while taken:
        taken = False
        for key in holders:
            if manager.num_free > 0 and manager.reserve(key, manager.block_size).ok:
                taken = True
    assert manager.num_free == 0
    rng.shuffle(holders)
    for key in holders:
        manager.free_request(key)
    assert manager.num_free == manager.num_blocks


def run_in_process(folder: Path, dtype: str, trace: list[dict], max_tokens: int, block_size: int, ops=None, device="cuda:0",
                   prepare=None, watch=None):
    """Replays a trace through the engine's Replayer in this process; returns (outputs, replayer).
    `prepare(replayer)` runs before the first step, `watch(replayer, record)` after every step and
    before the step's finished requests give their pages back."""
    from paged_attention_engine_b200.engine.llm import Engine
    from paged_attention_engine_b200.engine.replay import Replayer

    engine = Engine.from_pretrained(folder, dtype, device=device, ops=ops)
    replayer = Replayer(engine, max_tokens, block_size)
    if prepare is not None:
        prepare(replayer)
    outputs = {}
    for record in trace:
        if watch is None:
            logits = replayer.run(record)
        else:
            logits = replayer.run(dict(record, end=[]))
            watch(replayer, record)
            replayer.run({"step": record["step"], "entries": [], "end": record.get("end", [])})
        if logits is not None:
            outputs[record["step"]] = logits.float().cpu()
    return outputs, replayer


def run_trace_program(folder: Path, dtype: str, trace: list[dict], max_tokens: int, out_dir: Path, vocab: int,
                      block_size: int = 16, timeout: int = 900) -> dict[int, torch.Tensor]:
    """Replays a trace through bin/trace_run as a user would, one step after each `done`."""
    import subprocess
    import sys

    import numpy as np

    program = Path(__file__).resolve().parent.parent / "bin" / "trace_run"
    process = subprocess.Popen(
        [sys.executable, str(program), "--model", str(folder), "--dtype", dtype, "--out", str(out_dir),
         "--max-tokens", str(max_tokens), "--block-size", str(block_size)],
        stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True,
    )
    try:
        for record in trace:
            process.stdin.write(json.dumps(record) + "\n")
            process.stdin.flush()
            answer = process.stdout.readline().strip()
            assert answer == f"done {record['step']}", f"trace_run answered {answer!r}"
        process.stdin.close()
        assert process.wait(timeout=timeout) == 0
    finally:
        if process.poll() is None:
            process.kill()
    outputs = {}
    for record in trace:
        wanted = sum(len(e["want"]) for e in record["entries"])
        path = out_dir / f"{record['step']}.f32"
        if wanted:
            data = np.fromfile(str(path), dtype="<f4")
            assert data.size == wanted * vocab, f"{path}: {data.size} floats for {wanted} x {vocab}"
            outputs[record["step"]] = torch.from_numpy(data.reshape(wanted, vocab).copy())
        else:
            assert not path.exists()
    return outputs


def records_steps() -> bool:
    """Whether runners record steps as CUDA graphs here: not on the checked build of the kernels
    (PAE_BOUNDS=1), which hands its limits to the libraries between launches."""
    from paged_attention_engine_b200.kernels import ops

    return not ops.bounds_checked
