"""The layer sizes of the Qwen2.5-1.5B shape (hidden 1536, 12 heads over 2 kv heads of 128,
intermediate 8960, vocabulary 151936, tied head, theta 1e6), with two layers so that it stays
quick: the kernels at the sizes they are tuned for (tcgen05 products and attention, split
sums, SwiGLU in the epilogue), cut into portions and decoded, against the plain implementation
run on the GPU in float32. The same for the layer sizes of the 7B shape (hidden 3584, 28 heads
over 4 kv heads, intermediate 18944, untied head of 152064) and of the 32B shape (hidden 5120,
40 over 8, intermediate 27648, eps 1e-5), which the measured request streams run at."""

import pytest
import torch

import helpers
from faulty_ops import RecordingOps
from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

SHAPE = dict(
    architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=1536, num_attention_heads=12,
    num_key_value_heads=2, head_dim=128, intermediate_size=8960, vocab_size=151936, rope_theta=1e6,
    rms_norm_eps=1e-6, max_position_embeddings=32768, tie_word_embeddings=True, use_sliding_window=False,
)


SHAPE_7B = dict(
    architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=3584, num_attention_heads=28,
    num_key_value_heads=4, head_dim=128, intermediate_size=18944, vocab_size=152064, rope_theta=1e6,
    rms_norm_eps=1e-6, max_position_embeddings=32768, tie_word_embeddings=False, use_sliding_window=False,
)
SHAPE_32B = dict(
    architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=5120, num_attention_heads=40,
    num_key_value_heads=8, head_dim=128, intermediate_size=27648, vocab_size=152064, rope_theta=1e6,
    rms_norm_eps=1e-5, max_position_embeddings=32768, tie_word_embeddings=False, use_sliding_window=False,
)
LARGER = {"7b": SHAPE_7B, "32b": SHAPE_32B}


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    return helpers.write_model(tmp_path_factory.mktemp("real_shape"), SHAPE, 3, torch.bfloat16, sharpen=2.0)


@pytest.fixture(scope="module")
def oracle(folder):
    cfg = plain.read_config(folder)
    weights = {k: v.float().cuda() for k, v in plain.read_weights(folder).items()}
    requests = {"long": helpers.random_tokens(SHAPE["vocab_size"], 700, 1), "short": helpers.random_tokens(SHAPE["vocab_size"], 150, 2)}
    logits = {}
    for key, ids in requests.items():
        ids_gpu = torch.tensor(ids, device="cuda")
        hidden = plain.forward_hidden(ids_gpu, weights, cfg)
        rows = list(range(0, len(ids), 37)) + [len(ids) - 1]
        logits[key] = (rows, plain.linear(hidden[rows], plain.lm_head_weight(weights)).float().cpu())
    del weights
    torch.cuda.empty_cache()
    return requests, logits


@pytest.mark.parametrize("dtype_name", ["bfloat16", "float32"])
def test_portions_and_decoding_at_the_real_layer_sizes(folder, oracle, dtype_name):
    from paged_attention_engine_b200.engine.llm import Engine
    from paged_attention_engine_b200.engine.replay import Replayer
    from paged_attention_engine_b200.kernels import ops

    requests, logits = oracle
    dtype = torch.bfloat16 if dtype_name == "bfloat16" else torch.float32
    engine = Engine.from_pretrained(folder, dtype_name)
    replayer = Replayer(engine, max_tokens=1024, block_size=16)
    # `long`: a portion of 400 (tcgen05 attention and persistent products in bfloat16), one of 236
    # beside the whole of `short`, then single tokens; logits wanted at every 37th place.
    long_ids, short_ids = requests["long"], requests["short"]
    wanted = {key: set(rows) for key, (rows, _) in logits.items()}

    def entry(key, ids, start, count):
        want = [i for i in range(count) if start + i in wanted[key]]
        return {"id": key, "tokens": ids[start : start + count], "want": want}

    steps = [
        {"step": 0, "entries": [entry("long", long_ids, 0, 400)], "end": []},
        {"step": 1, "entries": [entry("long", long_ids, 400, 236), entry("short", short_ids, 0, 150)], "end": ["short"]},
    ]
    for i in range(636, 700):
        steps.append({"step": len(steps), "entries": [entry("long", long_ids, i, 1)], "end": ["long"] if i == 699 else []})
    got = {key: [] for key in requests}
    for record in steps:
        out = replayer.run(record)
        ops.check_device_errors()
        at = 0
        for e in record["entries"]:
            n = len(e["want"])
            if n:
                got[e["id"]].append(out[at : at + n].float().cpu())
                at += n
    for key, (rows, want) in logits.items():
        have = torch.cat(got[key])
        assert have.shape == want.shape
        gap = (have - want).abs().max().item()
        assert gap <= helpers.tolerance(dtype, want), f"{dtype_name}/{key}: max |dlogit| {gap:.3e} vs {helpers.tolerance(dtype, want):.3e}"


@pytest.mark.parametrize("dtype_name", ["bfloat16", "float32"])
def test_short_portions_after_a_long_one_at_the_real_layer_sizes(folder, dtype_name):
    """A prompt of 1,800 tokens whose first 1,280 come in one step and the rest in portions of
    192, 100 (beside another request's decoded tokens) and 228: the later portions are few query
    tiles over many keys, which the bfloat16 attention shares out over clusters of blocks."""
    from paged_attention_engine_b200.engine.llm import Engine
    from paged_attention_engine_b200.engine.replay import Replayer
    from paged_attention_engine_b200.kernels import ops

    dtype = torch.bfloat16 if dtype_name == "bfloat16" else torch.float32
    cfg = plain.read_config(folder)
    weights = {k: v.float().cuda() for k, v in plain.read_weights(folder).items()}
    ids = {"far": helpers.random_tokens(SHAPE["vocab_size"], 1800, 5), "near": helpers.random_tokens(SHAPE["vocab_size"], 90, 6)}
    rows = {"far": [1279, 1300, 1471, 1472, 1571, 1572, 1700, 1799], "near": [79, 80, 81, 82, 89]}
    want = {}
    for key in ids:
        hidden = plain.forward_hidden(torch.tensor(ids[key], device="cuda"), weights, cfg)
        want[key] = plain.linear(hidden[rows[key]], plain.lm_head_weight(weights)).float().cpu()
    del weights, hidden
    torch.cuda.empty_cache()

    recording = RecordingOps(ops)
    engine = Engine.from_pretrained(folder, dtype_name, ops=recording)
    replayer = Replayer(engine, max_tokens=2048, block_size=16)

    def entry(key, start, count):
        return {"id": key, "tokens": ids[key][start : start + count], "want": [r - start for r in rows[key] if start <= r < start + count]}

    steps = [
        [entry("far", 0, 1280), entry("near", 0, 80)],
        [entry("far", 1280, 192), entry("near", 80, 1)],
        [entry("far", 1472, 100), entry("near", 81, 1)],
        [entry("far", 1572, 228), entry("near", 82, 8)],
    ]
    got = {key: [] for key in ids}
    clusters = []
    for i, entries in enumerate(steps):
        out = replayer.run({"step": i, "entries": entries, "end": ["far", "near"] if i == len(steps) - 1 else []})
        ops.check_device_errors()
        if dtype_name == "bfloat16":
            clusters.append(recording.attention_calls[-1]["cluster"])
        at = 0
        for e in entries:
            n = len(e["want"])
            if n:
                got[e["id"]].append(out[at : at + n].float().cpu())
                at += n
    if dtype_name == "bfloat16":
        assert clusters[0] == 1 and min(clusters[1:]) >= 2, clusters
    for key in ids:
        have = torch.cat(got[key])
        assert have.shape == want[key].shape
        gap = (have - want[key]).abs().max().item()
        assert gap <= helpers.tolerance(dtype, want[key]), f"{dtype_name}/{key}: max |dlogit| {gap:.3e} vs {helpers.tolerance(dtype, want[key]):.3e}"


def test_a_long_prompt_whole_then_decoded_at_the_real_layer_sizes(folder):
    """8,192 tokens in one step (enough blocks that the paired tcgen05 attention is picked), then
    16 tokens one by one over the 8,192 keys (decode slices and their merge), in bfloat16."""
    from paged_attention_engine_b200.engine.llm import Engine
    from paged_attention_engine_b200.engine.replay import Replayer
    from paged_attention_engine_b200.kernels import ops

    cfg = plain.read_config(folder)
    weights = {k: v.float().cuda() for k, v in plain.read_weights(folder).items()}
    ids = helpers.random_tokens(SHAPE["vocab_size"], 8192 + 16, 9)
    rows = [0, 127, 128, 4095, 4096, 8191] + list(range(8192, 8192 + 16))
    hidden = plain.forward_hidden(torch.tensor(ids, device="cuda"), weights, cfg)
    want = plain.linear(hidden[rows], plain.lm_head_weight(weights)).float().cpu()
    del weights, hidden
    torch.cuda.empty_cache()

    recording = RecordingOps(ops)
    engine = Engine.from_pretrained(folder, "bfloat16", ops=recording)
    replayer = Replayer(engine, max_tokens=8192 + 64, block_size=16)
    got = [replayer.run({"step": 0, "entries": [{"id": "r", "tokens": ids[:8192], "want": rows[:6]}], "end": []}).float().cpu()]
    assert recording.attention_calls[-1] == {"kernel": "tcgen05", "cluster": 0}       # the paired kernel
    for i in range(16):
        step = {"step": 1 + i, "entries": [{"id": "r", "tokens": [ids[8192 + i]], "want": [0]}], "end": ["r"] if i == 15 else []}
        got.append(replayer.run(step).float().cpu())
    ops.check_device_errors()
    have = torch.cat(got)
    gap = (have - want).abs().max().item()
    assert gap <= helpers.tolerance(torch.bfloat16, want), f"max |dlogit| {gap:.3e} vs {helpers.tolerance(torch.bfloat16, want):.3e}"


@pytest.fixture(scope="module", params=list(LARGER))
def larger(request, tmp_path_factory):
    """(folder, shape, requests, rows and float32 logits of the plain model at those rows)."""
    import json

    from safetensors.torch import save_file

    from paged_attention_engine_b200.config import resolve
    from paged_attention_engine_b200.weights import random_tensors

    shape = LARGER[request.param]
    folder = tmp_path_factory.mktemp(f"shape_{request.param}")
    # Drawn on the GPU (gigabytes of normal variates take the CPU a minute) and written as a folder.
    # q and k are left as drawn: at these widths the scores already spread as far as the sharpened
    # ones of the 1.5B shape do (their deviation grows with the hidden size).
    tensors = random_tensors(shape, 5, torch.bfloat16, "cuda")
    save_file({k: v.cpu().contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    (folder / "config.json").write_text(json.dumps(resolve(shape)[0].to_dict()))
    del tensors
    cfg = plain.read_config(folder)
    weights = {k: v.float().cuda() for k, v in plain.read_weights(folder).items()}
    requests = {"long": helpers.random_tokens(shape["vocab_size"], 520, 21), "short": helpers.random_tokens(shape["vocab_size"], 100, 22)}
    logits = {}
    for key, ids in requests.items():
        hidden = plain.forward_hidden(torch.tensor(ids, device="cuda"), weights, cfg)
        rows = list(range(0, len(ids), 41)) + list(range(len(ids) - 24, len(ids)))
        rows = sorted(set(rows))
        logits[key] = (rows, plain.linear(hidden[rows], plain.lm_head_weight(weights)).float().cpu())
    del weights, hidden
    torch.cuda.empty_cache()
    yield folder, shape, requests, logits
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype_name", ["bfloat16", "float32"])
def test_portions_and_decoding_at_the_larger_layer_sizes(larger, dtype_name):
    """One long portion, a portion beside another request's whole prompt, a portion of 70 beside
    decoded tokens, then single tokens (two requests in a step, so products of 2 rows), with the
    products' K of 3584/5120 and 18944/27648 and query heads in groups of 7 and 5."""
    from paged_attention_engine_b200.engine.llm import Engine
    from paged_attention_engine_b200.engine.replay import Replayer
    from paged_attention_engine_b200.kernels import ops

    folder, shape, requests, logits = larger
    dtype = torch.bfloat16 if dtype_name == "bfloat16" else torch.float32
    engine = Engine.from_pretrained(folder, dtype_name)
    replayer = Replayer(engine, max_tokens=768, block_size=16)
    ids = requests
    wanted = {key: set(rows) for key, (rows, _) in logits.items()}

    def entry(key, start, count):
        want = [i for i in range(count) if start + i in wanted[key]]
        return {"id": key, "tokens": ids[key][start : start + count], "want": want}

    steps = [
        [entry("long", 0, 300)],
        [entry("long", 300, 126), entry("short", 0, 76)],
        [entry("long", 426, 70), entry("short", 76, 1)],
    ]
    for i in range(23):
        steps.append([entry("long", 496 + i, 1), entry("short", 77 + i, 1)])
    steps.append([entry("long", 519, 1)])
    got = {key: [] for key in requests}
    for i, entries in enumerate(steps):
        out = replayer.run({"step": i, "entries": entries, "end": ["long", "short"] if i == len(steps) - 1 else []})
        ops.check_device_errors()
        at = 0
        for e in entries:
            n = len(e["want"])
            if n:
                got[e["id"]].append(out[at : at + n].float().cpu())
                at += n
    for key, (rows, want) in logits.items():
        have = torch.cat(got[key])
        assert have.shape == want.shape
        assert torch.isfinite(have).all()
        gap = (have - want).abs().max().item()
        assert gap <= helpers.tolerance(dtype, want), f"{dtype_name}/{key}: max |dlogit| {gap:.3e} vs {helpers.tolerance(dtype, want):.3e}"
    del engine, replayer
    torch.cuda.empty_cache()
