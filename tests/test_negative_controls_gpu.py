"""Negative controls: the comparison with the plain model must FAIL when the engine is
wrong. One layer's attention is given a damaged block table or a shortened context
(tests/faulty_ops.py), in float32 and in bfloat16, at two tiny configurations and at the
layer sizes of the 1.5B shape; every time the logits must leave the tolerance that the
positive tests hold them to. The same runs without a fault stay inside it."""

import pytest
import torch

import helpers
from faulty_ops import FaultyOps
from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
REAL = dict(
    architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=1536, num_attention_heads=12,
    num_key_value_heads=2, head_dim=128, intermediate_size=8960, vocab_size=151936, rope_theta=1e6,
    rms_norm_eps=1e-6, max_position_embeddings=32768, tie_word_embeddings=True, use_sliding_window=False,
)
CASES = {
    # name: (configuration, page size, seed, sharpen, prompt tokens, decoded tokens, keys dropped)
    "tiny_a": (helpers.TINY_A, 4, 0, 4.0, 60, 12, 8),
    "tiny_b": (helpers.TINY_B, 16, 1, 4.0, 150, 12, 32),
    "real": (REAL, 16, 3, 2.0, 300, 8, 64),
}


@pytest.fixture(scope="module", params=list(CASES))
def case(request, tmp_path_factory):
    raw, page, seed, sharpen, prompt, decoded, drop = CASES[request.param]
    folder = helpers.write_model(tmp_path_factory.mktemp(f"neg_{request.param}"), raw, seed, torch.bfloat16, sharpen=sharpen)
    ids = helpers.random_tokens(raw["vocab_size"], prompt + decoded, 40 + seed)
    cfg = plain.read_config(folder)
    weights = {k: v.float().cuda() for k, v in plain.read_weights(folder).items()}
    hidden = plain.forward_hidden(torch.tensor(ids, device="cuda"), weights, cfg)
    # The first pages' rows too: attention does not depend on the ORDER of the keys it sees, so two
    # pages that change places show only at the queries that stand inside them (the causal rule
    # goes by a key's place in the table), and one wrong page among many is a small part of a
    # late query's keys but most of an early one's.
    rows = sorted(set(range(min(3 * page, prompt))) | set(range(max(0, prompt - 8), prompt + decoded)))
    oracle = plain.linear(hidden[rows], plain.lm_head_weight(weights)).float().cpu()
    del weights, hidden
    torch.cuda.empty_cache()
    return request.param, folder, raw, page, ids, prompt, rows, oracle, drop


def _run(case, dtype_name, fault, layer):
    from paged_attention_engine_b200.engine.llm import Engine
    from paged_attention_engine_b200.engine.replay import Replayer
    from paged_attention_engine_b200.kernels import ops

    name, folder, raw, page, ids, prompt, rows, oracle, drop = case
    wrapped = FaultyOps(ops, raw["num_hidden_layers"], layer, fault, drop) if fault else None
    engine = Engine.from_pretrained(folder, dtype_name, ops=wrapped)
    replayer = Replayer(engine, max_tokens=len(ids) + 64, block_size=page)
    replayer.runner.use_graphs = False          # the fault is put in by host code at every call
    got = [replayer.run({"step": 0, "entries": [{"id": "r", "tokens": ids[:prompt], "want": [r for r in rows if r < prompt]}], "end": []}).float().cpu()]
    for i in range(prompt, len(ids)):
        got.append(replayer.run({"step": i, "entries": [{"id": "r", "tokens": [ids[i]], "want": [0]}], "end": []}).float().cpu())
    ops.check_device_errors()
    gap = (torch.cat(got) - oracle).abs().max().item()
    made = wrapped.faults_made if wrapped else 0
    del engine, replayer
    torch.cuda.empty_cache()
    return gap, made


@pytest.mark.parametrize("dtype_name", list(DTYPES))
def test_without_a_fault_the_run_is_inside_the_tolerance(case, dtype_name):
    gap, _ = _run(case, dtype_name, None, 0)
    assert gap <= helpers.tolerance(DTYPES[dtype_name], case[7]), f"{case[0]}/{dtype_name}: {gap}"


@pytest.mark.parametrize("fault", ["swap_pages", "wrong_page", "drop_tile"])
@pytest.mark.parametrize("dtype_name", list(DTYPES))
def test_a_fault_in_one_layer_leaves_the_tolerance(case, dtype_name, fault):
    """The fault sits in the LAST layer only (the least a fault can be: every other layer, the
    cache and all other keys are right)."""
    last = case[2]["num_hidden_layers"] - 1
    gap, made = _run(case, dtype_name, fault, last)
    limit = helpers.tolerance(DTYPES[dtype_name], case[7])
    assert made > 0, "the fault was never put in"
    print(f"{case[0]}/{dtype_name}/{fault}: max |dlogit| {gap:.4f} = {gap / limit:.1f} x the tolerance")
    assert gap > limit, f"{case[0]}/{dtype_name}/{fault}: max |dlogit| {gap:.4f} is inside the tolerance {limit:.4f}: the tolerance does not bite"
