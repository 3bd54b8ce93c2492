"""Sizes off the beaten path: configurations drawn from a seeded generator (head sizes in steps
of 16 from 16 to 128, any number of heads and groups, widths, intermediate sizes and
vocabularies that are no powers of two, pages of 8 to 64, windows, tied and untied heads),
each replayed in mixed portions and single tokens and compared with the plain implementation,
in bfloat16 and in float32. Whatever kernel a size falls to (tcgen05, mma.sync or CUDA cores),
the logits must agree; a size that no kernel takes must be refused with a message, not computed
wrongly."""

import random

import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def _config(seed: int) -> tuple[dict, int]:
    rng = random.Random(seed)
    head_dim = rng.choice([16, 32, 48, 64, 80, 96, 112, 128])
    kv_heads = rng.choice([1, 2, 3, 5])
    groups = rng.choice([1, 2, 3, 4, 7])
    heads = kv_heads * groups
    hidden = 8 * rng.randint(6, 40)                      # a multiple of 8 (a TMA row pitch), rarely a power of two
    if rng.random() < 0.25:
        hidden += rng.choice([2, 4, 6])                  # and sometimes not even that: the CUDA-core products
    windowed = rng.random() < 0.3
    layers = rng.randint(1, 3)
    raw = dict(
        architectures=["Qwen2ForCausalLM"], num_hidden_layers=layers, hidden_size=hidden, num_attention_heads=heads,
        num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=rng.choice([16, 24, 40, 100, 176, 250]) + 16 * rng.randint(0, 9),
        vocab_size=rng.randint(50, 1100), rope_theta=rng.choice([1e4, 5e4, 1e6]), rms_norm_eps=rng.choice([1e-6, 1e-5, 3e-6]),
        max_position_embeddings=512, tie_word_embeddings=rng.random() < 0.5, use_sliding_window=windowed,
    )
    if windowed:
        raw.update(sliding_window=rng.randint(5, 60), max_window_layers=rng.randint(0, layers - 1) if layers > 1 else 0)
    return raw, rng.choice([8, 16, 16, 32, 64])


@pytest.mark.parametrize("seed", list(range(24)))
@pytest.mark.parametrize("dtype_name", ["bfloat16", "float32"])
def test_drawn_configuration_agrees_with_the_plain_implementation(tmp_path, seed, dtype_name):
    raw, page = _config(seed)
    dtype = torch.bfloat16 if dtype_name == "bfloat16" else torch.float32
    folder = helpers.write_model(tmp_path / "model", raw, seed, dtype, sharpen=3.0)
    rng = random.Random(100 + seed)
    requests = {f"r{i}": helpers.random_tokens(raw["vocab_size"], rng.choice([3, 40, 90, 150]), 10 * seed + i) for i in range(3)}
    requests["whole"] = helpers.random_tokens(raw["vocab_size"], rng.choice([70, 130, 200]), 10 * seed + 7)
    wants = {key: helpers.plain_logits(folder, ids) for key, ids in requests.items()}
    # mixed portions and single tokens; then every request whole (long portions take other kernels)
    for trace in (helpers.trace_mixed(requests, seed=seed, live_limit=3, decode_tail=4), helpers.trace_whole(requests)):
        outputs, replayer = helpers.run_in_process(folder, dtype_name, trace, helpers.max_live_tokens(trace, 64), page)
        got = helpers.collect(trace, outputs, requests)
        for key in requests:
            gap = (got[key] - wants[key]).abs().max().item()
            assert gap <= helpers.tolerance(dtype, wants[key]), f"seed {seed} {raw} page {page}: {key} off by {gap}"


@pytest.mark.parametrize("seed", list(range(8)))
@pytest.mark.parametrize("dtype_name", ["bfloat16", "float32"])
def test_drawn_configuration_generates_under_pressure(tmp_path, seed, dtype_name):
    """Eleven requests at once through the entry point, with a pool too small for all of them
    (requests are preempted and recomputed) and decode steps that replay padded graphs: every
    step's logits are the plain model's for the engine's own token history."""
    from paged_attention_engine_b200 import LLM, EventKind, Request

    raw, page = _config(50 + seed)
    dtype = torch.bfloat16 if dtype_name == "bfloat16" else torch.float32
    folder = helpers.write_model(tmp_path / "model", raw, seed, dtype, sharpen=3.0)
    rng = random.Random(200 + seed)
    prompts = {f"q{i}": tuple(helpers.random_tokens(raw["vocab_size"], rng.randint(1, 45), 20 * seed + i)) for i in range(11)}
    new_tokens = {rid: rng.randint(6, 20) for rid in prompts}
    needs = [-(-(len(p) + new_tokens[rid]) // page) for rid, p in prompts.items()]
    pool = max(max(needs) + 2, sum(needs) * 2 // 5)
    llm = LLM.from_pretrained(folder, dtype=dtype_name, num_blocks=pool, block_size=page, max_num_seqs=12,
                              max_num_batched_tokens=64, record_logits=True)
    for rid, prompt in prompts.items():
        assert llm.add_request(Request(rid, prompt, new_tokens[rid], temperature=0.0))
    out = llm.run_to_completion()
    for rid, prompt in prompts.items():
        assert len(out[rid]) == new_tokens[rid]
        helpers.teacher_forced_check(folder, dtype, prompt, out[rid], llm.scheduler.finished[rid].step_logits)
    assert llm.cache.manager.allocators[0].num_free == pool, "every page came back"
