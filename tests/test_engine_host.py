"""Everything above the kernels, on the CPU: the engine's own configuration, loader,
parts, cache manager, batch flattening and step function, with the kernels replaced by
the plain torch stand-in of tests/torch_ops.py, replayed in every way of cutting and
compared with the plain whole-sequence implementation."""

import pytest
import torch

import helpers
import torch_ops


def _requests(vocab, lengths, seed):
    return {f"r{i}": helpers.random_tokens(vocab, n, seed * 100 + i) for i, n in enumerate(lengths)}


@pytest.fixture(scope="module", params=list(helpers.TINY))
def tiny(request, tmp_path_factory):
    raw, page, seed = helpers.TINY[request.param]
    folder = helpers.write_model(tmp_path_factory.mktemp(request.param), raw, seed, torch.float32, sharpen=4.0)
    lengths = (1, 2, 33, 47, 64, 90, 17, 70)
    requests = _requests(raw["vocab_size"], lengths, seed)
    oracle = {k: helpers.plain_logits(folder, ids) for k, ids in requests.items()}
    return folder, raw, page, requests, oracle


def _compare(folder, page, trace, requests, oracle, max_tokens):
    outputs, replayer = helpers.run_in_process(folder, "float32", trace, max_tokens, page, ops=torch_ops, device="cpu")
    got = helpers.collect(trace, outputs, requests)
    for key, ids in requests.items():
        assert got[key].shape == oracle[key].shape
        gap = (got[key] - oracle[key]).abs().max().item()
        assert gap <= helpers.tolerance(torch.float32, oracle[key]), f"{key}: max |dlogit| {gap}"
    return replayer


def test_whole(tiny):
    folder, raw, page, requests, oracle = tiny
    _compare(folder, page, helpers.trace_whole(requests), requests, oracle, 128)


def test_tail_one_by_one(tiny):
    folder, raw, page, requests, oracle = tiny
    _compare(folder, page, helpers.trace_tail(requests), requests, oracle, 128)


def test_chunks(tiny):
    folder, raw, page, requests, oracle = tiny
    _compare(folder, page, helpers.trace_chunks(requests, seed=5), requests, oracle, 128)


def test_mixed_with_reuse(tiny):
    folder, raw, page, requests, oracle = tiny
    trace = helpers.trace_mixed(requests, seed=11)
    budget = helpers.max_live_tokens(trace)
    replayer = _compare(folder, page, trace, requests, oracle, budget)
    manager = replayer.manager
    total = sum(len(v) for v in requests.values())
    assert total > budget, "the trace must need more tokens than the pool holds, so that pages are used again"
    assert not manager.live_requests()
    for allocator in manager.allocators:
        assert allocator.num_free == allocator.num_blocks


def test_one_traversal_per_step(tiny):
    folder, raw, page, requests, oracle = tiny
    trace = helpers.trace_mixed(requests, seed=3)
    _, replayer = helpers.run_in_process(
        folder, "float32", trace, helpers.max_live_tokens(trace), page, ops=torch_ops, device="cpu"
    )
    assert replayer.runner.model.forward_pass_count == len(trace)


def test_entry_point_generates_what_the_plain_implementation_does(tmp_path):
    """Requests through LLM (scheduler, executor, sampler, cache manager) on stand-in
    kernels: greedy tokens equal the plain implementation's, under a pool so small that
    requests are preempted and recomputed, and under a token budget that cuts prompts."""
    from paged_attention_engine_b200 import LLM, Engine, Request
    from plain import qwen2_plain as plain

    raw, page, seed = helpers.TINY["tiny_a"]
    folder = helpers.write_model(tmp_path / "m", raw, seed, torch.float32, sharpen=4.0)
    engine = Engine.from_pretrained(folder, "float32", device="cpu", ops=torch_ops)
    llm = LLM(engine, num_blocks=14, block_size=page, max_num_seqs=4, max_num_batched_tokens=12, record_logits=True)
    prompts = [helpers.random_tokens(256, n, 40 + n) for n in (5, 11, 17, 3)]
    for i, prompt in enumerate(prompts):
        assert llm.add_request(Request(f"p{i}", tuple(prompt), 8))
    out = llm.run_to_completion()
    cfg, weights = plain.read_config(folder), plain.read_weights(folder)
    for i, prompt in enumerate(prompts):
        want, rows = plain.generate_greedy(prompt, 8, weights, cfg)
        assert list(out[f"p{i}"]) == want
        got_rows = torch.stack(llm.scheduler.finished[f"p{i}"].step_logits)
        assert (got_rows - rows).abs().max().item() <= helpers.tolerance(torch.float32, rows)
    from paged_attention_engine_b200 import EventKind
    assert llm.scheduler.events_of(EventKind.PREEMPT), "14 pages of 4 tokens cannot hold four such requests"
    assert llm.runner.model.forward_pass_count == llm.scheduler._step


def test_temperature_sampling_does_not_depend_on_the_batch(tmp_path):
    from paged_attention_engine_b200 import LLM, Engine, Request

    raw, page, seed = helpers.TINY["tiny_b"]
    folder = helpers.write_model(tmp_path / "m", raw, seed, torch.float32)
    engine = Engine.from_pretrained(folder, "float32", device="cpu", ops=torch_ops)
    prompts = {f"t{i}": tuple(helpers.random_tokens(509, n, 60 + n)) for i, n in enumerate((1, 7, 23))}

    def run(**options):
        llm = LLM(engine, block_size=page, **options)
        for rid, prompt in prompts.items():
            llm.add_request(Request(rid, prompt, 6, temperature=0.8, seed=1234))
        return llm.run_to_completion()

    together = run(num_blocks=64)
    alone = run(num_blocks=64, max_num_seqs=1)
    squeezed = run(num_blocks=5, max_num_batched_tokens=5)
    assert together == alone == squeezed
    greedy = LLM(engine, num_blocks=64, block_size=page)
    greedy.add_request(Request("t2", prompts["t2"], 6))
    assert greedy.run_to_completion()["t2"] != together["t2"]


def test_the_step_lists_the_requests_that_bring_more_than_one_token():
    """`multi_index`: the entries that bring a portion, in their order, when some entries do and some
    bring one token; None when all or none do (the portion kernels then cover every request)."""
    from paged_attention_engine_b200.cache.manager import CacheManager, KVGroupSpec
    from paged_attention_engine_b200.engine.batch import BatchBuilder, StepEntry

    manager = CacheManager((KVGroupSpec(num_kv_heads=1, head_dim=16, window=0, entries=(0,)),), 32, 8, 8)
    builder = BatchBuilder(manager, torch_ops, torch.float32, "cpu", 100)

    def build(lengths):
        entries = []
        for i, n in enumerate(lengths):
            manager.create_request(i)
            assert manager.reserve(i, n).ok
            entries.append(StepEntry(i, list(range(1, n + 1)), (n - 1,)))
        ctx = builder.build(entries)
        for i in range(len(lengths)):
            manager.free_request(i)
        return ctx

    mixed = build([1, 5, 1, 1, 9, 2, 1])
    assert mixed.multi_index.tolist() == [1, 4, 5] and mixed.num_single == 4
    assert build([1, 1, 1]).multi_index is None
    assert build([4, 2]).multi_index is None
    # the other integers lie where they did
    assert mixed.q_start.tolist() == [0, 1, 6, 7, 8, 17, 19, 20] and mixed.logit_rows.tolist() == [0, 5, 6, 7, 16, 18, 19]
