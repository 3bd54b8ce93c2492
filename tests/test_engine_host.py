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
