"""Replay on the GPU, through the engine's own kernels, in float32 and bfloat16, against
the plain whole-sequence implementation: each request alone and whole; most of it in one
step and the last 32 tokens one by one; portions of changing size down to two tokens;
and mixed, up to four live requests with so few pages that they are used again."""

import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
LENGTHS = (1, 2, 33, 47, 64, 90, 17, 70)


@pytest.fixture(scope="module", params=[(c, d) for c in helpers.TINY for d in DTYPES], ids=lambda p: f"{p[0]}-{p[1]}")
def case(request, tmp_path_factory):
    name, dtype_name = request.param
    raw, page, seed = helpers.TINY[name]
    dtype = DTYPES[dtype_name]
    folder = helpers.write_model(tmp_path_factory.mktemp(f"{name}_{dtype_name}"), raw, seed, dtype, sharpen=4.0)
    requests = {f"r{i}": helpers.random_tokens(raw["vocab_size"], n, seed * 100 + i) for i, n in enumerate(LENGTHS)}
    oracle = {k: helpers.plain_logits(folder, ids) for k, ids in requests.items()}
    return folder, raw, page, dtype_name, requests, oracle


def _compare(case, trace, max_tokens):
    folder, raw, page, dtype_name, requests, oracle = case
    outputs, replayer = helpers.run_in_process(folder, dtype_name, trace, max_tokens, page)
    got = helpers.collect(trace, outputs, requests)
    worst = 0.0
    for key in requests:
        assert got[key].shape == oracle[key].shape
        assert torch.isfinite(got[key]).all()
        gap = (got[key] - oracle[key]).abs()
        limit = helpers.tolerance(DTYPES[dtype_name], oracle[key])
        if gap.max().item() > limit:
            row = int(torch.nonzero(gap.max(dim=1).values > limit)[0])
            raise AssertionError(f"{key}: max |dlogit| {gap.max().item():.3e} > {limit:.3e}; first wrong token at place {row}")
        worst = max(worst, gap.max().item())
    return got, replayer


def test_whole(case):
    _compare(case, helpers.trace_whole(case[4]), 128)


def test_tail_one_by_one(case):
    _compare(case, helpers.trace_tail(case[4]), 128)


def test_chunks(case):
    _compare(case, helpers.trace_chunks(case[4], seed=5), 128)


def test_mixed_with_reuse(case):
    requests = case[4]
    trace = helpers.trace_mixed(requests, seed=11)
    budget = helpers.max_live_tokens(trace)
    assert sum(len(v) for v in requests.values()) > budget
    _, replayer = _compare(case, trace, budget)
    assert replayer.runner.model.forward_pass_count == len(trace)
    for allocator in replayer.manager.allocators:
        assert allocator.num_free == allocator.num_blocks


def test_mixed_on_a_fragmented_pool(case):
    """The mixed replay again, started on a pool whose free list is shuffled: the requests' pages
    are neither adjacent nor ascending (asserted: some block table must be non-monotonic, as in
    the reference's tests/test_parity.py:318-321), and the logits are those of the plain model."""
    folder, raw, page, dtype_name, requests, oracle = case
    trace = helpers.trace_mixed(requests, seed=17)
    budget = helpers.max_live_tokens(trace)
    tables = []

    def watch(replayer, record):
        for key in replayer.manager.live_requests():
            for group in range(len(replayer.manager.allocators)):
                tables.append(replayer.manager.block_table(key, group))

    outputs, replayer = helpers.run_in_process(
        folder, dtype_name, trace, budget, page, prepare=lambda r: helpers.fragment_pool(r.manager, seed=3), watch=watch)
    got = helpers.collect(trace, outputs, requests)
    for key in requests:
        gap = (got[key] - oracle[key]).abs().max().item()
        assert gap <= helpers.tolerance(DTYPES[dtype_name], oracle[key]), f"{key}: {gap}"
    long_tables = [[p for p in t if p >= 0] for t in tables]
    long_tables = [t for t in long_tables if len(t) >= 3]
    assert long_tables, "no request held three pages at once"
    assert any(t != sorted(t) for t in long_tables), "every block table was ascending: the pool was not fragmented"
    assert any(max(abs(a - b) for a, b in zip(t, t[1:])) > 1 for t in long_tables), "all pages were adjacent"
    for allocator in replayer.manager.allocators:
        assert allocator.num_free == allocator.num_blocks


def test_cuts_agree_with_each_other(case):
    """The same tokens cut in two ways give the same logits up to the rounding of sums."""
    folder, raw, page, dtype_name, requests, oracle = case
    a, _ = _compare(case, helpers.trace_whole(requests), 128)
    b, _ = _compare(case, helpers.trace_mixed(requests, seed=23), helpers.max_live_tokens(helpers.trace_mixed(requests, seed=23)))
    for key in requests:
        top = max(1.0, float(oracle[key].abs().max()))
        limit = (2e-5 if dtype_name == "float32" else 2.0 ** -6) * top
        assert (a[key] - b[key]).abs().max().item() <= limit


@pytest.mark.parametrize("dtype_name", list(DTYPES))
def test_trace_run_program(dtype_name, tmp_path):
    """bin/trace_run as a user runs it: JSON lines in, `done` lines and .f32 files out."""
    raw, page, seed = helpers.TINY["tiny_b"]
    folder = helpers.write_model(tmp_path / "model", raw, seed, DTYPES[dtype_name], sharpen=4.0)
    requests = {f"q{i}": helpers.random_tokens(raw["vocab_size"], n, 900 + i) for i, n in enumerate((40, 3, 75, 58, 21))}
    trace = helpers.trace_mixed(requests, seed=2)
    trace.append({"step": trace[-1]["step"] + 1, "entries": [{"id": "z", "tokens": [1, 2, 3], "want": []}], "end": ["z"]})
    outputs = helpers.run_trace_program(
        folder, dtype_name, trace, helpers.max_live_tokens(trace), tmp_path / "out", raw["vocab_size"]
    )
    got = helpers.collect(trace[:-1], outputs, requests)
    for key, ids in requests.items():
        oracle = helpers.plain_logits(folder, ids)
        gap = (got[key] - oracle).abs().max().item()
        assert gap <= helpers.tolerance(DTYPES[dtype_name], oracle), f"{key}: {gap}"
