"""Schedules that the other GPU tests do not reach: decode-only steps of more than 64
requests (every product takes another form beyond 64 rows, graphs pad the batch to
multiples of 8); decoders that wait a step for want of token budget while their last token
is still on the device; a windowed model with heads of 128 through the entry point under a
pool so small that the window's pages are given back and used again; and the error word of
the kernels' bounded waits, which the generation path must look at."""

import pytest
import torch

import helpers
from faulty_ops import RecordingOps
from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
REAL = dict(
    architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=1536, num_attention_heads=12,
    num_key_value_heads=2, head_dim=128, intermediate_size=8960, vocab_size=151936, rope_theta=1e6,
    rms_norm_eps=1e-6, max_position_embeddings=32768, tie_word_embeddings=True, use_sliding_window=False,
)
# Every layer windowed (one page group), heads of 128, pages of 16: the tcgen05 attention with
# table entries that the window has left behind.
WINDOWED = dict(
    architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=256, num_attention_heads=2,
    num_key_value_heads=1, head_dim=128, intermediate_size=512, vocab_size=1000, rope_theta=1e6,
    rms_norm_eps=1e-6, max_position_embeddings=1024, tie_word_embeddings=True, use_sliding_window=True,
    sliding_window=96, max_window_layers=0,
)


@pytest.fixture(scope="module", params=["tiny_d", "real"])
def wide(request, tmp_path_factory):
    """200 requests with short prompts and three more tokens each, and the plain model's logits
    at their last four places."""
    raw = helpers.TINY_D if request.param == "tiny_d" else REAL
    folder = helpers.write_model(tmp_path_factory.mktemp(f"wide_{request.param}"), raw, 7, torch.bfloat16, sharpen=2.0)
    gen = torch.Generator().manual_seed(77)
    lengths = torch.randint(4, 14, (200,), generator=gen).tolist()
    requests = {f"w{i}": helpers.random_tokens(raw["vocab_size"], n + 3, 1000 + i) for i, n in enumerate(lengths)}
    cfg = plain.read_config(folder)
    weights = {k: v.float().cuda() for k, v in plain.read_weights(folder).items()}
    oracle = {}
    for key, ids in requests.items():
        hidden = plain.forward_hidden(torch.tensor(ids, device="cuda"), weights, cfg)
        oracle[key] = plain.linear(hidden[-4:], plain.lm_head_weight(weights)).float().cpu()
    del weights, hidden
    torch.cuda.empty_cache()
    return request.param, folder, raw, requests, oracle


@pytest.mark.parametrize("count", [65, 100, 200])
@pytest.mark.parametrize("dtype_name", list(DTYPES))
def test_decode_only_steps_of_more_than_64_requests(wide, dtype_name, count):
    from paged_attention_engine_b200.engine.llm import Engine
    from paged_attention_engine_b200.engine.replay import Replayer
    from paged_attention_engine_b200.kernels import ops

    name, folder, raw, requests, oracle = wide
    keys = list(requests)[:count]
    engine = Engine.from_pretrained(folder, dtype_name)

    def run(use_graphs):
        replayer = Replayer(engine, max_tokens=count * 32, block_size=16, max_live=count)
        replayer.runner.use_graphs = use_graphs and replayer.runner.use_graphs
        # every prompt in one step, then three steps of `count` single tokens
        first = [{"id": k, "tokens": requests[k][:-3], "want": [len(requests[k]) - 4]} for k in keys]
        got = [replayer.run({"step": 0, "entries": first, "end": []}).float().cpu()]
        for step in range(3):
            entries = [{"id": k, "tokens": [requests[k][len(requests[k]) - 3 + step]], "want": [0]} for k in keys]
            got.append(replayer.run({"step": 1 + step, "entries": entries, "end": keys if step == 2 else []}).float().cpu())
        ops.check_device_errors()
        return torch.stack(got, dim=1), replayer.runner.graph_replays      # [count, 4, vocab]

    with_graphs, replays = run(True)
    eager, none = run(False)
    assert (replays >= 2 or not helpers.records_steps()) and none == 0       # the first decode step records its graph, the others replay it
    assert torch.equal(with_graphs, eager), "a replayed graph holds the launches of the eager step: the same bits"
    for i, key in enumerate(keys):
        gap = (with_graphs[i] - oracle[key]).abs().max().item()
        assert gap <= helpers.tolerance(DTYPES[dtype_name], oracle[key]), f"{name}/{dtype_name}/{key}: {gap}"
    del engine
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype_name", list(DTYPES))
def test_decoders_wait_for_token_budget_with_their_token_on_the_device(tmp_path_factory, dtype_name):
    """Decoders never outnumber the token budget by the scheduler's own doing (each of them used a
    token of it in the step before), so the budget is cut while eight requests decode: from then
    on three of them wait every step, the first time with the token they sampled a step earlier
    still on the device, not yet read back. The tokens are those of the synchronous executor
    under the same cut, and in float32 those of a run whose budget is never cut."""
    from paged_attention_engine_b200 import LLM, Request

    raw, page, seed = helpers.TINY["tiny_b"]
    folder = helpers.write_model(tmp_path_factory.mktemp(f"defer_{dtype_name}"), raw, seed, DTYPES[dtype_name], sharpen=4.0)
    prompts = {f"d{i}": tuple(helpers.random_tokens(raw["vocab_size"], 3 + 2 * i, 800 + i)) for i in range(8)}

    def run(asynchronous, cut_to):
        llm = LLM.from_pretrained(folder, dtype=dtype_name, num_blocks=64, block_size=page, max_num_seqs=8,
                                  max_num_batched_tokens=256, asynchronous=asynchronous)
        for rid, prompt in prompts.items():
            assert llm.add_request(Request(rid, prompt, 10 + int(rid[1:]), temperature=0.6 if int(rid[1:]) % 2 else 0.0, seed=9))
        waited_with_pending = waited = 0
        for step in range(10_000):
            if not (llm.scheduler.waiting or llm.scheduler.running):
                break
            if step == 3 and cut_to is not None:
                assert len(llm.scheduler.running) == 8
                llm.scheduler.max_num_batched_tokens = cut_to
            pending = {s.request_id for s in llm.scheduler.running if s.generated and s.generated[-1] < 0}
            result = llm.step()
            waited += len(result.deferred)
            waited_with_pending += len(pending & set(result.deferred))
        llm.scheduler.resolve()
        return {rid: tuple(seq.generated) for rid, seq in llm.scheduler.finished.items()}, waited, waited_with_pending, llm

    late, waited, pending_waits, llm = run(True, 5)
    assert llm.executor.asynchronous
    assert waited > 10
    assert pending_waits > 0, "no decoder ever waited with its token still on the device"
    now, waited_now, pending_now, _ = run(False, 5)
    assert waited_now == waited and pending_now == 0       # the synchronous executor reads every token at once
    assert late == now
    assert all(len(v) == 10 + int(rid[1:]) and min(v) >= 0 for rid, v in late.items())
    if dtype_name == "float32":
        roomy, none, _, _ = run(True, None)
        assert none == 0 and late == roomy


@pytest.mark.parametrize("dtype_name", list(DTYPES))
def test_windowed_heads_of_128_through_the_entry_point_with_pages_reused(tmp_path_factory, dtype_name):
    """Prompts of some hundred tokens in portions of up to 160 through a model whose layers all
    see the last 96 keys, pages of 16, three requests at a time in a pool of 40 pages: a request
    alone would need up to 24 pages without the window; with it pages return as the window
    passes them and are handed out again, to the same and to other requests."""
    from paged_attention_engine_b200 import LLM, Request
    from paged_attention_engine_b200.engine.llm import Engine
    from paged_attention_engine_b200.kernels import ops

    folder = helpers.write_model(tmp_path_factory.mktemp(f"windowed_{dtype_name}"), WINDOWED, 11, DTYPES[dtype_name], sharpen=3.0)
    recording = RecordingOps(ops)
    engine = Engine.from_pretrained(folder, dtype_name, ops=recording)
    llm = LLM(engine, num_blocks=40, block_size=16, max_num_seqs=3, max_num_batched_tokens=200, record_logits=True)
    lengths = (150, 330, 97, 260, 64, 201)
    prompts = {f"v{i}": tuple(helpers.random_tokens(WINDOWED["vocab_size"], n, 900 + i)) for i, n in enumerate(lengths)}
    for rid, prompt in prompts.items():
        assert llm.add_request(Request(rid, prompt, 40))
    handed_out = 0
    free_before = llm.cache.manager.num_free
    while llm.scheduler.waiting or llm.scheduler.running:
        llm.step()
        free_now = llm.cache.manager.num_free
        handed_out += max(0, free_before - free_now)
        free_before = free_now
    llm.scheduler.resolve()
    ops.check_device_errors()
    assert handed_out > 40, f"only {handed_out} pages were handed out from a pool of 40: none was used again"
    assert llm.cache.manager.num_free == 40
    if dtype_name == "bfloat16":
        kernels = {call.get("kernel") for call in recording.attention_calls}
        assert "tcgen05" in kernels, kernels
    for rid, prompt in prompts.items():
        seq = llm.scheduler.finished[rid]
        assert len(seq.generated) == 40
        helpers.teacher_forced_check(folder, DTYPES[dtype_name], prompt, seq.generated, seq.step_logits)


@pytest.mark.parametrize("asynchronous", [True, False])
def test_a_wait_that_gave_up_stops_generation(tmp_path_factory, asynchronous):
    """A tcgen05 kernel that gives up on a bounded wait writes its role code into the device's
    error word and leaves an output that means nothing. The word is set here from the host (no
    wait is made to run out): the step that follows must raise when its tokens are looked at,
    not hand them out, and the word must be clear afterwards."""
    from paged_attention_engine_b200 import LLM, Request
    from paged_attention_engine_b200.kernels import ops

    raw, page, seed = helpers.TINY["tiny_b"]
    folder = helpers.write_model(tmp_path_factory.mktemp(f"flag_{asynchronous}"), raw, seed, torch.bfloat16)
    llm = LLM.from_pretrained(folder, dtype="bfloat16", num_blocks=32, block_size=page, asynchronous=asynchronous)
    assert llm.add_request(Request("x", tuple(helpers.random_tokens(raw["vocab_size"], 9, 1)), 8))
    llm.step()
    llm.scheduler.resolve()
    ops.error_flag("cuda:0").fill_(5)
    with pytest.raises(ops.KernelError, match="role code 5"):
        llm.step()
        llm.scheduler.resolve()
    assert int(ops.error_flag("cuda:0").item()) == 0
    ops.check_device_errors()
