"""Generation through the entry point on the GPU: greedy tokens against the plain
implementation, decode steps through captured graphs against eager steps, long decoding,
the first tokens of a sequence, preemption and recompute under a tiny pool."""

import pytest
import torch

import helpers
from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _folder(tmp_path_factory, name, dtype_name, sharpen=4.0):
    raw, page, seed = helpers.TINY[name]
    folder = helpers.write_model(tmp_path_factory.mktemp(f"{name}_{dtype_name}"), raw, seed, DTYPES[dtype_name], sharpen=sharpen)
    return folder, raw, page


_teacher_forced_check = helpers.teacher_forced_check


@pytest.mark.parametrize("name", list(helpers.TINY))
@pytest.mark.parametrize("dtype_name", list(DTYPES))
def test_greedy_generation_through_the_entry_point(tmp_path_factory, name, dtype_name):
    from paged_attention_engine_b200 import LLM, Request

    folder, raw, page = _folder(tmp_path_factory, name, dtype_name)
    llm = LLM.from_pretrained(folder, dtype=dtype_name, num_blocks=64, block_size=page, max_num_seqs=4,
                              max_num_batched_tokens=24, record_logits=True)
    prompts = {f"p{i}": tuple(helpers.random_tokens(raw["vocab_size"], n, 300 + n)) for i, n in enumerate((5, 11, 17, 1, 30))}
    for rid, prompt in prompts.items():
        assert llm.add_request(Request(rid, prompt, 8))
    out = llm.run_to_completion()
    cfg, weights = plain.read_config(folder), {k: v.float() for k, v in plain.read_weights(folder).items()}
    for rid, prompt in prompts.items():
        assert len(out[rid]) == 8
        _teacher_forced_check(folder, DTYPES[dtype_name], prompt, out[rid], llm.scheduler.finished[rid].step_logits)
        if dtype_name == "float32":
            want, _ = plain.generate_greedy(list(prompt), 8, weights, cfg)
            assert list(out[rid]) == want
    assert llm.runner.graph_replays > 0 or not helpers.records_steps(), "decode steps are expected to run as captured graphs"


@pytest.mark.parametrize("dtype_name", list(DTYPES))
def test_graph_steps_equal_eager_steps(tmp_path_factory, dtype_name):
    """The captured graph holds the same launches as the eager step: the logits are the same bits."""
    from paged_attention_engine_b200 import LLM, Request

    folder, raw, page = _folder(tmp_path_factory, "tiny_b", dtype_name)
    prompts = {f"g{i}": tuple(helpers.random_tokens(raw["vocab_size"], n, 400 + n)) for i, n in enumerate((9, 16, 33))}

    def run(use_graphs):
        llm = LLM.from_pretrained(folder, dtype=dtype_name, num_blocks=64, block_size=page, record_logits=True,
                                  use_graphs=use_graphs)
        for rid, prompt in prompts.items():
            llm.add_request(Request(rid, prompt, 20, temperature=0.7, seed=11))
        out = llm.run_to_completion()
        return out, {rid: torch.stack(llm.scheduler.finished[rid].step_logits) for rid in prompts}, llm.runner.graph_replays

    out_g, logits_g, replays = run(True)
    out_e, logits_e, none = run(False)
    assert (replays > 10 or not helpers.records_steps()) and none == 0
    assert out_g == out_e
    for rid in prompts:
        assert torch.equal(logits_g[rid], logits_e[rid])


@pytest.mark.parametrize("config_name", ["tiny_b", "tiny_d"])
def test_padded_graph_steps_equal_eager_steps(tmp_path_factory, config_name):
    """Eleven, ten and nine requests decode through the graph of twelve (then of ten): rows that
    pad a step up to its graph's batch size change nothing for the real ones, whose tokens and
    logits are the same bits as without graphs; the requests end at different steps, so the
    batch shrinks through several graphs."""
    from paged_attention_engine_b200 import LLM, Request
    from paged_attention_engine_b200.engine.runner import ModelRunner

    assert [ModelRunner.graph_batch(n) for n in (1, 8, 9, 11, 16, 17, 33, 64)] == [1, 8, 10, 12, 16, 20, 40, 64]
    folder, raw, page = _folder(tmp_path_factory, config_name, "bfloat16")
    lengths = (9, 16, 33, 5, 21, 2, 40, 12, 7, 30, 18)
    prompts = {f"p{i}": tuple(helpers.random_tokens(raw["vocab_size"], n, 700 + n)) for i, n in enumerate(lengths)}

    def run(use_graphs):
        llm = LLM.from_pretrained(folder, dtype="bfloat16", num_blocks=128, block_size=page, record_logits=True,
                                  use_graphs=use_graphs, max_num_seqs=16)
        for i, (rid, prompt) in enumerate(prompts.items()):
            llm.add_request(Request(rid, prompt, 6 + 2 * i, temperature=0.5 if i % 2 else 0.0, seed=3))
        out = llm.run_to_completion()
        sizes = sorted({key[0] for key in llm.runner.graphs})
        return out, {rid: torch.stack(llm.scheduler.finished[rid].step_logits) for rid in prompts}, sizes

    out_g, logits_g, sizes = run(True)
    out_e, logits_e, none = run(False)
    assert (12 in sizes and 10 in sizes and 11 not in sizes and 9 not in sizes or not helpers.records_steps()) and not none
    assert out_g == out_e
    for rid in prompts:
        assert torch.equal(logits_g[rid], logits_e[rid]), rid


@pytest.mark.parametrize("dtype_name", list(DTYPES))
def test_long_decoding_and_first_tokens(tmp_path_factory, dtype_name):
    """A one-token prompt decoded far past several page edges and graph widths: the first
    tokens of a sequence, and every later one, against the plain model."""
    from paged_attention_engine_b200 import LLM, Request

    folder, raw, page = _folder(tmp_path_factory, "tiny_c", dtype_name, sharpen=3.0)
    llm = LLM.from_pretrained(folder, dtype=dtype_name, num_blocks=80, block_size=page, record_logits=True)
    prompt = (7,)
    llm.add_request(Request("long", prompt, 300))
    out = llm.run_to_completion()
    assert len(out["long"]) == 300
    _teacher_forced_check(folder, DTYPES[dtype_name], prompt, out["long"], llm.scheduler.finished["long"].step_logits)


@pytest.mark.parametrize("dtype_name", list(DTYPES))
def test_preemption_and_recompute_on_the_gpu(tmp_path_factory, dtype_name):
    from paged_attention_engine_b200 import LLM, EventKind, Request

    folder, raw, page = _folder(tmp_path_factory, "tiny_b", dtype_name)
    prompts = {f"s{i}": tuple(helpers.random_tokens(raw["vocab_size"], n, 500 + n)) for i, n in enumerate((20, 31, 12, 40))}

    def run(num_blocks):
        llm = LLM.from_pretrained(folder, dtype=dtype_name, num_blocks=num_blocks, block_size=page, record_logits=True)
        for rid, prompt in prompts.items():
            assert llm.add_request(Request(rid, prompt, 24))
        return llm.run_to_completion(), llm

    roomy, _ = run(64)
    tight, llm = run(7)          # 112 token slots for four requests that grow to 44..64 tokens each
    assert llm.scheduler.events_of(EventKind.PREEMPT)
    for rid, prompt in prompts.items():
        _teacher_forced_check(folder, DTYPES[dtype_name], prompt, tight[rid], llm.scheduler.finished[rid].step_logits)
    if dtype_name == "float32":
        assert tight == roomy


@pytest.mark.parametrize("dtype_name", list(DTYPES))
@pytest.mark.parametrize("temperature", [0.0, 0.8])
def test_tokens_fed_forward_on_the_device_equal_tokens_read_back(tmp_path_factory, dtype_name, temperature):
    """The asynchronous executor leaves sampled tokens on the device, feeds them to the next step
    there and reads them a step later; the synchronous one reads each step's tokens before it
    plans the next. Same requests, same pool (small enough to preempt), same tokens."""
    from paged_attention_engine_b200 import LLM, EventKind, Request

    folder, raw, page = _folder(tmp_path_factory, "tiny_b", dtype_name)
    prompts = {f"a{i}": tuple(helpers.random_tokens(raw["vocab_size"], n, 600 + n)) for i, n in enumerate((20, 31, 1, 12, 40, 5))}

    def run(asynchronous):
        llm = LLM.from_pretrained(folder, dtype=dtype_name, num_blocks=9, block_size=page, max_num_seqs=4,
                                  max_num_batched_tokens=48, asynchronous=asynchronous)
        for rid, prompt in prompts.items():
            assert llm.add_request(Request(rid, prompt, 30, temperature=temperature, seed=5))
        out = llm.run_to_completion()
        return out, llm

    late, llm = run(True)
    assert llm.executor.asynchronous and llm.scheduler.events_of(EventKind.PREEMPT)
    now, _ = run(False)
    assert late == now
    assert all(len(v) == 30 and min(v) >= 0 for v in late.values())


def test_command_line_generates_what_the_entry_point_generates(tmp_path):
    """`python -m paged_attention_engine_b200 generate`, from a model folder and from a
    configuration with random weights, prints the tokens that LLM.generate returns."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    from paged_attention_engine_b200 import LLM

    raw, page, seed = helpers.TINY["tiny_b"]
    folder = helpers.write_model(tmp_path / "model", raw, seed, torch.bfloat16)
    config = tmp_path / "cfg.json"
    config.write_text(json.dumps(raw))
    prompts = [helpers.random_tokens(raw["vocab_size"], 21, 5), helpers.random_tokens(raw["vocab_size"], 3, 6)]
    want = LLM.from_pretrained(folder, dtype="bfloat16", num_blocks=64, block_size=page).generate(prompts, max_new_tokens=9)
    root = Path(__file__).resolve().parent.parent
    common = ["--dtype", "bfloat16", "--num-blocks", "64", "--block-size", str(page), "--max-new-tokens", "9"]
    for p in prompts:
        common += ["--prompt-ids", ",".join(str(t) for t in p)]
    for source in (["--model", str(folder)], ["--random", str(config), "--weights-seed", str(seed)]):
        done = subprocess.run([sys.executable, "-m", "paged_attention_engine_b200", "generate", *source, *common],
                              cwd=root, capture_output=True, text=True, timeout=600)
        assert done.returncode == 0, done.stderr[-2000:]
        rows = [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]
        assert [tuple(r["token_ids"]) for r in rows] == [tuple(w) for w in want], source


@pytest.mark.parametrize("dtype_name", list(DTYPES))
def test_a_step_whose_shape_comes_again_is_recorded_and_replayed(tmp_path_factory, dtype_name):
    """Steps that are not decode-only: the same shape (a portion of 70 tokens from position 0 beside
    a portion of 33, then 21 more tokens of the first beside one decoded token of the second, in
    the same state slots) comes four times with other tokens and other pages. The first time it runs eagerly, the second time
    it is recorded, then replayed; every time the logits are the bits of a runner that records nothing."""
    from paged_attention_engine_b200.engine.batch import StepEntry
    from paged_attention_engine_b200.engine.llm import Engine

    folder, raw, page = _folder(tmp_path_factory, "tiny_d", dtype_name)
    engine = Engine.from_pretrained(folder, dtype_name)
    rounds = [{name: helpers.random_tokens(raw["vocab_size"], n, 900 + 10 * r + i) for i, (name, n) in enumerate((("a", 91), ("b", 34)))}
              for r in range(4)]

    def run(use_graphs):
        cache = engine.new_paged_cache(40, page, 4)
        runner = engine.new_runner(cache)
        runner.use_graphs = use_graphs and runner.use_graphs
        got = []
        for r, tokens in enumerate(rounds):
            for name in tokens:
                runner.begin_request(name)
            if r == 2:        # other pages from here on: a request that stays holds some
                runner.begin_request("keep")
                assert cache.manager.reserve("keep", 3 * page).ok
            for name in tokens:
                assert cache.manager.reserve(name, len(tokens[name])).ok
            first = runner.step([StepEntry("a", tokens["a"][:70], (0, 69)), StepEntry("b", tokens["b"][:33], (32,))])
            got.append(first.logits.float().cpu().clone())
            second = runner.step([StepEntry("a", tokens["a"][70:], (20,)), StepEntry("b", tokens["b"][33:], (0,))])
            got.append(second.logits.float().cpu().clone())
            for name in reversed(list(tokens)):      # the slot freed last is handed out first: "a" and "b" meet theirs again
                runner.end_request(name)
        return got, runner.shape_graph_replays, len(runner.shape_graphs)

    recorded, replays, kept = run(True)
    eager, none, nothing = run(False)
    assert (replays == 4 and kept == 2) or not helpers.records_steps(), "two shapes, each eager once, recorded once and replayed twice"
    assert none == 0 and nothing == 0
    for step, (a, b) in enumerate(zip(recorded, eager)):
        assert torch.equal(a, b), f"step {step}"


def test_recordings_by_shape_are_few(tmp_path_factory):
    """The least recently used recording goes when more shapes come again than are kept."""
    from paged_attention_engine_b200.engine.batch import StepEntry
    from paged_attention_engine_b200.engine.llm import Engine

    folder, raw, page = _folder(tmp_path_factory, "tiny_b", "bfloat16")
    engine = Engine.from_pretrained(folder, "bfloat16")
    cache = engine.new_paged_cache(16, page, 2)
    runner = engine.new_runner(cache)
    runner.SHAPE_GRAPHS = 2
    for length in (5, 6, 7, 5, 6, 7, 7, 5):
        runner.begin_request("x")
        assert cache.manager.reserve("x", length).ok
        runner.step([StepEntry("x", helpers.random_tokens(raw["vocab_size"], length, length), (length - 1,))])
        runner.end_request("x")
    keys = [key[0][0][0] for key in runner.shape_graphs]
    # 5, 6 and 7 are recorded at their second coming, 5 goes when 7 comes; the third 7 is a replay; the third 5 starts over
    assert (keys == [6, 7] and runner.shape_graph_replays == 1) or not helpers.records_steps(), (keys, runner.shape_graph_replays)


@pytest.mark.parametrize("dtype_name", list(DTYPES))
def test_the_same_prompts_again_through_the_entry_point(tmp_path_factory, dtype_name):
    """One prompt at a time, four times over, sampled with a temperature: from the second time on
    the prompt's step has a shape that came before (same length, same state slot) and from the
    third on it is replayed from its recording, with the sampler's rows and the asynchronous
    token hand-over inside. Tokens and logits are those of an engine that records nothing."""
    from paged_attention_engine_b200 import LLM, Request

    folder, raw, page = _folder(tmp_path_factory, "tiny_b", dtype_name)
    prompts = [tuple(helpers.random_tokens(raw["vocab_size"], n, 500 + 7 * r + n)) for r in range(4) for n in (23, 23, 70)]

    def run(use_graphs):
        llm = LLM.from_pretrained(folder, dtype=dtype_name, num_blocks=64, block_size=page, record_logits=False,
                                  use_graphs=use_graphs, max_num_seqs=2)
        out = {}
        for i, prompt in enumerate(prompts):
            llm.add_request(Request(f"q{i}", prompt, 5, temperature=0.8, seed=17))
            out.update(llm.run_to_completion())
        return out, llm.runner.shape_graph_replays

    recorded, replays = run(True)
    eager, none = run(False)
    assert none == 0 and (replays >= 6 or not helpers.records_steps()), replays
    assert recorded == eager
