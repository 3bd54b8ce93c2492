"""The assembly is general: with parts defined HERE, in the test, and registered under new
names, a model is built, given pages and state by the cache manager, and stepped, without
a change to any file of the package.

  * `running_mean` is a mixer with state of its own and no keys or values: it adds to every
    token the mean of all tokens of its request so far. Its state (a sum and a count per
    request) lives in the cache manager's state slots, is zero for a new request, carries
    over portions and steps, and belongs to one request only.
  * the schedule names a layer twice (shared weights, a cache per run), and lets an entry
    read the keys and values that an earlier entry wrote.
  * `top1_experts` is a feed-forward with routing: router logits in float32, every token
    goes to the one expert with the highest logit, an expert is a small SiLU-gated network.
  * `stretched_rotary` is another position encoding: rotation angles of positions divided by a
    factor, for a chosen part of the frequencies only (the rest are not rotated). The
    package's attention part uses it through the same `table(ctx)` as its own.

  * `decayed_sum` is a second mixer with state, written so that a step depends on the batch only
    through device tensors (it finds its requests' slots in `ctx.state_slot`): a model that holds
    it keeps its decode steps as recorded CUDA graphs, and replayed steps give the bits of eager ones.
  * `sandwich_norm` is another arrangement of a layer: a norm before AND after each branch
    (four norms, with roles of its own names). The block kind declares its parts; the
    loader, the random weights, the cache plan and the model follow that declaration.

These are toys for the test, not models of anything.
"""

import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def _register_toys():
    from paged_attention_engine_b200.parts import MIXERS, Part, StateNeed

    if "running_mean" in MIXERS.names():
        return

    @MIXERS.register("running_mean")
    class RunningMean(Part):
        """params: hidden_size. No tensors, no pages; state [hidden + 1] per request."""

        graph_safe = False      # forward() loops over the step's requests on the host

        @classmethod
        def state_need(cls, spec):
            return StateNeed((int(spec.params["hidden_size"]) + 1,), torch.float32)

        def forward(self, ctx, x, residual, cache):
            out = residual.clone()
            at = 0
            for slot, count in zip(ctx.host_state_slots, ctx.host_q_lens):
                state = cache.state[slot]
                rows = x[at : at + count].float()
                sums = state[:-1] + rows.cumsum(0)
                counts = state[-1] + torch.arange(1, count + 1, device=x.device, dtype=torch.float32)
                out[at : at + count] += (sums / counts[:, None]).to(out.dtype)
                state[:-1] = sums[-1]
                state[-1] = counts[-1]
                at += count
            return out

    from paged_attention_engine_b200.parts import FEED_FORWARDS, POSITION_ENCODINGS, TensorSpec

    @FEED_FORWARDS.register("top1_experts")
    class Top1Experts(Part):
        """params: hidden_size, intermediate_size, experts. tensors: router.weight [E, H] and, per
        expert e, experts.e.gate_up.weight [2 I, H] and experts.e.down.weight [H, I]."""

        graph_safe = False      # the routing is read back to the host

        @classmethod
        def tensor_specs(cls, spec):
            h, i, e = (int(spec.params[k]) for k in ("hidden_size", "intermediate_size", "experts"))
            specs = [TensorSpec(spec.tensor_name("router.weight"), (e, h), "matrix")]
            for x in range(e):
                specs.append(TensorSpec(spec.tensor_name(f"experts.{x}.gate_up.weight"), (2 * i, h), "matrix"))
                specs.append(TensorSpec(spec.tensor_name(f"experts.{x}.down.weight"), (h, i), "matrix"))
            return specs

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.experts = int(spec.params["experts"])
            self.router = tensors[spec.tensor_name("router.weight")]
            self.gate_up = [tensors[spec.tensor_name(f"experts.{x}.gate_up.weight")] for x in range(self.experts)]
            self.down = [tensors[spec.tensor_name(f"experts.{x}.down.weight")] for x in range(self.experts)]

        def forward(self, ctx, x, residual):
            ops = self.ops
            x = ops.materialized(x)
            logits = ops.materialized(ops.linear(x, self.router, out_dtype=torch.float32))     # float32 router logits
            choice = logits.argmax(dim=-1)
            out = residual.clone()
            for e in range(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    hidden = ops.silu_mul(ops.linear(x[rows].contiguous(), self.gate_up[e]))
                    out[rows] += ops.materialized(ops.linear(hidden, self.down[e])).to(out.dtype)
            return out

    @POSITION_ENCODINGS.register("stretched_rotary")
    class StretchedRotary(Part):
        """params: head_dim, theta, factor, rotated (how many of the head_dim / 2 frequencies rotate)."""

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            d, theta = int(spec.params["head_dim"]), float(spec.params["theta"])
            inv_freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.int64).to(torch.float32) / d))
            inv_freq = inv_freq / float(spec.params["factor"])
            inv_freq[int(spec.params["rotated"]):] = 0.0          # angle 0: cosine 1, sine 0
            self.inv_freq = inv_freq.to(runtime.device)
            self._key = ("stretched_rotary", d, theta, float(spec.params["factor"]), int(spec.params["rotated"]))

        def table(self, ctx):
            if self._key not in ctx.memo:
                ctx.memo[self._key] = self.ops.rotary_table(ctx.positions, self.inv_freq)
            return ctx.memo[self._key]


def _spec(hidden, vocab, schedule_kind):
    from paged_attention_engine_b200.config import ModelSpec, PartSpec, ScheduleEntry

    def norm(prefix):
        return PartSpec("rms_norm", {"size": hidden, "eps": 1e-5}, prefix)

    attention = PartSpec("gqa_attention", {
        "hidden_size": hidden, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16, "qkv_bias": True, "scale": 0.25,
        "window": 0, "position_encoding": {"kind": "rotary", "head_dim": 16, "theta": 1e4}}, "l0.attn")
    layers = (
        helpers.decoder_layer(norm("l0.n1"), attention, norm("l0.n2"),
                  PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": 48}, "l0.ff")),
        helpers.decoder_layer(norm("l1.n1"), PartSpec("running_mean", {"hidden_size": hidden}), norm("l1.n2"),
                  PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": 40}, "l1.ff")),
    )
    schedule = {
        "stateful": (ScheduleEntry(0), ScheduleEntry(1)),
        "twice": (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)),
        "shared_cache": (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0, cache_from=0)),
    }[schedule_kind]
    return ModelSpec("toy", vocab, hidden, 256, PartSpec("token_embedding", {"vocab_size": vocab, "hidden_size": hidden}, "emb"),
                     layers, schedule, norm("final"), PartSpec("lm_head", {"vocab_size": vocab, "hidden_size": hidden, "tied_to": "emb.weight"}, "head"))


def _plain_forward(spec, w, ids):
    """The same toy model written out whole-sequence with the plain implementation's functions."""
    from plain import qwen2_plain as plain

    x = w["emb.weight"][torch.tensor(ids)]
    n = len(ids)
    cos, sin = plain.rotary_tables(plain.rotary_inv_freq(16, 1e4), torch.arange(n), torch.float32)
    cfg = plain.PlainConfig(2, x.shape[1], 4, 2, 16, 48, w["emb.weight"].shape[0], 1e-5, 1e4, True, (0, 0))
    kv_of_entry = {}
    for position, entry in enumerate(spec.schedule):
        p = f"l{entry.layer}."
        normed = plain.rms_norm(x, w[p + "n1.weight"], 1e-5)
        if entry.layer == 0:
            source = normed if entry.cache_from is None else kv_of_entry[entry.cache_from]
            kv_of_entry[position] = normed
            q = plain.apply_rotary(plain.linear(normed, w[p + "attn.q_proj.weight"], w[p + "attn.q_proj.bias"]).view(n, 4, 16), cos, sin)
            k = plain.apply_rotary(plain.linear(source, w[p + "attn.k_proj.weight"], w[p + "attn.k_proj.bias"]).view(n, 2, 16), cos, sin)
            v = plain.linear(source, w[p + "attn.v_proj.weight"], w[p + "attn.v_proj.bias"]).view(n, 2, 16)
            x = x + plain.linear(plain.attention(q, k, v, 0.25).reshape(n, 64), w[p + "attn.o_proj.weight"])
        else:
            x = x + normed.cumsum(0) / torch.arange(1, n + 1)[:, None]
        normed = plain.rms_norm(x, w[p + "n2.weight"], 1e-5)
        x = x + plain.swiglu(normed, w[p + "ff.gate_proj.weight"], w[p + "ff.up_proj.weight"], w[p + "ff.down_proj.weight"])
    return plain.linear(plain.rms_norm(x, w["final.weight"], 1e-5), w["emb.weight"])


@pytest.mark.parametrize("schedule_kind", ["stateful", "twice", "shared_cache"])
def test_toy_model_is_registered_built_and_stepped(schedule_kind):
    from paged_attention_engine_b200.engine.batch import StepEntry
    from paged_attention_engine_b200.engine.llm import Engine
    from paged_attention_engine_b200.kernels import ops
    from paged_attention_engine_b200.parts import Runtime
    from paged_attention_engine_b200.weights import collect_tensor_specs, place_tensors
    from paged_attention_engine_b200.weights.random_init import draw

    _register_toys()
    hidden, vocab = 64, 97
    spec = _spec(hidden, vocab, schedule_kind)
    gen = torch.Generator().manual_seed(9)
    raw = {name: draw(t, gen) * (5.0 if ".q_proj." in name or ".k_proj." in name else 1.0)
           for name, t in sorted(collect_tensor_specs(spec).items())}
    runtime = Runtime(ops, torch.float32, torch.device("cuda:0"))
    engine = Engine(None, spec, place_tensors(dict(raw), spec, torch.float32, runtime.device), runtime)

    plan = engine.cache_plan
    assert len(plan.state_needs) == sum(1 for e in spec.schedule if e.layer == 1)
    owners = [pos for pos, e in enumerate(spec.schedule) if e.layer == 0 and e.cache_from is None]
    assert plan.groups[0].entries == tuple(owners)

    cache = engine.new_paged_cache(num_blocks=24, block_size=8, max_num_seqs=3)
    runner = engine.new_runner(cache)
    requests = {"a": helpers.random_tokens(vocab, 41, 1), "b": helpers.random_tokens(vocab, 23, 2), "c": helpers.random_tokens(vocab, 30, 3)}
    trace = helpers.trace_mixed(requests, seed=4, live_limit=2, decode_tail=6)
    outputs = {}
    for record in trace:
        entries = []
        for item in record["entries"]:
            if not cache.manager.is_live(item["id"]):
                assert runner.begin_request(item["id"])
            assert cache.manager.reserve(item["id"], len(item["tokens"])).ok
            entries.append(StepEntry(item["id"], item["tokens"], item["want"]))
        outputs[record["step"]] = runner.step(entries).logits.float().cpu()
        for key in record["end"]:
            runner.end_request(key)
    got = helpers.collect(trace, outputs, requests)
    for key, ids in requests.items():
        want = _plain_forward(spec, raw, ids)
        gap = (got[key] - want).abs().max().item()
        assert gap <= helpers.tolerance(torch.float32, want), f"{schedule_kind}/{key}: {gap}"
    assert cache.manager.slots.num_free == 3 and cache.manager.allocators[0].num_free == 24


def _routed_spec(hidden, vocab):
    from paged_attention_engine_b200.config import ModelSpec, PartSpec, ScheduleEntry

    def norm(prefix):
        return PartSpec("rms_norm", {"size": hidden, "eps": 1e-5}, prefix)

    def attention(prefix):
        return PartSpec("gqa_attention", {
            "hidden_size": hidden, "num_heads": 4, "num_kv_heads": 1, "head_dim": 16, "qkv_bias": True, "scale": 0.25,
            "window": 0, "position_encoding": {"kind": "stretched_rotary", "head_dim": 16, "theta": 1e4, "factor": 4.0, "rotated": 5}},
            prefix)

    layers = (
        helpers.decoder_layer(norm("l0.n1"), attention("l0.attn"), norm("l0.n2"),
                  PartSpec("top1_experts", {"hidden_size": hidden, "intermediate_size": 24, "experts": 3}, "l0.ff")),
        helpers.decoder_layer(norm("l1.n1"), attention("l1.attn"), norm("l1.n2"),
                  PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": 48}, "l1.ff")),
    )
    return ModelSpec("toy_routed", vocab, hidden, 256, PartSpec("token_embedding", {"vocab_size": vocab, "hidden_size": hidden}, "emb"),
                     layers, (ScheduleEntry(0), ScheduleEntry(1)), norm("final"),
                     PartSpec("lm_head", {"vocab_size": vocab, "hidden_size": hidden, "tied_to": "emb.weight"}, "head"))


def _plain_routed_forward(w, ids):
    """The routed toy model, whole sequence, with the plain implementation's functions."""
    from plain import qwen2_plain as plain

    x = w["emb.weight"][torch.tensor(ids)]
    n = len(ids)
    inv_freq = plain.rotary_inv_freq(16, 1e4) / 4.0
    inv_freq[5:] = 0.0
    cos, sin = plain.rotary_tables(inv_freq, torch.arange(n), torch.float32)
    for layer in (0, 1):
        p = f"l{layer}."
        normed = plain.rms_norm(x, w[p + "n1.weight"], 1e-5)
        q = plain.apply_rotary(plain.linear(normed, w[p + "attn.q_proj.weight"], w[p + "attn.q_proj.bias"]).view(n, 4, 16), cos, sin)
        k = plain.apply_rotary(plain.linear(normed, w[p + "attn.k_proj.weight"], w[p + "attn.k_proj.bias"]).view(n, 1, 16), cos, sin)
        v = plain.linear(normed, w[p + "attn.v_proj.weight"], w[p + "attn.v_proj.bias"]).view(n, 1, 16)
        x = x + plain.linear(plain.attention(q, k, v, 0.25).reshape(n, 64), w[p + "attn.o_proj.weight"])
        normed = plain.rms_norm(x, w[p + "n2.weight"], 1e-5)
        if layer == 0:
            choice = plain.linear(normed, w[p + "ff.router.weight"]).argmax(dim=-1)
            update = torch.zeros_like(x)
            for e in range(3):
                rows = choice == e
                gate_up = plain.linear(normed[rows], w[p + f"ff.experts.{e}.gate_up.weight"])
                inner = gate_up.shape[1] // 2
                hidden = torch.nn.functional.silu(gate_up[:, :inner]) * gate_up[:, inner:]
                update[rows] = plain.linear(hidden, w[p + f"ff.experts.{e}.down.weight"])
            x = x + update
        else:
            x = x + plain.swiglu(normed, w[p + "ff.gate_proj.weight"], w[p + "ff.up_proj.weight"], w[p + "ff.down_proj.weight"])
    return plain.linear(plain.rms_norm(x, w["final.weight"], 1e-5), w["emb.weight"]), choice


def test_routed_feed_forward_and_another_position_encoding():
    """A feed-forward that routes tokens to experts and a position encoding that is not the
    package's, both defined above, in a model that is built and stepped in portions and single
    tokens like any other; compared with the same model written out whole."""
    from paged_attention_engine_b200.engine.batch import StepEntry
    from paged_attention_engine_b200.engine.llm import Engine
    from paged_attention_engine_b200.kernels import ops
    from paged_attention_engine_b200.parts import Runtime
    from paged_attention_engine_b200.weights import collect_tensor_specs, place_tensors
    from paged_attention_engine_b200.weights.random_init import draw

    _register_toys()
    hidden, vocab = 64, 89
    spec = _routed_spec(hidden, vocab)
    gen = torch.Generator().manual_seed(19)
    raw = {}
    for name, t in sorted(collect_tensor_specs(spec).items()):
        scale = 5.0 if ".q_proj." in name or ".k_proj." in name else (25.0 if "router" in name else 1.0)
        raw[name] = draw(t, gen) * scale        # a sharp router: no token sits on the fence between two experts
    runtime = Runtime(ops, torch.float32, torch.device("cuda:0"))
    engine = Engine(None, spec, place_tensors(dict(raw), spec, torch.float32, runtime.device), runtime)
    assert not engine.model.graph_safe, "the routing reads the step on the host: no graph is recorded"
    cache = engine.new_paged_cache(num_blocks=24, block_size=8, max_num_seqs=3)
    runner = engine.new_runner(cache)
    requests = {"a": helpers.random_tokens(vocab, 37, 5), "b": helpers.random_tokens(vocab, 26, 6), "c": helpers.random_tokens(vocab, 19, 7)}
    trace = helpers.trace_mixed(requests, seed=8, live_limit=2, decode_tail=5)
    outputs = {}
    for record in trace:
        entries = []
        for item in record["entries"]:
            if not cache.manager.is_live(item["id"]):
                assert runner.begin_request(item["id"])
            assert cache.manager.reserve(item["id"], len(item["tokens"])).ok
            entries.append(StepEntry(item["id"], item["tokens"], item["want"]))
        outputs[record["step"]] = runner.step(entries).logits.float().cpu()
        for key in record["end"]:
            runner.end_request(key)
    got = helpers.collect(trace, outputs, requests)
    used = set()
    for key, ids in requests.items():
        want, choice = _plain_routed_forward(raw, ids)
        used |= set(choice.tolist())
        gap = (got[key] - want).abs().max().item()
        assert gap <= helpers.tolerance(torch.float32, want), f"{key}: {gap}"
    assert used == {0, 1, 2}, "every expert got tokens"
    assert cache.manager.allocators[0].num_free == 24


def _register_sandwich():
    from paged_attention_engine_b200.parts import BLOCKS, Block

    if "sandwich_norm" in BLOCKS.names():
        return

    @BLOCKS.register("sandwich_norm")
    class SandwichNorm(Block):
        """x += after_mixer(mixer(before_mixer(x))); x += after_ff(ff(before_ff(x)))."""

        roles = {"before_mixer": "norm", "token_mixer": "mixer", "after_mixer": "norm",
                 "before_ff": "norm", "ff": "feed_forward", "after_ff": "norm"}

        def forward(self, ctx, hidden, layer, cache):
            ops = ctx.ops
            hidden = ops.materialized(hidden)
            zero = torch.zeros_like(hidden)
            branch = layer.token_mixer.forward(ctx, layer.before_mixer.forward(ctx, hidden), zero, cache)
            hidden = hidden + ops.materialized(layer.after_mixer.forward(ctx, branch))
            branch = layer.ff.forward(ctx, layer.before_ff.forward(ctx, hidden), zero)
            return hidden + ops.materialized(layer.after_ff.forward(ctx, branch))


def test_a_block_kind_declares_its_own_parts():
    """A layer with four norms under role names that no file of the package knows: the tensors
    of all six parts are found by the loader's walk, pages go to the role that needs them, and the
    model steps in portions and single tokens like any other."""
    from paged_attention_engine_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from paged_attention_engine_b200.engine.batch import StepEntry
    from paged_attention_engine_b200.engine.llm import Engine
    from paged_attention_engine_b200.kernels import ops
    from paged_attention_engine_b200.parts import Runtime
    from paged_attention_engine_b200.weights import collect_tensor_specs, place_tensors
    from paged_attention_engine_b200.weights.random_init import draw
    from plain import qwen2_plain as plain

    _register_sandwich()
    hidden, vocab, eps = 48, 71, 1e-5

    def norm(prefix):
        return PartSpec("rms_norm", {"size": hidden, "eps": eps}, prefix)

    def layer(p, inner):
        return LayerSpec("sandwich_norm", {
            "before_mixer": norm(p + "n1"), "after_mixer": norm(p + "n2"), "before_ff": norm(p + "n3"), "after_ff": norm(p + "n4"),
            "token_mixer": PartSpec("gqa_attention", {
                "hidden_size": hidden, "num_heads": 3, "num_kv_heads": 1, "head_dim": 16, "qkv_bias": True, "scale": 0.25,
                "window": 0, "position_encoding": {"kind": "rotary", "head_dim": 16, "theta": 1e4}}, p + "attn"),
            "ff": PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": inner}, p + "ff"),
        })

    spec = ModelSpec("toy_sandwich", vocab, hidden, 256, PartSpec("token_embedding", {"vocab_size": vocab, "hidden_size": hidden}, "emb"),
                     (layer("l0.", 32), layer("l1.", 40)), (ScheduleEntry(0), ScheduleEntry(1)), norm("final"),
                     PartSpec("lm_head", {"vocab_size": vocab, "hidden_size": hidden, "tied_to": "emb.weight"}, "head"))
    names = collect_tensor_specs(spec)
    assert {"l0.n1.weight", "l0.n4.weight", "l1.n3.weight", "l1.attn.q_proj.bias", "l0.ff.down_proj.weight"} <= set(names)
    with pytest.raises(ValueError, match="missing: after_ff"):
        collect_tensor_specs(ModelSpec(
            "broken", vocab, hidden, 256, spec.embedding,
            (LayerSpec("sandwich_norm", {k: v for k, v in spec.layers[0].parts.items() if k != "after_ff"}),),
            (ScheduleEntry(0),), spec.final_norm, spec.head))

    gen = torch.Generator().manual_seed(29)
    raw = {name: draw(t, gen) * (5.0 if ".q_proj." in name or ".k_proj." in name else 1.0) for name, t in sorted(names.items())}
    runtime = Runtime(ops, torch.float32, torch.device("cuda:0"))
    engine = Engine(None, spec, place_tensors(dict(raw), spec, torch.float32, runtime.device), runtime)
    assert len(engine.cache_plan.groups) == 1 and engine.cache_plan.groups[0].entries == (0, 1)
    cache = engine.new_paged_cache(num_blocks=24, block_size=8, max_num_seqs=3)
    runner = engine.new_runner(cache)
    requests = {"a": helpers.random_tokens(vocab, 33, 11), "b": helpers.random_tokens(vocab, 21, 12), "c": helpers.random_tokens(vocab, 27, 13)}
    trace = helpers.trace_mixed(requests, seed=6, live_limit=2, decode_tail=5)
    outputs = {}
    for record in trace:
        entries = []
        for item in record["entries"]:
            if not cache.manager.is_live(item["id"]):
                assert runner.begin_request(item["id"])
            assert cache.manager.reserve(item["id"], len(item["tokens"])).ok
            entries.append(StepEntry(item["id"], item["tokens"], item["want"]))
        outputs[record["step"]] = runner.step(entries).logits.float().cpu()
        for key in record["end"]:
            runner.end_request(key)
    got = helpers.collect(trace, outputs, requests)

    def whole(ids):
        x = raw["emb.weight"][torch.tensor(ids)]
        n = len(ids)
        cos, sin = plain.rotary_tables(plain.rotary_inv_freq(16, 1e4), torch.arange(n), torch.float32)
        for p in ("l0.", "l1."):
            y = plain.rms_norm(x, raw[p + "n1.weight"], eps)
            q = plain.apply_rotary(plain.linear(y, raw[p + "attn.q_proj.weight"], raw[p + "attn.q_proj.bias"]).view(n, 3, 16), cos, sin)
            k = plain.apply_rotary(plain.linear(y, raw[p + "attn.k_proj.weight"], raw[p + "attn.k_proj.bias"]).view(n, 1, 16), cos, sin)
            v = plain.linear(y, raw[p + "attn.v_proj.weight"], raw[p + "attn.v_proj.bias"]).view(n, 1, 16)
            branch = plain.linear(plain.attention(q, k, v, 0.25).reshape(n, 48), raw[p + "attn.o_proj.weight"])
            x = x + plain.rms_norm(branch, raw[p + "n2.weight"], eps)
            y = plain.rms_norm(x, raw[p + "n3.weight"], eps)
            branch = plain.swiglu(y, raw[p + "ff.gate_proj.weight"], raw[p + "ff.up_proj.weight"], raw[p + "ff.down_proj.weight"])
            x = x + plain.rms_norm(branch, raw[p + "n4.weight"], eps)
        return plain.linear(plain.rms_norm(x, raw["final.weight"], eps), raw["emb.weight"])

    for key, ids in requests.items():
        want = whole(ids)
        gap = (got[key] - want).abs().max().item()
        assert gap <= helpers.tolerance(torch.float32, want), f"{key}: {gap}"
    assert cache.manager.allocators[0].num_free == 24


def _register_decayed_sum():
    from paged_attention_engine_b200.parts import MIXERS, Part, StateNeed

    if "decayed_sum" in MIXERS.names():
        return

    @MIXERS.register("decayed_sum")
    class DecayedSum(Part):
        """out[t] = residual[t] + s[t] with s[t] = decay * s[t - 1] + x[t] per request; the state is
        s after the request's last token. params: hidden_size, decay. No tensors, no pages.
        Every index it uses is a device tensor of the step, so its steps can be recorded."""

        graph_safe = True

        @classmethod
        def state_need(cls, spec):
            return StateNeed((int(spec.params["hidden_size"]),), torch.float32)

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.decay = float(spec.params["decay"])

        def forward(self, ctx, x, residual, cache):
            slots = ctx.state_slot.long()[ctx.seq_index.long()]          # [tokens]: each token's state slot
            rows = x.float()
            if ctx.max_q_len == 1:                                        # single tokens: one update each, on the device
                state = cache.state[slots] * self.decay + rows
                cache.state.index_copy_(0, slots, state)
                return residual + state.to(residual.dtype)
            out = residual.clone()                                        # portions: token by token within a request
            at = 0
            for slot, count in zip(ctx.host_state_slots, ctx.host_q_lens):
                state = cache.state[slot]
                for i in range(count):
                    state = state * self.decay + rows[at + i]
                    out[at + i] += state.to(out.dtype)
                cache.state[slot] = state
                at += count
            return out


def test_a_stateful_mixer_whose_decode_steps_are_recorded():
    """State of fixed size per request does not cost the model its CUDA graphs when the mixer reads
    the step through device tensors only: decode steps are replayed from recordings (padding rows
    use the spare state slot), and give the same bits as without graphs; the state is zero for a
    new request and follows the request over portions and single tokens."""
    from paged_attention_engine_b200.config import ModelSpec, PartSpec, ScheduleEntry
    from paged_attention_engine_b200.engine.batch import StepEntry
    from paged_attention_engine_b200.engine.llm import Engine
    from paged_attention_engine_b200.kernels import ops
    from paged_attention_engine_b200.parts import Runtime
    from paged_attention_engine_b200.weights import collect_tensor_specs, place_tensors
    from paged_attention_engine_b200.weights.random_init import draw
    from plain import qwen2_plain as plain

    _register_decayed_sum()
    hidden, vocab, decay = 64, 83, 0.75

    def norm(prefix):
        return PartSpec("rms_norm", {"size": hidden, "eps": 1e-5}, prefix)

    layers = tuple(
        helpers.decoder_layer(norm(f"l{i}.n1"), PartSpec("decayed_sum", {"hidden_size": hidden, "decay": decay}), norm(f"l{i}.n2"),
                              PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": 48}, f"l{i}.ff"))
        for i in range(2))
    spec = ModelSpec("toy_decayed", vocab, hidden, 256, PartSpec("token_embedding", {"vocab_size": vocab, "hidden_size": hidden}, "emb"),
                     layers, (ScheduleEntry(0), ScheduleEntry(1)), norm("final"),
                     PartSpec("lm_head", {"vocab_size": vocab, "hidden_size": hidden, "tied_to": "emb.weight"}, "head"))
    gen = torch.Generator().manual_seed(31)
    raw = {name: draw(t, gen) for name, t in sorted(collect_tensor_specs(spec).items())}
    runtime = Runtime(ops, torch.float32, torch.device("cuda:0"))
    engine = Engine(None, spec, place_tensors(dict(raw), spec, torch.float32, runtime.device), runtime)
    assert engine.model.graph_safe and not engine.cache_plan.groups and len(engine.cache_plan.state_needs) == 2
    requests = {"a": helpers.random_tokens(vocab, 19, 41), "b": helpers.random_tokens(vocab, 12, 42), "c": helpers.random_tokens(vocab, 27, 43)}

    def run(use_graphs):
        cache = engine.new_paged_cache(num_blocks=8, block_size=8, max_num_seqs=4)
        runner = engine.new_runner(cache, use_graphs=use_graphs)
        rows = {k: [] for k in requests}
        for k, ids in requests.items():            # the first five tokens as a portion, beside nothing
            assert runner.begin_request(k) and cache.manager.reserve(k, 5).ok
            rows[k].append(runner.step([StepEntry(k, ids[:5], tuple(range(5)))]).logits.float().cpu().clone())
        for i in range(5, 27):                      # then single tokens of whoever has some left: 3, 2 and 1 requests a step
            entries = []
            for k, ids in requests.items():
                if i < len(ids):
                    assert cache.manager.reserve(k, 1).ok
                    entries.append(StepEntry(k, (ids[i],), (0,)))
            out = runner.step(entries).logits.float().cpu().clone()
            for j, e in enumerate(entries):
                rows[e.key].append(out[j : j + 1])
        for k in requests:
            runner.end_request(k)
        assert cache.manager.slots.num_free == 4
        return {k: torch.cat(v) for k, v in rows.items()}, runner.graph_replays

    recorded, replays = run(True)
    eager, none = run(False)
    assert (replays >= 15 or not helpers.records_steps()) and none == 0
    for k, ids in requests.items():
        assert torch.equal(recorded[k], eager[k]), k
        x = raw["emb.weight"][torch.tensor(ids)]
        for p in ("l0.", "l1."):
            y = plain.rms_norm(x, raw[p + "n1.weight"], 1e-5)
            state, mixed = torch.zeros(hidden), []
            for row in y:
                state = state * decay + row
                mixed.append(state)
            x = x + torch.stack(mixed)
            y = plain.rms_norm(x, raw[p + "n2.weight"], 1e-5)
            x = x + plain.swiglu(y, raw[p + "ff.gate_proj.weight"], raw[p + "ff.up_proj.weight"], raw[p + "ff.down_proj.weight"])
        want = plain.linear(plain.rms_norm(x, raw["final.weight"], 1e-5), raw["emb.weight"])
        gap = (recorded[k] - want).abs().max().item()
        assert gap <= helpers.tolerance(torch.float32, want), f"{k}: {gap}"
