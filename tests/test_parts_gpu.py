"""Each part alone on the GPU against the plain implementation's function for the same part,
at sizes of its own (not a model's), in float32 and bfloat16; and generality of the
assembly: a layer run twice, a layer reading another entry's cache, a mixer with state of
its own registered from the test, with no change to the package's files."""

import pytest
import torch

import helpers
from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def runtime_of():
    from paged_attention_engine_b200.kernels import ops
    from paged_attention_engine_b200.parts import Runtime

    return lambda dtype: Runtime(ops, dtype, torch.device("cuda:0"))


def _limit(dtype, want):
    return (5e-5 if dtype == torch.float32 else 2.0 ** -6) * max(1.0, float(want.abs().max()))


class _Ctx:
    """The least a part needs of a step context."""

    def __init__(self, **fields):
        self.memo = {}
        self.__dict__.update(fields)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rms_norm_part(runtime_of, dtype):
    from paged_attention_engine_b200.config import PartSpec
    from paged_attention_engine_b200.parts import NORMS

    spec = PartSpec("rms_norm", {"size": 200, "eps": 3e-5}, "n")
    weight = 1 + 0.1 * torch.randn(200)
    part = NORMS.get("rms_norm")(spec, {"n.weight": weight.cuda()}, runtime_of(dtype))
    x = (torch.randn(13, 200) * 2).to(dtype)
    got = part.forward(_Ctx(), x.cuda()).float().cpu()
    want = plain.rms_norm(x.float(), weight, 3e-5)
    assert (got - want).abs().max().item() <= _limit(dtype, want)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(runtime_of, dtype):
    from paged_attention_engine_b200.config import PartSpec
    from paged_attention_engine_b200.parts import FEED_FORWARDS

    hidden, inter = 72, 200
    spec = PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": inter}, "ff")
    w = {
        "ff.gate_proj.weight": (torch.randn(inter, hidden) * 0.1).to(dtype),
        "ff.up_proj.weight": (torch.randn(inter, hidden) * 0.1).to(dtype),
        "ff.down_proj.weight": (torch.randn(hidden, inter) * 0.1).to(dtype),
    }
    part = FEED_FORWARDS.get("swiglu")(spec, {k: v.cuda() for k, v in w.items()}, runtime_of(dtype))
    x, residual = torch.randn(9, hidden).to(dtype), torch.randn(9, hidden).to(dtype)
    got = runtime_of(dtype).ops.materialized(part.forward(_Ctx(), x.cuda(), residual.cuda())).float().cpu()
    want = residual.float() + plain.swiglu(x.float(), *(w[f"ff.{n}_proj.weight"].float() for n in ("gate", "up", "down")))
    assert (got - want).abs().max().item() <= _limit(dtype, want)


@pytest.mark.parametrize("theta,d", [(1e4, 16), (1e6, 128), (5e4, 48)])
def test_rotary_part(runtime_of, theta, d):
    from paged_attention_engine_b200.config import PartSpec
    from paged_attention_engine_b200.parts import POSITION_ENCODINGS

    part = POSITION_ENCODINGS.get("rotary")(PartSpec("rotary", {"head_dim": d, "theta": theta}), {}, runtime_of(torch.float32))
    positions = torch.tensor([0, 1, 5, 100, 2047, 30000], dtype=torch.int32)
    ctx = _Ctx(positions=positions.cuda())
    table = part.table(ctx).cpu()
    assert part.table(ctx) is part.table(ctx), "one table per step, shared by the layers"
    cos, sin = plain.rotary_tables(plain.rotary_inv_freq(d, theta), positions, torch.float32)
    assert (table[:, : d // 2] - cos[:, : d // 2]).abs().max().item() <= 2e-6
    assert (table[:, d // 2 :] - sin[:, : d // 2]).abs().max().item() <= 2e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tied", [True, False])
def test_embedding_and_head_parts(runtime_of, dtype, tied):
    from paged_attention_engine_b200.config import PartSpec
    from paged_attention_engine_b200.parts import EMBEDDINGS, HEADS

    vocab, hidden = 301, 40
    tensors = {"emb.weight": (torch.randn(vocab, hidden) * 0.1).to(dtype).cuda()}
    if not tied:
        tensors["head.weight"] = (torch.randn(vocab, hidden) * 0.1).to(dtype).cuda()
    rt = runtime_of(dtype)
    emb = EMBEDDINGS.get("token_embedding")(PartSpec("token_embedding", {"vocab_size": vocab, "hidden_size": hidden}, "emb"), tensors, rt)
    head = HEADS.get("lm_head")(
        PartSpec("lm_head", {"vocab_size": vocab, "hidden_size": hidden, "tied_to": "emb.weight" if tied else None}, "head"), tensors, rt)
    ids = torch.tensor([0, 300, 7, 7], dtype=torch.int32)
    rows = emb.forward(_Ctx(token_ids=ids.cuda()))
    assert torch.equal(rows.cpu(), tensors["emb.weight"].cpu()[ids.long()])
    logits = head.forward(_Ctx(), rows)
    assert logits.dtype == torch.float32
    table = tensors["emb.weight" if tied else "head.weight"].float().cpu()
    want = plain.linear(rows.float().cpu(), table)
    assert (logits.cpu() - want).abs().max().item() <= _limit(torch.float32 if dtype == torch.float32 else torch.bfloat16, want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [0, 9])
def test_attention_part_alone(runtime_of, dtype, window):
    """The mixer over its own little cache: two portions and single tokens of one request
    against plain whole-sequence attention."""
    from paged_attention_engine_b200.cache import CacheManager, PagedKVCache, plan_cache
    from paged_attention_engine_b200.config import ModelSpec, PartSpec, ScheduleEntry
    from paged_attention_engine_b200.engine.batch import BatchBuilder, StepEntry
    from paged_attention_engine_b200.parts import MIXERS

    hidden, heads, kv_heads, d = 56, 6, 2, 32
    params = {"hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": d, "qkv_bias": True,
              "scale": d ** -0.5, "window": window, "position_encoding": {"kind": "rotary", "head_dim": d, "theta": 1e4}}
    mixer_spec = PartSpec("gqa_attention", params, "a")
    norm = PartSpec("rms_norm", {"size": hidden, "eps": 1e-6}, "n")
    spec = ModelSpec("test", 8, hidden, 512, PartSpec("token_embedding", {"vocab_size": 8, "hidden_size": hidden}, "e"),
                     (helpers.decoder_layer(norm, mixer_spec, norm, PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": 8}, "f")),),
                     (ScheduleEntry(0),), norm, PartSpec("lm_head", {"vocab_size": 8, "hidden_size": hidden, "tied_to": "e.weight"}, "h"))
    gen = torch.Generator().manual_seed(5)
    w = {}
    for name, rows in (("q_proj", heads * d), ("k_proj", kv_heads * d), ("v_proj", kv_heads * d)):
        w[f"a.{name}.weight"] = (torch.randn(rows, hidden, generator=gen) * 0.3).to(dtype)
        w[f"a.{name}.bias"] = torch.randn(rows, generator=gen) * 0.1
    w["a.o_proj.weight"] = (torch.randn(hidden, heads * d, generator=gen) * 0.1).to(dtype)
    rt = runtime_of(dtype)
    mixer = MIXERS.get("gqa_attention")(mixer_spec, {k: v.cuda() for k, v in w.items()}, rt)
    plan = plan_cache(spec)
    manager = CacheManager(plan.groups, 16, 16, 2)
    cache = PagedKVCache(plan, manager, dtype, "cuda:0")
    builder = BatchBuilder(manager, rt.ops, dtype, "cuda:0")
    total = 45
    x = torch.randn(total, hidden, generator=gen).to(dtype)
    residual = torch.randn(total, hidden, generator=gen).to(dtype)
    manager.create_request("r")
    got, at = [], 0
    for n in (20, 1, 17, 1, 6):
        manager.reserve("r", n)
        ctx = builder.build([StepEntry("r", [0] * n, ())])
        got.append(rt.ops.materialized(mixer.forward(ctx, x[at : at + n].cuda(), residual[at : at + n].cuda(), cache.entry_cache(0))).float().cpu())
        manager.advance("r", n)
        at += n
    cfg = plain.PlainConfig(1, hidden, heads, kv_heads, d, 8, 8, 1e-6, 1e4, True, (window,))
    cos, sin = plain.rotary_tables(plain.rotary_inv_freq(d, 1e4), torch.arange(total), torch.float32)
    pw = {k.replace("a.", "p."): v.float() for k, v in w.items()}
    want = residual.float() + plain.attention_layer(x.float(), pw, "p.", cfg, cos, sin, window)
    assert (torch.cat(got) - want).abs().max().item() <= _limit(dtype, want)
