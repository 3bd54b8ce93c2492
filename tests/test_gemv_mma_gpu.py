"""The products of up to 24 tokens as single mma.sync kernels (csrc/gemv_mma.cu) against the plain
reference, each kind alone and at other sizes than the engine's: o and down (+ residual),
gate|up with SiLU x up, q|k|v with bias, rotation and page write; each with and without the
RMSNorm of its input folded in; every built launch shape; the same bits whatever the batch; what
is refused; where the kernels layer sends a product to them; and the path of a wait that runs out."""

import ctypes

import pytest
import torch

import torch_ops as ref

pytestmark = pytest.mark.gpu

SHAPES = [(8, 2, 4), (8, 2, 2), (8, 3, 3), (8, 3, 4), (8, 3, 2)]
QKV, RESIDUAL, GATE_UP = 0, 1, 2


@pytest.fixture(scope="module")
def ops():
    from paged_attention_engine_b200.kernels import ops as kernel_ops

    kernel_ops.use_tensor_cores = True
    yield kernel_ops
    lib = kernel_ops._lib("gemv_mma")
    for kind in range(3):
        lib.pae_linear_few_tokens_configure(kind, 0, 0, 0)
    kernel_ops.few_token_products_everywhere = False
    kernel_ops.use_few_token_products = True


def _rand(shape, seed, std=1.0):
    gen = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=gen) * std).to(torch.bfloat16).cuda()


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def _call(ops, name, *args):
    lib = ops._lib("gemv_mma")
    code = getattr(lib, name)(*args)
    if code:
        raise ops.KernelError(lib.pae_last_error().decode())


def _flag(ops):
    return ops.error_flag("cuda:0").data_ptr()


def _linear(ops, x, w, residual=None, norm=None, eps=0.0):
    out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.bfloat16, device="cuda")
    _call(ops, "pae_linear_few_tokens", _ptr(out), _ptr(x), _ptr(w), _ptr(residual), _ptr(norm), eps, x.shape[0], w.shape[0],
          w.shape[1], _flag(ops), 0)
    return out


def _swiglu(ops, x, w, norm=None, eps=0.0):
    out = torch.empty((x.shape[0], w.shape[0] // 2), dtype=torch.bfloat16, device="cuda")
    _call(ops, "pae_linear_swiglu_few_tokens", _ptr(out), _ptr(x), _ptr(w), _ptr(norm), eps, x.shape[0], w.shape[0], w.shape[1],
          _flag(ops), 0)
    return out


def _qkv(ops, x, w, bias, norm, eps, table, slots, keys, values, heads, kv_heads, d, page):
    out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.bfloat16, device="cuda")
    _call(ops, "pae_qkv_few_tokens", _ptr(out), _ptr(x), _ptr(w), _ptr(bias), _ptr(norm), eps, _ptr(table), _ptr(slots), _ptr(keys),
          _ptr(values), x.shape[0], heads, kv_heads, d, page, w.shape[1], _flag(ops), 0)
    return out


def _close(got, want, what, scale=2.0 ** -7):
    limit = scale * max(1.0, float(want.float().abs().max()))
    gap = (got.float().cpu() - want.float().cpu()).abs().max().item()
    assert gap <= limit, f"{what}: max gap {gap:.3e} > {limit:.3e}"


def _norm_weight(k, seed):
    gen = torch.Generator().manual_seed(seed)
    return (1 + 0.2 * torch.randn(k, generator=gen)).cuda()


@pytest.mark.parametrize("tokens", [1, 3, 8, 9, 16, 17, 24])
@pytest.mark.parametrize("n,k", [(1536, 8960), (1536, 1536), (509, 128), (136, 64), (3001, 320), (24, 4096)])
@pytest.mark.parametrize("normed,residual", [(False, True), (False, False), (True, True)])
def test_o_and_down(ops, tokens, n, k, normed, residual):
    x = _rand((tokens, k), 1)
    w = _rand((n, k), 2, 0.05)
    r = _rand((tokens, n), 3) if residual else None
    gamma = _norm_weight(k, 4) if normed else None
    if not ops._lib("gemv_mma").pae_linear_few_tokens_supports(RESIDUAL, tokens, n, k, int(normed)):
        assert normed and ((tokens > 8 and k == 8960) or (tokens > 16 and k == 4096)), "only these normed operands are too large for shared memory"
        with pytest.raises(ops.KernelError, match="shared memory"):
            _linear(ops, x, w, r, gamma, 1e-5)
        return
    got = _linear(ops, x, w, r, gamma, 1e-5)
    ops.check_device_errors()
    source = ref.rms_norm(x.cpu(), gamma.cpu(), 1e-5) if normed else x.cpu()
    want = ref.linear(source, w.cpu(), None, None if r is None else r.cpu(), out_dtype=torch.float32)
    _close(got, want, f"[{tokens},{n},{k}]")


@pytest.mark.parametrize("tokens", [1, 5, 8, 12, 16, 21, 24])
@pytest.mark.parametrize("inter,k", [(8960, 1536), (176, 64), (48, 320), (2000, 256)])
@pytest.mark.parametrize("normed", [True, False])
def test_gate_up_with_silu(ops, tokens, inter, k, normed):
    x = _rand((tokens, k), 10)
    gate, up = _rand((inter, k), 11, 0.05), _rand((inter, k), 12, 0.05)
    w = ops.interleave_gate_up(gate, up)
    gamma = _norm_weight(k, 13) if normed else None
    got = _swiglu(ops, x, w, gamma, 1e-6)
    ops.check_device_errors()
    source = ref.rms_norm(x.cpu(), gamma.cpu(), 1e-6) if normed else x.cpu()
    want = ref.silu_mul(ref.linear(source, torch.cat([gate, up]).cpu()).to(torch.bfloat16))
    _close(got, want, f"[{tokens},{inter},{k}]", 2.0 ** -6)


@pytest.mark.parametrize("tokens", [1, 7, 8, 11, 16, 19, 24])
@pytest.mark.parametrize("heads,kv_heads,d,page,k", [(12, 2, 128, 16, 1536), (3, 1, 32, 16, 64), (5, 5, 48, 8, 320), (4, 2, 64, 16, 256),
                                                      (2, 1, 80, 16, 128)])
@pytest.mark.parametrize("normed", [True, False])
def test_qkv_with_bias_rotation_and_page_write(ops, tokens, heads, kv_heads, d, page, k, normed):
    pages = 6
    width = (heads + 2 * kv_heads) * d
    x = _rand((tokens, k), 20)
    w = _rand((width, k), 21, 0.05)
    bias = torch.randn(width, generator=torch.Generator().manual_seed(22)).cuda()
    gamma = _norm_weight(k, 23) if normed else None
    positions = torch.arange(40, 40 + tokens, dtype=torch.int32).cuda()
    inv_freq = (1.0 / (1e4 ** (torch.arange(0, d, 2).float() / d))).cuda()
    table = ops.rotary_table(positions, inv_freq)
    slots = torch.randperm(pages * page, generator=torch.Generator().manual_seed(24))[:tokens].to(torch.int32).cuda()
    keys = torch.zeros(pages, kv_heads, page, d, dtype=torch.bfloat16).cuda()
    values = torch.zeros_like(keys)
    got = _qkv(ops, x, w, bias, gamma, 1e-6, table, slots, keys, values, heads, kv_heads, d, page)
    ops.check_device_errors()
    source = ref.rms_norm(x.cpu(), gamma.cpu(), 1e-6) if normed else x.cpu()
    want_keys, want_values = torch.zeros_like(keys).cpu(), torch.zeros_like(values).cpu()
    want = ref.rotary_qk_cache_write(ref.linear(source, w.cpu(), bias.cpu()).to(torch.bfloat16), table.cpu(), slots.cpu(), want_keys,
                                     want_values, heads, kv_heads, d, page)
    _close(got, want, "qkv", 2.0 ** -6)
    _close(keys, want_keys, "keys", 2.0 ** -6)
    _close(values, want_values, "values", 2.0 ** -6)
    # what went to the pages is what stands in the output, bit for bit, and nothing else was written
    view = got.view(tokens, heads + 2 * kv_heads, d)
    page_of, offset = (slots // page).long(), (slots % page).long()
    assert torch.equal(keys[page_of, :, offset], view[:, heads:heads + kv_heads])
    assert torch.equal(values[page_of, :, offset], view[:, heads + kv_heads:])
    assert int((keys != 0).any(-1).sum()) <= tokens * kv_heads


def test_a_token_without_a_slot_is_not_written_and_parts_may_be_absent(ops):
    heads, kv_heads, d, page, k, tokens = 3, 1, 32, 16, 128, 5
    width = (heads + 2 * kv_heads) * d
    x, w = _rand((tokens, k), 30), _rand((width, k), 31, 0.05)
    slots = torch.tensor([4, -1, 9, -1, 17], dtype=torch.int32).cuda()
    keys = torch.zeros(2, kv_heads, page, d, dtype=torch.bfloat16).cuda()
    values = torch.zeros_like(keys)
    got = _qkv(ops, x, w, None, None, 0.0, None, slots, keys, values, heads, kv_heads, d, page)
    ops.check_device_errors()
    _close(got, ref.linear(x.cpu(), w.cpu()), "no bias, no rotation")
    written = (keys != 0).any(-1).any(1).flatten().nonzero().flatten().tolist()
    assert written == [4, 9, 17]
    alone = _qkv(ops, x, w, None, None, 0.0, None, None, None, None, heads, kv_heads, d, page)
    assert torch.equal(alone, got)


@pytest.mark.parametrize("tokens", [4, 13, 22])
def test_every_built_shape_gives_the_same_bits(ops, tokens):
    """Stages and chunks per stage change when a piece of a weight row arrives, not the order of a sum."""
    lib = ops._lib("gemv_mma")
    x, xi = _rand((tokens, 1536), 40), _rand((tokens, 2240), 41, 0.3)
    wo, wd = _rand((1536, 1536), 42, 0.05), _rand((1536, 2240), 43, 0.05)
    wg = ops.interleave_gate_up(_rand((2240, 1536), 44, 0.05), _rand((2240, 1536), 45, 0.05))
    r, gamma = _rand((tokens, 1536), 46), _norm_weight(1536, 47)
    products = (lambda: _linear(ops, x, wo, r), lambda: _linear(ops, xi, wd, r), lambda: _swiglu(ops, x, wg, gamma, 1e-6),
                lambda: _linear(ops, x, wo, None, gamma, 1e-6))
    results = [[] for _ in products]
    try:
        for warps, stages, boxes in SHAPES:
            for kind in range(3):
                assert lib.pae_linear_few_tokens_configure(kind, warps, stages, boxes) == 0
            for product, seen in zip(products, results):
                try:
                    seen.append(product())
                except ops.KernelError as refused:      # activations beside the weights in the widest rings
                    assert "shared memory" in str(refused) and (tokens > 8 or (stages, boxes) == (3, 4))
    finally:
        for kind in range(3):
            assert lib.pae_linear_few_tokens_configure(kind, 0, 0, 0) == 0
    ops.check_device_errors()
    for product, seen in zip(products, results):
        assert len(seen) >= 4 or (tokens > 8 and len(seen) >= 1)
        seen.append(product())                         # the library's own choice
        for other in seen[1:]:
            assert torch.equal(seen[0], other)
    assert lib.pae_linear_few_tokens_configure(1, 3, 3, 3) != 0, "a shape that was not built is refused"


def test_a_tokens_product_does_not_depend_on_the_batch(ops):
    """Alone, among 7 others, among 23 others: the same sums in the same order, in every kind."""
    x = _rand((24, 1536), 50)
    gamma = _norm_weight(1536, 51)
    wo = _rand((2048, 1536), 52, 0.05)
    wg = ops.interleave_gate_up(_rand((640, 1536), 53, 0.05), _rand((640, 1536), 54, 0.05))
    whole = (_linear(ops, x, wo), _linear(ops, x, wo, None, gamma, 1e-6), _swiglu(ops, x, wg, gamma, 1e-6),
             _qkv(ops, x, wo, None, gamma, 1e-6, None, None, None, None, 12, 2, 128, 16))
    for count in (1, 8, 9, 16, 17):
        part_x = x[:count].contiguous()
        part = (_linear(ops, part_x, wo), _linear(ops, part_x, wo, None, gamma, 1e-6), _swiglu(ops, part_x, wg, gamma, 1e-6),
                _qkv(ops, part_x, wo, None, gamma, 1e-6, None, None, None, None, 12, 2, 128, 16))
        for a, b in zip(part, whole):
            assert torch.equal(a, b[:count]), f"{count} tokens"


def test_what_is_refused(ops):
    x, w = _rand((4, 128), 60), _rand((64, 128), 61)
    with pytest.raises(ops.KernelError, match="25 tokens"):
        _linear(ops, _rand((25, 128), 62), w)
    with pytest.raises(ops.KernelError, match="multiple of 64"):
        _linear(ops, _rand((4, 96), 63), _rand((64, 96), 64))
    with pytest.raises(ops.KernelError, match="16-byte boundary"):
        _linear(ops, _rand((5, 128), 65).flatten()[4:4 + 4 * 128].view(4, 128), w)
    with pytest.raises(ops.KernelError, match="blocks of 16 gate and 16 up"):
        _swiglu(ops, x, _rand((48, 128), 66))
    with pytest.raises(ops.KernelError, match="head_dim 24"):
        _qkv(ops, x, _rand((96, 128), 67), None, None, 0.0, None, None, None, None, 2, 1, 24, 16)
    # a normed operand of 16 tokens x 16,384 does not fit shared memory beside any ring
    wide = _rand((16, 16384), 68)
    with pytest.raises(ops.KernelError, match="shared memory"):
        _linear(ops, wide, _rand((32, 16384), 69), None, _norm_weight(16384, 70), 1e-6)
    lib = ops._lib("gemv_mma")
    assert lib.pae_linear_few_tokens_supports(RESIDUAL, 16, 32, 16384, 1) == 0
    assert lib.pae_linear_few_tokens_supports(RESIDUAL, 16, 32, 16384, 0) != 0
    assert lib.pae_linear_few_tokens_supports(RESIDUAL, 25, 32, 128, 0) == 0
    ops.check_device_errors()


def test_where_the_kernels_layer_sends_a_product(ops):
    """To these kernels where all blocks of the launch run at once (the library answers 2): the four products of
    the 1536-wide model do, q|k|v and gate|up of the 3584-wide one do not and stay with tcgen05."""
    lib = ops._lib("gemv_mma")
    sms = ops._lib("gemm_tcgen05").pae_sm_count()
    small = [(QKV, 2048, 1536, 1), (RESIDUAL, 1536, 1536, 0), (GATE_UP, 17920, 1536, 1), (RESIDUAL, 1536, 8960, 0)]
    assert [lib.pae_linear_few_tokens_supports(kind, 8, n, k, normed) for kind, n, k, normed in small] == [2, 2, 2, 2]
    if sms <= 148:
        assert lib.pae_linear_few_tokens_supports(QKV, 8, 4608, 3584, 1) == 1
        assert lib.pae_linear_few_tokens_supports(GATE_UP, 8, 37888, 3584, 1) == 1
    x, gamma = _rand((8, 1536), 80), _norm_weight(1536, 81)
    wo, r = _rand((1536, 1536), 82, 0.05), _rand((8, 1536), 83)
    product = ops.linear(x, wo, residual=r)
    assert isinstance(product, torch.Tensor), "finished output, nothing left to sum"
    pending_norm = ops.rms_norm(product, gamma, 1e-6)
    assert isinstance(pending_norm, ops.PendingNorm) and pending_norm.value is None, "the norm waits for the product that takes it"
    big = _rand((6144, 1536), 84, 0.05)        # 384 blocks: more than run at once
    if sms <= 148:
        taken = ops.linear(pending_norm, big)
        assert pending_norm.value is not None, "a product that does not fold the norm in has it computed"
        _close(ops.materialized(taken), ref.linear(ref.rms_norm(product.cpu(), gamma.cpu(), 1e-6), big.cpu()), "norm, then tcgen05")
    _close(ops.materialized(ops.rms_norm(product, gamma, 1e-6)), ref.rms_norm(product.cpu(), gamma.cpu(), 1e-6), "the norm alone")
    ops.use_few_token_products = False
    try:
        assert isinstance(ops.linear(x, wo, residual=r), ops.PendingSum)
        assert isinstance(ops.rms_norm(x, gamma, 1e-6), torch.Tensor)
    finally:
        ops.use_few_token_products = True
    ops.few_token_products_everywhere = True
    try:
        everywhere = ops.linear(ops.rms_norm(product, gamma, 1e-6), big)
        assert isinstance(everywhere, torch.Tensor)
        _close(everywhere, ref.linear(ref.rms_norm(product.cpu(), gamma.cpu(), 1e-6), big.cpu()), "two waves of blocks")
    finally:
        ops.few_token_products_everywhere = False
    ops.check_device_errors()


def test_a_wait_that_runs_out_is_reported_and_the_next_call_is_right(ops):
    """Warp 3 of every block announces its second stage and never asks for it: its wait gives up
    after a few thousand polls, the kernel ends by itself, the error word says 8."""
    tokens, n, k = 6, 512, 4096
    x, w = _rand((tokens, k), 90), _rand((n, k), 91, 0.05)
    out = torch.empty((tokens, n), dtype=torch.bfloat16, device="cuda")
    ops.check_device_errors()
    _call(ops, "pae_linear_few_tokens_selftest_giveup", _ptr(out), _ptr(x), _ptr(w), tokens, n, k, 3, 1, _flag(ops), 0)
    torch.cuda.synchronize()                     # the kernel came back by itself
    assert int(ops.error_flag("cuda:0").item()) == 8
    with pytest.raises(ops.KernelError, match="role code 8"):
        ops.check_device_errors()
    ops.check_device_errors()                    # the word was cleared
    _close(_linear(ops, x, w), ref.linear(x.cpu(), w.cpu()), "the call after")
    ops.check_device_errors()
