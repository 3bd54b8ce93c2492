"""The tcgen05 products against the plain reference: the many-token form and the few-token
(swapped, split-K) form, at sizes with ragged edges in every dimension. The mma.sync kernels
that take products of up to 24 tokens where they are faster are switched off in this module
(tests/test_gemv_mma_gpu.py is theirs)."""

import pytest
import torch

import torch_ops as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from paged_attention_engine_b200.kernels import ops as kernel_ops

    kernel_ops.use_tensor_cores = True
    before = kernel_ops.use_few_token_products
    kernel_ops.use_few_token_products = False
    yield kernel_ops
    kernel_ops.use_few_token_products = before


def _rand(shape, seed, std=1.0):
    gen = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=gen) * std).to(torch.bfloat16).cuda()


def _check(ops, m, n, k, bias, residual, out_dtype):
    x = _rand((m, k), 1)
    w = _rand((n, k), 2, 0.05)
    b = torch.randn(n).cuda() if bias else None
    r = None
    if residual:
        r = _rand((m, n), 3) if out_dtype == torch.bfloat16 else torch.randn(m, n).cuda()
    got = ops.materialized(ops.linear(x, w, b, r, out_dtype=out_dtype))
    ops.check_device_errors()
    want = ref.linear(x.cpu(), w.cpu(), None if b is None else b.cpu(), None if r is None else r.cpu(), out_dtype=torch.float32)
    assert got.dtype == out_dtype and tuple(got.shape) == (m, n)
    limit = (2.0 ** -7 if out_dtype == torch.bfloat16 else 1e-4) * max(1.0, float(want.abs().max()))
    gap = (got.float().cpu() - want).abs().max().item()
    assert gap <= limit, f"[{m},{n},{k}] max gap {gap:.3e} > {limit:.3e}"


@pytest.mark.parametrize("m", [1, 8, 16, 17, 33, 64])
@pytest.mark.parametrize("n,k", [(2048, 1536), (1536, 8960), (509, 96), (136, 72), (3000, 264)])
def test_few_tokens(ops, m, n, k):
    _check(ops, m, n, k, bias=True, residual=True, out_dtype=torch.bfloat16)


@pytest.mark.parametrize("m,n,k", [(65, 128, 64), (129, 1536, 1536), (300, 130, 264), (2048, 2048, 1536), (515, 509, 96), (128, 24, 200)])
@pytest.mark.parametrize("extras", [(False, False), (True, False), (True, True)])
def test_many_tokens(ops, m, n, k, extras):
    _check(ops, m, n, k, bias=extras[0], residual=extras[1], out_dtype=torch.bfloat16)


def _expected_planes(m, n, k, sms):
    """The rule of `pae_linear_tcgen05_plane_count`, restated: as many K ranges per output tile as
    fill the SMs, each of at least 8 k-blocks of 64 where K is long (32 k-blocks and more; the
    tiles are then 256, 192 or 176 columns wide) and of at least 4 where it is short (tiles of 128
    and 64 columns too); 1 when the tiles fill half of the SMs by themselves, when K has fewer than
    8 k-blocks, or for few tokens or narrow outputs."""
    up = lambda a, b: -(-a // b)
    k_blocks = up(k, 64)
    if m <= 64 or n < 256 or k_blocks < 8:
        return 1
    tiles_a = up(m, 128)
    widths = (256, 192, 176) if k_blocks >= 32 else (256, 192, 176, 128, 64)
    width = min(widths, key=lambda w: (up(tiles_a * up(n, w), sms) * (w + 32), -w))
    tiles = tiles_a * up(n, width)
    if tiles * 2 > sms:
        return 1
    planes = min(sms // tiles, k_blocks // (8 if k_blocks >= 32 else 4))
    if planes < 2:
        return 1
    return up(k_blocks, up(k_blocks, planes))


def test_the_plane_rule_at_148_sms():
    """What the rule gives on a B200 (148 SMs), as a record of the sizes it was tuned at."""
    cases = [(65, 1536, 8960, 16), (128, 1536, 8960, 16), (300, 1536, 8960, 5), (1024, 1536, 8960, 2),
             (130, 520, 2056, 4), (2048, 1536, 8960, 1), (128, 1536, 1536, 6), (128, 2048, 1536, 4), (300, 2048, 1536, 1)]
    assert [_expected_planes(m, n, k, 148) for m, n, k, _ in cases] == [p for *_, p in cases]


@pytest.mark.parametrize("m,n,k", [(65, 1536, 8960), (128, 1536, 8960), (300, 1536, 8960), (1024, 1536, 8960),
                                   (130, 520, 2056), (2048, 1536, 8960), (128, 1536, 1536), (128, 2048, 1536), (200, 3584, 18944),
                                   (100, 5120, 27648), (70, 3001, 520)])
@pytest.mark.parametrize("extras", [(False, False), (True, True)])
def test_few_output_tiles_and_a_long_k_share_k_over_blocks(ops, m, n, k, extras):
    """A down projection for a few hundred tokens has a handful of output tiles: each tile's K
    is shared out over blocks that write float32 planes, which the consumer adds up. The plane
    count is what fills this device's SMs, 1 when the tiles do already or K is short."""
    lib = ops._lib("gemm_tcgen05")
    import ctypes
    planes = _expected_planes(m, n, k, lib.pae_sm_count())
    assert lib.pae_linear_tcgen05_plane_count(ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k)) == planes
    x = _rand((m, k), 1)
    w = _rand((n, k), 2, 0.05)
    # Up to 128 tokens over a K of 2,048 and more stay with the swapped product (its splits, not planes);
    # the many-token kernel and its plane rule are asked for those sizes all the same.
    for long_k_limit in (ops.SWAPPED_MAX_TOKENS_LONG_K, ops.SWAPPED_MAX_TOKENS):
        ops.SWAPPED_MAX_TOKENS_LONG_K = long_k_limit
        try:
            pending = ops.linear(x, w)
            if ops._swapped(m, k):
                assert tuple(pending.partial.shape) == (lib.pae_linear_swapped_splits(n, k), m, n)
            else:
                assert isinstance(pending, ops.PendingSum) == (planes > 1)
                if planes > 1:
                    assert tuple(pending.partial.shape) == (planes, m, n)
            _check(ops, m, n, k, bias=extras[0], residual=extras[1], out_dtype=torch.bfloat16)
        finally:
            ops.SWAPPED_MAX_TOKENS_LONG_K = 128


def test_a_wait_that_runs_out_is_reported_and_the_next_call_is_right(ops):
    """The kernels' only failure detection is the bounded wait on an mbarrier. The self-test
    kernel is the few-token product whose producer never loads one k-block (nothing is in
    flight for it): the MMA issuer's wait for that stage runs out after a few thousand polls, the
    block leaves by its give-up path (loads in flight waited for, tensor memory freed), and
    the error word holds the role's code. Afterwards the context is intact and an ordinary
    product is right."""
    import ctypes
    from ctypes import c_int, c_void_p

    lib = ops._lib("gemm_tcgen05")
    m, n, k = 8, 2048, 1536
    x = _rand((m, k), 1)
    w = _rand((n, k), 2, 0.05)
    ops.check_device_errors()
    splits = lib.pae_linear_swapped_splits(c_int(n), c_int(k))
    partial = torch.zeros((splits, m, n), dtype=torch.float32, device="cuda")
    flag = ops.error_flag("cuda:0")
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    code = lib.pae_linear_tcgen05_selftest_giveup(c_void_p(partial.data_ptr()), c_void_p(x.data_ptr()), c_void_p(w.data_ptr()),
                                                  c_int(m), c_int(n), c_int(k), c_int(1), c_void_p(flag.data_ptr()), stream)
    assert code == 0, lib.pae_last_error().decode()
    torch.cuda.synchronize()                     # the kernel came back by itself
    assert int(flag.item()) == 2, "the MMA issuer's wait (role 2) is the one that runs out"
    with pytest.raises(ops.KernelError, match="role code 2"):
        ops.check_device_errors()
    ops.check_device_errors()                    # the word was cleared
    _check(ops, m, n, k, bias=True, residual=True, out_dtype=torch.bfloat16)
    _check(ops, 300, n, k, bias=True, residual=False, out_dtype=torch.bfloat16)


@pytest.mark.parametrize("m,n,k", [(4, 151936, 1536), (70, 3001, 520), (8, 509, 96)])
def test_float32_logits(ops, m, n, k):
    _check(ops, m, n, k, bias=False, residual=False, out_dtype=torch.float32)


def test_agrees_with_the_cuda_core_kernel(ops):
    x = _rand((40, 1536), 5)
    w = _rand((1000, 1536), 6, 0.05)
    fast = ops.materialized(ops.linear(x, w))
    ops.use_tensor_cores = False
    try:
        slow = ops.linear(x, w)
    finally:
        ops.use_tensor_cores = True
    assert (fast.float() - slow.float()).abs().max().item() <= 2.0 ** -7 * float(slow.float().abs().max())


def test_a_tokens_product_does_not_depend_on_the_batch(ops):
    """Alone, among 7 others, among 63 others: the same sums in the same order."""
    x = _rand((64, 1536), 7)
    w = _rand((2048, 1536), 8, 0.05)
    whole = ops.materialized(ops.linear(x, w))
    for count in (1, 8, 24):
        part = ops.materialized(ops.linear(x[:count].contiguous(), w))
        assert torch.equal(part, whole[:count]), f"{count} tokens"


def _pending(ops, m, n, k, bias, residual, seed):
    x = _rand((m, k), seed)
    w = _rand((n, k), seed + 1, 0.05)
    b = torch.randn(n).cuda() if bias else None
    r = _rand((m, n), seed + 2) if residual else None
    ops.fuse_split_sums = True
    pending = ops.linear(x, w, b, r)
    assert isinstance(pending, ops.PendingSum), "a step of few tokens leaves its product to be summed"
    ops.fuse_split_sums = False
    try:
        plain = ops.linear(x, w, b, r)
    finally:
        ops.fuse_split_sums = True
    return pending, plain


def test_sum_fused_into_rms_norm(ops):
    pending, plain = _pending(ops, 8, 1536, 8960, bias=False, residual=True, seed=30)
    weight = (1 + 0.1 * torch.randn(1536)).cuda()
    normed = ops.rms_norm(pending, weight, 1e-6)
    assert torch.equal(ops.materialized(pending), plain), "the summed residual stream is the same bits"
    want = ops.rms_norm(plain, weight, 1e-6)
    # The two norm kernels add the squares in different orders: one rounding step apart at most.
    assert (normed.float() - want.float()).abs().max().item() <= 2.0 ** -7 * float(want.float().abs().max())


def test_sum_fused_into_silu_mul(ops):
    pending, plain = _pending(ops, 5, 2 * 176, 96, bias=False, residual=False, seed=40)
    assert torch.equal(ops.silu_mul(pending), ops.silu_mul(plain))


@pytest.mark.parametrize("heads,kv_heads,d,page", [(12, 2, 128, 16), (3, 1, 32, 16), (5, 5, 48, 8)])
def test_sum_fused_into_rotation_and_page_write(ops, heads, kv_heads, d, page):
    tokens, pages = 7, 6
    width = (heads + 2 * kv_heads) * d
    pending, plain = _pending(ops, tokens, width, 264, bias=True, residual=False, seed=50)
    positions = torch.arange(40, 40 + tokens, dtype=torch.int32).cuda()
    inv_freq = (1.0 / (1e4 ** (torch.arange(0, d, 2).float() / d))).cuda()
    table = ops.rotary_table(positions, inv_freq)
    slots = torch.randperm(pages * page)[:tokens].to(torch.int32).cuda()
    caches = [torch.zeros(pages, kv_heads, page, d, dtype=torch.bfloat16).cuda() for _ in range(4)]
    fused = ops.rotary_qk_cache_write(pending, table, slots, caches[0], caches[1], heads, kv_heads, d, page)
    unfused = ops.rotary_qk_cache_write(plain.clone(), table, slots, caches[2], caches[3], heads, kv_heads, d, page)
    def where(a, b):
        bad = (a != b).nonzero()
        return f"{bad.shape[0]} of {a.numel()} differ, first at {bad[0].tolist() if bad.shape[0] else None}: " \
               f"{a[tuple(bad[0])].item() if bad.shape[0] else ''} != {b[tuple(bad[0])].item() if bad.shape[0] else ''}; " \
               f"pending against plain: {(ops.materialized(pending) != plain).sum().item()} differ"

    assert torch.equal(fused, unfused), "qkv: " + where(fused, unfused)
    assert torch.equal(caches[0], caches[2]), "keys: " + where(caches[0], caches[2])
    assert torch.equal(caches[1], caches[3]), "values: " + where(caches[1], caches[3])


@pytest.mark.parametrize("m", [1, 8, 64, 65, 300, 2048])
@pytest.mark.parametrize("inter,k", [(8960, 1536), (176, 64), (256, 96), (2000, 264)])
def test_swiglu_inside_the_product(ops, m, inter, k):
    """silu(gate) * up in the product's epilogue (many tokens), in the split sum (few tokens) and as
    a kernel of its own give the same bits, and agree with the plain reference."""
    x = _rand((m, k), 60)
    gate = _rand((inter, k), 61, 0.05)
    up = _rand((inter, k), 62, 0.05)
    w = ops.interleave_gate_up(gate, up)
    assert w is not None and tuple(w.shape) == (2 * inter, k)
    assert torch.equal(w[:16], gate[:16]) and torch.equal(w[16:32], up[:16]) and torch.equal(w[32:48], gate[16:32])
    got = ops.linear_swiglu(x, w)
    ops.check_device_errors()
    ops.use_tensor_cores = False
    try:
        apart = ops.silu_mul(ops.linear(x, w), 16)
    finally:
        ops.use_tensor_cores = True
    want = ref.silu_mul(ref.linear(x.cpu(), torch.cat([gate, up]).cpu()).to(torch.bfloat16))
    limit = 2.0 ** -6 * max(1e-3, float(want.float().abs().max()))
    assert (got.float().cpu() - want.float()).abs().max().item() <= limit
    assert (got.float() - apart.float()).abs().max().item() <= limit
    assert ops.interleave_gate_up(gate[:24], up[:24]) is None, "an intermediate size that is no multiple of 16 stays apart"


@pytest.mark.parametrize("tokens", [65, 300, 2048])
@pytest.mark.parametrize("heads,kv_heads,d,page,k", [(12, 2, 128, 16, 1536), (4, 2, 64, 16, 256), (6, 3, 32, 8, 96), (5, 5, 128, 32, 264)])
def test_qkv_finished_in_the_products_epilogue(ops, tokens, heads, kv_heads, d, page, k):
    """q|k|v for a prompt's portion: bias, rotation and page write in the epilogue of the product
    give the same bits as the product followed by the rotation kernel."""
    width = (heads + 2 * kv_heads) * d
    x = _rand((tokens, k), 70)
    w = _rand((width, k), 71, 0.05)
    bias = torch.randn(width).cuda()
    positions = torch.arange(11, 11 + tokens, dtype=torch.int32).cuda()
    inv_freq = (1.0 / (1e4 ** (torch.arange(0, d, 2).float() / d))).cuda()
    table = ops.rotary_table(positions, inv_freq)
    pages = -(-tokens // page) + 3
    slots = torch.randperm(pages * page)[:tokens].to(torch.int32)
    slots[5] = -1                                    # a token whose page write is switched off
    slots = slots.cuda()
    caches = [torch.zeros(pages, kv_heads, page, d, dtype=torch.bfloat16).cuda() for _ in range(4)]
    before = ops.launches
    fused = ops.qkv_projection(x, w, bias, table, slots, caches[0], caches[1], heads, kv_heads, d, page)
    # one kernel, unless the output has so few tiles that K is shared out over blocks: then the
    # kernel that adds the planes up rotates and writes
    planes = ops._lib("gemm_tcgen05").pae_linear_tcgen05_plane_count(tokens, width, k)
    assert ops.launches - before == (1 if planes == 1 else 2), f"{planes} planes"
    assert planes == 1 or tokens == 65
    ops.check_device_errors()
    ops.fuse_qkv_epilogue = False
    try:
        apart = ops.qkv_projection(x, w, bias, table, slots, caches[2], caches[3], heads, kv_heads, d, page)
    finally:
        ops.fuse_qkv_epilogue = True
    assert torch.equal(fused, apart)
    assert torch.equal(caches[0], caches[2]) and torch.equal(caches[1], caches[3])
    # and without a position encoding or pages to write
    plain = ops.qkv_projection(x, w, bias, None, None, caches[0], caches[1], heads, kv_heads, d, page)
    assert torch.equal(plain, ops.materialized(ops.linear(x, w, bias)))
