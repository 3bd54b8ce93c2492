"""Each kernel alone against its plain reference (tests/torch_ops.py), at sizes other than
the engine's tiny models: widths and vocabularies that are no power of two, head sizes in
steps of 16, odd numbers of heads and groups, page sizes from 1 up."""

import pytest
import torch

import torch_ops as ref

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from paged_attention_engine_b200.kernels import ops as kernel_ops

    return kernel_ops


def _close(got, want, dtype, scale=1.0):
    got, want = got.float().cpu(), want.float().cpu()
    limit = (2e-5 if dtype == torch.float32 else 2.0 ** -7) * max(1.0, float(want.abs().max())) * scale
    gap = (got - want).abs().max().item()
    assert gap <= limit, f"max gap {gap:.3e} > {limit:.3e}"


def _rand(shape, dtype, seed, std=1.0):
    gen = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=gen) * std).to(dtype).cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width", [(1, 8), (7, 100), (33, 1536), (5, 4104)])
def test_rms_norm(ops, dtype, rows, width):
    x = _rand((rows, width), dtype, 1, 3.0)
    w = (1 + 0.1 * torch.randn(width)).cuda()
    _close(ops.rms_norm(x, w, 1e-5), ref.rms_norm(x.cpu(), w.cpu(), 1e-5), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gather_and_embedding(ops, dtype):
    table = _rand((301, 72), dtype, 2)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32).cuda()
    assert torch.equal(ops.embedding(ids, table).cpu(), table.cpu()[ids.cpu().long()])
    assert torch.equal(ops.gather_rows(table, ids[:2]).cpu(), table.cpu()[[0, 300]])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,n,k", [(1, 509, 96), (5, 64, 176), (70, 130, 257), (129, 1536, 1536), (8, 3001, 520)])
@pytest.mark.parametrize("extras", ["plain", "bias", "bias+residual"])
def test_linear(ops, dtype, m, n, k, extras):
    x = _rand((m, k), dtype, 3)
    w = _rand((n, k), dtype, 4, 0.05)
    bias = torch.randn(n).cuda() if "bias" in extras else None
    res = _rand((m, n), dtype, 5) if "residual" in extras else None
    want = ref.linear(x.cpu(), w.cpu(), None if bias is None else bias.cpu(), None if res is None else res.cpu())
    _close(ops.materialized(ops.linear(x, w, bias, res)), want, dtype)


def test_linear_mixed_types(ops):
    x = _rand((9, 200), torch.bfloat16, 6)
    w32 = _rand((77, 200), torch.float32, 7, 0.05)
    w16 = w32.to(torch.bfloat16)
    _close(ops.linear(x, w32), ref.linear(x.cpu(), w32.cpu()), torch.bfloat16)
    out = ops.materialized(ops.linear(x, w16, out_dtype=torch.float32))
    assert out.dtype == torch.float32
    _close(out, ref.linear(x.cpu().float(), w16.cpu().float()), torch.float32)


def test_linear_rows_do_not_depend_on_the_batch(ops):
    """A token's product is the same bits whether it runs alone or among others."""
    x = _rand((37, 300), torch.float32, 8)
    w = _rand((190, 300), torch.float32, 9, 0.05)
    whole = ops.linear(x, w)
    for r in (0, 13, 36):
        assert torch.equal(ops.linear(x[r : r + 1].contiguous(), w)[0], whole[r])


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(ops, dtype):
    gu = _rand((11, 2 * 173), dtype, 10, 4.0)
    _close(ops.silu_mul(gu), ref.silu_mul(gu.cpu()), dtype)


@pytest.mark.parametrize("theta,half", [(1e4, 8), (1e6, 64)])
def test_rotary_table(ops, theta, half):
    positions = torch.tensor([0, 1, 2, 77, 4095, 32767], dtype=torch.int32).cuda()
    inv_freq = (1.0 / (theta ** (torch.arange(0, 2 * half, 2).float() / (2 * half)))).cuda()
    got = ops.rotary_table(positions, inv_freq).cpu()
    angle = positions.cpu().float()[:, None] * inv_freq.cpu()[None, :]
    want = torch.cat((angle.double().cos(), angle.double().sin()), dim=-1).float()
    assert (got - want).abs().max().item() <= 2e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,d,page", [(4, 2, 16, 4), (3, 1, 32, 16), (7, 7, 48, 1), (12, 2, 128, 16)])
def test_rotary_and_cache_write(ops, dtype, heads, kv_heads, d, page):
    tokens, pages = 19, 9
    qkv = _rand((tokens, (heads + 2 * kv_heads) * d), dtype, 11)
    positions = torch.arange(100, 100 + tokens, dtype=torch.int32).cuda()
    inv_freq = (1.0 / (1e4 ** (torch.arange(0, d, 2).float() / d))).cuda()
    table = ops.rotary_table(positions, inv_freq)
    slots = torch.randperm(pages * page)[:tokens].to(torch.int32) if pages * page >= tokens else None
    if slots is None:
        pages = tokens
        slots = torch.randperm(pages * page)[:tokens].to(torch.int32)
    keys = torch.zeros(pages, kv_heads, page, d, dtype=dtype).cuda()
    values = torch.zeros_like(keys)
    want_qkv, want_k, want_v = qkv.cpu().clone(), keys.cpu().clone(), values.cpu().clone()
    ref.rotary_qk_cache_write(want_qkv, table.cpu(), slots, want_k, want_v, heads, kv_heads, d, page)
    ops.rotary_qk_cache_write(qkv, table, slots.cuda(), keys, values, heads, kv_heads, d, page)
    _close(qkv, want_qkv, dtype)
    _close(keys, want_k, dtype)
    _close(values, want_v, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize(
    "heads,kv_heads,d,page,window",
    [(4, 2, 16, 4, 0), (3, 1, 32, 16, 0), (5, 5, 48, 8, 24), (6, 3, 64, 1, 0), (12, 2, 128, 16, 0), (2, 1, 256, 32, 40)],
)
def test_paged_attention(ops, dtype, heads, kv_heads, d, page, window):
    """Portions at offsets, single tokens and whole prompts in one batch, over shuffled pages."""
    gen = torch.Generator().manual_seed(12)
    q_lens = [1, 37, 5, 1, 64]
    pos0 = [70, 0, 29, 0, 101]
    kv_lens = [p + n for p, n in zip(pos0, q_lens)]
    width = max(-(-n // page) for n in kv_lens)
    total_pages = sum(-(-n // page) for n in kv_lens) + 3
    order = torch.randperm(total_pages, generator=gen).tolist()
    table = torch.full((len(q_lens), width), -1, dtype=torch.int32)
    for b, n in enumerate(kv_lens):
        for i in range(-(-n // page)):
            table[b, i] = order.pop()
    keys = (torch.randn(total_pages, kv_heads, page, d, generator=gen)).to(dtype)
    values = (torch.randn(total_pages, kv_heads, page, d, generator=gen)).to(dtype)
    # One far key per request gets a large score, so that missing it cannot hide.
    qkv = torch.randn(sum(q_lens), (heads + 2 * kv_heads) * d, generator=gen).to(dtype)
    q_start = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), dtype=torch.int32)
    args = dict(num_heads=heads, num_kv_heads=kv_heads, head_dim=d, page_size=page, max_q_len=max(q_lens),
                max_kv_len=max(kv_lens), scale=d ** -0.5 * 3.0, window=window)
    tensors = [qkv, keys, values, table, q_start, torch.tensor(pos0, dtype=torch.int32), torch.tensor(kv_lens, dtype=torch.int32)]
    want = ref.paged_attention(*tensors, **args)
    got = ops.paged_attention(*[t.cuda() for t in tensors], **args)
    _close(got, want, dtype, scale=2.0)


@pytest.mark.parametrize("vocab", [5, 509, 151936])
def test_sampling(ops, vocab):
    gen = torch.Generator().manual_seed(13)
    rows = 6
    logits = torch.randn(rows, vocab, generator=gen)
    logits[0, vocab // 2] = logits[0, vocab - 1] = 9.0        # a tie: the lower index wins
    temperature = torch.tensor([0.0, 0.0, 0.7, 1.0, 1.3, 0.7])
    seed = torch.tensor([1, 1, 1, 2**40 + 5, 7, 1], dtype=torch.int64)
    key = torch.tensor([0, 1, 2, 3, 4, 2], dtype=torch.int32)
    index = torch.tensor([0, 0, 5, 6, 7, 5], dtype=torch.int32)
    lo = (seed & 0xFFFFFFFF).to(torch.int64)
    lo = torch.where(lo >= 2**31, lo - 2**32, lo).to(torch.int32)
    hi = (seed >> 32).to(torch.int32)
    got = ops.sample(logits.cuda(), temperature.cuda(), lo.cuda(), hi.cuda(), key.cuda(), index.cuda()).cpu()
    assert got[0].item() == vocab // 2
    assert got[1].item() == int(torch.argmax(logits[1]))
    logits[5] = logits[2]
    got2 = ops.sample(logits.cuda(), temperature.cuda(), lo.cuda(), hi.cuda(), key.cuda(), index.cuda()).cpu()
    # the same call can also leave every row's token where the next step's embedding looks for it
    last = torch.full((40,), -7, dtype=torch.int32).cuda()
    rows_of = torch.tensor([4, 0, 9, 2, 7, 11], dtype=torch.int32).cuda()                # wanted place r is this token row,
    entry_of = torch.tensor([1, 0, 0, 4, 4, 4, 4, 2, 2, 3, 3, 5], dtype=torch.int32).cuda()   # a token row belongs to this entry,
    slot_of = torch.tensor([3, 9, 0, 31, 17, 22], dtype=torch.int32).cuda()                # whose state slot this is
    got3 = ops.sample(logits.cuda(), temperature.cuda(), lo.cuda(), hi.cuda(), key.cuda(), index.cuda(),
                      keep=(last, rows_of, entry_of, slot_of)).cpu()
    assert torch.equal(got3, got2)
    want_last = torch.full((40,), -7, dtype=torch.int32)
    ref.scatter_tokens(want_last, got2, rows_of.cpu(), entry_of.cpu(), slot_of.cpu())
    assert torch.equal(last.cpu(), want_last) and int((want_last != -7).sum()) == rows
    assert got2[5] == got2[2], "the same counters and logits draw the same token whatever the row"
    # The device's float32 scores may order two near-equal candidates otherwise than the
    # float64 restatement: the token drawn must score within 1e-4 of the restatement's best.
    from plain import qwen2_plain as plain
    for r in range(2, 5):
        # the vectorised restatement at every vocabulary (at 151,936 the draw is two kernels and scratch) ...
        scores = ref.gumbel_scores(logits[r], float(temperature[r]), lo[r], hi[r], key[r], index[r])
        assert scores[got[r]].item() >= scores.max().item() - 1e-4, f"row {r}: drew {int(got[r])}, the best is {int(scores.argmax())}"
        if vocab <= 509:
            # ... which the plain implementation's entry-by-entry one agrees with
            slow = plain.sample_scores(logits[r], float(temperature[r]), int(seed[r]), int(key[r]), int(index[r]))
            assert (slow - scores).abs().max().item() <= 1e-9


def _paged_case(gen, q_lens, pos0, heads, kv_heads, d, page, dtype, spike=True, late_spike=False):
    """Random queries, keys and values over shuffled pages. With `spike`, one far key of every
    request (its key 3) is made to score high for every query, so that missing it shows. With
    `late_spike`, a key 40 places before a request's end scores far higher still than anything
    before it: a row's maximum then jumps by more than 2^8 in the middle of its walk over the keys."""
    kv_lens = [p + n for p, n in zip(pos0, q_lens)]
    width = max(-(-n // page) for n in kv_lens)
    total_pages = sum(-(-n // page) for n in kv_lens) + 5
    order = torch.randperm(total_pages, generator=gen).tolist()
    table = torch.full((len(q_lens), width), -1, dtype=torch.int32)
    for b, n in enumerate(kv_lens):
        for i in range(-(-n // page)):
            table[b, i] = order.pop()
    keys = torch.randn(total_pages, kv_heads, page, d, generator=gen)
    values = torch.randn(total_pages, kv_heads, page, d, generator=gen)
    qkv = torch.randn(sum(q_lens), (heads + 2 * kv_heads) * d, generator=gen)
    if spike:
        direction = torch.randn(d, generator=gen)
        direction /= direction.norm()
        q_view = qkv.view(sum(q_lens), heads + 2 * kv_heads, d)
        q_view[:, :heads] += 3.0 * direction
        for b, n in enumerate(kv_lens):
            j = min(3, n - 1)
            keys[table[b, j // page], :, j % page] += 3.0 * direction
            if late_spike and n > 80:
                j = n - 40
                keys[table[b, j // page], :, j % page] += 40.0 * direction
    q_start = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), dtype=torch.int32)
    tensors = [qkv.to(dtype), keys.to(dtype), values.to(dtype), table, q_start,
               torch.tensor(pos0, dtype=torch.int32), torch.tensor(kv_lens, dtype=torch.int32)]
    return tensors, kv_lens


@pytest.mark.parametrize("heads,kv_heads,d,page,window", [(4, 2, 128, 16, 0), (6, 1, 64, 64, 0), (2, 2, 128, 32, 700)])
@pytest.mark.parametrize("late_spike", [False, True])
def test_short_portions_over_long_contexts_share_their_keys_over_a_cluster(ops, heads, kv_heads, d, page, window, late_spike):
    """A few query tiles over thousands of keys: the launch is small enough that each query
    tile's keys are shared out over a cluster of blocks by itself. One far key (the request's
    key 3, in the first block's share) scores high for every query, with `late_spike` another
    near the end (the last block's share) far higher, so a share that is dropped, or merged with
    the wrong weight, shows."""
    gen = torch.Generator().manual_seed(37)
    q_lens, pos0 = [130, 64], [3000, 1900]
    tensors, kv_lens = _paged_case(gen, q_lens, pos0, heads, kv_heads, d, page, torch.bfloat16, late_spike=late_spike)
    args = dict(num_heads=heads, num_kv_heads=kv_heads, head_dim=d, page_size=page, max_q_len=max(q_lens),
                max_kv_len=max(kv_lens), scale=d ** -0.5, window=window)
    want = ref.paged_attention(*tensors, **args)
    info = {}
    got = ops.paged_attention(*[t.cuda() for t in tensors], **args, info=info)
    ops.check_device_errors()
    assert info["kernel"] == "tcgen05" and info["cluster"] >= (2 if window else 4), info
    _close(got, want, torch.bfloat16, scale=2.0)
    alone = ops.paged_attention(*[t.cuda() for t in tensors], **args, form=1, info=info)
    assert info["cluster"] == 1
    assert (got.float() - alone.float()).abs().max().item() <= 2.0 ** -6 * float(alone.float().abs().max())


@pytest.mark.parametrize("heads,kv_heads,d,page,window", [
    (12, 2, 128, 16, 0), (16, 1, 64, 32, 0), (3, 1, 32, 16, 0), (28, 4, 128, 16, 300), (8, 8, 64, 48, 0), (6, 2, 128, 64, 33),
])
def test_decode_attention_over_long_contexts(ops, heads, kv_heads, d, page, window):
    """Single tokens over contexts from one key to thousands, cut into slices and merged."""
    gen = torch.Generator().manual_seed(21)
    kv = [4096, 777, 17, 1, 16, 2049, 65]
    tensors, kv_lens = _paged_case(gen, [1] * len(kv), [n - 1 for n in kv], heads, kv_heads, d, page, torch.bfloat16)
    args = dict(num_heads=heads, num_kv_heads=kv_heads, head_dim=d, page_size=page, max_q_len=1,
                max_kv_len=max(kv_lens), scale=d ** -0.5, window=window)
    want = ref.paged_attention(*tensors, **args)
    got = ops.paged_attention(*[t.cuda() for t in tensors], **args, num_single=len(kv))
    _close(got, want, torch.bfloat16, scale=2.0)


@pytest.mark.parametrize("heads,kv_heads,d,page,window", [
    (12, 2, 128, 16, 0), (4, 4, 64, 16, 0), (3, 1, 32, 32, 0), (6, 3, 128, 16, 100), (2, 1, 64, 64, 17),
])
def test_prefill_attention_portions_at_offsets(ops, heads, kv_heads, d, page, window):
    """Portions of prompts at any offset (ragged against the 64-token blocks and the pages),
    beside single tokens, in one launch."""
    gen = torch.Generator().manual_seed(22)
    q_lens = [300, 1, 65, 2, 64, 1, 129]
    pos0 = [0, 500, 1000, 31, 64, 0, 77]
    tensors, kv_lens = _paged_case(gen, q_lens, pos0, heads, kv_heads, d, page, torch.bfloat16)
    args = dict(num_heads=heads, num_kv_heads=kv_heads, head_dim=d, page_size=page, max_q_len=max(q_lens),
                max_kv_len=max(kv_lens), scale=d ** -0.5, window=window)
    want = ref.paged_attention(*tensors, **args)
    got = ops.paged_attention(*[t.cuda() for t in tensors], **args)
    _close(got, want, torch.bfloat16, scale=2.0)
    # Knowing how many requests bring one token only changes how their keys are sliced: the
    # same sums in another order.
    got2 = ops.paged_attention(*[t.cuda() for t in tensors], **args, num_single=2)
    assert (got.float() - got2.float()).abs().max().item() <= 2.0 ** -7 * float(got.float().abs().max())


def test_tensor_core_attention_agrees_with_the_cuda_core_kernel(ops):
    gen = torch.Generator().manual_seed(23)
    q_lens, pos0 = [1, 40, 1, 7], [99, 3, 0, 60]
    tensors, kv_lens = _paged_case(gen, q_lens, pos0, 6, 2, 64, 16, torch.bfloat16)
    args = dict(num_heads=6, num_kv_heads=2, head_dim=64, page_size=16, max_q_len=40, max_kv_len=max(kv_lens),
                scale=0.125, window=0)
    fast = ops.paged_attention(*[t.cuda() for t in tensors], **args)
    ops.use_tensor_cores = False
    try:
        slow = ops.paged_attention(*[t.cuda() for t in tensors], **args)
    finally:
        ops.use_tensor_cores = True
    assert (fast.float() - slow.float()).abs().max().item() <= 2.0 ** -6 * float(slow.float().abs().max())


@pytest.mark.parametrize("heads,kv_heads,d,page,window", [
    (12, 2, 128, 16, 0), (4, 4, 64, 16, 0), (3, 1, 128, 32, 0), (6, 3, 128, 16, 100), (2, 1, 64, 64, 17), (5, 5, 128, 128, 0),
])
@pytest.mark.parametrize("form,late_spike", [(1, False), (2, False), (1, True), (2, True), (4, False), (4, True), (8, True),
                                             (16, False), (0, True)])
def test_tcgen05_prefill_attention(ops, heads, kv_heads, d, page, window, form, late_spike):
    """The tcgen05 kernels (form 1: 128-key tiles, one block per SM; form 2: 64-key tiles, the
    output kept in tensor memory, two blocks per SM; forms 4, 8, 16: the first with a query
    tile's keys shared out over a cluster of 2, 4, 8 blocks, whose outputs the first block
    merges, some of them with no keys at all; 0: whichever the launch's size picks): portions of
    64 tokens and more at offsets that are ragged against the 128-row tiles, the pages and the
    key tiles, beside shorter portions and single tokens."""
    gen = torch.Generator().manual_seed(31)
    q_lens = [300, 1, 129, 2, 128, 1, 65, 700]
    pos0 = [0, 500, 1000, 31, 64, 0, 77, 5]
    tensors, kv_lens = _paged_case(gen, q_lens, pos0, heads, kv_heads, d, page, torch.bfloat16, late_spike=late_spike)
    args = dict(num_heads=heads, num_kv_heads=kv_heads, head_dim=d, page_size=page, max_q_len=max(q_lens),
                max_kv_len=max(kv_lens), scale=d ** -0.5, window=window)
    want = ref.paged_attention(*tensors, **args)
    assert ops.use_tcgen05_attention
    info = {}
    got = ops.paged_attention(*[t.cuda() for t in tensors], **args, form=form, info=info)
    assert info["kernel"] == "tcgen05" and (form == 0 or info["cluster"] == {1: 1, 2: 0}.get(form, form // 2)), info
    ops.check_device_errors()
    _close(got, want, torch.bfloat16, scale=2.0)
    ops.use_tcgen05_attention = False
    try:
        other = ops.paged_attention(*[t.cuda() for t in tensors], **args)
    finally:
        ops.use_tcgen05_attention = True
    assert (got.float() - other.float()).abs().max().item() <= 2.0 ** -6 * float(other.float().abs().max())


@pytest.mark.parametrize("heads,kv_heads,d,page,window", [(12, 2, 128, 16, 0), (4, 4, 64, 32, 90)])
@pytest.mark.parametrize("kernel", ["tcgen05", "mma"])
def test_portion_kernels_launched_for_the_listed_requests_only(ops, heads, kv_heads, d, page, window, kernel):
    """Many requests that bring one token beside a few portions: with the list of those that bring
    more than one, the portion kernels launch blocks for them only; the result is the bits of a
    launch that covers every request and lets the blocks of the others return. A list of the wrong
    length is refused."""
    gen = torch.Generator().manual_seed(41)
    q_lens = [1] * 9 + [130] + [1] * 7 + [66, 1, 1, 2] + [1] * 5
    pos0 = [int(v) for v in torch.randint(0, 600, (len(q_lens),), generator=gen)]
    tensors, kv_lens = _paged_case(gen, q_lens, pos0, heads, kv_heads, d, page, torch.bfloat16)
    args = dict(num_heads=heads, num_kv_heads=kv_heads, head_dim=d, page_size=page, max_q_len=max(q_lens),
                max_kv_len=max(kv_lens), scale=d ** -0.5, window=window, num_single=q_lens.count(1))
    multi = torch.tensor([i for i, n in enumerate(q_lens) if n > 1], dtype=torch.int32).cuda()
    want = ref.paged_attention(*tensors, **{k: v for k, v in args.items() if k != "num_single"})
    on_device = [t.cuda() for t in tensors]
    ops.use_tcgen05_attention = kernel == "tcgen05"
    try:
        info = {}
        listed = ops.paged_attention(*on_device, **args, multi_index=multi, info=info)
        everyone = ops.paged_attention(*on_device, **args)
        assert info["kernel"] == kernel
        with pytest.raises(ops.KernelError, match="requests listed"):
            ops.paged_attention(*on_device, **args, multi_index=multi[:2])
    finally:
        ops.use_tcgen05_attention = True
    ops.check_device_errors()
    assert torch.equal(listed, everyone)
    _close(listed, want, torch.bfloat16, scale=2.0)


@pytest.mark.parametrize("heads,kv_heads,d,page,window", [(4, 2, 128, 16, 100), (6, 3, 64, 32, 70), (2, 1, 128, 16, 257), (4, 4, 64, 16, 33)])
@pytest.mark.parametrize("form", ["mma", 1, 2, 0])
def test_windowed_attention_over_a_table_with_released_pages(ops, heads, kv_heads, d, page, window, form):
    """A windowed layer as the cache manager leaves it: the table entries of the pages that the
    window has passed are -1 and the pages themselves hold something else by now (here: NaN, as
    do all pages that no request owns). No kernel may read through such an entry, whichever tile
    size it rounds the window's first key down to."""
    gen = torch.Generator().manual_seed(41)
    q_lens = [200, 1, 70, 1, 129, 64]
    pos0 = [300, 500, 1000, 90, 64, 37]
    tensors, kv_lens = _paged_case(gen, q_lens, pos0, heads, kv_heads, d, page, torch.bfloat16)
    qkv, keys, values, table, q_start, q_pos0, kv_len = tensors
    owned = set()
    for b, p0 in enumerate(pos0):
        released = max(p0 - window + 1, 0) // page          # what CacheManager.advance gives back before this step
        table[b, :released] = -1
        owned |= {int(x) for x in table[b] if x >= 0}
    for pid in range(keys.shape[0]):
        if pid not in owned:
            keys[pid] = float("nan")
            values[pid] = float("nan")
    args = dict(num_heads=heads, num_kv_heads=kv_heads, head_dim=d, page_size=page, max_q_len=max(q_lens),
                max_kv_len=max(kv_lens), scale=d ** -0.5, window=window)
    want = ref.paged_attention(*tensors, **args)
    assert torch.isfinite(want).all()
    info = {}
    if form == "mma":
        ops.use_tcgen05_attention = False
    try:
        got = ops.paged_attention(*[t.cuda() for t in tensors], **args, form=0 if form == "mma" else form, info=info)
    finally:
        ops.use_tcgen05_attention = True
    assert info["kernel"] == ("mma" if form == "mma" else "tcgen05"), info
    ops.check_device_errors()
    assert torch.isfinite(got).all(), "a kernel read a page that the table no longer names"
    _close(got, want, torch.bfloat16, scale=2.0)
    # the CUDA-core kernel in both dtypes
    ops.use_tensor_cores = False
    try:
        slow = ops.paged_attention(*[t.cuda() for t in tensors], **args)
        slow32 = ops.paged_attention(*[t.cuda().float() if t.is_floating_point() else t.cuda() for t in tensors], **args)
    finally:
        ops.use_tensor_cores = True
    assert torch.isfinite(slow).all() and torch.isfinite(slow32).all()
    _close(slow, want, torch.bfloat16, scale=2.0)
