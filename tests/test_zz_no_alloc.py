"""The allocation-free decode attention entry point (csrc/attention_decode_noalloc.h),
called through its exported C symbol as a program without torch's allocator would call it,
against the regular entry point that takes a scratch buffer from the caller, and against
plain attention over the same pages written out in torch (tests/torch_ops.py), which
shares nothing with either.

Some users of these libraries cannot allocate device memory when they call: the serving
process has handed all spare memory to the cache pool, the decode loop cannot afford the
device-wide synchronisation of cudaMalloc, or the host program has no allocator but
cudaMalloc itself. For them the scratch of the decode kernel lives inside the library.

This file is named so that pytest collects it last: a run that stops at the first failure
has then already run every other test. It must pass alone in a fresh process, and after
all the others.
"""

import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def libraries():
    from paged_attention_engine_b200.kernels import build

    paths = build.ensure_built(["attention_mma", "attention_decode_noalloc"])
    regular = ctypes.CDLL(str(paths["attention_mma"]))
    noalloc = ctypes.CDLL(str(paths["attention_decode_noalloc"]))
    for lib in (regular, noalloc):
        lib.pae_last_error.restype = ctypes.c_char_p
    regular.pae_decode_scratch_floats.restype = ctypes.c_longlong
    noalloc.pae_noalloc_scratch_capacity.restype = ctypes.c_longlong
    return regular, noalloc


def _case(seed, kv_lens, heads, kv_heads, d, page):
    gen = torch.Generator().manual_seed(seed)
    seqs = len(kv_lens)
    width = max(-(-n // page) for n in kv_lens)
    pages = sum(-(-n // page) for n in kv_lens) + 2
    order = torch.randperm(pages, generator=gen).tolist()
    table = torch.full((seqs, width), -1, dtype=torch.int32)
    for b, n in enumerate(kv_lens):
        for i in range(-(-n // page)):
            table[b, i] = order.pop()
    return dict(
        qkv=torch.randn(seqs, (heads + 2 * kv_heads) * d, generator=gen).to(torch.bfloat16).cuda(),
        keys=torch.randn(pages, kv_heads, page, d, generator=gen).to(torch.bfloat16).cuda(),
        values=torch.randn(pages, kv_heads, page, d, generator=gen).to(torch.bfloat16).cuda(),
        table=table.cuda(),
        q_start=torch.arange(seqs + 1, dtype=torch.int32).cuda(),
        kv_len=torch.tensor(kv_lens, dtype=torch.int32).cuda(),
        seqs=seqs, heads=heads, kv_heads=kv_heads, d=d, page=page, width=width,
    )


def _ptr(t):
    return c_void_p(t.data_ptr())


def _common_args(c, out, slice_keys, max_slices, window):
    return [
        _ptr(out), _ptr(c["qkv"]), _ptr(c["keys"]), _ptr(c["values"]), _ptr(c["table"]), c_int(c["width"]),
        _ptr(c["q_start"]), _ptr(c["kv_len"]), c_int(c["seqs"]), c_int(c["heads"]), c_int(c["kv_heads"]), c_int(c["d"]),
        c_int(c["page"]), c_float(c["d"] ** -0.5), c_int(window), c_int(slice_keys), c_int(max_slices),
    ]


def _both(libraries, c, slice_keys, window=0):
    regular, noalloc = libraries
    max_slices = -(-(int(c["kv_len"].max()) + 15) // slice_keys)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    shape = (c["seqs"], c["heads"] * c["d"])
    want = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
    floats = regular.pae_decode_scratch_floats(c_int(c["seqs"]), c_int(c["heads"]), c_int(c["d"]), c_int(max_slices))
    scratch = torch.empty(floats, dtype=torch.float32, device="cuda")
    code = regular.pae_paged_attention_decode(*_common_args(c, want, slice_keys, max_slices, window), _ptr(scratch), stream)
    assert code == 0, regular.pae_last_error().decode()
    got = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
    code = noalloc.pae_paged_attention_decode_noalloc(*_common_args(c, got, slice_keys, max_slices, window), stream)
    assert code == 0, noalloc.pae_last_error().decode()
    torch.cuda.synchronize()
    return got, want


def _plain(c, window=0):
    """The same attention in plain torch on the CPU: every request's one query over its pages."""
    import torch_ops

    kv = c["kv_len"].cpu()
    out = torch_ops.paged_attention(
        c["qkv"].cpu(), c["keys"].cpu(), c["values"].cpu(), c["table"].cpu(), c["q_start"].cpu(), kv - 1, kv,
        c["heads"], c["kv_heads"], c["d"], c["page"], 1, int(kv.max()), c["d"] ** -0.5, window)
    return out.float()


def test_two_calls_in_a_row_match_the_entry_point_with_caller_scratch(libraries):
    """The second call differs in every size from the first, so what the first left in the
    shared array lies under other slices, heads and requests of the second. Contexts of one
    key, of exactly one slice, of an exact number of slices and one key more pin the first
    and the last slice and a slice's edge."""
    first = _case(1, [4096, 700, 17, 1, 2049, 64, 65, 128], heads=12, kv_heads=2, d=128, page=16)
    got, want = _both(libraries, first, slice_keys=64)
    # The same kernels over another buffer: the tolerance of the other kernel tests
    # (2**-7 of the largest value) holds with room to spare; in fact the bits agree.
    limit = 2.0 ** -7 * max(1.0, float(want.float().abs().max()))
    assert (got.float() - want.float()).abs().max().item() <= limit
    assert torch.isfinite(got.float()).all()
    # Against plain attention (the kernels round probabilities to bfloat16: twice the budget, as
    # the other attention tests allow).
    plain = _plain(first)
    assert (got.float().cpu() - plain).abs().max().item() <= 2 * 2.0 ** -7 * max(1.0, float(plain.abs().max()))
    second = _case(2, [333, 64, 1500, 256, 1], heads=6, kv_heads=3, d=64, page=32)
    got2, want2 = _both(libraries, second, slice_keys=128, window=200)
    limit2 = 2.0 ** -7 * max(1.0, float(want2.float().abs().max()))
    assert (got2.float() - want2.float()).abs().max().item() <= limit2
    plain2 = _plain(second, window=200)
    assert (got2.float().cpu() - plain2).abs().max().item() <= 2 * 2.0 ** -7 * max(1.0, float(plain2.abs().max()))
    # And the first again, after the array has held the second's partial results.
    got3, _ = _both(libraries, first, slice_keys=64)
    assert torch.equal(got3, got)


def test_more_scratch_than_the_library_holds_is_refused(libraries):
    _, noalloc = libraries
    capacity = noalloc.pae_noalloc_scratch_capacity()
    assert capacity == 2 * 1024 * 1024
    c = _case(3, [64] * 4, heads=12, kv_heads=2, d=128, page=16)
    out = torch.full((4, 12 * 128), 7.0, dtype=torch.bfloat16, device="cuda")
    # 4 requests x 12 heads x 400 slices x 130 floats = 2,496,000 > 2,097,152
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    code = noalloc.pae_paged_attention_decode_noalloc(*_common_args(c, out, 16, 400, 0), stream)
    assert code != 0
    message = noalloc.pae_last_error().decode()
    assert "floats of scratch" in message and "2097152" in message
    torch.cuda.synchronize()
    assert (out.float() == 7.0).all(), "a refused call must not launch anything"


def test_more_slices_than_the_merge_takes_are_refused_before_anything_runs(libraries):
    """1 request x 1 head x 10,000 slices fit the library's array (1,300,000 floats), but the merge
    step keeps a weight per slice in shared memory and takes fewer: the call must be refused
    as a whole, with nothing launched and the output untouched."""
    _, noalloc = libraries
    c = _case(4, [64], heads=1, kv_heads=1, d=128, page=16)
    out = torch.full((1, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    code = noalloc.pae_paged_attention_decode_noalloc(*_common_args(c, out, 16, 10000, 0), stream)
    assert code != 0
    assert "more than the merge takes" in noalloc.pae_last_error().decode()
    torch.cuda.synchronize()
    assert (out.float() == 7.0).all(), "a refused call must not launch anything"
    # and the next ordinary call is served
    got, want = _both(libraries, c, slice_keys=16)
    assert torch.equal(got, want)
