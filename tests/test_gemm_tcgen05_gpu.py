"""The tcgen05 products against the plain reference: the many-token form and the few-token
(swapped, split-K) form, at sizes with ragged edges in every dimension."""

import pytest
import torch

import torch_ops as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from paged_attention_engine_b200.kernels import ops as kernel_ops

    kernel_ops.use_tensor_cores = True
    return kernel_ops


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
    got = ops.linear(x, w, b, r, out_dtype=out_dtype)
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


@pytest.mark.parametrize("m,n,k", [(4, 151936, 1536), (70, 3001, 520), (8, 509, 96)])
def test_float32_logits(ops, m, n, k):
    _check(ops, m, n, k, bias=False, residual=False, out_dtype=torch.float32)


def test_agrees_with_the_cuda_core_kernel(ops):
    x = _rand((40, 1536), 5)
    w = _rand((1000, 1536), 6, 0.05)
    fast = ops.linear(x, w)
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
    whole = ops.linear(x, w)
    for count in (1, 8, 24):
        part = ops.linear(x[:count].contiguous(), w)
        assert torch.equal(part, whole[:count]), f"{count} tokens"
