"""GPU tests of the memory budget: ``max_gpu_mem`` bounds what a product allocates on the device, as the reference's
budget contract asserts for its own products (falkon/tests/conftest.py:22-59: peak allocated memory during the call
stays below the configured limit).  Over budget, the rows of the large operand are processed in chunks; when not
even the smallest chunk fits, MemoryError (falkon/utils/helpers.py:83-84).
"""
import numpy as np
import pytest
import torch

from oracle import falkon_oracle as fo

pytestmark = pytest.mark.gpu

MIB = 2**20


def _peak_of(fn):
    from falkon_b200 import _lib

    _lib.release_workspaces()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    base = torch.cuda.memory_allocated()
    torch.cuda.reset_peak_memory_stats()
    out = fn()
    torch.cuda.synchronize()
    return out, torch.cuda.max_memory_allocated() - base


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64], ids=["f32", "f64"])
def test_products_stay_within_max_gpu_mem(dtype):
    from falkon_b200 import FalkonOptions
    from falkon_b200.kernels import GaussianKernel

    n, m, d = (1_200_000, 1500, 28) if dtype == torch.float32 else (600_000, 800, 12)
    g = torch.Generator(device="cuda").manual_seed(3)
    X = torch.randn(n, d, generator=g, device="cuda", dtype=dtype)
    C = X[:m].contiguous()
    v = torch.randn(m, 1, generator=g, device="cuda", dtype=dtype)
    w = torch.randn(n, 1, generator=g, device="cuda", dtype=dtype)
    # positive entries: a sum of 1e6 terms of random sign has a condition number of ~1e3, which would turn the
    # fp32 rounding of two different summation orders (chunked or not) into a 1e-4 difference
    y = torch.rand(n, 1, generator=g, device="cuda", dtype=dtype) + 0.1
    k = GaussianKernel(5.0)
    limit = (192 if dtype == torch.float32 else 32) * MIB
    tight = FalkonOptions(max_gpu_mem=limit)
    tol = 2e-6 if dtype == torch.float32 else 1e-12

    free_out, free_peak = _peak_of(lambda: k.dmmv(X, C, v, w))
    assert free_peak > limit  # the problem is large enough for the budget to matter
    got, peak = _peak_of(lambda: k.dmmv(X, C, v, w, opt=tight))
    assert peak <= limit, f"dmmv peak {peak / MIB:.0f} MiB over a budget of {limit / MIB:.0f} MiB"
    assert fo.rel_l2(got.cpu().numpy(), free_out.cpu().numpy()) <= tol

    want = k.mmv(X, C, v)
    got, peak = _peak_of(lambda: k.mmv(X, C, v, opt=tight))  # rows of X1 in chunks
    assert peak <= limit + want.numel() * want.element_size()
    assert fo.rel_l2(got.cpu().numpy(), want.cpu().numpy()) <= tol

    want = k.mmv(C, X, y)
    got, peak = _peak_of(lambda: k.mmv(C, X, y, opt=tight))  # reduction side in chunks, accumulated
    assert peak <= limit
    assert fo.rel_l2(got.cpu().numpy(), want.cpu().numpy()) <= tol


def test_impossible_budget_raises_memory_error():
    from falkon_b200 import FalkonOptions
    from falkon_b200.kernels import GaussianKernel

    X = torch.randn(100_000, 28, device="cuda")
    C = X[:20_000].contiguous()
    v = torch.randn(20_000, 1, device="cuda")
    with pytest.raises(MemoryError):
        GaussianKernel(5.0).dmmv(X, C, v, None, opt=FalkonOptions(max_gpu_mem=1 * MIB))


def test_accumulate_flag_through_the_c_abi():
    """FLK_FLAG_ACCUMULATE adds to what `out` holds: two half-problems summed equal the whole."""
    from falkon_b200 import _lib

    g = torch.Generator(device="cuda").manual_seed(5)
    n, m, d = 3000, 700, 9
    X = torch.randn(n, d, generator=g, device="cuda")
    C = torch.randn(m, d, generator=g, device="cuda")
    v = torch.randn(m, 2, generator=g, device="cuda")
    w = torch.randn(n, 2, generator=g, device="cuda")
    sig = np.array([2.0])
    whole = _lib.call_fdmmv(_lib.FLK_GAUSSIAN, sig, X, C, v, w, torch.empty(m, 2, device="cuda")).clone()
    out = torch.empty(m, 2, device="cuda")
    _lib.call_fdmmv(_lib.FLK_GAUSSIAN, sig, X[:1700], C, v, w[:1700], out)
    _lib.call_fdmmv(_lib.FLK_GAUSSIAN, sig, X[1700:], C, v, w[1700:], out, flags=_lib.FLAG_ACCUMULATE)
    assert fo.rel_l2(out.cpu().numpy(), whole.cpu().numpy()) <= 2e-6
    whole = _lib.call_fmmv(_lib.FLK_GAUSSIAN, sig, X, C, v, torch.empty(n, 2, device="cuda")).clone()
    out = torch.empty(n, 2, device="cuda")
    _lib.call_fmmv(_lib.FLK_GAUSSIAN, sig, X, C[:300], v[:300], out)
    _lib.call_fmmv(_lib.FLK_GAUSSIAN, sig, X, C[300:], v[300:], out, flags=_lib.FLAG_ACCUMULATE)
    assert fo.rel_l2(out.cpu().numpy(), whole.cpu().numpy()) <= 2e-6
