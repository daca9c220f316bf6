"""CPU tests of the blocked split-TF32 linear algebra of the preconditioner (on the CPU the TF32 switch has no
effect, so these check the algebra: exact split, block structure, chunked accumulation, failure codes)."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from falkon_b200.preconditioner.tensor_core_la import (  # noqa: E402
    addmm_nt_3xtf32_, cholesky_lower_3xtf32, split_tf32, triu_times_transpose_3xtf32)


def test_split_is_exact_and_hi_is_tf32():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(257, 33, generator=g) * torch.logspace(-20, 20, 33)
    hi, lo = split_tf32(x)
    assert torch.equal(hi + lo, x)
    assert int((hi.view(torch.int32) & 8191).abs().max()) == 0
    assert float((lo.abs() / x.abs()).max()) < 2.0**-10
    hi2, lo2 = split_tf32(x.t())  # non-contiguous input
    assert torch.equal(hi2 + lo2, x.t())
    with pytest.raises(TypeError):
        split_tf32(x.double())


def test_addmm_chunks():
    g = torch.Generator().manual_seed(1)
    A, B = torch.randn(70, 333, generator=g), torch.randn(50, 333, generator=g)
    acc = torch.ones(70, 50)
    addmm_nt_3xtf32_(acc, *split_tf32(A), *split_tf32(B), alpha=-2.0, k_chunk=100)
    want = 1.0 - 2.0 * (A.double() @ B.double().T)
    assert float((acc.double() - want).norm() / want.norm()) < 1e-6


@pytest.mark.parametrize("m,block", [(700, 256), (512, 256), (100, 256)])
def test_triu_times_transpose(m, block):
    g = torch.Generator().manual_seed(2)
    T = torch.triu(torch.randn(m, m, generator=g))
    for view in (T, T.t().contiguous().t()):  # row-major and transposed-view input
        out = triu_times_transpose_3xtf32(view, block=block, k_chunk=96)
        want = T.double() @ T.double().T
        assert float((out.double() - want).norm() / want.norm()) < 1e-6
        assert torch.equal(out, out.T)


@pytest.mark.parametrize("m,panel,trailing", [(900, 128, 256), (300, 512, 512), (1000, 250, 300)])
def test_blocked_cholesky(m, panel, trailing):
    g = torch.Generator().manual_seed(3)
    X = torch.randn(m, 5, generator=g)
    K = torch.exp(-0.125 * torch.cdist(X, X).pow(2)) + 0.5 * torch.eye(m)
    work = K.clone()
    work[0, 1:] = float("nan")  # the strict upper triangle is never read
    L, info = cholesky_lower_3xtf32(work, panel=panel, trailing=trailing, k_chunk=64)
    assert info == 0 and L.data_ptr() == work.data_ptr()
    assert float(L.triu(1).abs().max()) == 0.0
    ref = torch.linalg.cholesky(K.double())
    assert float((L.double() - ref).norm() / ref.norm()) < 2e-5
    bad = K.clone()
    bad[m // 2, m // 2] = -1.0
    _, info = cholesky_lower_3xtf32(bad, panel=panel, trailing=trailing)
    assert info == m // 2 + 1  # order of the first leading minor that is not positive definite
    with pytest.raises(ValueError):
        cholesky_lower_3xtf32(K.double())


@pytest.mark.parametrize("m,block", [(700, 128), (512, 128), (100, 128), (1, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_blocked_triangular_solves(m, block, dtype):
    from falkon_b200.preconditioner.tri_solve import BlockedTriangular

    g = torch.Generator().manual_seed(4)
    L = torch.tril(torch.randn(m, m, generator=g, dtype=torch.float64)) + 20.0 * torch.eye(m, dtype=torch.float64)
    L = L.to(dtype).contiguous()
    bt = BlockedTriangular(L, block=block)
    tol = 1e-4 if dtype == torch.float32 else 1e-12
    for shape in ((m,), (m, 3)):
        b = torch.randn(*shape, generator=g, dtype=torch.float64).to(dtype)
        x = bt.solve(b)
        assert x.shape == b.shape
        assert float((L.double() @ x.double() - b.double()).abs().max()) < tol * 20
        x = bt.solve_t(b)
        assert float((L.double().T @ x.double() - b.double()).abs().max()) < tol * 20
    with pytest.raises(ValueError):
        bt.solve(torch.zeros(m + 1, dtype=dtype))
    with pytest.raises(ValueError):
        BlockedTriangular(L.t() if m > 1 else torch.zeros(2, 3, dtype=dtype))
