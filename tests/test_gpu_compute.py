"""GPU tests of the two small entry points next to the products: the dense kernel block
(``Kernel.compute`` -> ``flk_fmm``) and the row-norm routine (``flk_square_norm``).

``compute`` is the reference's extension point (falkon/kernels/diff_kernel.py:90-91,
falkon/kernels/kernel.py:462-505); the tests have the shape of the reference's custom-kernel tests
(falkon/tests/test_custom_kernel.py:33-98: the block, then ``mmv`` / ``dmmv`` against products formed from the
block), applied to the built-in kernels.  ``flk_square_norm`` replaces ``falkon::square_norm``
(falkon/c_ext/ops/cuda/cuda_square_norm.cu:48-61).

Tolerances: block entries 1e-5 absolute in fp32 (values lie in (0, 1]), 1e-12 in fp64; products rel-L2 1e-4 /
1e-10; norms rtol 1e-6 / 1e-13 against the CPU oracle's accumulation in the data's dtype.
"""
import numpy as np
import pytest
import torch

from oracle import falkon_oracle as fo

pytestmark = pytest.mark.gpu

N, M, D, T = 300, 170, 12, 3


def _data(dtype, seed=92):
    rng = np.random.default_rng(seed)
    A = rng.random((N, D)).astype(dtype)
    B = rng.random((M, D)).astype(dtype)
    v = rng.random((M, T)).astype(dtype)
    w = rng.random((N, T)).astype(dtype)
    return A, B, v, w


def _kernels():
    from falkon_b200.kernels import GaussianKernel, LaplacianKernel, MaternKernel

    vec = torch.linspace(0.8, 2.0, D, dtype=torch.float64)
    return [
        ("gaussian", GaussianKernel(1.3), "gaussian", 1.3, None),
        ("gaussian-vec", GaussianKernel(vec), "gaussian", vec.numpy(), None),
        ("laplacian", LaplacianKernel(2.0), "laplacian", 2.0, None),
        ("matern15", MaternKernel(1.7, nu=1.5), "matern", 1.7, 1.5),
        ("matern25", MaternKernel(1.7, nu=2.5), "matern", 1.7, 2.5),
    ]


@pytest.mark.parametrize("dtype", [np.float32, np.float64], ids=["f32", "f64"])
@pytest.mark.parametrize("order", ["C", "F"])
def test_compute_writes_the_block_into_out(dtype, order):
    A, B, v, w = _data(dtype)
    tol = 1e-5 if dtype == np.float32 else 1e-12
    for name, k, oname, sigma, nu in _kernels():
        Ad, Bd = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
        if order == "F":
            out = torch.empty(M, N, dtype=Ad.dtype, device="cuda").t()
        else:
            out = torch.empty(N, M, dtype=Ad.dtype, device="cuda")
        ptr = out.data_ptr()
        res = k.compute(Ad, Bd, out, False)
        assert res.data_ptr() == ptr, name  # written in place and returned
        want = fo.dense_kernel_fp64(A, B, oname, sigma, nu)
        got = res.cpu().numpy().astype(np.float64)
        assert np.abs(got - want).max() <= tol, f"{name}: {np.abs(got - want).max():.3e}"
        # the same block from the reference's algorithm in the data's dtype
        ref = fo.kernel_block(torch.from_numpy(A), torch.from_numpy(B), oname, sigma, nu).numpy()
        assert np.abs(got - ref).max() <= 10 * tol, name


def test_compute_diag():
    A, _, _, _ = _data(np.float64)
    A2 = A + 0.01
    for name, k, oname, sigma, nu in _kernels():
        out = torch.empty(N, dtype=torch.float64, device="cuda")
        res = k.compute(torch.from_numpy(A).cuda(), torch.from_numpy(A2).cuda(), out, True)
        assert res.data_ptr() == out.data_ptr()
        want = np.diag(fo.dense_kernel_fp64(A, A2, oname, sigma, nu))
        np.testing.assert_allclose(res.cpu().numpy(), want, rtol=1e-10, atol=1e-12, err_msg=name)


@pytest.mark.parametrize("dtype", [np.float32, np.float64], ids=["f32", "f64"])
def test_products_agree_with_products_formed_from_compute(dtype):
    """mmv / dmmv (fused kernels, no block in memory) against K @ v and K^T (K v + w) with K from compute."""
    A, B, v, w = _data(dtype)
    tol = 1e-4 if dtype == np.float32 else 1e-10
    Ad, Bd, vd, wd = (torch.from_numpy(a).cuda() for a in (A, B, v, w))
    for name, k, *_ in _kernels():
        K = k.compute(Ad, Bd, torch.empty(N, M, dtype=Ad.dtype, device="cuda"), False).double()
        assert fo.rel_l2(k.mmv(Ad, Bd, vd).cpu().numpy(), (K @ vd.double()).cpu().numpy()) <= tol, name
        want = (K.T @ (K @ vd.double() + wd.double())).cpu().numpy()
        out = torch.empty(M, T, dtype=Ad.dtype, device="cuda")
        k.dmmv(Ad, Bd, vd, wd, out=out)
        assert fo.rel_l2(out.cpu().numpy(), want) <= tol, name


def test_compute_argument_errors():
    from falkon_b200.kernels import GaussianKernel

    k = GaussianKernel(1.0)
    A = torch.zeros(5, 3, device="cuda")
    B = torch.zeros(4, 3, device="cuda")
    with pytest.raises(ValueError):
        k.compute(A, B, torch.empty(5, 5, device="cuda"), False)
    with pytest.raises(TypeError):
        k.compute(A, B, torch.empty(5, 4, device="cuda", dtype=torch.float64), False)
    with pytest.raises(ValueError):
        k.compute(A, B, torch.empty(5, device="cuda"), True)  # diag needs n == m


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64], ids=["f32", "f64"])
@pytest.mark.parametrize("order", ["C", "F"])
@pytest.mark.parametrize("n,d", [(1, 1), (63, 5), (64, 64), (1000, 28), (4097, 130)])
def test_square_norm_against_oracle(dtype, order, n, d):
    from falkon_b200 import _lib

    g = torch.Generator().manual_seed(n * 1000 + d)
    X = torch.randn(n, d, generator=g, dtype=dtype)
    Xd = X.cuda()
    if order == "F":
        Xd = Xd.t().contiguous().t()
        assert Xd.stride(0) == 1 or n == 1 or d == 1
    rtol = 1e-6 if dtype == torch.float32 else 1e-13
    got = _lib.call_square_norm(Xd)
    want = fo.square_norm_rows(X).reshape(-1)
    torch.testing.assert_close(got.cpu(), want, rtol=rtol * max(1, d ** 0.5), atol=0)
    # scalar length-scale: norms of X / sigma, as the distance kernels use the routine
    got_s = _lib.call_square_norm(Xd, sigma=2.5)
    want_s = fo.square_norm_rows(X / torch.tensor(2.5, dtype=dtype)).reshape(-1)
    torch.testing.assert_close(got_s.cpu(), want_s, rtol=rtol * max(1, d ** 0.5), atol=0)


def test_square_norm_refuses_what_it_cannot_do():
    from falkon_b200 import _lib

    X = torch.randn(10, 4, device="cuda")
    with pytest.raises(NotImplementedError):
        _lib.call_square_norm(X, sigma=[1.0, 2.0, 3.0, 4.0])
    with pytest.raises(ValueError):
        _lib.call_square_norm(X, sigma=[1.0, 2.0])
    with pytest.raises(ValueError):
        _lib.call_square_norm(X, out=torch.empty(9, device="cuda"))
    assert _lib.call_square_norm(torch.empty(0, 4, device="cuda")).numel() == 0
