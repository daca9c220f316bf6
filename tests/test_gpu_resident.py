"""GPU tests of resident operands: what a product prepares from X1 / X2 stays in the workspace and is kept by the next
product when the operand is the same unchanged tensor (falkon_b200/_lib.py: _tensor_key, FLK_FLAG_KEEP_X1 / _X2).
The cache must be invisible: identical results with and without it, and any in-place edit of an operand (which bumps
torch's version counter) must be seen.
"""
import numpy as np
import pytest
import torch

from oracle import falkon_oracle as fo

pytestmark = pytest.mark.gpu


def _setup(dtype, n=6000, m=900, d=28, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    X = torch.randn(n, d, generator=g, device="cuda", dtype=dtype)
    C = torch.randn(m, d, generator=g, device="cuda", dtype=dtype)
    vs = [torch.randn(m, 1, generator=g, device="cuda", dtype=dtype) for _ in range(3)]
    w = torch.randn(n, 1, generator=g, device="cuda", dtype=dtype)
    return X, C, vs, w


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64], ids=["f32", "f64"])
def test_kept_operands_give_identical_results_with_fewer_launches(dtype):
    from falkon_b200 import _lib
    from falkon_b200.kernels import GaussianKernel

    X, C, vs, w = _setup(dtype)
    k = GaussianKernel(5.0)
    fresh, fresh_launches = [], []
    for v in vs:
        _lib.forget_resident()
        before = _lib.launch_count()
        fresh.append(k.dmmv(X, C, v, w).clone())
        fresh_launches.append(_lib.launch_count() - before)
    _lib.forget_resident()
    kept_launches = []
    for i, v in enumerate(vs):
        before = _lib.launch_count()
        got = k.dmmv(X, C, v, w)
        kept_launches.append(_lib.launch_count() - before)
        assert torch.equal(got, fresh[i]), i  # bit for bit: the kept images are the images a fresh call builds
    assert kept_launches[0] == fresh_launches[0]
    assert kept_launches[1] < fresh_launches[1] and kept_launches[2] == kept_launches[1]
    # K v alone keeps its operands the same way
    _lib.forget_resident()
    a = k.mmv(X, C, vs[0]).clone()
    before = _lib.launch_count()
    b = k.mmv(X, C, vs[0])
    assert torch.equal(a, b) and _lib.launch_count() - before < fresh_launches[0]


def test_in_place_edit_of_an_operand_is_seen():
    from falkon_b200.kernels import GaussianKernel

    X, C, vs, w = _setup(torch.float32, seed=1)
    k = GaussianKernel(5.0)
    first = k.dmmv(X, C, vs[0], w).clone()
    again = k.dmmv(X, C, vs[0], w).clone()
    assert torch.equal(first, again)
    X.mul_(1.5)  # same storage, same shape: only the version counter tells
    edited = k.dmmv(X, C, vs[0], w).cpu().numpy()
    want = fo.dense_fdmmv_fp64(X.cpu().numpy(), C.cpu().numpy(), vs[0].cpu().numpy(), w.cpu().numpy(), "gaussian", 5.0)
    assert fo.rel_l2(edited, want) <= 1e-5
    assert fo.rel_l2(first.cpu().numpy(), want) > 1e-2
    C[:10] += 1.0
    edited2 = k.dmmv(X, C, vs[0], w).cpu().numpy()
    want2 = fo.dense_fdmmv_fp64(X.cpu().numpy(), C.cpu().numpy(), vs[0].cpu().numpy(), w.cpu().numpy(), "gaussian", 5.0)
    assert fo.rel_l2(edited2, want2) <= 1e-5


def test_other_sizes_kernels_and_sigmas_are_never_kept():
    from falkon_b200.kernels import GaussianKernel, LaplacianKernel

    X, C, vs, w = _setup(torch.float32, seed=2)
    Xn, Cn, vn, wn = (t.cpu().numpy() for t in (X, C, vs[0], w))
    GaussianKernel(5.0).dmmv(X, C, vs[0], w)
    got = GaussianKernel(3.0).dmmv(X, C, vs[0], w).cpu().numpy()  # other length-scale, same tensors
    assert fo.rel_l2(got, fo.dense_fdmmv_fp64(Xn, Cn, vn, wn, "gaussian", 3.0)) <= 1e-5
    got = LaplacianKernel(3.0).dmmv(X, C, vs[0], w).cpu().numpy()  # other kernel function
    assert fo.rel_l2(got, fo.dense_fdmmv_fp64(Xn, Cn, vn, wn, "laplacian", 3.0)) <= 1e-5
    got = GaussianKernel(3.0).dmmv(X[:3000], C, vs[0], w[:3000]).cpu().numpy()  # a view with the same address
    assert fo.rel_l2(got, fo.dense_fdmmv_fp64(Xn[:3000], Cn, vn, wn[:3000], "gaussian", 3.0)) <= 1e-5
    v2 = torch.cat([vs[0], vs[1]], dim=1).contiguous()
    w2 = torch.cat([w, w], dim=1).contiguous()
    got = GaussianKernel(3.0).dmmv(X, C, v2, w2).cpu().numpy()  # two vector columns: another layout
    assert fo.rel_l2(got, fo.dense_fdmmv_fp64(Xn, Cn, v2.cpu().numpy(), w2.cpu().numpy(), "gaussian", 3.0)) <= 1e-5


def test_range_flag_of_a_kept_operand_is_kept_too():
    """A row that fp16 cannot carry sends the call to the SIMT kernels; that range flag belongs to the operand and must
    survive when its images are kept."""
    from falkon_b200 import _lib
    from falkon_b200.kernels import GaussianKernel

    X, C, vs, w = _setup(torch.float32, seed=3)
    X[5] = 4000.0  # |x / sigma| = 800: beyond the fp16 images
    k = GaussianKernel(5.0)
    want = None
    for i in range(3):
        got = k.dmmv(X, C, vs[0], w)
        assert _lib.range_flag(X.device) == 1, i
        if want is None:
            want = fo.dense_fdmmv_fp64(X.cpu().numpy(), C.cpu().numpy(), vs[0].cpu().numpy(), w.cpu().numpy(),
                                       "gaussian", 5.0)
        assert fo.rel_l2(got.cpu().numpy(), want) <= 1e-5, i
    # a vector entry that is not finite opens the SIMT path for one call only
    X2, C2, vs2, w2 = _setup(torch.float32, seed=4)
    ok = k.dmmv(X2, C2, vs2[0], w2).clone()
    bad = vs2[0].clone()
    bad[3] = float("inf")
    k.mmv(X2, C2, vs2[0])
    k.mmv(X2, C2, bad)
    assert _lib.range_flag(X2.device) == 1
    k.mmv(X2, C2, vs2[0])
    assert _lib.range_flag(X2.device) == 0
    assert torch.equal(k.dmmv(X2, C2, vs2[0], w2), ok)


def test_inference_tensors_are_not_kept():
    from falkon_b200 import _lib
    from falkon_b200.kernels import GaussianKernel

    k = GaussianKernel(5.0)
    with torch.inference_mode():
        X, C, vs, w = _setup(torch.float32, seed=5)
        a = k.dmmv(X, C, vs[0], w).clone()
        before = _lib.launch_count()
        b = k.dmmv(X, C, vs[0], w)
        second = _lib.launch_count() - before
        _lib.forget_resident()
        before = _lib.launch_count()
        k.dmmv(X, C, vs[0], w)
        assert _lib.launch_count() - before == second  # nothing was kept: no version counter to trust
        assert torch.equal(a, b)
