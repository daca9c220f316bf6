"""GPU parity of the backward pass: ``Kernel.mmv`` / ``Kernel.__call__`` under autograd against the
gradients the reference itself computed (tests/golden/grad_*.npz), against the CPU oracle, and -- at a size
with several row blocks -- against an fp64 autograd evaluation of the dense formula.

Tolerances (rel-L2): 1e-4 in fp32, 1e-9 in fp64.
"""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

from grad_cases import build_grad_inputs, grad_cases  # noqa: E402

from oracle import falkon_grad_oracle as go  # noqa: E402
from oracle import falkon_oracle as fo  # noqa: E402

pytestmark = pytest.mark.gpu
CASES = grad_cases()


def _tol(case):
    return 1e-4 if case["dtype"] == "float32" else 1e-9


def _make_kernel(case, requires_grad=True):
    from falkon_b200.kernels import GaussianKernel, LaplacianKernel, MaternKernel

    sigma = torch.tensor(case["sigma"], dtype=torch.float64)
    if requires_grad:
        sigma.requires_grad_()
    if case["kernel"] == "gaussian":
        return GaussianKernel(sigma)
    if case["kernel"] == "laplacian":
        return LaplacianKernel(sigma)
    return MaternKernel(sigma, nu=case["nu"])


def _golden(case):
    return np.load(os.path.join(ROOT, "tests", "golden", case["name"] + ".npz"))


@pytest.mark.parametrize("where", ["cuda", "cpu"])
@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_mmv_backward_matches_reference(case, where):
    X1n, X2n, vn, Gn, _ = build_grad_inputs(case)
    ref = _golden(case)
    X1, X2, v = (torch.from_numpy(a).to(where).requires_grad_() for a in (X1n, X2n, vn))
    k = _make_kernel(case)
    out = k.mmv(X1, X2, v)
    assert out.requires_grad and out.device.type == where
    assert fo.rel_l2(out.detach().cpu().numpy(), ref["mmv_out"]) < _tol(case)
    out.backward(torch.from_numpy(Gn).to(where))
    for name, t in (("mmv_dX1", X1), ("mmv_dX2", X2), ("mmv_dv", v), ("mmv_dsigma", k.sigma)):
        assert t.grad is not None and t.grad.device == t.device and t.grad.dtype == t.dtype, name
        assert tuple(t.grad.shape) == ref[name].shape, name
        assert fo.rel_l2(t.grad.cpu().numpy(), ref[name]) < _tol(case), name


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_kernel_matrix_backward_matches_reference(case):
    X1n, X2n, _, _, Sn = build_grad_inputs(case)
    ref = _golden(case)
    X1, X2 = (torch.from_numpy(a).cuda().requires_grad_() for a in (X1n, X2n))
    k = _make_kernel(case)
    K = k(X1, X2)
    assert K.requires_grad
    K.backward(torch.from_numpy(Sn).cuda())
    for name, t in (("mm_dX1", X1), ("mm_dX2", X2), ("mm_dsigma", k.sigma)):
        assert fo.rel_l2(t.grad.cpu().numpy(), ref[name]) < _tol(case), name


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_kgrad_abi_matches_oracle(case):
    """flk_kgrad itself, through the C ABI, against the closed-form pair weights of the oracle; both forms of
    the upstream gradient, C- and F-ordered outputs."""
    from falkon_b200 import _lib

    X1n, X2n, vn, Gn, Sn = build_grad_inputs(case)
    kid = {"gaussian": 0, "laplacian": 1}.get(case["kernel"], {1.5: 2, 2.5: 3}.get(case["nu"]))
    sigma = np.asarray(case["sigma"], dtype=np.float64)
    X1, X2, v, G, S = (torch.from_numpy(a).cuda() for a in (X1n, X2n, vn, Gn, Sn))
    n, m = X1.shape[0], X2.shape[0]
    want = go.pair_weights(X1n, X2n, Gn, vn, case["kernel"], sigma, case["nu"]).numpy()
    out = torch.empty((n, m), dtype=X1.dtype, device="cuda")
    _lib.call_kgrad(kid, sigma, X1, X2, G, v, out)
    assert fo.rel_l2(out.cpu().numpy(), want) < _tol(case)
    out_f = torch.empty((m, n), dtype=X1.dtype, device="cuda").t()
    _lib.call_kgrad(kid, sigma, X1, X2, G.t().contiguous().t(), v, out_f)
    assert fo.rel_l2(out_f.cpu().numpy(), want) < _tol(case)
    want = go.pair_weights(X1n, X2n, Sn, None, case["kernel"], sigma, case["nu"]).numpy()
    _lib.call_kgrad(kid, sigma, X1, X2, S, None, out)
    assert fo.rel_l2(out.cpu().numpy(), want) < _tol(case)


def _dense_autograd_fp64(X1, X2, v, G, kernel, sigma, nu):
    x1, x2, vv = (t.detach().double().requires_grad_() for t in (X1, X2, v))
    sig = sigma.detach().double().to(X1.device).requires_grad_()
    d2 = torch.cdist(x1 / sig, x2 / sig).pow(2).clamp_min(1e-20)
    r = d2.sqrt()
    if kernel == "gaussian":
        K = torch.exp(-0.5 * d2)
    elif kernel == "laplacian":
        K = torch.exp(-r)
    elif nu == 1.5:
        K = (1 + 3**0.5 * r) * torch.exp(-(3**0.5) * r)
    else:
        K = (1 + 5**0.5 * r + 5.0 / 3.0 * d2) * torch.exp(-(5**0.5) * r)
    return torch.autograd.grad(K @ vv, [x1, x2, vv, sig], grad_outputs=G.double())


@pytest.mark.parametrize("kernel,nu", [("gaussian", None), ("matern", 2.5), ("laplacian", None)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64], ids=["f32", "f64"])
def test_mmv_backward_many_row_blocks(kernel, nu, dtype):
    """n x m weights far above one L2-sized block (several launches of flk_kgrad, ragged last block)."""
    from falkon_b200.kernels import GaussianKernel, LaplacianKernel, MaternKernel

    n, m, d, t = 40_037, 3_001, 28, 4
    g = torch.Generator(device="cuda").manual_seed(77)
    X1 = torch.randn(n, d, generator=g, device="cuda", dtype=dtype).requires_grad_()
    X2 = torch.randn(m, d, generator=g, device="cuda", dtype=dtype).requires_grad_()
    v = torch.randn(m, t, generator=g, device="cuda", dtype=dtype).requires_grad_()
    G = torch.randn(n, t, generator=g, device="cuda", dtype=dtype)
    sigma = torch.tensor([6.0], dtype=torch.float64, requires_grad=True)
    k = {"gaussian": lambda: GaussianKernel(sigma), "laplacian": lambda: LaplacianKernel(sigma),
         "matern": lambda: MaternKernel(sigma, nu=nu)}[kernel]()
    k.mmv(X1, X2, v).backward(G)
    want = _dense_autograd_fp64(X1, X2, v, G, kernel, sigma, nu)
    tol = 1e-4 if dtype == torch.float32 else 1e-9
    for name, got, ref in zip(("dX1", "dX2", "dv", "dsigma"), (X1.grad, X2.grad, v.grad, k.sigma.grad), want):
        err = fo.rel_l2(got.double().cpu().numpy(), ref.cpu().numpy())
        assert err < tol, (name, err)


def test_backward_contract():
    from falkon_b200.kernels import GaussianKernel

    g = torch.Generator().manual_seed(5)
    X1 = torch.randn(100, 3, generator=g).cuda()
    X2 = torch.randn(20, 3, generator=g).cuda()
    v = torch.randn(20, 2, generator=g).cuda().requires_grad_()
    k = GaussianKernel(2.0)
    # only v requires a gradient: nothing else gets one, sigma included
    out = k.mmv(X1, X2, v)
    out.sum().backward()
    assert v.grad is not None and k.sigma.grad is None
    want = k.mmv(X2, X1, torch.ones(100, 2, device="cuda"))  # K^T 1
    assert fo.rel_l2(v.grad.cpu().numpy(), want.cpu().numpy()) < 1e-5
    # a caller-provided output is written in place and carries the graph
    buf = torch.empty(100, 2, device="cuda")
    v.grad = None
    out = k.mmv(X1, X2, v, out=buf)
    assert out.data_ptr() == buf.data_ptr() and out.requires_grad
    out.sum().backward()
    assert fo.rel_l2(v.grad.cpu().numpy(), want.cpu().numpy()) < 1e-5
    # no graph without gradients enabled
    with torch.no_grad():
        assert not k.mmv(X1, X2, v).requires_grad
    # the double product stays non-differentiable, as in the reference (fmmv.py:1028-1031)
    with pytest.raises(NotImplementedError):
        k.dmmv(X1, X2, v, None)
    # second-order use is not claimed
    X1g = X1.clone().requires_grad_()
    out = k.mmv(X1g, X2, v.detach())
    (gx,) = torch.autograd.grad(out.sum(), X1g, create_graph=True)
    assert not gx.requires_grad
    # differentiable diagonal
    Xa = torch.randn(50, 3, generator=g).cuda().requires_grad_()
    Xb = torch.randn(50, 3, generator=g).cuda()
    dg = k(Xa, Xb, diag=True)
    dg.sum().backward()
    want = torch.exp(-0.5 * ((Xa.detach() - Xb) / 2.0).pow(2).sum(1))
    assert fo.rel_l2(dg.detach().cpu().numpy(), want.cpu().numpy()) < 1e-6 and Xa.grad is not None
