"""CPU tests of the backward-pass oracle and of the host-side gradient algebra.

1. The oracle (oracle/falkon_grad_oracle.py) against gradients the reference itself computed
   (tests/golden/grad_*.npz, written by tests/golden/make_golden_grad.py).
2. ``falkon_b200.mmv_ops.grad.kernel_backward`` -- the products that turn the pair weights of ``flk_kgrad``
   into gradients -- with the two library calls replaced by their CPU restatements.
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

CASES = grad_cases()
KIDS = {"gaussian": 0, "laplacian": 1}


def _tol(case):
    return 2e-5 if case["dtype"] == "float32" else 1e-11


def _golden(case):
    return np.load(os.path.join(ROOT, "tests", "golden", case["name"] + ".npz"))


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_grad_oracle_matches_reference(case):
    X1, X2, v, G, S = build_grad_inputs(case)
    ref = _golden(case)
    got = go.mmv_grads(X1, X2, v, G, case["kernel"], case["sigma"], case["nu"])
    for name, g in zip(("mmv_dX1", "mmv_dX2", "mmv_dv", "mmv_dsigma"), got):
        assert g.shape == ref[name].shape
        assert fo.rel_l2(g, ref[name]) < _tol(case), name
    got = go.mm_grads(X1, X2, S, case["kernel"], case["sigma"], case["nu"])
    for name, g in zip(("mm_dX1", "mm_dX2", "mm_dsigma"), got):
        assert fo.rel_l2(g, ref[name]) < _tol(case), name


def _kernel_of(kid):
    return {0: ("gaussian", None), 1: ("laplacian", None), 2: ("matern", 1.5), 3: ("matern", 2.5)}[kid]


def _kid(case):
    if case["kernel"] == "matern":
        return {0.5: 1, 1.5: 2, 2.5: 3, float("inf"): 0}[case["nu"]]
    return KIDS[case["kernel"]]


@pytest.fixture
def fake_library(monkeypatch):
    """Replaces the two C-ABI calls of kernel_backward with CPU restatements, so that its torch algebra
    (row blocks, the products with W, the sigma reduction) is testable without a GPU."""
    from falkon_b200 import _lib

    def call_kgrad(kernel_id, sigma, X1, X2, G, v, out, flags=0):
        name, nu = _kernel_of(kernel_id)
        out.copy_(go.pair_weights(X1, X2, G, v, name, sigma, nu))
        return out

    def call_fdmmv(kernel_id, sigma, X1, X2, v, w, out, flags=0, host=False, device=None):
        name, nu = _kernel_of(kernel_id)
        assert v is None
        out.copy_(fo.kernel_block(X1, X2, name, torch.as_tensor(sigma), nu).t() @ w)
        return out

    monkeypatch.setattr(_lib, "call_kgrad", call_kgrad)
    monkeypatch.setattr(_lib, "call_fdmmv", call_fdmmv)


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_kernel_backward_algebra(case, fake_library, monkeypatch):
    from falkon_b200.mmv_ops import grad as grad_mod

    # several row blocks, the last one ragged
    monkeypatch.setattr(grad_mod, "_W_BLOCK_BYTES", 64 * case["m"] * np.dtype(case["dtype"]).itemsize)
    X1, X2, v, G, S = (torch.from_numpy(a) for a in build_grad_inputs(case))
    ref = _golden(case)
    sigma = torch.tensor(case["sigma"], dtype=torch.float64)
    tol = 5 * _tol(case)
    g = grad_mod.kernel_backward(_kid(case), sigma, X1, X2, G, v, [True, True, True, True])
    for name, got in zip(("mmv_dX1", "mmv_dX2", "mmv_dv", "mmv_dsigma"), g):
        assert got.dtype == (torch.float64 if name == "mmv_dsigma" else X1.dtype)
        assert tuple(got.shape) == ref[name].shape
        assert fo.rel_l2(got.numpy(), ref[name]) < tol, name
    g = grad_mod.kernel_backward(_kid(case), sigma, X1, X2, S, None, [True, True, False, True])
    assert g[2] is None
    for name, got in zip(("mm_dX1", "mm_dX2", None, "mm_dsigma"), g):
        if name is not None:
            assert fo.rel_l2(got.numpy(), ref[name]) < tol, name
    # only what is asked for is computed
    g = grad_mod.kernel_backward(_kid(case), sigma, X1, X2, G, v, [False, False, True, False])
    assert g[0] is None and g[1] is None and g[3] is None and g[2] is not None
    g = grad_mod.kernel_backward(_kid(case), sigma, X1, X2, G, v, [True, False, False, False])
    assert g[0] is not None and g[1] is None and g[2] is None and g[3] is None
