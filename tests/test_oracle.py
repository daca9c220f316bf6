"""Pins the CPU oracle (oracle/falkon_oracle.py) against outputs of the reference itself.

The .npz fixtures were produced by tests/golden/make_golden.py from the reference's own
Kernel.mmv / Kernel.dmmv; tolerances are those of the reference's kernel tests
(falkon/tests/test_kernels.py:74-81: fp32 1e-4, fp64 1e-8 element-wise) plus the benchmark's
relative-L2 bars (1e-4 fp32, 1e-10 fp64).
"""
import os

import numpy as np
import pytest
import torch

from cases import all_cases, build_inputs
from oracle import falkon_oracle as fo

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = all_cases()


def _t(a):
    return None if a is None else torch.from_numpy(a)


def _tols(case):
    return (1e-4, 1e-4, 5e-5) if case["dtype"] == "float32" else (1e-8, 1e-8, 1e-11)


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_matches_reference_outputs(case):
    gold = np.load(os.path.join(GOLD, case["name"] + ".npz"))
    inp = build_inputs(case)
    X, C, v, w, y = (_t(inp[k]) for k in ("X", "C", "v", "w", "y"))
    rtol, atol, l2 = _tols(case)
    kw = dict(kernel=case["kernel"], sigma=case["sigma"], nu=case["nu"])
    if "mmv" in case["ops"]:
        got = fo.fmmv(X, C, v, **kw).numpy()[gold["mmv_rows"]]
        if case["family"] == "reftest":  # element-wise bars of the reference's own tests
            np.testing.assert_allclose(got, gold["mmv"], rtol=rtol, atol=atol)
        assert fo.rel_l2(got, gold["mmv"]) <= l2
    if "dmmv" in case["ops"]:
        got = fo.fdmmv(X, C, v, w, **kw).numpy()
        assert fo.rel_l2(got, gold["dmmv"]) <= l2
    if "dmmv_now" in case["ops"]:
        got = fo.fdmmv(X, C, v, None, **kw).numpy()
        assert fo.rel_l2(got, gold["dmmv_now"]) <= l2
    if "mmv_t" in case["ops"]:
        got = fo.fmmv(C, X, y, **kw).numpy()
        assert fo.rel_l2(got, gold["mmv_t"]) <= l2


SMALL = [c for c in CASES if c["family"] == "reftest"]


@pytest.mark.parametrize("case", SMALL, ids=[c["name"] for c in SMALL])
def test_reference_outputs_match_explicit_difference_truth(case):
    """The stored reference outputs agree with the fp64 explicit-difference definition
    (the role of falkon/tests/naive_kernels.py) within the reference's own tolerances."""
    gold = np.load(os.path.join(GOLD, case["name"] + ".npz"))
    inp = build_inputs(case)
    rtol, atol, _ = _tols(case)
    if case["dtype"] == "float64":
        rtol = atol = 4e-8  # Laplacian-type kernels amplify the norm-expansion cancellation
    truth = fo.dense_fdmmv_fp64(inp["X"], inp["C"], inp["v"], inp["w"], case["kernel"], case["sigma"], case["nu"])
    np.testing.assert_allclose(gold["dmmv"], truth, rtol=rtol, atol=atol)
    truth = fo.dense_fmmv_fp64(inp["X"], inp["C"], inp["v"], case["kernel"], case["sigma"], case["nu"])
    np.testing.assert_allclose(gold["mmv"], truth[gold["mmv_rows"]], rtol=rtol, atol=atol)


def test_oracle_block_length_only_changes_rounding():
    case = [c for c in CASES if c["name"] == "rt_large_gauss_32"][0]
    inp = build_inputs(case)
    X, C, v, w = (_t(inp[k]) for k in ("X", "C", "v", "w"))
    a = fo.fdmmv(X, C, v, w, "gaussian", [3.0], max_block_elems=None).numpy()
    b = fo.fdmmv(X, C, v, w, "gaussian", [3.0], max_block_elems=250 * 40).numpy()
    assert fo.rel_l2(a, b) < 1e-5


def test_oracle_v_none_and_errors():
    rng = np.random.default_rng(0)
    X = torch.from_numpy(rng.standard_normal((50, 4)))
    C = X[:7].clone()
    w = torch.from_numpy(rng.standard_normal((50, 2)))
    got = fo.fdmmv(X, C, None, w, "gaussian", 2.0).numpy()
    truth = fo.dense_fdmmv_fp64(X.numpy(), C.numpy(), None, w.numpy(), "gaussian", 2.0)
    np.testing.assert_allclose(got, truth, rtol=1e-9, atol=1e-9)
    with pytest.raises(ValueError):
        fo.fdmmv(X, C, None, None, "gaussian", 2.0)
    with pytest.raises(ValueError):
        fo.kernel_block(X, C, "matern", 2.0, nu=3.5)
