"""Seeded inputs of the golden cases for the rows next to the hot path: the kernel matrix (fmm), the
preconditioner and the full ``Falkon.fit`` (conjugate gradient around dmmv).  Inputs are regenerated
from numpy's PCG64 generator; the fixtures (fit_*.npz) hold only what the reference computed."""
from __future__ import annotations

import numpy as np


def fit_cases():
    return [
        # benchmark configuration 1's data (N = 20000, d = 10, M = 1000, Gaussian sigma = 3) as a regression fit
        dict(name="fit_c1_32", dtype="float32", n=20000, d=10, m=1000, t=1, kernel="gaussian", sigma=3.0, nu=None,
             penalty=1e-6, maxiter=20, seed=11, data="randn_regression", weighted=False),
        dict(name="fit_c1_64", dtype="float64", n=20000, d=10, m=1000, t=1, kernel="gaussian", sigma=3.0, nu=None,
             penalty=1e-6, maxiter=20, seed=11, data="randn_regression", weighted=False),
        # benchmark configuration 3 reduced (mixture data, +-1 labels with 5 % flips, sigma = 5, lambda = 1e-7)
        dict(name="fit_c3_small_32", dtype="float32", n=100000, d=28, m=2000, t=1, kernel="gaussian", sigma=5.0,
             nu=None, penalty=1e-7, maxiter=20, seed=13, data="mixture_labels", weighted=False),
        # multi-output Matern fit in fp64 and a re-weighted least-squares fit
        dict(name="fit_matern_multi_64", dtype="float64", n=6000, d=12, m=400, t=3, kernel="matern", sigma=4.0,
             nu=2.5, penalty=1e-5, maxiter=15, seed=17, data="randn_regression", weighted=False),
        dict(name="fit_weighted_32", dtype="float32", n=8000, d=6, m=300, t=1, kernel="gaussian", sigma=2.0, nu=None,
             penalty=1e-5, maxiter=15, seed=19, data="mixture_labels", weighted=True),
    ]


def fit_case_by_name(name):
    for c in fit_cases():
        if c["name"] == name:
            return c
    raise KeyError(name)


def build_fit_inputs(case):
    """Returns X (n, d), Y (n, t) as numpy arrays of the case's dtype."""
    dt = np.dtype(case["dtype"])
    n, d, t = case["n"], case["d"], case["t"]
    rng = np.random.default_rng(7000 + case["seed"])
    if case["data"] == "randn_regression":
        X = rng.standard_normal((n, d))
        W = rng.standard_normal((d, t)) / np.sqrt(d)
        Y = np.sin(X @ W) + 0.1 * rng.standard_normal((n, t))
    elif case["data"] == "mixture_labels":
        z = rng.integers(0, 2, size=(n, 1))
        X = rng.standard_normal((n, d)) + (2 * z - 1) * 0.5
        flip = rng.random((n, 1)) < 0.05
        Y = np.where(flip, -(2 * z - 1), 2 * z - 1).astype(np.float64)
        if t > 1:
            Y = np.repeat(Y, t, axis=1)
    else:
        raise ValueError(case["data"])
    return X.astype(dt), Y.astype(dt)


def weight_fn_numpy(Y):
    """Weights of the re-weighted case: positive class 2.0, negative class 1.0."""
    return np.where(Y[:, :1] > 0, 2.0, 1.0)
