"""Seeded inputs of the golden cases for the backward pass of ``k(X1, X2) @ v`` and of ``k(X1, X2)``.
Inputs are regenerated from numpy's PCG64 generator; the fixtures (grad_*.npz) hold only the gradients the
reference computed."""
from __future__ import annotations

import numpy as np


def grad_cases():
    cases = []
    for dtype, tag in (("float32", "32"), ("float64", "64")):
        cases += [
            dict(name=f"grad_gauss_{tag}", dtype=dtype, n=300, m=40, d=5, t=3, kernel="gaussian", sigma=[2.0],
                 nu=None, seed=1),
            dict(name=f"grad_gauss_vec_{tag}", dtype=dtype, n=257, m=65, d=4, t=1, kernel="gaussian",
                 sigma=[1.5, 2.0, 2.5, 3.0], nu=None, seed=2),
            dict(name=f"grad_laplace_{tag}", dtype=dtype, n=200, m=30, d=6, t=2, kernel="laplacian", sigma=[3.0],
                 nu=None, seed=3),
            dict(name=f"grad_matern15_{tag}", dtype=dtype, n=150, m=33, d=7, t=2, kernel="matern", sigma=[2.5],
                 nu=1.5, seed=4),
            dict(name=f"grad_matern25_vec_{tag}", dtype=dtype, n=130, m=70, d=3, t=17, kernel="matern",
                 sigma=[2.0, 3.0, 4.0], nu=2.5, seed=5),
        ]
    # a wider problem: d above one shared-memory step, t above one step, rows not a multiple of the tile
    cases.append(dict(name="grad_gauss_wide_64", dtype="float64", n=333, m=129, d=40, t=20, kernel="gaussian",
                      sigma=[6.0], nu=None, seed=6))
    return cases


def grad_case_by_name(name):
    for c in grad_cases():
        if c["name"] == name:
            return c
    raise KeyError(name)


def build_grad_inputs(case):
    """X1 (n, d), X2 (m, d), v (m, t), G (n, t) = upstream gradient of k(X1, X2) v, S (n, m) = upstream
    gradient of k(X1, X2); numpy arrays of the case's dtype.  X2 is drawn independently of X1 (no coincident
    points, where the Laplacian's derivative is singular)."""
    dt = np.dtype(case["dtype"])
    n, m, d, t = case["n"], case["m"], case["d"], case["t"]
    rng = np.random.default_rng(9000 + case["seed"])
    X1 = rng.standard_normal((n, d))
    X2 = rng.standard_normal((m, d))
    v = rng.standard_normal((m, t))
    G = rng.standard_normal((n, t))
    S = rng.standard_normal((n, m))
    return tuple(a.astype(dt) for a in (X1, X2, v, G, S))
