"""Seeded inputs for the golden parity cases.

Each case is described by a small dict; `build_inputs(case)` regenerates its inputs from
numpy's PCG64 generator, so only the reference's *outputs* are stored in the .npz fixtures.
The first group reproduces the shapes, seeds and Uniform[0,1) distribution of the
reference's own kernel tests (falkon/tests/test_kernels.py:32-71, :529-545;
falkon/tests/gen_random.py:17-22).  The second group are the benchmark configurations at
sizes the CPU reference finishes in seconds.
"""
from __future__ import annotations

import numpy as np

INF = float("inf")


def _uniform(seed, a, b, dtype):
    return np.random.default_rng(seed).random(size=(a, b), dtype=np.float32).astype(dtype)


def _ref_test_case(name, kernel, sigma, nu, dtype, n=20, m=5, d=3, t=2):
    return dict(name=name, family="reftest", kernel=kernel, sigma=sigma, nu=nu, dtype=dtype,
                n=n, m=m, d=d, t=t, ops=("mmv", "dmmv", "dmmv_now"))


def all_cases():
    cases = []
    for dt in ("float32", "float64"):
        s = dt[-2:]
        cases += [
            _ref_test_case(f"rt_gauss_single_{s}", "gaussian", [3.0], None, dt),
            _ref_test_case(f"rt_gauss_vec_{s}", "gaussian", [3.0, 3.0, 3.0], None, dt),
            _ref_test_case(f"rt_gauss_vec2_{s}", "gaussian", [1.0, 2.5, 0.7], None, dt),
            _ref_test_case(f"rt_laplace_{s}", "laplacian", [3.0], None, dt),
            _ref_test_case(f"rt_laplace_vec_{s}", "laplacian", [2.0, 1.0, 3.0], None, dt),
            _ref_test_case(f"rt_matern05_{s}", "matern", [3.0], 0.5, dt),
            _ref_test_case(f"rt_matern15_{s}", "matern", [3.0], 1.5, dt),
            _ref_test_case(f"rt_matern25_{s}", "matern", [3.0], 2.5, dt),
            _ref_test_case(f"rt_matern25_vec_{s}", "matern", [2.0, 1.0, 3.0], 2.5, dt),
            _ref_test_case(f"rt_materninf_{s}", "matern", [3.0], INF, dt),
        ]
    # multi-block case of the reference (n=1500, m=250, d=3, t=2, fp32, sigma=3)
    cases.append(_ref_test_case("rt_large_gauss_32", "gaussian", [3.0], None, "float32", n=1500, m=250))
    # benchmark configurations (c1 full size; c2, c4, c5 reduced)
    cases += [
        dict(name="c1_full", family="config", cfg=1, kernel="gaussian", sigma=[3.0], nu=None, dtype="float32",
             n=20000, m=1000, d=10, t=1, dist="randn", w="zeros", ops=("mmv", "dmmv", "mmv_t")),
        dict(name="c2_small", family="config", cfg=2, kernel="gaussian", sigma=[5.0], nu=None, dtype="float32",
             n=20000, m=2000, d=28, t=1, dist="mixture", w="randn", ops=("mmv", "dmmv", "mmv_t")),
        dict(name="c4_small_32", family="config", cfg=4, kernel="gaussian", sigma=[1.0], nu=None, dtype="float32",
             n=20000, m=2000, d=9, t=1, dist="uniform", w="zeros", ops=("dmmv",)),
        dict(name="c4_small_64", family="config", cfg=4, kernel="gaussian", sigma=[1.0], nu=None, dtype="float64",
             n=20000, m=2000, d=9, t=1, dist="uniform", w="zeros", ops=("dmmv",)),
        dict(name="c5_small", family="config", cfg=5, kernel="matern", sigma=[10.0], nu=2.5, dtype="float64",
             n=4000, m=600, d=128, t=32, dist="randn", w="randn", ops=("mmv", "dmmv")),
        dict(name="c5_small_32", family="config", cfg=5, kernel="matern", sigma=[10.0], nu=2.5, dtype="float32",
             n=4000, m=600, d=128, t=32, dist="randn", w="randn", ops=("dmmv",)),
        dict(name="lap_mid_32", family="config", cfg=6, kernel="laplacian", sigma=[4.0], nu=None, dtype="float32",
             n=6000, m=700, d=17, t=3, dist="randn", w="randn", ops=("mmv", "dmmv")),
        dict(name="mat15_mid_32", family="config", cfg=7, kernel="matern", sigma=[4.0], nu=1.5, dtype="float32",
             n=6000, m=700, d=5, t=2, dist="randn", w="randn", ops=("mmv", "dmmv")),
    ]
    return cases


def case_by_name(name):
    for c in all_cases():
        if c["name"] == name:
            return c
    raise KeyError(name)


def build_inputs(case):
    """Returns dict of numpy arrays: X (n,d), C (m,d), v (m,t), w (n,t) or None, y (n,t)."""
    dt = np.dtype(case["dtype"])
    n, m, d, t = case["n"], case["m"], case["d"], case["t"]
    if case["family"] == "reftest":
        X = _uniform(92, n, d, dt)
        C = _uniform(93, m, d, dt)
        v = _uniform(94, m, t, dt)
        w = _uniform(95, n, t, dt)
        return dict(X=X, C=C, v=v, w=w, y=w)
    cfg = case["cfg"]
    rx = np.random.default_rng(1000 + cfg)
    if case["dist"] == "randn":
        X = rx.standard_normal((n, d))
    elif case["dist"] == "uniform":
        X = rx.random((n, d))
    elif case["dist"] == "mixture":
        z = rx.integers(0, 2, size=(n, 1))
        X = rx.standard_normal((n, d)) + (2 * z - 1) * 0.5
    else:
        raise ValueError(case["dist"])
    X = X.astype(dt)
    idx = np.random.default_rng(2000 + cfg).choice(n, size=m, replace=False)
    C = np.ascontiguousarray(X[idx])
    v = np.random.default_rng(3000 + cfg).standard_normal((m, t)).astype(dt)
    wr = np.random.default_rng(4000 + cfg).standard_normal((n, t)).astype(dt)
    w = None if case["w"] == "zeros" else wr
    return dict(X=X, C=C, v=v, w=w, y=wr)
