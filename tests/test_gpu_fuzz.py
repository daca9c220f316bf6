"""Seeded random shapes through every fp32 path (resident and K-loop tensor-core kernels, 4- and 32-column
epilogues, one- and two-segment grids, chunked reductions) against the library's own fp64 kernels, which share
no code with them beyond the operand preparation.  Tolerance: rel-L2 <= 1e-4 (the fp32 bar), and the two
products of an fdmmv must agree with each other (K^T u computed by fdmmv and by fmmv on swapped operands).
"""
import numpy as np
import pytest
import torch

from oracle import falkon_oracle as fo

pytestmark = pytest.mark.gpu


def _cases():
    rng = np.random.default_rng(20240607)
    out = []
    for i in range(36):
        d = int(rng.choice([1, 2, 5, 9, 10, 19, 20, 28, 30, 31, 33, 64, 100, 200]))
        t = int(rng.choice([1, 1, 1, 2, 3, 4, 5, 8, 20, 33, 40]))
        n = int(rng.integers(1, 300_000)) if i % 3 else int(rng.integers(1, 3000))
        m = int(rng.integers(1, 6000)) if i % 4 else int(rng.integers(1, 200))
        if n * m * max(d, 8) * max(t, 4) > 4e12:  # keep the fp64 check in the seconds range
            n = max(1, int(4e12 / (m * max(d, 8) * max(t, 4))))
        kernel = ["gaussian", "laplacian", "matern15", "matern25"][i % 4]
        out.append((i, n, m, d, t, kernel))
    return out


CASES = _cases()


def _kernel(name, sigma):
    from falkon_b200.kernels import GaussianKernel, LaplacianKernel, MaternKernel

    if name == "gaussian":
        return GaussianKernel(sigma)
    if name == "laplacian":
        return LaplacianKernel(sigma)
    return MaternKernel(sigma, nu=1.5 if name == "matern15" else 2.5)


@pytest.mark.parametrize("case", CASES, ids=[f"{c[5]}_n{c[1]}_m{c[2]}_d{c[3]}_t{c[4]}" for c in CASES])
def test_random_shape_against_fp64_kernels(case):
    from falkon_b200 import _lib

    seed, n, m, d, t, name = case
    g = torch.Generator(device="cuda").manual_seed(1000 + seed)
    X = torch.randn(n, d, generator=g, device="cuda")
    C = torch.randn(m, d, generator=g, device="cuda") if seed % 2 else X[torch.randint(0, n, (m,), generator=g, device="cuda")]
    C = C.contiguous()
    v = torch.randn(m, t, generator=g, device="cuda")
    w = torch.randn(n, t, generator=g, device="cuda")
    k = _kernel(name, 1.5 * float(d) ** 0.5)
    Xd, Cd, vd, wd = X.double(), C.double(), v.double(), w.double()
    u32, u64 = k.mmv(X, C, v), k.mmv(Xd, Cd, vd)
    assert fo.rel_l2(u32.cpu().numpy(), u64.cpu().numpy()) < 1e-4
    o32, o64 = k.dmmv(X, C, v, w), k.dmmv(Xd, Cd, vd, wd)
    assert fo.rel_l2(o32.cpu().numpy(), o64.cpu().numpy()) < 1e-4
    # the second sweep of fdmmv against the single product on swapped operands
    kt = k.mmv(C, X, w)
    o_w = k.dmmv(X, C, None, w)
    assert fo.rel_l2(o_w.cpu().numpy(), kt.cpu().numpy()) < 2e-5
    assert _lib.tc_status(X.device) == 0 and _lib.range_flag(X.device) == 0
