"""Seeded random shapes through every fp32 path (resident and K-loop tensor-core kernels, 4- and 32-column
epilogues, one- and two-segment grids, chunked reductions) against the library's own fp64 kernels, which share
no code with them beyond the operand preparation.  Tolerance: rel-L2 <= 1e-4 (the fp32 bar), and the two
products of an fdmmv must agree with each other (K^T u computed by fdmmv and by fmmv on swapped operands).
"""
import os

import numpy as np
import pytest
import torch

from oracle import falkon_oracle as fo

pytestmark = pytest.mark.gpu


def _cases():
    # FLK_FUZZ_SEED / FLK_FUZZ_CASES widen the sweep for a longer soak run
    rng = np.random.default_rng(int(os.environ.get("FLK_FUZZ_SEED", "20240607")))
    out = []
    for i in range(int(os.environ.get("FLK_FUZZ_CASES", "36"))):
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


def _host_cases():
    rng = np.random.default_rng(77)
    out = []
    for i in range(8):
        n = int(rng.choice([1000, 262_144, 262_145, 300_001, 524_288, 700_000]))
        m = int(rng.integers(1, 3000))
        d = int(rng.choice([3, 9, 28, 40]))
        t = int(rng.choice([1, 2, 5]))
        out.append((i, n, m, d, t, ["gaussian", "laplacian", "matern15", "matern25"][i % 4], ["C", "F"][i % 2]))
    return out


HOST_CASES = _host_cases()


@pytest.mark.parametrize("case", HOST_CASES, ids=[f"{c[5]}_n{c[1]}_m{c[2]}_d{c[3]}_t{c[4]}_{c[6]}" for c in HOST_CASES])
def test_host_operands_match_device_operands(case):
    """Host tensors (staged, from 262,144 rows on in row chunks through the copy stream) give the result of the
    same call on device tensors, in either memory order."""
    seed, n, m, d, t, name, order = case
    g = torch.Generator().manual_seed(500 + seed)
    X = torch.randn(n, d, generator=g)
    C = torch.randn(m, d, generator=g)
    v = torch.randn(m, t, generator=g)
    w = torch.randn(n, t, generator=g)
    if order == "F":
        X, w = X.t().contiguous().t(), w.t().contiguous().t()
    k = _kernel(name, 1.5 * float(d) ** 0.5)
    k.params.flk_devices = [torch.cuda.current_device()]
    dev = [a.cuda() for a in (X, C, v, w)]
    got, want = k.dmmv(X, C, v, w), k.dmmv(*dev)
    assert got.device.type == "cpu"
    assert fo.rel_l2(got.numpy(), want.cpu().numpy()) < 1e-5
    got, want = k.mmv(X, C, v), k.mmv(*dev[:3])
    assert fo.rel_l2(got.numpy(), want.cpu().numpy()) < 1e-5
