"""GPU tests of the folded Gaussian single-column sweep: log2 |v_j| is carried in the exponent of the reduction-side
operand image and the rows are sorted by the sign of v_j (csrc/flk_fold.cuh), so the sweep's epilogue is one
exponential and a signed add per kernel value.  Checked against the fp64 explicit-difference truth (rel-L2 <= 1e-4,
the fp32 bar; in practice ~1e-6 or better) and against the same product with the fold switched off
(FLK_FLAG_NO_FOLD), for sign patterns and sizes that exercise the partition: empty sign classes, tile boundaries,
zeros, a wide dynamic range, non-finite entries (which must reach the SIMT kernels).
"""
import numpy as np
import pytest
import torch

from oracle import falkon_oracle as fo

pytestmark = pytest.mark.gpu

D = 28
SIGMA = 5.0


def _kernel(flags=0):
    from falkon_b200 import FalkonOptions
    from falkon_b200.kernels import GaussianKernel

    k = GaussianKernel(SIGMA, opt=FalkonOptions())
    k.params.flk_flags = flags
    return k


def _data(n, m, seed):
    rng = np.random.default_rng(seed)
    X = (rng.standard_normal((n, D)) + 0.5).astype(np.float32)
    C = (rng.standard_normal((m, D)) - 0.5).astype(np.float32)
    return X, C, rng


def _signs(pattern, m, rng):
    v = np.abs(rng.standard_normal((m, 1))) + 0.1
    if pattern == "positive":
        return v
    if pattern == "negative":
        return -v
    if pattern == "alternating":
        return v * np.where(np.arange(m)[:, None] % 2 == 0, 1.0, -1.0)
    if pattern == "blocks":  # long runs of one sign, changing inside tiles
        return v * np.where((np.arange(m)[:, None] // 37) % 2 == 0, 1.0, -1.0)
    if pattern == "one_negative":
        v[m // 2] *= -1.0
        return v
    if pattern == "zeros":  # a third exact zeros (both signs of zero), the rest mixed
        s = rng.standard_normal((m, 1))
        s[::3] = 0.0
        s[1::6] = -0.0
        return s
    return rng.standard_normal((m, 1))


@pytest.mark.parametrize("pattern", ["positive", "negative", "alternating", "blocks", "one_negative", "zeros", "random"])
@pytest.mark.parametrize("m", [1, 2, 127, 128, 129, 255, 256, 257, 640, 1000])
def test_mmv_sign_patterns(pattern, m):
    from falkon_b200 import _lib

    n = 300
    X, C, rng = _data(n, m, seed=m * 7 + len(pattern))
    v = _signs(pattern, m, rng).astype(np.float32)
    Xd, Cd, vd = (torch.from_numpy(a).cuda() for a in (X, C, v))
    got = _kernel().mmv(Xd, Cd, vd).cpu().numpy()
    want = fo.dense_fmmv_fp64(X, C, v, "gaussian", SIGMA)
    scale = np.abs(fo.dense_kernel_fp64(X, C, "gaussian", SIGMA) @ np.abs(v.astype(np.float64))).max()
    # (an all-zero vector leaves at most 2^-126 per null column: the absolute floor)
    assert np.abs(got - want).max() <= 2e-6 * scale + 1e-30, f"{np.abs(got - want).max():.3e} vs scale {scale:.3e}"
    plain = _kernel(_lib.FLAG_NO_FOLD).mmv(Xd, Cd, vd).cpu().numpy()
    assert np.abs(got - plain).max() <= 2e-6 * scale + 1e-30
    assert _lib.range_flag(Xd.device) == 0 and _lib.tc_status(Xd.device) == 0


@pytest.mark.parametrize("n,m", [(1, 1), (5, 3), (513, 130), (2000, 777), (4096, 1024)])
@pytest.mark.parametrize("variant", ["vw", "v_only", "w_only"])
def test_dmmv_both_sweeps_folded(n, m, variant):
    X, C, rng = _data(n, m, seed=n + m)
    v = rng.standard_normal((m, 1)).astype(np.float32) if variant != "w_only" else None
    w = rng.standard_normal((n, 1)).astype(np.float32) if variant != "v_only" else None
    dev = lambda a: None if a is None else torch.from_numpy(a).cuda()
    got = _kernel().dmmv(dev(X), dev(C), dev(v), dev(w)).cpu().numpy()
    want = fo.dense_fdmmv_fp64(X, C, v, w, "gaussian", SIGMA)
    assert fo.rel_l2(got, want) <= 1e-5, fo.rel_l2(got, want)


def test_wide_dynamic_range_of_the_vector():
    """Entries from 1e-25 to 1e12: magnitudes are stored relative to the largest one; tiny entries may be flushed,
    which the tolerance (relative to the largest term) allows."""
    n, m = 400, 900
    X, C, rng = _data(n, m, seed=3)
    v = (rng.standard_normal((m, 1)) * 10.0 ** rng.uniform(-25, 12, size=(m, 1))).astype(np.float32)
    Xd, Cd, vd = (torch.from_numpy(a).cuda() for a in (X, C, v))
    got = _kernel().mmv(Xd, Cd, vd).cpu().numpy().astype(np.float64)
    want = fo.dense_fmmv_fp64(X, C, v, "gaussian", SIGMA)
    assert fo.rel_l2(got, want) <= 1e-5
    # all entries tiny: the scale is taken from the largest entry, so nothing is lost
    v2 = (rng.standard_normal((m, 1)) * 1e-30).astype(np.float32)
    got2 = _kernel().mmv(Xd, Cd, torch.from_numpy(v2).cuda()).cpu().numpy().astype(np.float64)
    assert fo.rel_l2(got2, fo.dense_fmmv_fp64(X, C, v2, "gaussian", SIGMA)) <= 1e-5


def test_zero_vector_gives_zero():
    n, m = 300, 500
    X, C, _ = _data(n, m, seed=4)
    Xd, Cd = torch.from_numpy(X).cuda(), torch.from_numpy(C).cuda()
    out = _kernel().mmv(Xd, Cd, torch.zeros(m, 1, device="cuda"))
    assert float(out.abs().max()) <= 1e-30  # null rows contribute 2^-200 (flushed) or at most 2^-126 each
    out2 = _kernel().dmmv(Xd, Cd, torch.zeros(m, 1, device="cuda"), None)
    assert float(out2.abs().max()) <= 1e-25


@pytest.mark.parametrize("bad", [float("inf"), float("-inf"), float("nan")])
def test_non_finite_entries_take_the_simt_path(bad):
    from falkon_b200 import _lib

    n, m = 200, 300
    X, C, rng = _data(n, m, seed=5)
    v = rng.standard_normal((m, 1)).astype(np.float32)
    v[17] = bad
    Xd, Cd, vd = (torch.from_numpy(a).cuda() for a in (X, C, v))
    got = _kernel().mmv(Xd, Cd, vd)
    assert _lib.range_flag(Xd.device) == 1  # the image builder handed over to the SIMT kernels
    K = torch.from_numpy(fo.dense_kernel_fp64(X, C, "gaussian", SIGMA)).float()
    want = K @ torch.from_numpy(v)
    assert torch.equal(torch.isnan(got.cpu()), torch.isnan(want))
    assert torch.equal(torch.isinf(got.cpu()), torch.isinf(want))


def test_fortran_order_and_vector_sigma():
    from falkon_b200 import FalkonOptions
    from falkon_b200.kernels import GaussianKernel

    n, m = 700, 333
    X, C, rng = _data(n, m, seed=6)
    sig = np.linspace(3.0, 7.0, D)
    v = rng.standard_normal((m, 1)).astype(np.float32)
    w = rng.standard_normal((n, 1)).astype(np.float32)
    k = GaussianKernel(torch.from_numpy(sig), opt=FalkonOptions())
    Xf = torch.from_numpy(X).cuda().t().contiguous().t()
    Cf = torch.from_numpy(C).cuda().t().contiguous().t()
    got = k.dmmv(Xf, Cf, torch.from_numpy(v).cuda(), torch.from_numpy(w).cuda()).cpu().numpy()
    assert fo.rel_l2(got, fo.dense_fdmmv_fp64(X, C, v, w, "gaussian", sig)) <= 1e-5


def test_bitwise_repeatable():
    n, m = 3000, 2000
    X, C, rng = _data(n, m, seed=8)
    v = rng.standard_normal((m, 1)).astype(np.float32)
    w = rng.standard_normal((n, 1)).astype(np.float32)
    args = [torch.from_numpy(a).cuda() for a in (X, C, v, w)]
    a = _kernel().dmmv(*args).clone()
    b = _kernel().dmmv(*args)
    assert torch.equal(a, b)


@pytest.mark.parametrize("share_negative", [0.5, 0.2])
def test_strongly_cancelling_sums_keep_their_accuracy(share_negative):
    """A flat kernel matrix (all distances alike) times a vector of random signs: every output is the small
    difference of two large one-signed sums (500 to 800 times larger here).  The folded sweep stores the rows sorted
    by sign; a chunk that summed all positive tiles before the negative ones let its fp32 running sums grow to the
    size of the one-sided sum and lost up to 1e-4 of relative accuracy at 2e5 rows (growing with the square root of
    the row count).  Each chunk now takes an equal share of both sign ranges and walks them interleaved.

    What is asserted: the error is below 2e-7 of sum_j k_ij |v_j| (measured: 1e-9 and 3e-8), and when both signs
    have the same magnitudes also below 1e-5 of the result itself (measured 6e-7, the level of the unfolded sweep).
    With sign-correlated magnitudes (second case: negative entries four times larger) the folded sweep keeps a small
    differential bias between the two one-signed sums -- |v_j| sits in the exponent, so terms of different magnitude
    pass through different roundings of the fp32 accumulator of the exponent GEMM, which the unfolded sweep applies
    to all terms alike (2.5e-5 of the result at an 800-fold cancellation, against 9e-7); FLK_FLAG_NO_FOLD is the
    switch for data that cancels harder than the fp32 bar of 1e-4 allows."""
    from falkon_b200 import _lib
    from falkon_b200.kernels import GaussianKernel

    d, r, s = 20, 512, 200_000
    g = torch.Generator(device="cuda").manual_seed(17)
    X1 = torch.randn(r, d, generator=g, device="cuda")
    X2 = torch.randn(s, d, generator=g, device="cuda")
    v = torch.rand(s, 1, generator=g, device="cuda") + 0.5
    v = torch.where(torch.rand(s, 1, generator=g, device="cuda") < share_negative, -v, v)
    if share_negative != 0.5:  # keep the cancellation: both one-signed sums equally large
        v = torch.where(v < 0, v * (1.0 - share_negative) / share_negative, v)
    k = GaussianKernel(float(d) ** 0.5)
    want = k.mmv(X1.double(), X2.double(), v.double()).cpu().numpy()
    one_sided = k.mmv(X1.double(), X2.double(), v.double().abs()).cpu().numpy()
    got = k.mmv(X1, X2, v).cpu().numpy()
    k.params.flk_flags = _lib.FLAG_NO_FOLD
    unfolded = k.mmv(X1, X2, v).cpu().numpy()
    err, err_unfolded = fo.rel_l2(got, want), fo.rel_l2(unfolded, want)
    forward = float(np.linalg.norm(got - want) / np.linalg.norm(one_sided))
    print(f"share of negative entries {share_negative}: folded {err:.2e} ({forward:.2e} of the one-sided sums), "
          f"unfolded {err_unfolded:.2e}; cancellation {np.linalg.norm(one_sided) / np.linalg.norm(want):.0f}x")
    assert forward < 2e-7
    assert err < 1e-4
    if share_negative == 0.5:
        assert err < 1e-5
