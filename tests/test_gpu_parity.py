"""GPU parity tests: the CUDA path (through the C ABI) against the reference-generated golden
outputs, the CPU oracle and the fp64 explicit-difference truth.

Tolerances: relative L2 <= 1e-4 (fp32) and <= 1e-10 (fp64), the benchmark's parity bars; on the
reference's own test shapes additionally the element-wise bars of falkon/tests/test_kernels.py:74-81
(fp32 rtol = atol = 1e-4; fp64 1e-8, Laplacian-type 4e-8).
"""
import os

import numpy as np
import pytest
import torch

from cases import all_cases, build_inputs, case_by_name
from oracle import falkon_oracle as fo

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = all_cases()
L2_TOL = {"float32": 1e-4, "float64": 1e-10}


def make_kernel(case, **opt_kw):
    from falkon_b200 import FalkonOptions
    from falkon_b200.kernels import GaussianKernel, LaplacianKernel, MaternKernel

    opt = FalkonOptions(**opt_kw)
    sigma = torch.tensor(case["sigma"], dtype=torch.float64)
    if case["kernel"] == "gaussian":
        return GaussianKernel(sigma, opt=opt)
    if case["kernel"] == "laplacian":
        return LaplacianKernel(sigma, opt=opt)
    return MaternKernel(sigma, nu=float(case["nu"]), opt=opt)


def dev(a):
    return None if a is None else torch.from_numpy(a).cuda()


class _Flags:
    """FalkonOptions carries no backend switch; tests select the SIMT / tensor-core kernel through
    the `flk_flags` attribute that falkon_b200.mmv_ops reads from the option object."""


def with_flags(kernel, flags):
    kernel.params.flk_flags = flags
    return kernel


@pytest.mark.parametrize("flags", [0, 1], ids=["auto", "simt"])
@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_against_reference_golden(case, flags):
    gold = np.load(os.path.join(GOLD, case["name"] + ".npz"))
    inp = build_inputs(case)
    X, C, v, w, y = (dev(inp[k]) for k in ("X", "C", "v", "w", "y"))
    k = with_flags(make_kernel(case), flags)
    tol = L2_TOL[case["dtype"]]
    elementwise = case["family"] == "reftest"
    if case["dtype"] == "float32":
        rtol = atol = 1e-4
    else:
        rtol = atol = 4e-8 if case["kernel"] != "gaussian" else 1e-8

    def check(got, want, what):
        got = got.cpu().numpy()
        assert np.isfinite(got).all(), what
        err = fo.rel_l2(got, want)
        assert err <= tol, f"{what}: rel-L2 {err:.3e} > {tol}"
        if elementwise:
            np.testing.assert_allclose(got, want, rtol=rtol, atol=atol, err_msg=what)

    if "mmv" in case["ops"]:
        check(k.mmv(X, C, v)[torch.from_numpy(gold["mmv_rows"]).cuda()], gold["mmv"], "mmv")
    if "dmmv" in case["ops"]:
        check(k.dmmv(X, C, v, w), gold["dmmv"], "dmmv")
    if "dmmv_now" in case["ops"]:
        check(k.dmmv(X, C, v, None), gold["dmmv_now"], "dmmv (w=None)")
    if "mmv_t" in case["ops"]:
        check(k.mmv(C, X, y), gold["mmv_t"], "mmv transposed (reduction over data rows)")


@pytest.mark.parametrize("flags", [0, 1], ids=["auto", "simt"])
@pytest.mark.parametrize("name", ["rt_gauss_vec2_32", "rt_matern25_vec_64", "rt_large_gauss_32"])
@pytest.mark.parametrize("order", ["C", "F"])
def test_memory_orders_out_reuse_and_host_inputs(name, order, flags):
    """Both memory orders are legal, `out` must be reused, and CPU tensors run through the host
    entry points (falkon/tests/test_kernels.py:152, :188, :222)."""
    case = case_by_name(name)
    gold = np.load(os.path.join(GOLD, name + ".npz"))
    inp = build_inputs(case)
    k = with_flags(make_kernel(case), flags)
    tol = L2_TOL[case["dtype"]]

    def conv(a, cuda):
        t = torch.from_numpy(np.asfortranarray(a) if order == "F" else np.ascontiguousarray(a))
        if order == "F":
            assert t.stride(0) == 1
        return t.cuda() if cuda else t

    for cuda in (True, False):
        X, C, v, w = (conv(inp[k_], cuda) for k_ in ("X", "C", "v", "w"))
        out = torch.empty(C.shape[0], v.shape[1], dtype=X.dtype, device=X.device)
        res = k.dmmv(X, C, v, w, out=out)
        assert res.data_ptr() == out.data_ptr()
        assert fo.rel_l2(res.cpu().numpy(), gold["dmmv"]) <= tol
        res2 = k.dmmv(X, C, v, w)
        assert res2.device == X.device
        if order == "F":
            assert res2.stride(0) == 1  # output follows X1's memory order
        assert fo.rel_l2(res2.cpu().numpy(), gold["dmmv"]) <= tol
        out = torch.empty(X.shape[0], v.shape[1], dtype=X.dtype, device=X.device)
        res = k.mmv(X, C, v, out=out)
        assert res.data_ptr() == out.data_ptr()
        assert fo.rel_l2(res.cpu().numpy()[gold["mmv_rows"]], gold["mmv"]) <= tol


SHAPES = [
    # n, m, d, t
    (1, 1, 1, 1),
    (5, 3, 2, 1),
    (127, 129, 7, 1),
    (129, 127, 28, 2),
    (257, 255, 30, 3),
    (300, 70, 31, 5),
    (513, 300, 9, 4),
    (1000, 17, 3, 33),
    (300, 700, 12, 70),   # fp32: resident tensor-core kernel with 32 vector columns per pass
    (400, 300, 100, 40),  # fp32: K-loop tensor-core kernel with 32 vector columns per pass
    (70, 1000, 64, 1),
    (260, 130, 130, 2),
]


@pytest.mark.parametrize("dtype", ["float32", "float64"])
@pytest.mark.parametrize("kernel,nu", [("gaussian", None), ("laplacian", None), ("matern", 1.5), ("matern", 2.5)])
@pytest.mark.parametrize("shape", SHAPES, ids=[f"n{n}_m{m}_d{d}_t{t}" for n, m, d, t in SHAPES])
def test_ragged_shapes_against_oracle(shape, kernel, nu, dtype):
    """Sizes that are not multiples of any tile, every kernel function, both kernels (SIMT and,
    where it applies, tensor-core), checked against the CPU oracle and the fp64 truth."""
    n, m, d, t = shape
    rng = np.random.default_rng(n * 1000 + m * 10 + d + t)
    X = rng.standard_normal((n, d)).astype(dtype)
    C = rng.standard_normal((m, d)).astype(dtype)
    v = rng.standard_normal((m, t)).astype(dtype)
    w = rng.standard_normal((n, t)).astype(dtype)
    sigma = [1.5 + 0.25 * np.sqrt(d)]
    case = dict(kernel=kernel, sigma=sigma, nu=nu)
    truth_mmv = fo.dense_fmmv_fp64(X, C, v, kernel, sigma[0], nu)
    truth_dmmv = fo.dense_fdmmv_fp64(X, C, v, w, kernel, sigma[0], nu)
    orc_dmmv = fo.fdmmv(torch.from_numpy(X), torch.from_numpy(C), torch.from_numpy(v), torch.from_numpy(w),
                        kernel, sigma, nu).numpy()
    # distance-based kernels of random points: fp32 cancellation is mild, fp64 bar is the benchmark's
    tol = 1e-4 if dtype == "float32" else 1e-10
    for flags in (0, 1):
        k = with_flags(make_kernel(case), flags)
        got = k.mmv(dev(X), dev(C), dev(v)).cpu().numpy()
        assert fo.rel_l2(got, truth_mmv) <= tol, f"mmv flags={flags}"
        got = k.dmmv(dev(X), dev(C), dev(v), dev(w)).cpu().numpy()
        assert fo.rel_l2(got, truth_dmmv) <= tol, f"dmmv flags={flags}"
        assert fo.rel_l2(got, orc_dmmv) <= tol, f"dmmv vs oracle flags={flags}"
        got = k.dmmv(dev(X), dev(C), None, dev(w)).cpu().numpy()
        assert fo.rel_l2(got, fo.dense_fdmmv_fp64(X, C, None, w, kernel, sigma[0], nu)) <= tol, "dmmv v=None"


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64], ids=["f32", "f64"])
def test_empty_operands(dtype):
    """Zero rows on either side: empty or all-zero results of the right shape, no launch failure, and the
    context stays usable."""
    from falkon_b200.kernels import GaussianKernel

    k = GaussianKernel(2.0)
    g = torch.Generator().manual_seed(9)
    X = torch.randn(50, 4, generator=g, dtype=dtype).cuda()
    C = torch.randn(7, 4, generator=g, dtype=dtype).cuda()
    v = torch.randn(7, 2, generator=g, dtype=dtype).cuda()
    w = torch.randn(50, 2, generator=g, dtype=dtype).cuda()
    out = k.mmv(X[:0], C, v)
    assert tuple(out.shape) == (0, 2)
    out = k.mmv(X, C[:0], v[:0])
    assert tuple(out.shape) == (50, 2) and float(out.abs().max()) == 0.0
    out = k.dmmv(X[:0], C, v, w[:0])
    assert tuple(out.shape) == (7, 2) and float(out.abs().max()) == 0.0
    out = k.dmmv(X, C[:0], v[:0], w)
    assert tuple(out.shape) == (0, 2)
    K = k(X[:0], C)
    assert tuple(K.shape) == (0, 7)
    # host operands too
    out = k.dmmv(X[:0].cpu(), C.cpu(), v.cpu(), w[:0].cpu())
    assert tuple(out.shape) == (7, 2) and float(out.abs().max()) == 0.0
    ref = fo.dense_fdmmv_fp64(X.cpu().numpy(), C.cpu().numpy(), v.cpu().numpy(), w.cpu().numpy(), "gaussian", 2.0)
    assert fo.rel_l2(k.dmmv(X, C, v, w).cpu().numpy(), ref) < (1e-4 if dtype == torch.float32 else 1e-10)


@pytest.mark.parametrize("d", [8, 48], ids=["resident", "kloop"])
def test_long_reductions_keep_fp32_accuracy(d):
    """Reduction over millions of rows (the K^T u sweep of a large fit): the error against an fp64 evaluation
    does not grow with the length of the reduction (it stays at the level of a 65,536-row problem, below 1e-6 for
    the resident kernel).  A single running fp32 sum per thread over a whole chunk reaches several 1e-6 here,
    which is enough to make an fp32 conjugate gradient at lambda = 1e-7 drift; the kernels sum in two levels."""
    from falkon_b200.kernels import GaussianKernel

    n, m = 4_000_000, 1024
    g = torch.Generator(device="cuda").manual_seed(12)
    X = torch.randn(n, d, generator=g, device="cuda")
    C = X[torch.randperm(n, generator=g, device="cuda")[:m]].contiguous()
    y = torch.randn(n, 2, generator=g, device="cuda")
    k = GaussianKernel(float(d) ** 0.5)
    errs = []
    for rows in (65_536, n):
        got = k.mmv(C, X[:rows], y[:rows])
        want = k.mmv(C.double(), X[:rows].double(), y[:rows].double())
        errs.append(fo.rel_l2(got.cpu().numpy(), want.cpu().numpy()))
        got = k.dmmv(X[:rows], C, None, y[:rows])
        errs.append(fo.rel_l2(got.cpu().numpy(), want.cpu().numpy()))
    small, big = max(errs[:2]), max(errs[2:])
    assert big < 2.0 * small + 5e-7, errs
    assert big < (1e-6 if d <= 30 else 1e-4), errs


@pytest.mark.parametrize("d,t", [(48, 1), (64, 1), (64, 2), (20, 2), (96, 1)])
def test_vector_tiles_are_not_overwritten_under_their_readers(d, t):
    """Few output rows, a long reduction, few features: the epilogue is the slow side, the bulk-copy producer runs
    ahead until it waits for the very vector tile the epilogue is reading, and refills it the moment it is
    released.  The release has to wait for the loads of that tile (a data dependency on the sums they feed plus a
    proxy fence before the arrive); without it the results were wrong in a few rows and changed from run to run."""
    from falkon_b200.kernels import GaussianKernel

    g = torch.Generator(device="cuda").manual_seed(5)
    X1 = torch.randn(1024, d, generator=g, device="cuda")
    X2 = torch.randn(65_536, d, generator=g, device="cuda")
    v = torch.randn(65_536, t, generator=g, device="cuda")
    k = GaussianKernel(float(d) ** 0.5)
    want = k.mmv(X1.double(), X2.double(), v.double()).cpu().numpy()
    outs = [k.mmv(X1, X2, v).cpu().numpy() for _ in range(4)]
    for got in outs:
        assert fo.rel_l2(got, want) < 2e-5
    for got in outs[1:]:
        assert np.array_equal(got, outs[0])  # and bitwise the same every time


def test_duplicate_points_clamp():
    """Centres that are exact copies of data rows (distance 0): the clamp keeps sqrt() finite and
    the diagonal entries equal to 1 (falkon/kernels/distance_kernel.py:100)."""
    rng = np.random.default_rng(5)
    X = rng.standard_normal((300, 6)).astype(np.float32) * 3
    C = X[:40].copy()
    v = np.eye(40, dtype=np.float32)[:, :4].copy()
    from falkon_b200.kernels import GaussianKernel, LaplacianKernel, MaternKernel

    for k in (GaussianKernel(2.0), LaplacianKernel(2.0), MaternKernel(2.0, 1.5), MaternKernel(2.0, 2.5)):
        for flags in (0, 1):
            with_flags(k, flags)
            out = k.mmv(dev(X), dev(C), dev(v)).cpu().numpy()
            assert np.isfinite(out).all()
            for j in range(4):  # row j of X equals centre j: K[j, j] = 1
                assert abs(out[j, j] - 1.0) < 2e-3


def test_run_to_run_determinism():
    """Two runs give bit-identical results (the reference's stress test demands run-to-run
    equality, falkon/tests/test_stress_multi_core.py:224): no atomics on the result path."""
    case = case_by_name("c2_small")
    inp = build_inputs(case)
    X, C, v, w = (dev(inp[k]) for k in ("X", "C", "v", "w"))
    for flags in (0, 1):
        k = with_flags(make_kernel(case), flags)
        a = k.dmmv(X, C, v, w).clone()
        b = k.dmmv(X, C, v, w).clone()
        assert torch.equal(a, b)
        a = k.mmv(C, X, w).clone()
        b = k.mmv(C, X, w).clone()
        assert torch.equal(a, b)


def test_tensor_core_kernel_is_used_and_clean():
    from falkon_b200 import _lib

    lib = _lib.load()
    assert lib.flk_check_device() == 0, _lib.last_error()
    assert lib.flk_uses_tensor_cores(0, 0, 28, 1, 0) == 1
    case = case_by_name("c2_small")
    inp = build_inputs(case)
    X, C, v, w = (dev(inp[k]) for k in ("X", "C", "v", "w"))
    k = with_flags(make_kernel(case), 2)  # FORCE_TC: fails instead of falling back to SIMT
    before = _lib.launch_count()
    out = k.dmmv(X, C, v, w)
    assert _lib.launch_count() - before >= 7
    assert _lib.tc_status(X.device) == 0
    gold = np.load(os.path.join(GOLD, "c2_small.npz"))
    assert fo.rel_l2(out.cpu().numpy(), gold["dmmv"]) <= 1e-4
    k64 = with_flags(make_kernel(case_by_name("c4_small_64")), 2)
    with pytest.raises(NotImplementedError):
        k64.mmv(X.double(), C.double(), v.double())


@pytest.mark.parametrize("kernel,nu", [("gaussian", None), ("matern", 2.5)])
def test_rows_beyond_fp16_range_take_the_simt_path(kernel, nu):
    """The tensor-core operand images are fp16; a row whose scaled squared norm does not fit is
    detected on the device and the SIMT kernels produce the result instead.  The answer must be as
    accurate as for in-range data, with FORCE_TC set or not (the flag only refuses unsupported
    dtype / feature counts up front, it does not disable the device-side switch)."""
    from falkon_b200 import _lib
    from falkon_b200.kernels import GaussianKernel, MaternKernel

    rng = np.random.default_rng(77)
    n, m, d = 1500, 700, 12
    X = rng.standard_normal((n, d)).astype(np.float32)
    X[7] *= 3000.0       # |x / sigma|^2 ~ 2.7e7: far outside what fp16 images carry
    X[1203, 3] = 900.0   # a single large coordinate
    C = X[:m].copy()     # includes row 7, so K has an exact 1 on an out-of-range diagonal entry
    v = rng.standard_normal((m, 2)).astype(np.float32)
    w = rng.standard_normal((n, 2)).astype(np.float32)
    for flags in (0, 2):
        k = GaussianKernel(2.0) if kernel == "gaussian" else MaternKernel(2.0, nu=nu)
        k = with_flags(k, flags)
        got = k.dmmv(dev(X), dev(C), dev(v), dev(w)).cpu().numpy()
        assert _lib.tc_status(torch.device("cuda", torch.cuda.current_device())) == 0
        want = fo.dense_fdmmv_fp64(X, C, v, w, kernel, 2.0, nu)
        assert np.isfinite(got).all()
        assert fo.rel_l2(got, want) <= 1e-4
        got = k.mmv(dev(X), dev(C), dev(v)).cpu().numpy()
        assert fo.rel_l2(got, fo.dense_fmmv_fp64(X, C, v, kernel, 2.0, nu)) <= 1e-4


@pytest.mark.parametrize("order", ["C", "F"])
def test_large_host_inputs_travel_in_row_chunks(order):
    """From 262,144 rows up the host-buffer entry points copy X1 (and w) in row chunks through a copy stream
    and, for fdmmv, sum the per-chunk results: the answer must equal the one-piece device call to rounding,
    for row-major and column-major host matrices and a row count that is not a multiple of anything."""
    from falkon_b200.kernels import GaussianKernel, MaternKernel

    g = torch.Generator().manual_seed(31)
    n, m, d, t = 300_017, 257, 11, 2
    X = torch.randn(n, d, generator=g)
    C = X[torch.randperm(n, generator=g)[:m]].contiguous()
    v = torch.randn(m, t, generator=g)
    w = torch.randn(n, t, generator=g)
    if order == "F":
        X = X.T.contiguous().T
        w = w.T.contiguous().T
    for k in (GaussianKernel(3.0), MaternKernel(3.0, nu=1.5)):
        dev_out = k.dmmv(X.cuda(), C.cuda(), v.cuda(), w.cuda()).cpu()
        host_out = k.dmmv(X, C, v, w)
        assert host_out.device.type == "cpu"
        assert float((host_out - dev_out).norm() / dev_out.norm()) <= 2e-6
        host_out2 = k.dmmv(X, C, None, w)  # w only: K^T w
        dev_out2 = k.dmmv(X.cuda(), C.cuda(), None, w.cuda()).cpu()
        assert float((host_out2 - dev_out2).norm() / dev_out2.norm()) <= 2e-6
        dev_u = k.mmv(X.cuda(), C.cuda(), v.cuda()).cpu()
        host_u = k.mmv(X, C, v)
        assert torch.equal(host_u, dev_u)  # K v has no cross-chunk sum: bit-identical
    # fp64 through the SIMT kernel
    k = GaussianKernel(3.0)
    a = k.dmmv(X.double(), C.double(), v.double(), w.double())
    b = k.dmmv(X.double().cuda(), C.double().cuda(), v.double().cuda(), w.double().cuda()).cpu()
    assert float((a - b).norm() / b.norm()) <= 1e-13


def test_errors_surface_as_python_exceptions():
    from falkon_b200.kernels import GaussianKernel

    k = GaussianKernel(1.0)
    X = torch.randn(64, 4, device="cuda")
    C = torch.randn(8, 4, device="cuda")
    v = torch.randn(8, 1, device="cuda")
    with pytest.raises(ValueError):
        k.mmv(X[:, ::2], C[:, ::2], v)  # neither stride is 1
    with pytest.raises(TypeError):
        k.mmv(X, C.double(), v)
    with pytest.raises(ValueError):
        k.dmmv(X, C, None, None)
    with pytest.raises(RuntimeError):
        from falkon_b200 import FalkonOptions

        k.mmv(X, C, v, opt=FalkonOptions(use_cpu=True))
    Xg = X.clone().requires_grad_()
    with pytest.raises(NotImplementedError):
        k.dmmv(Xg, C, v, None)
    # the context survives all of the above
    assert torch.isfinite(k.mmv(X, C, v)).all()


@pytest.mark.parametrize("flags", [0, 1], ids=["auto", "simt"])
def test_full_size_config2_properties(flags):
    """Benchmark configuration 2 at full size (N = 1e6, d = 28, M = 20000): linearity in v,
    agreement of sampled outputs with an fp64 evaluation, and SIMT / tensor-core agreement."""
    n, m, d = 1_000_000, 20_000, 28
    g = torch.Generator(device="cuda").manual_seed(1002)
    z = (torch.rand(n, 1, generator=g, device="cuda") < 0.5).float()
    X = torch.randn(n, d, generator=g, device="cuda") + (2 * z - 1) * 0.5
    idx = torch.randperm(n, generator=g, device="cuda")[:m]
    C = X[idx].contiguous()
    v1 = torch.randn(m, 1, generator=g, device="cuda")
    v2 = torch.randn(m, 1, generator=g, device="cuda")
    w = torch.randn(n, 1, generator=g, device="cuda")
    from falkon_b200.kernels import GaussianKernel

    k = with_flags(GaussianKernel(5.0), flags)
    u = k.mmv(X, C, v1)
    # sampled rows of K v against fp64
    rows = torch.arange(0, n, n // 64, device="cuda")[:64]
    truth = fo.dense_fmmv_fp64(X[rows].cpu().numpy(), C.cpu().numpy(), v1.cpu().numpy(), "gaussian", 5.0)
    assert fo.rel_l2(u[rows].cpu().numpy(), truth) <= 1e-4
    # sampled entries of K^T (K v + w): out_j = sum_i k(x_i, c_j) (u_i + w_i) in fp64
    out = k.dmmv(X, C, v1, w)
    cols = torch.arange(0, m, m // 8, device="cuda")[:8]
    uu = (u.double() + w.double())
    Xd, Cd = X.double() / 5.0, C[cols].double() / 5.0
    d2 = (Xd * Xd).sum(1, keepdim=True) - 2 * Xd @ Cd.t() + (Cd * Cd).sum(1)[None, :]
    truth = (torch.exp(-0.5 * d2.clamp_min(0)).t() @ uu).cpu().numpy()
    assert fo.rel_l2(out[cols].cpu().numpy(), truth) <= 1e-4
    # linearity: dmmv(v1 + v2, w) - dmmv(v1, w) = dmmv(v2, None)
    lhs = k.dmmv(X, C, v1 + v2, w) - out
    rhs = k.dmmv(X, C, v2, None)
    assert fo.rel_l2(lhs.cpu().numpy(), rhs.cpu().numpy()) <= 2e-4
    # the other kernel gives the same answer
    other = with_flags(GaussianKernel(5.0), 1 - flags)
    assert fo.rel_l2(other.dmmv(X, C, v1, w).cpu().numpy(), out.cpu().numpy()) <= 1e-4
