"""CPU tests of the host-side mirror of the reference's operator API (no GPU work)."""
import dataclasses

import numpy as np
import pytest
import torch

from falkon_b200 import FalkonOptions
from falkon_b200.kernels import GaussianKernel, Kernel, LaplacianKernel, MaternKernel, validate_sigma
from falkon_b200.mmv_ops import fdmmv, fmmv
from falkon_b200.mmv_ops.utils import create_output_mat, is_contig, is_f_contig
from falkon_b200 import _lib


def test_options_match_reference_field_list():
    # names and defaults of falkon/options.py:168-181, :205-208, :223-227, :257-259, :281-283
    expected = {
        "debug": False, "use_cpu": False, "max_gpu_mem": np.inf, "max_cpu_mem": np.inf,
        "compute_arch_speed": False, "no_single_kernel": True, "min_cuda_pc_size_32": 10000,
        "min_cuda_pc_size_64": 30000, "min_cuda_iter_size_32": 300_000_000, "min_cuda_iter_size_64": 900_000_000,
        "never_store_kernel": False, "store_kernel_d_threshold": 1200, "num_fmm_streams": 2, "memory_slack": 0.9,
        "keops_acc_dtype": "auto", "keops_sum_scheme": "auto", "keops_active": "auto", "keops_memory_slack": 0.7,
        "cg_epsilon_32": 1e-7, "cg_epsilon_64": 1e-15, "cg_tolerance": 1e-7, "cg_full_gradient_every": 10,
        "cg_differential_convergence": False, "pc_epsilon_32": 1e-5, "pc_epsilon_64": 1e-13,
        "cpu_preconditioner": False, "chol_force_in_core": False, "chol_force_ooc": False,
        "chol_par_blk_multiplier": 2,
    }
    assert dataclasses.asdict(FalkonOptions()) == expected
    o = FalkonOptions(max_gpu_mem=1.0, keops_active="no")
    merged = dataclasses.replace(FalkonOptions(debug=True), **dataclasses.asdict(o))
    assert merged.max_gpu_mem == 1.0 and merged.keops_active == "no" and merged.debug is False
    assert o.cg_epsilon(torch.float32) == 1e-7 and o.pc_epsilon(torch.float64) == 1e-13
    with pytest.raises(TypeError):
        o.cg_epsilon(torch.float16)
    assert o.get_base_options().max_gpu_mem == 1.0


def test_sigma_and_nu_validation():
    assert validate_sigma(3).dtype == torch.float64 and validate_sigma(3).shape == (1,)
    assert validate_sigma(torch.tensor([[1.0], [2.0]])).shape == (2,)
    with pytest.raises(ValueError):
        validate_sigma(torch.eye(3))
    with pytest.raises(TypeError):
        validate_sigma(None)
    k = MaternKernel(2.0, 2.5)
    assert k.nu == 2.5 and k.name == "2.5-matern" and k.nondiff_params == {"nu": 2.5}
    assert list(k.diff_params) == ["sigma"]
    assert MaternKernel(2.0, 0.5)._flk_spec()[0] == _lib.FLK_LAPLACIAN
    assert MaternKernel(2.0, float("inf"))._flk_spec()[0] == _lib.FLK_GAUSSIAN
    with pytest.raises(ValueError):
        MaternKernel(2.0, 3.5)
    with pytest.raises(TypeError):
        MaternKernel(2.0, 2)
    g = GaussianKernel(torch.tensor([1.0, 2.0, 3.0]))
    kid, sig = g._flk_spec()
    assert kid == _lib.FLK_GAUSSIAN and sig.dtype == np.float64 and sig.tolist() == [1.0, 2.0, 3.0]
    d = g.detach()
    assert isinstance(d, GaussianKernel) and d.params is g.params
    assert "GaussianKernel" in repr(g) and "Laplacian" in str(LaplacianKernel(1.0))


def test_dimension_and_dtype_errors_follow_reference():
    k = GaussianKernel(1.0)
    X, C, v, w = torch.randn(10, 3), torch.randn(4, 3), torch.randn(4, 2), torch.randn(10, 2)
    with pytest.raises(ValueError, match="One of v and w"):
        k.dmmv(X, C, None, None)
    with pytest.raises(ValueError, match="must be 2D"):
        k.mmv(X[0], C, v)
    with pytest.raises(ValueError, match="Dimensions of matrix v"):
        k.mmv(X, C, torch.randn(5, 2))
    with pytest.raises(ValueError, match="Dimensions of matrix w"):
        k.dmmv(X, C, v, torch.randn(9, 2))
    with pytest.raises(ValueError, match="Output dimension"):
        k.dmmv(X, C, v, w, out=torch.empty(10, 2))
    with pytest.raises(TypeError):
        k.mmv(X.double(), C, v)
    # the kernel matrix validates like the reference (falkon/kernels/kernel.py:107-133)
    with pytest.raises(ValueError):
        k(X, C[:, :2])
    with pytest.raises(ValueError):
        k(X, C, out=torch.empty(3, 3))
    with pytest.raises(TypeError):
        k(X.double(), C)
    with pytest.raises(ValueError):
        k(X, C, diag=True)  # different numbers of rows


def test_products_fail_loudly_without_gpu_or_with_use_cpu():
    k = GaussianKernel(1.0)
    X, C, v = torch.randn(10, 3), torch.randn(4, 3), torch.randn(4, 1)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        k.mmv(X, C, v, opt=FalkonOptions(use_cpu=True))
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="needs a CUDA device"):
            k.mmv(X, C, v)
        with pytest.raises(RuntimeError, match="needs a CUDA device"):
            k.dmmv(X, C, v, None)
    with pytest.raises(NotImplementedError):
        fdmmv(X, C, v, None, k, None, True, FalkonOptions())  # positional, differentiable=True
    with pytest.raises(ValueError, match="memory contiguous"):
        fmmv(torch.randn(10, 6)[:, ::2], C, v, k, opt=FalkonOptions())

    class Custom(Kernel):
        def compute(self, X1, X2, out, diag, **kw):
            return out

    # a kernel that only implements `compute` takes the blocked path through its own compute -- on the GPU only
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="needs a CUDA device"):
            Custom("custom", None).mmv(X, C, v)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        Custom("custom", None).dmmv(X, C, v, None, opt=FalkonOptions(use_cpu=True))


def test_output_allocation_rules():
    Xc = torch.empty(6, 3)
    Xf = torch.empty(3, 6).t()
    assert is_contig(Xc) and is_contig(Xf) and is_f_contig(Xf, strict=True) and not is_f_contig(Xc, strict=True)
    cpu = torch.device("cpu")
    o = create_output_mat(None, [cpu, cpu], (6, 2), torch.float32, "cuda", Xc)
    assert o.shape == (6, 2) and o.stride() == (2, 1) and o.device.type == "cpu"
    o = create_output_mat(None, [cpu, cpu], (6, 2), torch.float64, "cuda", Xf)
    assert o.stride() == (1, 6) and o.dtype == torch.float64
    given = torch.empty(6, 2)
    assert create_output_mat(given, [cpu], (6, 2), torch.float32, "cuda", Xc) is given


def test_incore_falkon_requires_cuda_tensors():
    from falkon_b200 import InCoreFalkon

    model = InCoreFalkon(kernel=GaussianKernel(1.0), penalty=1e-3, M=5)
    with pytest.raises(ValueError, match="CUDA tensors"):
        model.fit(torch.randn(20, 3), torch.randn(20, 1))


def test_falkon_constructor_validation():
    from falkon_b200 import Falkon, FalkonOptions

    with pytest.raises(ValueError, match="M must be specified"):
        Falkon(kernel=GaussianKernel(1.0), penalty=1e-3, M=None)
    with pytest.raises(ValueError, match="not valid"):
        Falkon(kernel=GaussianKernel(1.0), penalty=1e-3, M=5, center_selection="kmeans")
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        Falkon(kernel=GaussianKernel(1.0), penalty=1e-3, M=5, options=FalkonOptions(use_cpu=True))
    model = Falkon(kernel=GaussianKernel(1.0), penalty=1e-3, M=5)
    with pytest.raises(RuntimeError, match="has not been trained"):
        model.predict(torch.randn(4, 3))
    with pytest.raises(ValueError, match="same number of samples"):
        model.fit(torch.randn(20, 3), torch.randn(19, 1))


def test_option_merge_keeps_the_extra_attributes():
    """``dataclasses.replace`` drops attributes that are not dataclass fields; the per-call merge must carry
    flk_flags / flk_devices / pc_tensor_cores from the kernel's own options and let the call's options override."""
    from falkon_b200.options import merge_options

    base = FalkonOptions(debug=True)
    base.flk_flags = _lib.FLAG_FORCE_SIMT
    base.flk_devices = [1]
    k = GaussianKernel(1.0, opt=base)
    assert k._merged(None) is base
    call = FalkonOptions(max_gpu_mem=5.0)
    m = k._merged(call)
    assert m.max_gpu_mem == 5.0 and m.debug is False  # fields: the call's options win, as in the reference
    assert m.flk_flags == _lib.FLAG_FORCE_SIMT and m.flk_devices == [1]  # extras survive the merge
    call.flk_flags = _lib.FLAG_FORCE_TC
    m = k._merged(call)
    assert m.flk_flags == _lib.FLAG_FORCE_TC and m.flk_devices == [1]
    assert not hasattr(merge_options(FalkonOptions(), FalkonOptions()), "flk_flags")
    # a narrower option object (the reference passes BaseOptions subsets around) merges field by field
    from falkon_b200.options import BaseOptions

    assert merge_options(base, BaseOptions(max_cpu_mem=7.0)).max_cpu_mem == 7.0


def test_c_abi_guard_rejects_mismatched_operands():
    """The ctypes layer refuses operands whose shape, dtype or placement disagree before any pointer reaches the
    library (the kernels trust the sizes they are given)."""
    X, C, v, w = torch.randn(10, 3), torch.randn(4, 3), torch.randn(4, 2), torch.randn(10, 2)
    out_m, out_n = torch.empty(4, 2), torch.empty(10, 2)
    sig = np.array([1.0])
    with pytest.raises(ValueError, match="v has shape"):
        _lib.call_fmmv(0, sig, X, C, torch.randn(5, 2), out_n, host=True)
    with pytest.raises(ValueError, match="out has shape"):
        _lib.call_fmmv(0, sig, X, C, v, torch.empty(9, 2), host=True)
    with pytest.raises(TypeError, match="Data types"):
        _lib.call_fmmv(0, sig, X, C, v.double(), out_n, host=True)
    with pytest.raises(ValueError, match="X2 has shape"):
        _lib.call_fmmv(0, sig, X, torch.randn(4, 5), v, out_n, host=True)
    with pytest.raises(ValueError, match="w has shape"):
        _lib.call_fdmmv(0, sig, X, C, v, torch.randn(9, 2), out_m, host=True)
    with pytest.raises(ValueError, match="out has shape"):
        _lib.call_fdmmv(0, sig, X, C, v, w, torch.empty(4, 3), host=True)
    with pytest.raises(TypeError, match="Data types"):
        _lib.call_fdmmv(0, sig, X, C, v, w.double(), out_m, host=True)
    with pytest.raises(ValueError, match="One of v and w"):
        _lib.call_fdmmv(0, sig, X, C, None, None, out_m, host=True)
    with pytest.raises(ValueError, match="must be 2-D"):
        _lib.call_fmmv(0, sig, X, C, v[:, 0], out_n, host=True)
    with pytest.raises(ValueError, match="CUDA device"):
        _lib.call_fmmv(0, sig, X, C, v, out_n)  # device entry point given host tensors
    with pytest.raises(ValueError, match="CUDA device"):
        _lib.call_fmm(0, sig, X, C, torch.empty(10, 4))
    with pytest.raises(ValueError, match="CUDA device"):
        _lib.call_kgrad(0, sig, X, C, torch.randn(10, 2), v, torch.empty(10, 4))


def test_falkon_passes_extra_attributes_down():
    """The estimator hands its options to every product as ``opt=``; a forced tensor-core path on fp64 data must
    therefore surface as NotImplementedError from inside fit, not be silently dropped.  Checked here through the
    merge alone (no GPU): the options the products see carry the flag."""
    from falkon_b200 import Falkon

    o = FalkonOptions()
    o.flk_flags = _lib.FLAG_FORCE_TC
    model = Falkon(kernel=GaussianKernel(1.0), penalty=1e-3, M=5, options=o)
    assert model.kernel._merged(model.options).flk_flags == _lib.FLAG_FORCE_TC


def test_rows_within_budget_uses_the_workspace_queries():
    """Chunk sizing under a memory budget is host arithmetic over the C ABI's workspace queries."""
    lib = _lib.load()

    def need(r):
        return lib.flk_fdmmv_workspace_bytes(_lib.FLK_F32, _lib.FLK_GAUSSIAN, r, 50_000, 28, 1, 0)

    n = 10_000_000
    assert _lib.rows_within_budget(need, n, None) == n
    assert _lib.rows_within_budget(need, n, float("inf")) == n
    assert _lib.rows_within_budget(need, n, need(n)) == n
    budget = 1 * 2**30
    r = _lib.rows_within_budget(need, n, budget)
    assert 0 < r < n and r % 512 == 0 and need(r) <= budget < need(r + 1024)
    with pytest.raises(MemoryError, match="not enough"):
        _lib.rows_within_budget(need, n, 1 * 2**20)
    # the budget rule of the products: min(free, max_gpu_mem) * memory_slack; no limit -> None on a CPU-only box
    from falkon_b200.mmv_ops.fmmv import device_budget

    assert device_budget(FalkonOptions(), torch.device("cpu")) is None
    assert device_budget(FalkonOptions(max_gpu_mem=1000.0, memory_slack=0.5), torch.device("cpu")) == 500.0
