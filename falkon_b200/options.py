"""Option dataclasses of the operator API.

Field names and defaults are those of the reference's option classes
(falkon/options.py:164-303: BaseOptions :168-181, KeopsOptions :205-208,
ConjugateGradientOptions :223-227, PreconditionerOptions :257-259, CholeskyOptions :281-283),
so option objects written for the reference configure this package unchanged and
``dataclasses.replace(kernel.params, **dataclasses.asdict(opt))`` (falkon/kernels/kernel.py:283-285)
keeps working.  On the kernel-vector-product path most of them have nothing left to control:
no n x m block is ever allocated, so the memory budgets are accepted and ignored, and KeOps is
never consulted.  ``use_cpu=True`` is rejected by the products (there is no CPU path here).
"""
from dataclasses import dataclass

import numpy as np
import torch

__all__ = (
    "BaseOptions",
    "KeopsOptions",
    "ConjugateGradientOptions",
    "PreconditionerOptions",
    "CholeskyOptions",
    "FalkonOptions",
    "EXTRA_ATTRS",
    "merge_options",
)


@dataclass
class BaseOptions:
    debug: bool = False
    use_cpu: bool = False
    max_gpu_mem: float = np.inf
    max_cpu_mem: float = np.inf
    compute_arch_speed: bool = False
    no_single_kernel: bool = True
    min_cuda_pc_size_32: int = 10000
    min_cuda_pc_size_64: int = 30000
    min_cuda_iter_size_32: int = 10_000 * 10 * 3_000
    min_cuda_iter_size_64: int = 30_000 * 10 * 3_000
    never_store_kernel: bool = False
    store_kernel_d_threshold: int = 1200
    num_fmm_streams: int = 2
    memory_slack: float = 0.9

    def get_base_options(self):
        return BaseOptions(**{f: getattr(self, f) for f in BaseOptions.__dataclass_fields__})


@dataclass
class KeopsOptions:
    keops_acc_dtype: str = "auto"
    keops_sum_scheme: str = "auto"
    keops_active: str = "auto"
    keops_memory_slack: float = 0.7

    def get_keops_options(self):
        return KeopsOptions(**{f: getattr(self, f) for f in KeopsOptions.__dataclass_fields__})


@dataclass
class ConjugateGradientOptions:
    cg_epsilon_32: float = 1e-7
    cg_epsilon_64: float = 1e-15
    cg_tolerance: float = 1e-7
    cg_full_gradient_every: int = 10
    cg_differential_convergence: bool = False

    def cg_epsilon(self, dtype):
        if dtype == torch.float32:
            return self.cg_epsilon_32
        if dtype == torch.float64:
            return self.cg_epsilon_64
        raise TypeError(f"Data-type {str(dtype)} invalid")

    def get_conjgrad_options(self):
        return ConjugateGradientOptions(
            **{f: getattr(self, f) for f in ConjugateGradientOptions.__dataclass_fields__}
        )


@dataclass
class PreconditionerOptions:
    pc_epsilon_32: float = 1e-5
    pc_epsilon_64: float = 1e-13
    cpu_preconditioner: bool = False

    def pc_epsilon(self, dtype):
        if dtype == torch.float32:
            return self.pc_epsilon_32
        if dtype == torch.float64:
            return self.pc_epsilon_64
        raise TypeError(f"Data-type {str(dtype)} invalid")

    def get_pc_options(self):
        return PreconditionerOptions(**{f: getattr(self, f) for f in PreconditionerOptions.__dataclass_fields__})


@dataclass(frozen=False)
class CholeskyOptions:
    chol_force_in_core: bool = False
    chol_force_ooc: bool = False
    chol_par_blk_multiplier: int = 2

    def get_chol_options(self):
        return CholeskyOptions(**{f: getattr(self, f) for f in CholeskyOptions.__dataclass_fields__})


@dataclass()
class FalkonOptions(BaseOptions, ConjugateGradientOptions, PreconditionerOptions, CholeskyOptions, KeopsOptions):
    """Global options; the union of all option groups (falkon/options.py:293-303)."""

    pass


# Attributes of this package that are not fields of the reference's option classes (so that the field list
# stays the reference's): plain attributes set on an option object.
#   flk_flags        FLK_FLAG_* bits handed to the C ABI (force the SIMT or the tensor-core kernels)
#   flk_devices      list of CUDA ordinals a host-operand product may spread over
#   pc_tensor_cores  False selects the library factorisations in the fp32 preconditioner
EXTRA_ATTRS = ("flk_flags", "flk_devices", "pc_tensor_cores")


def merge_options(base, override):
    """Options of one call: ``override``'s fields on top of ``base`` (falkon/kernels/kernel.py:283-285).

    ``dataclasses.replace`` rebuilds the object from its fields and so drops the extra attributes above;
    they are carried over here: ``base``'s first, then ``override``'s where it sets them."""
    import dataclasses

    if override is None:
        return base
    fields = {f.name for f in dataclasses.fields(base)}
    merged = dataclasses.replace(base, **{k: v for k, v in dataclasses.asdict(override).items() if k in fields})
    for src in (base, override):
        for name in EXTRA_ATTRS:
            if name in getattr(src, "__dict__", {}):
                setattr(merged, name, getattr(src, name))
    return merged
