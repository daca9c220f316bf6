"""falkon_b200: B200-native implicit kernel-matrix products behind Falkon's operator API.

    from falkon_b200 import FalkonOptions
    from falkon_b200.kernels import GaussianKernel
    k = GaussianKernel(sigma=5.0)
    out = k.dmmv(X, C, v, w)          # K(X,C)^T (K(X,C) v + w), computed by hand-written sm_100a kernels

The CUDA library (falkon_b200/libfalkon_b200.so, C ABI in include/falkon_b200.h) is loaded on first
use; there is no CPU fallback.
"""
from .options import FalkonOptions  # noqa: F401
from . import center_selection, kernels, mmv_ops, models, optim, preconditioner  # noqa: F401
from .models import Falkon, InCoreFalkon  # noqa: F401

__version__ = "0.2.0"
__all__ = ("FalkonOptions", "Falkon", "InCoreFalkon", "kernels", "mmv_ops", "optim", "preconditioner", "models", "center_selection")
