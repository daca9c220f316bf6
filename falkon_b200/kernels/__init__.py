from .kernel import Kernel
from .distance_kernel import DiffKernel, GaussianKernel, LaplacianKernel, MaternKernel, validate_sigma

__all__ = ("Kernel", "DiffKernel", "GaussianKernel", "LaplacianKernel", "MaternKernel", "validate_sigma")
