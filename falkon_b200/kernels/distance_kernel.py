"""Distance kernels: Gaussian, Laplacian, Matern (nu in 0.5, 1.5, 2.5, inf).

Constructor arguments, attributes (``sigma``, ``nu``, ``diff_params``, ``nondiff_params``,
``detach``) and validation follow falkon/kernels/distance_kernel.py:20-38, :314-432, :435-507,
:510-630 and falkon/kernels/diff_kernel.py:14-145.  The arithmetic itself lives in the CUDA library;
each class only tells it which kernel function and length-scale to use (``_flk_spec``).
"""
from typing import Any, Dict, Optional, Union

import numpy as np
import torch
from torch import nn

from .. import _lib
from ..options import FalkonOptions
from .kernel import Kernel


def validate_sigma(sigma: Union[float, torch.Tensor]) -> torch.Tensor:
    """float -> fp64 tensor [1]; 1-element tensor kept; vector flattened; matrices rejected."""
    if isinstance(sigma, torch.Tensor):
        if sigma.numel() == 1:
            return sigma
        if sigma.dim() == 1 or (sigma.dim() == 2 and sigma.shape[1] == 1):
            return sigma.reshape(-1)
        raise ValueError("sigma must be a scalar or a vector.")
    try:
        return torch.tensor([float(sigma)], dtype=torch.float64)
    except TypeError:
        raise TypeError("Sigma must be a scalar or a tensor.") from None


class DiffKernel(Kernel):
    """Kernel whose hyper-parameters are registered as ``nn.Parameter`` s
    (falkon/kernels/diff_kernel.py:46-59)."""

    def __init__(self, name, options, **kernel_params):
        super().__init__(name=name, opt=options)
        self._other_params = {}
        for k, v in kernel_params.items():
            if isinstance(v, torch.Tensor):
                self.register_parameter(k, nn.Parameter(v, requires_grad=v.requires_grad))
            else:
                self._other_params[k] = v
                setattr(self, k, v)

    @property
    def diff_params(self) -> Dict[str, torch.Tensor]:
        return dict(self.named_parameters())

    @property
    def nondiff_params(self) -> Dict[str, Any]:
        return self._other_params

    def compute(self, X1, X2, out, diag, **kwargs):
        """Dense kernel block ``k(X1, X2)`` written into ``out`` (n x m, or (n,) with ``diag=True``) and returned:
        the extension point of falkon/kernels/diff_kernel.py:90-91 (``core_fn(X1, X2, out=out, diag=diag,
        **params)``).  The block is evaluated by ``flk_fmm`` in the dtype of the data, as the reference's core
        functions do (the fp64 upcast of ``no_single_kernel`` belongs to ``fmm``, not to ``compute``).  The
        products ``mmv`` / ``dmmv`` never call this: they do not form the block."""
        from ..mmv_ops.fmm import compute_block

        if kwargs:
            raise NotImplementedError("Distance kernels take no per-row keyword tensors.")
        return compute_block(self, X1, X2, out, diag)

    def dmmv(self, X1, X2, v, w, out=None, opt=None):
        """Same entry as falkon/kernels/diff_kernel.py:127-145: validates, then calls the chosen
        implementation POSITIONALLY as ``(X1, X2, v, w, kernel, out, differentiable, opt)``."""
        X1, X2, v, w, out = self._check_dmmv_dimensions(X1, X2, v, w, out)
        params = self._merged(opt)
        dmmv_impl = self._decide_dmmv_impl(X1, X2, v, w, params)
        diff = torch.is_grad_enabled() and any(
            t.requires_grad for t in [X1, X2, v, w] + list(self.diff_params.values()) if t is not None
        )
        return dmmv_impl(X1, X2, v, w, self, out, diff, params)

    def _sigma_numpy(self) -> np.ndarray:
        return self.sigma.detach().to(device="cpu", dtype=torch.float64).reshape(-1).numpy()


class GaussianKernel(DiffKernel):
    r"""``k(x, x') = exp(-|x - x'|^2 / (2 sigma^2))``; ``sigma`` a scalar or a length-d vector."""

    kernel_name = "gaussian"

    def __init__(self, sigma: Union[float, torch.Tensor], opt: Optional[FalkonOptions] = None):
        sigma = validate_sigma(sigma)
        super().__init__(self.kernel_name, opt, sigma=sigma)

    def _flk_spec(self):
        return _lib.FLK_GAUSSIAN, self._sigma_numpy()

    def detach(self) -> "GaussianKernel":
        return GaussianKernel(self.sigma.detach(), opt=self.params)

    def __repr__(self):
        return f"GaussianKernel(sigma={self.sigma})"

    def __str__(self):
        return f"Gaussian kernel<{self.sigma}>"


class LaplacianKernel(DiffKernel):
    r"""``k(x, x') = exp(-|x - x'| / sigma)``."""

    kernel_name = "laplacian"

    def __init__(self, sigma: Union[float, torch.Tensor], opt: Optional[FalkonOptions] = None):
        sigma = validate_sigma(sigma)
        super().__init__(self.kernel_name, opt, sigma=sigma)

    def _flk_spec(self):
        return _lib.FLK_LAPLACIAN, self._sigma_numpy()

    def detach(self) -> "LaplacianKernel":
        return LaplacianKernel(self.sigma.detach(), opt=self.params)

    def __repr__(self):
        return f"LaplacianKernel(sigma={self.sigma})"

    def __str__(self):
        return f"Laplaciankernel<{self.sigma}>"


class MaternKernel(DiffKernel):
    """Matern kernel for ``nu`` in {0.5, 1.5, 2.5, inf}; 0.5 is the Laplacian and inf the Gaussian
    kernel (falkon/kernels/distance_kernel.py:235-238)."""

    _valid_nu_values = frozenset({0.5, 1.5, 2.5, float("inf")})

    def __init__(self, sigma: Union[float, torch.Tensor], nu: Union[float, torch.Tensor],
                 opt: Optional[FalkonOptions] = None):
        sigma = validate_sigma(sigma)
        nu = self.validate_nu(nu)
        self.kernel_name = f"{nu:.1f}-matern"
        super().__init__(self.kernel_name, opt, sigma=sigma, nu=nu)

    @staticmethod
    def validate_nu(nu: Union[torch.Tensor, float]) -> float:
        if isinstance(nu, torch.Tensor):
            if nu.requires_grad:
                raise ValueError(
                    "The nu parameter of the Matern kernel is not differentiable, and must not require gradients."
                )
            try:
                out_nu = round(nu.item(), ndigits=2)
            except (ValueError, RuntimeError):
                raise ValueError(f"nu={nu} is not convertible to a scalar.") from None
        elif isinstance(nu, float):
            out_nu = round(nu, ndigits=2)
        else:
            raise TypeError(f"nu must be a float or a tensor, not a {type(nu)}")
        if out_nu not in MaternKernel._valid_nu_values:
            raise ValueError(f"The given value of nu = {out_nu} can only take values {MaternKernel._valid_nu_values}.")
        return out_nu

    def _flk_spec(self):
        nu = self.nondiff_params["nu"]
        kid = {0.5: _lib.FLK_LAPLACIAN, 1.5: _lib.FLK_MATERN15, 2.5: _lib.FLK_MATERN25,
               float("inf"): _lib.FLK_GAUSSIAN}[nu]
        return kid, self._sigma_numpy()

    def detach(self) -> "MaternKernel":
        return MaternKernel(self.sigma.detach(), self.nondiff_params["nu"], opt=self.params)

    def __repr__(self):
        return f"MaternKernel(sigma={self.sigma}, nu={self.nondiff_params['nu']:.1f})"

    def __str__(self):
        return f"Matern kernel<{self.sigma}, {self.nondiff_params['nu']:.1f}>"
