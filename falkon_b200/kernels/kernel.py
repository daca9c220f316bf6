"""Operator API: the abstract ``Kernel`` with ``mmv`` / ``dmmv``.

Mirrors the public surface of the reference's ``Kernel`` (falkon/kernels/kernel.py:14-577) on the
kernel-vector-product path: argument validation and error types (:43-105), per-call option
merging (:283-285), and the implementation-choice hooks ``_decide_mmv_impl`` /
``_decide_dmmv_impl`` (:298-334, :419-459) through which a backend is plugged in.  The hooks here
return the CUDA-backed :func:`falkon_b200.mmv_ops.fmmv` / :func:`fdmmv`.
"""
from abc import ABC, abstractmethod
from typing import Dict, Optional

import torch

from ..mmv_ops.fmm import fmm
from ..mmv_ops.fmmv import fdmmv, fmmv
from ..options import FalkonOptions, merge_options


def _same_dtype(*tensors) -> bool:
    dts = {t.dtype for t in tensors if t is not None}
    return len(dts) <= 1


def _same_device(*tensors) -> bool:
    devs = {t.device for t in tensors if t is not None}
    return len(devs) <= 1


class Kernel(torch.nn.Module, ABC):
    """Abstract kernel.  ``name`` is a short label, ``opt`` the base options of every operation."""

    def __init__(self, name: str, opt: Optional[FalkonOptions]):
        super().__init__()
        self.name = name
        if opt is None:
            opt = FalkonOptions()
        self.params: FalkonOptions = opt

    # ---- validation (falkon/kernels/kernel.py:43-105) ----
    @staticmethod
    def _check_dmmv_dimensions(X1, X2, v, w, out):
        if v is None and w is None:
            raise ValueError("One of v and w must be specified to run fdMMV.")
        if X1.dim() != 2:
            raise ValueError("Matrix X1 must be 2D.")
        if X2.dim() != 2:
            raise ValueError("Matrix X2 must be 2D.")
        if v is not None and v.dim() == 1:
            v = v.reshape((-1, 1))
        if v is not None and v.dim() != 2:
            raise ValueError(f"v must be a vector or a 2D matrix. Found {len(v.shape)}D.")
        if w is not None and w.dim() == 1:
            w = w.reshape((-1, 1))
        if w is not None and w.dim() != 2:
            raise ValueError(f"w must be a vector or a 2D matrix. Found {len(w.shape)}D.")
        T = v.size(1) if v is not None else w.size(1)
        M = X2.size(0)
        if out is not None and out.shape != (M, T):
            raise ValueError(f"Output dimension is incorrect. Expected ({M}, {T}) found {out.shape}")
        if v is not None and v.shape != (M, T):
            raise ValueError(f"Dimensions of matrix v are incorrect: Expected ({M}, {T}) found {v.shape}")
        if w is not None and w.shape != (X1.size(0), T):
            raise ValueError(f"Dimensions of matrix w are incorrect: Expected ({X1.size(0)}, {T}) found {w.shape}")
        if X1.size(1) != X2.size(1):
            raise ValueError(f"X1 and X2 must have the same number of features ({X1.size(1)} vs {X2.size(1)}).")
        if not _same_dtype(X1, X2, v, w, out):
            raise TypeError("Data types of input matrices must be equal.")
        return X1, X2, v, w, out

    @staticmethod
    def _check_mmv_dimensions(X1, X2, v, out):
        if X1.dim() != 2:
            raise ValueError("Matrix X1 must be 2D.")
        if X2.dim() != 2:
            raise ValueError("Matrix X2 must be 2D.")
        if v.dim() == 1:
            v = v.reshape((-1, 1))
        if v.dim() != 2:
            raise ValueError(f"v must be a vector or a 2D matrix. Found {len(v.shape)}D.")
        if out is not None and out.shape != (X1.size(0), v.size(1)):
            raise ValueError(f"Output dimension is incorrect. Expected ({X1.size(0)}, {v.size(1)}) found {out.shape}")
        if v.shape != (X2.size(0), v.size(1)):
            raise ValueError(
                f"Dimensions of matrix v are incorrect: Expected ({X2.size(0)}, {v.size(1)}) found {v.shape}"
            )
        if X1.size(1) != X2.size(1):
            raise ValueError(f"X1 and X2 must have the same number of features ({X1.size(1)} vs {X2.size(1)}).")
        if not _same_dtype(X1, X2, v, out):
            raise TypeError("Data types of input matrices must be equal.")
        return X1, X2, v, out

    @staticmethod
    def _check_device_properties(*args, fn_name: str, opt: FalkonOptions):
        if not _same_device(*args):
            raise RuntimeError(f"All input arguments to {fn_name} must be on the same device")

    def _merged(self, opt: Optional[FalkonOptions]) -> FalkonOptions:
        return merge_options(self.params, opt)

    # ---- the kernel matrix itself (falkon/kernels/kernel.py:135-193) ----
    @staticmethod
    def _check_mm_dimensions(X1, X2, diag, out):
        if X1.dim() != 2:
            raise ValueError("Matrix X1 must be 2D.")
        if X2.dim() != 2:
            raise ValueError("Matrix X2 must be 2D.")
        N, M = X1.size(0), X2.size(0)
        if X1.size(1) != X2.size(1):
            raise ValueError(f"X1 and X2 must have the same number of features ({X1.size(1)} vs {X2.size(1)}).")
        if diag:
            if N != M:
                raise ValueError(f"With diag=True X1 and X2 must have the same number of rows ({N} vs {M}).")
            if out is not None and out.shape != (N,):
                raise ValueError(f"Output dimension is incorrect. Expected ({N},) found {tuple(out.shape)}")
        elif out is not None and out.shape != (N, M):
            raise ValueError(f"Output dimension is incorrect. Expected ({N}, {M}) found {tuple(out.shape)}")
        if not _same_dtype(X1, X2, out):
            raise TypeError("Data types of input matrices must be equal.")
        return X1, X2, out

    def __call__(self, X1, X2, diag: bool = False, out=None, opt=None, kwargs_m1=None, kwargs_m2=None):
        """``k(X1, X2)``: X1 (N x D), X2 (M x D) -> (N x M), or the diagonal (N,) with ``diag=True``.
        ``out`` is written in place when given.  Signature of falkon/kernels/kernel.py:135-193."""
        X1, X2, out = self._check_mm_dimensions(X1, X2, diag, out)
        params = self._merged(opt)
        mm_impl = self._decide_mm_impl(X1, X2, diag, params)
        return mm_impl(kernel=self, opt=params, out=out, diag=diag, X1=X1, X2=X2, kwargs_m1=kwargs_m1,
                       kwargs_m2=kwargs_m2)

    def _decide_mm_impl(self, X1, X2, diag: bool, opt: FalkonOptions):
        return fmm

    # ---- K v ----
    def mmv(
        self,
        X1: torch.Tensor,
        X2: torch.Tensor,
        v: torch.Tensor,
        out: Optional[torch.Tensor] = None,
        opt: Optional[FalkonOptions] = None,
        kwargs_m1: Optional[Dict[str, torch.Tensor]] = None,
        kwargs_m2: Optional[Dict[str, torch.Tensor]] = None,
    ):
        """``k(X1, X2) @ v``: X1 (N x D), X2 (M x D), v (M x T) or (M,) -> (N x T).
        ``out`` is written in place when given.  Signature of falkon/kernels/kernel.py:226-296."""
        X1, X2, v, out = self._check_mmv_dimensions(X1, X2, v, out)
        params = self._merged(opt)
        mmv_impl = self._decide_mmv_impl(X1, X2, v, params)
        return mmv_impl(X1=X1, X2=X2, v=v, kernel=self, out=out, opt=params, kwargs_m1=kwargs_m1, kwargs_m2=kwargs_m2)

    def _decide_mmv_impl(self, X1, X2, v, opt: FalkonOptions):
        return fmmv

    # ---- K^T (K v + w) ----
    def dmmv(
        self,
        X1: torch.Tensor,
        X2: torch.Tensor,
        v: Optional[torch.Tensor],
        w: Optional[torch.Tensor],
        out: Optional[torch.Tensor] = None,
        opt: Optional[FalkonOptions] = None,
        kwargs_m1: Optional[Dict[str, torch.Tensor]] = None,
        kwargs_m2: Optional[Dict[str, torch.Tensor]] = None,
    ):
        """``k(X1, X2)^T (k(X1, X2) v + w)``: v (M x T) or None, w (N x T) or None -> (M x T).
        Signature of falkon/kernels/kernel.py:336-417."""
        X1, X2, v, w, out = self._check_dmmv_dimensions(X1, X2, v, w, out)
        params = self._merged(opt)
        dmmv_impl = self._decide_dmmv_impl(X1, X2, v, w, params)
        return dmmv_impl(
            X1=X1, X2=X2, v=v, w=w, kernel=self, out=out, differentiable=False, opt=params,
            kwargs_m1=kwargs_m1, kwargs_m2=kwargs_m2,
        )

    def _decide_dmmv_impl(self, X1, X2, v, w, opt: FalkonOptions):
        return fdmmv

    @abstractmethod
    def compute(self, X1: torch.Tensor, X2: torch.Tensor, out: torch.Tensor, diag: bool, **kwargs) -> torch.Tensor:
        """Dense kernel block (the reference's extension point, falkon/kernels/kernel.py:462-505).
        Not used by the CUDA products; concrete kernels may leave it unimplemented."""

    def extra_mem(self, is_differentiable, is_sparse, dtype, density1=None, density2=None) -> Dict[str, float]:
        """Extra memory per block in the reference's block-size model (falkon/kernels/kernel.py:542).
        Nothing n x m is ever allocated here."""
        return {}

    def __str__(self):
        return f"<{self.name} kernel>"
