"""CPU restatement of Falkon's blocked kernel-vector products (test infrastructure only).

This module is the parity oracle for the CUDA path: a plain CPU restatement, in torch CPU
tensor operations, of the algorithm the reference runs for ``fmmv`` / ``fdmmv`` with
``FalkonOptions(use_cpu=True, keops_active="no")``.  It is *not* part of the product: only the
test-suite, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py``
import it.  The product path (``falkon_b200``) never imports this file and has no CPU fallback.

Why torch CPU ops and not numpy: the reference *is* a sequence of torch CPU ops on this path
(``torch.addmm`` -> MKL/OpenBLAS GEMM, in-place ATen element-wise passes, a row-norm reduction),
so restating it with the same primitives reproduces the same rounding behaviour (fp32 GEMM and
fp32 element-wise passes) and the same multi-threaded CPU cost, which is what the timed CPU
baseline must represent.  An independent numpy/fp64 dense evaluation (`dense_kernel_fp64`) that
uses explicit differences instead of the norm expansion is provided next to it for small cases.

Parity pinning: this restatement is checked (tests/test_oracle.py) against outputs of the
reference itself, generated in the build container by tests/golden/make_golden.py from the
reference's own ``Kernel.mmv`` / ``Kernel.dmmv`` and stored under tests/golden/*.npz, on the
shapes, seeds and distributions of the reference's tests (falkon/tests/test_kernels.py:32-71,
:529-591) and on reduced versions of the benchmark configurations.

Reference citations (paths inside the reference project):
  * squared distances by norm expansion, clamp at 1e-20 ... falkon/kernels/distance_kernel.py:88-101
  * Gaussian core ........................................ falkon/kernels/distance_kernel.py:140-159
  * Laplacian core ....................................... falkon/kernels/distance_kernel.py:182-204
  * Matern core (nu = 0.5, 1.5, 2.5, inf) ................ falkon/kernels/distance_kernel.py:228-271
  * row-wise squared norm ................................ falkon/c_ext/ops/cpu/cpu_square_norm.cpp:13-53
  * blocked K v  (loop over row and column blocks) ....... falkon/mmv_ops/fmmv.py:309-402
  * blocked K^T (K v + w) (loop over row blocks) ......... falkon/mmv_ops/fmmv.py:683-767
"""
from __future__ import annotations

import math
from typing import Optional, Union

import numpy as np
import torch

SQRT3 = math.sqrt(3.0)
SQRT5 = math.sqrt(5.0)

KERNEL_NAMES = ("gaussian", "laplacian", "matern")


def _as_sigma(sigma: Union[float, torch.Tensor, np.ndarray], like: torch.Tensor) -> torch.Tensor:
    """Length-scale as a tensor of the data's dtype, shape [1] or [d].

    The reference stores sigma as an fp64 parameter and casts it to the data dtype at every
    call (falkon/kernels/distance_kernel.py:20-38, :148).
    """
    if not isinstance(sigma, torch.Tensor):
        sigma = torch.as_tensor(np.atleast_1d(np.asarray(sigma, dtype=np.float64)))
    sigma = sigma.detach().reshape(-1)
    if sigma.numel() not in (1, like.shape[1]):
        raise ValueError("sigma must have 1 or d entries")
    return sigma.to(dtype=like.dtype)


def square_norm_rows(x: torch.Tensor) -> torch.Tensor:
    """Row-wise sum of squares, accumulated in the input dtype, shape [n, 1].

    Restates ``falkon::square_norm(x, -1, keepdim=True)``
    (falkon/c_ext/ops/cpu/cpu_square_norm.cpp:13-53).
    """
    return (x * x).sum(dim=1, keepdim=True)


def sq_dist_block(a: torch.Tensor, b: torch.Tensor, an: torch.Tensor, bn: torch.Tensor) -> torch.Tensor:
    """``clamp_min(|a_i|^2 - 2 a_i.b_j + |b_j|^2, 1e-20)`` for all (i, j).

    Same operation order as falkon/kernels/distance_kernel.py:88-101: a GEMM with
    ``alpha=-2, beta=1`` on the row norms, then the column norms are added, then the clamp.
    """
    blk = torch.addmm(an, a, b.t(), alpha=-2.0, beta=1.0)
    blk.add_(bn.t())
    blk.clamp_min_(1e-20)
    return blk


def kernel_block(
    x1: torch.Tensor,
    x2: torch.Tensor,
    kernel: str,
    sigma: Union[float, torch.Tensor],
    nu: Optional[float] = None,
) -> torch.Tensor:
    """Dense kernel block k(x1, x2) computed the way the reference computes it.

    ``kernel`` is "gaussian", "laplacian" or "matern" (with ``nu`` in {0.5, 1.5, 2.5, inf}).
    Follows rbf_core / laplacian_core / matern_core
    (falkon/kernels/distance_kernel.py:140-159, :182-204, :228-271): inputs are divided by
    sigma first, norms are taken of the scaled inputs, and the element-wise epilogue runs in
    the data dtype.
    """
    if kernel not in KERNEL_NAMES:
        raise ValueError(f"unknown kernel {kernel!r}")
    if kernel == "matern":
        if nu is None:
            raise ValueError("matern needs nu")
        if nu == 0.5:
            kernel = "laplacian"
        elif nu == float("inf"):
            kernel = "gaussian"
        elif nu not in (1.5, 2.5):
            raise ValueError("nu must be one of 0.5, 1.5, 2.5, inf")
    s = _as_sigma(sigma, x1)
    a = x1 / s
    b = x2 / s
    d2 = sq_dist_block(a, b, square_norm_rows(a), square_norm_rows(b))
    if kernel == "gaussian":
        d2.mul_(-0.5)
        d2.exp_()
        return d2
    if kernel == "laplacian":
        d2.sqrt_()
        d2.neg_()
        d2.exp_()
        return d2
    if nu == 1.5:
        d2.sqrt_()
        d2.mul_(SQRT3)
        e = torch.neg(d2)
        e.exp_()
        d2.add_(1.0).mul_(e)
        return d2
    # nu == 2.5
    r = torch.sqrt(d2)
    r.mul_(SQRT5)
    d2.mul_(5.0 / 3.0).add_(r).add_(1.0)
    r.neg_().exp_()
    d2.mul_(r)
    return d2


def _rows_per_block(n: int, m: int, d: int, t: int, max_block_elems: Optional[int]) -> int:
    """Row-block length such that the n_blk x m kernel block plus its side buffers fit a budget.

    The reference sizes the block from a byte budget (falkon/mmv_ops/fmmv.py:488-544); the
    block length only changes the order of floating-point accumulation across blocks.
    """
    if max_block_elems is None:
        return n
    per_row = m + t + 2 * d + 2
    return int(max(1, min(n, max_block_elems // per_row)))


def _as_2d(v: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if v is not None and v.dim() == 1:
        return v.reshape(-1, 1)
    return v


def fmmv(
    x1: torch.Tensor,
    x2: torch.Tensor,
    v: torch.Tensor,
    kernel: str,
    sigma: Union[float, torch.Tensor],
    nu: Optional[float] = None,
    max_block_elems: Optional[int] = 64 * 2**20,
) -> torch.Tensor:
    """``k(x1, x2) @ v`` evaluated block by block over the rows of ``x1``; result [n, t].

    Restates the loop of mmv_run_thread (falkon/mmv_ops/fmmv.py:358-391): for every row block
    the kernel block is formed and multiplied into the output rows.  (The reference may also
    split the columns; that changes only the accumulation order.)
    """
    v = _as_2d(v)
    n, d = x1.shape
    m, t = v.shape
    if x2.shape != (m, d):
        raise ValueError("shape mismatch between x2 and v")
    out = torch.zeros(n, t, dtype=x1.dtype)
    blk = _rows_per_block(n, m, d, t, max_block_elems)
    for i in range(0, n, blk):
        kb = kernel_block(x1[i : i + blk], x2, kernel, sigma, nu)
        out[i : i + blk].addmm_(kb, v)
    return out


def fdmmv(
    x1: torch.Tensor,
    x2: torch.Tensor,
    v: Optional[torch.Tensor],
    w: Optional[torch.Tensor],
    kernel: str,
    sigma: Union[float, torch.Tensor],
    nu: Optional[float] = None,
    max_block_elems: Optional[int] = 64 * 2**20,
) -> torch.Tensor:
    """``k(x1, x2)^T (k(x1, x2) v + w)`` block by block over the rows of ``x1``; result [m, t].

    Restates dmmv_run_thread (falkon/mmv_ops/fmmv.py:740-760): per row block
    ``u = w_blk + K v`` then ``out += K^T u``.  ``w=None`` means a zero ``w``; ``v=None`` means
    ``out = K^T w`` (the operator-level contract, falkon/kernels/kernel.py:350-353).
    """
    v = _as_2d(v)
    w = _as_2d(w)
    if v is None and w is None:
        raise ValueError("One of v and w must be specified")
    n, d = x1.shape
    m = x2.shape[0]
    t = v.shape[1] if v is not None else w.shape[1]
    out = torch.zeros(m, t, dtype=x1.dtype)
    blk = _rows_per_block(n, m, d, t, max_block_elems)
    for i in range(0, n, blk):
        kb = kernel_block(x1[i : i + blk], x2, kernel, sigma, nu)
        if w is not None:
            u = w[i : i + blk].clone()
        else:
            u = torch.zeros(kb.shape[0], t, dtype=x1.dtype)
        if v is not None:
            u.addmm_(kb, v)
        out.addmm_(kb.t(), u)
    return out


def dense_kernel_fp64(
    x1: np.ndarray,
    x2: np.ndarray,
    kernel: str,
    sigma: Union[float, np.ndarray],
    nu: Optional[float] = None,
) -> np.ndarray:
    """Independent fp64 evaluation by explicit differences (no norm expansion, no clamp).

    Plays the role of the reference's naive test kernels (falkon/tests/naive_kernels.py:23-61):
    the mathematical definition, used as ground truth on small shapes.
    """
    a = np.asarray(x1, dtype=np.float64) / np.asarray(sigma, dtype=np.float64)
    b = np.asarray(x2, dtype=np.float64) / np.asarray(sigma, dtype=np.float64)
    d2 = np.zeros((a.shape[0], b.shape[0]))
    for k in range(a.shape[1]):
        diff = a[:, k][:, None] - b[:, k][None, :]
        d2 += diff * diff
    if kernel == "matern":
        if nu == 0.5:
            kernel = "laplacian"
        elif nu == float("inf"):
            kernel = "gaussian"
    if kernel == "gaussian":
        return np.exp(-0.5 * d2)
    r = np.sqrt(d2)
    if kernel == "laplacian":
        return np.exp(-r)
    if nu == 1.5:
        s = SQRT3 * r
        return (1.0 + s) * np.exp(-s)
    if nu == 2.5:
        s = SQRT5 * r
        return (1.0 + s + s * s / 3.0) * np.exp(-s)
    raise ValueError("unsupported kernel / nu")


def dense_fmmv_fp64(x1, x2, v, kernel, sigma, nu=None) -> np.ndarray:
    """fp64 ``K v`` from the explicit-difference kernel."""
    v = np.asarray(v, dtype=np.float64)
    if v.ndim == 1:
        v = v[:, None]
    return dense_kernel_fp64(x1, x2, kernel, sigma, nu) @ v


def dense_fdmmv_fp64(x1, x2, v, w, kernel, sigma, nu=None) -> np.ndarray:
    """fp64 ``K^T (K v + w)`` from the explicit-difference kernel."""
    k = dense_kernel_fp64(x1, x2, kernel, sigma, nu)
    t = (np.asarray(v).reshape(len(x2), -1) if v is not None else np.asarray(w).reshape(len(x1), -1)).shape[1]
    u = np.zeros((k.shape[0], t))
    if v is not None:
        u += k @ np.asarray(v, dtype=np.float64).reshape(k.shape[1], -1)
    if w is not None:
        u += np.asarray(w, dtype=np.float64).reshape(k.shape[0], -1)
    return k.T @ u


def rel_l2(a, b) -> float:
    """Relative L2 error ``|a - b| / |b|`` in fp64 (the parity measure of the benchmark spec)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / (den if den > 0 else 1.0))
