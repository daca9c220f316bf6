"""CPU restatement of the rows next to the hot path (test infrastructure only): kernel matrix,
Falkon preconditioner, conjugate gradient and the full fit.

Like falkon_oracle.py this file is the parity checker, never the product: only tests import it.
It restates, with torch CPU operations, what the reference runs with
``FalkonOptions(use_cpu=True, keops_active="no")``:

  * kernel matrix with the fp64 upcast of fp32 data ...... falkon/mmv_ops/fmm.py:298-388, :619-622
  * preconditioner  T = chol(K_MM + eps M I),
    A = chol(T T^T / M + lambda I), triangular solves .... falkon/preconditioner/flk_preconditioner.py:94-299
  * plain conjugate gradient (eps-regularised divisions,
    squared tolerance, full gradient every k iterations) . falkon/optim/conjgrad.py:48-203
  * Falkon operator and right-hand side .................. falkon/optim/conjgrad.py:242-256, :279-307
  * fit: centres by default_rng(seed).choice, alpha = T^-1 A^-1 beta
      ..................................................... falkon/models/falkon.py:205-298, falkon/center_selection.py:187-248

Pinned (tests/test_fit_oracle.py) against tests/golden/fit_*.npz, which hold what the reference's own
``Falkon.fit`` / ``FalkonPreconditioner`` / ``Kernel.__call__`` returned in the build container
(tests/golden/make_golden_fit.py).
"""
from __future__ import annotations

from typing import Callable, Optional

import numpy as np
import torch

from . import falkon_oracle as fo

PC_EPS = {torch.float32: 1e-5, torch.float64: 1e-13}     # falkon/options.py:257-258
CG_EPS = {torch.float32: 1e-7, torch.float64: 1e-15}     # falkon/options.py:223-224
CG_TOL = 1e-7                                            # falkon/options.py:225
CG_FULL_GRAD_EVERY = 10                                  # falkon/options.py:226


def kernel_matrix(x1: torch.Tensor, x2: torch.Tensor, kernel: str, sigma, nu=None, no_single_kernel: bool = True):
    """k(x1, x2) as the reference's fmm returns it: fp32 inputs are evaluated in fp64 and cast back
    when ``no_single_kernel`` (its default) is set (falkon/mmv_ops/fmm.py:619-622, :334-367)."""
    if x1.dtype == torch.float32 and no_single_kernel:
        return fo.kernel_block(x1.double(), x2.double(), kernel, sigma, nu).to(torch.float32)
    return fo.kernel_block(x1, x2, kernel, sigma, nu)


class Preconditioner:
    """T and A of flk_preconditioner.py:94-155 as two upper-triangular matrices."""

    def __init__(self, centres: torch.Tensor, kernel: str, sigma, nu, penalty: float,
                 weights: Optional[torch.Tensor] = None):
        C = kernel_matrix(centres, centres, kernel, sigma, nu)
        M = C.shape[0]
        C.diagonal().add_(PC_EPS[C.dtype] * M)                     # :117
        self.T = torch.linalg.cholesky(C, upper=True)              # :118-124 (T^T T = K_MM)
        TTt = self.T @ self.T.T                                    # LAUUM, :137-143
        if weights is not None:                                    # :131-152
            s = weights.reshape(-1).to(TTt.dtype).sqrt()
            TTt = TTt * s.reshape(-1, 1) * s.reshape(1, -1)
        TTt = TTt / M                                              # :155
        TTt.diagonal().add_(penalty)                               # :157
        self.A = torch.linalg.cholesky(TTt, upper=True)            # :159

    def invA(self, v):
        return torch.linalg.solve_triangular(self.A, v, upper=True)

    def invAt(self, v):
        return torch.linalg.solve_triangular(self.A.T, v, upper=False)

    def invT(self, v):
        return torch.linalg.solve_triangular(self.T, v, upper=True)

    def invTt(self, v):
        return torch.linalg.solve_triangular(self.T.T, v, upper=False)

    def apply(self, v):
        return self.invT(self.invA(v))

    def apply_t(self, v):
        return self.invAt(self.invTt(v))


def conjugate_gradient(B: torch.Tensor, mmv: Callable[[torch.Tensor], torch.Tensor], max_iter: int) -> torch.Tensor:
    """conjgrad.py:98-203 with X0 = None and the default options."""
    R = B.clone()
    X = torch.zeros_like(B)
    eps = CG_EPS[B.dtype]
    tol = CG_TOL ** 2
    P = R.clone()
    Rsold = R.square().sum(dim=0)
    for it in range(max_iter):
        AP = mmv(P)
        alpha = Rsold / (torch.sum(P * AP, dim=0) + eps)
        X = X + P * alpha.reshape(1, -1)
        if (it + 1) % CG_FULL_GRAD_EVERY == 0:
            R = B - mmv(X)
        else:
            R = R - AP * alpha.reshape(1, -1)
        Rsnew = R.square().sum(dim=0)
        if bool(torch.all(Rsnew < tol)):
            break
        Rsold = Rsold + eps   # the reference regularises Rsold in place (Rsold.add_(m_eps))
        P = P * (Rsnew / Rsold).reshape(1, -1) + R
        Rsold = Rsnew
    return X


def falkon_fit(X: torch.Tensor, Y: torch.Tensor, kernel: str, sigma, nu, penalty: float, M: int, maxiter: int,
               seed: int, weights: Optional[torch.Tensor] = None, max_block_elems: int = 64 * 2**20):
    """Returns (alpha, beta, centre indices).  ``weights`` (n x 1) selects re-weighted least squares."""
    n = X.shape[0]
    idx = np.random.default_rng(seed).choice(n, size=M, replace=False)          # center_selection.py:213
    C = X[torch.from_numpy(idx)]
    pc = Preconditioner(C, kernel, sigma, nu, penalty, weights=None if weights is None else weights[idx])
    y_over_n = Y / n
    if weights is not None:
        y_over_n = y_over_n * weights
    B = fo.fmmv(C, X, y_over_n, kernel, sigma, nu, max_block_elems=max_block_elems)   # conjgrad.py:296
    B = pc.apply_t(B)                                                                 # :297

    def mmv(sol):                                                                     # :242-256
        v = pc.invA(sol)
        v_t = pc.invT(v)
        if weights is None:
            cc = fo.fdmmv(X, C, v_t, None, kernel, sigma, nu, max_block_elems=max_block_elems)
        else:                                                                         # :258-273
            cc = fo.fmmv(X, C, v_t, kernel, sigma, nu, max_block_elems=max_block_elems) * weights
            cc = fo.fmmv(C, X, cc, kernel, sigma, nu, max_block_elems=max_block_elems)
        return pc.invAt(pc.invTt(cc / n) + penalty * v)

    beta = conjugate_gradient(B, mmv, maxiter)
    return pc.apply(beta), beta, idx


def krr_gradient_norm(X, Y, C, alpha, kernel: str, sigma, nu, penalty: float, weights=None,
                      max_block_elems: int = 64 * 2**20) -> float:
    """How well ``alpha`` solves the Nystrom ridge problem, as a backward error evaluated in fp64:

        || K_mn W (K_nm alpha - Y) / n + penalty K_mm alpha ||  /  || K_mn W Y / n ||

    (the gradient of the objective the fit minimises, falkon/models/falkon.py:34-60, relative to its value at
    alpha = 0).  Unlike alpha itself this is not amplified by the conditioning of the preconditioner's factors, so
    two fp32 solvers of equal quality give comparable values."""
    X, Y, C, alpha = (t.double() for t in (X, Y, C, alpha))
    n = X.shape[0]
    w = None if weights is None else weights.double()
    resid = fo.fmmv(X, C, alpha, kernel, sigma, nu, max_block_elems=max_block_elems) - Y
    y0 = Y
    if w is not None:
        resid, y0 = resid * w, Y * w
    g = fo.fmmv(C, X, resid / n, kernel, sigma, nu, max_block_elems=max_block_elems)
    g = g + penalty * (kernel_matrix(C, C, kernel, sigma, nu) @ alpha)
    g0 = fo.fmmv(C, X, y0 / n, kernel, sigma, nu, max_block_elems=max_block_elems)
    return float(g.norm() / g0.norm())
