"""Conjugate-gradient solvers around the kernel-vector products.

``ConjugateGradient.solve`` is the plain multi-right-hand-side CG of falkon/optim/conjgrad.py:48-203
(same recurrences, the same ``cg_epsilon`` regularisation of the two divisions, the same squared
tolerance test, the full-gradient refresh every ``cg_full_gradient_every`` iterations and optional
per-column "differential" convergence).  ``FalkonConjugateGradient`` wraps it with the Falkon
operator  beta -> A^-T (T^-T (K_nm^T K_nm T^-1 A^-1 beta / n) + lambda A^-1 beta)
(conjgrad.py:242-256) whose middle term is ONE ``dmmv`` call per iteration -- the hot path of this
package.

All vectors live on the GPU for the whole solve.  Per iteration the host reads one scalar (the
"all columns converged" flag, as the reference does); nothing else synchronises.  ``kernel`` may be
a kernel object or a ``ShardedKernelOps``: with row shards the right-hand side and every dmmv are
all-reduced over the process group and ``n`` is the global number of rows.
"""
import functools
import time
from typing import Callable, List, Optional

import torch

from ..options import ConjugateGradientOptions, FalkonOptions

__all__ = ("Optimizer", "ConjugateGradient", "FalkonConjugateGradient", "StopOptimizationException")


class StopOptimizationException(Exception):
    def __init__(self, message):
        super().__init__()
        self.message = message


class Optimizer:
    """Base class of the solvers (an empty shell, as in the reference)."""

    def __init__(self):
        pass


class ConjugateGradient(Optimizer):
    def __init__(self, opt: Optional[ConjugateGradientOptions] = None):
        super().__init__()
        self.params = opt or ConjugateGradientOptions()
        self.num_iter = None

    def solve(
        self,
        X0: Optional[torch.Tensor],
        B: torch.Tensor,
        mmv: Callable[[torch.Tensor], torch.Tensor],
        max_iter: int,
        callback: Optional[Callable[[int, torch.Tensor, float], None]] = None,
    ) -> torch.Tensor:
        """Solves A X = B for X (n x t) given only ``mmv(V) = A V``.

        ``callback(iteration, X, elapsed_seconds)`` runs after every iteration and may raise
        ``StopOptimizationException`` to stop early.
        """
        t_start = time.time()
        if X0 is None:
            R = B.clone()
            X = torch.zeros_like(B)
        else:
            R = B - mmv(X0)
            X = X0
        eps = self.params.cg_epsilon(X.dtype)
        full_grad_every = self.params.cg_full_gradient_every or max_iter * 2
        tol = self.params.cg_tolerance ** 2
        diff_conv = self.params.cg_differential_convergence and X.shape[1] > 1

        P = R.clone()
        Rsold = R.square().sum(dim=0)
        e_train = time.time() - t_start

        x_done: List[torch.Tensor] = []   # converged columns, in the order they converged
        idx_done: List[int] = []          # their original column indices
        idx_live = torch.arange(X.shape[1])
        X_orig = X

        for self.num_iter in range(max_iter):
            t_start = time.time()
            AP = mmv(P)
            alpha = Rsold / (torch.sum(P * AP, dim=0).add_(eps))
            X.addcmul_(P, alpha.reshape(1, -1))
            if (self.num_iter + 1) % full_grad_every == 0:
                R = B - mmv(X)
            else:
                R.addcmul_(AP, alpha.reshape(1, -1), value=-1.0)
            Rsnew = R.square().sum(dim=0)
            converged = torch.less(Rsnew, tol)
            if bool(torch.all(converged)):
                break
            if diff_conv and bool(torch.any(converged)):
                conv_cpu = converged.cpu()
                for i in torch.where(conv_cpu)[0].tolist():
                    idx_done.append(int(idx_live[i]))
                    x_done.append(X[:, i].clone())
                keep = ~converged
                idx_live = idx_live[~conv_cpu]
                P, R, B, X = P[:, keep], R[:, keep], B[:, keep], X[:, keep]
                Rsnew, Rsold = Rsnew[keep], Rsold[keep]
            P = P.mul_((Rsnew / Rsold.add_(eps)).reshape(1, -1)).add_(R)
            Rsold = Rsnew
            e_train += time.time() - t_start
            if callback is not None:
                try:
                    callback(self.num_iter + 1, X, e_train)
                except StopOptimizationException as e:
                    print(f"Optimization stopped from callback: {e.message}")
                    break
        if diff_conv:
            for col, j in zip(x_done, idx_done):
                X_orig[:, j].copy_(col)
            for i, j in enumerate(idx_live.tolist()):
                if X_orig[:, j].data_ptr() != X[:, i].data_ptr():
                    X_orig[:, j].copy_(X[:, i])
            X = X_orig
        return X


class FalkonConjugateGradient(Optimizer):
    r"""Preconditioned CG for the Nystrom KRR system
    :math:`\tilde B^\top H \tilde B \beta = \tilde B^\top K_{nm}^\top Y`, :math:`H = K_{nm}^\top K_{nm} + \lambda n K_{mm}`
    (falkon/optim/conjgrad.py:206-330).

    Parameters
    ----------
    kernel
        Kernel object (``mmv`` / ``dmmv``), or a ``falkon_b200.sharded.ShardedKernelOps`` when every
        process holds a row shard of X and Y.
    preconditioner
        An initialised ``FalkonPreconditioner`` built on the same centres.
    opt
        Options for the CG solver and the kernel products.
    weight_fn
        Optional ``weight_fn(Y, X, indices) -> (n x 1) weights`` for re-weighted least squares.
    """

    def __init__(self, kernel, preconditioner, opt: Optional[FalkonOptions] = None, weight_fn=None):
        super().__init__()
        self.kernel = kernel
        self.preconditioner = preconditioner
        self.params = opt or FalkonOptions()
        self.optimizer = ConjugateGradient(self.params.get_conjgrad_options())
        self.weight_fn = weight_fn

    @property
    def is_weighted(self) -> bool:
        return self.weight_fn is not None

    # K(M, X) y summed over all rows of X: one all-reduced product when the rows are sharded
    def _mmv_t(self, M, X, y):
        if hasattr(self.kernel, "mmv_t"):
            return self.kernel.mmv_t(M, X, y)
        return self.kernel.mmv(M, X, y, opt=self.params)

    def _dmmv(self, X, M, v):
        if hasattr(self.kernel, "mmv_t"):  # sharded ops: kernel options are bound inside
            return self.kernel.dmmv(X, M, v, None)
        return self.kernel.dmmv(X, M, v, None, opt=self.params)

    def falkon_mmv(self, sol, penalty, X, M, n: int):
        prec = self.preconditioner
        v = prec.invA(sol)
        v_t = prec.invT(v)
        cc = self._dmmv(X, M, v_t)
        # A^-T (T^-T (cc / n) + penalty * v)
        cc_ = prec.invTt(cc.div_(n)).add_(v.mul_(penalty))
        return prec.invAt(cc_)

    def weighted_falkon_mmv(self, sol, penalty, X, M, y_weights, n: int):
        prec = self.preconditioner
        v = prec.invA(sol)
        v_t = prec.invT(v)
        if hasattr(self.kernel, "mmv_t"):
            cc = self.kernel.mmv(X, M, v_t).mul_(y_weights)
        else:
            cc = self.kernel.mmv(X, M, v_t, opt=self.params).mul_(y_weights)
        cc = self._mmv_t(M, X, cc)
        cc_ = prec.invTt(cc.div_(n)).add_(v.mul_(penalty))
        return prec.invAt(cc_)

    def solve(self, X, M, Y, _lambda, initial_solution, max_iter, callback=None, n: Optional[int] = None):
        """Returns beta, the solution in the preconditioned space (alpha = preconditioner.apply(beta)).
        ``n`` defaults to the number of rows of ``Y``; pass the global row count when X, Y are shards."""
        if n is None:
            n = Y.size(0)
        y_over_n = Y / n
        y_weights = None
        if self.is_weighted:
            y_weights = self.weight_fn(Y, X, torch.arange(Y.shape[0]))
            y_over_n.mul_(y_weights)
        B = self._mmv_t(M, X, y_over_n)
        B = self.preconditioner.apply_t(B)
        if self.is_weighted:
            mmv = functools.partial(self.weighted_falkon_mmv, penalty=_lambda, X=X, M=M, y_weights=y_weights, n=n)
        else:
            mmv = functools.partial(self.falkon_mmv, penalty=_lambda, X=X, M=M, n=n)
        return self.optimizer.solve(initial_solution, B, mmv, max_iter, callback)

    def solve_val_rhs(self, Xtr, Xval, M, Y, _lambda, initial_solution, max_iter, callback=None):
        """Same system with the right-hand side built from a validation set (conjgrad.py:309-326)."""
        n = Xtr.size(0)
        B = self._mmv_t(M, Xval, Y / n)
        B = self.preconditioner.apply_t(B)
        mmv = functools.partial(self.falkon_mmv, penalty=_lambda, X=Xtr, M=M, n=n)
        return self.optimizer.solve(initial_solution, B, mmv, max_iter, callback)
