"""Conjugate-gradient solvers around the kernel-vector products, laid out for a device that never waits for the host.

Public surface of falkon/optim/conjgrad.py (``ConjugateGradient(opt).solve(X0, B, mmv, max_iter, callback)``,
``FalkonConjugateGradient(kernel, preconditioner, opt, weight_fn).solve(...)`` / ``solve_val_rhs(...)``,
``StopOptimizationException``), and its arithmetic: the standard CG recurrences with ``cg_epsilon`` added to both
denominators, the squared-tolerance test on the residual norms, a recomputed residual every
``cg_full_gradient_every`` iterations, optional per-column ("differential") convergence
(falkon/optim/conjgrad.py:95-186).

What is different is where the control flow lives.  The reference decides on the host, every iteration, whether to
stop (``if torch.all(converged)``), which forces a device synchronisation per iteration.  Here one iteration is a
FIXED sequence of launches -- the operator (two triangular solves, one ``dmmv``, two triangular solves), four
reductions and a handful of fused element-wise updates -- with every decision carried as data on the device:

* ``state.live``   (t,) 0/1 per column: columns that still move.  A column that met the tolerance is frozen when
  differential convergence is on; all columns are frozen from the iteration in which every one of them has met it
  (the reference's ``break``).  A frozen column has step lengths of exactly zero, so the iterate the caller gets is
  the one the reference would have returned at that iteration.
* ``state.iterations`` device counter of the iterations that did move something (``num_iter`` is read from it once,
  at the end).

The host looks at the "all frozen" flag only every ``cg_full_gradient_every`` iterations (to leave early), and not at
all when that option is 0.  A user callback, when given, is called after every iteration as in the reference; whether it
synchronises is its own business.
"""
import dataclasses
import time
from typing import Callable, Optional

import torch

from ..options import ConjugateGradientOptions, FalkonOptions

__all__ = ("Optimizer", "ConjugateGradient", "FalkonConjugateGradient", "StopOptimizationException")


class StopOptimizationException(Exception):
    def __init__(self, message):
        super().__init__()
        self.message = message


class Optimizer:
    """Base class of the solvers."""


@dataclasses.dataclass
class _CgState:
    """Everything one iteration reads and writes; all tensors live on the solve's device."""

    x: torch.Tensor          # (m, t) iterate
    r: torch.Tensor          # (m, t) residual
    p: torch.Tensor          # (m, t) search direction
    rho: torch.Tensor        # (t,) squared residual norms
    live: torch.Tensor       # (t,) 1.0 while the column still moves, else 0.0
    iterations: torch.Tensor  # () int64: iterations in which at least one column moved


def _cg_iteration(state: _CgState, b: torch.Tensor, apply_a: Callable, eps: float, tol_sq: float,
                  refresh_residual: bool, per_column_stop: bool) -> None:
    """One CG iteration, in place, with no host decision: frozen columns (live == 0) get zero step lengths."""
    ap = apply_a(state.p)
    state.iterations += (state.live.max() > 0).to(torch.int64)
    # step length per column; zero for frozen columns
    alpha = state.rho / ((state.p * ap).sum(dim=0) + eps) * state.live
    state.x.addcmul_(state.p, alpha.unsqueeze(0))
    if refresh_residual:
        fresh = b - apply_a(state.x)
        state.r = torch.where(state.live.unsqueeze(0) > 0, fresh, state.r)
    else:
        state.r.addcmul_(ap, alpha.unsqueeze(0), value=-1.0)
    rho_new = state.r.square().sum(dim=0)
    met = (rho_new < tol_sq).to(state.live.dtype)
    # the reference leaves its loop when every column has met the tolerance, BEFORE updating the direction
    all_met = met.min()
    live_next = state.live * (1.0 - all_met)
    if per_column_stop:
        live_next = live_next * (1.0 - met)
    beta = rho_new / (state.rho + eps) * live_next
    # p <- beta p + r for the columns that go on; frozen columns keep a direction that is never used again
    state.p = torch.where(live_next.unsqueeze(0) > 0, state.p * beta.unsqueeze(0) + state.r, state.p)
    state.rho = torch.where(state.live > 0, rho_new, state.rho)
    state.live = live_next


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
        """Solves A X = B for X (m x t) given only ``mmv(V) = A V``.

        ``callback(iteration, X, elapsed_seconds)`` runs after every iteration and may raise
        ``StopOptimizationException`` to stop early.  ``self.num_iter`` afterwards holds the index of the last
        iteration that changed the iterate (the reference's loop variable at exit).
        """
        t_begin = time.time()
        eps = self.params.cg_epsilon(B.dtype)
        tol_sq = self.params.cg_tolerance ** 2
        refresh_every = self.params.cg_full_gradient_every or 0
        per_column = bool(self.params.cg_differential_convergence) and B.shape[1] > 1
        if X0 is None:
            x, r = torch.zeros_like(B), B.clone()
        else:
            x, r = X0, B - mmv(X0)
        state = _CgState(x=x, r=r, p=r.clone(), rho=r.square().sum(dim=0),
                         live=torch.ones(B.shape[1], dtype=B.dtype, device=B.device),
                         iterations=torch.zeros((), dtype=torch.int64, device=B.device))
        elapsed = time.time() - t_begin
        launched = 0
        for it in range(max_iter):
            t_it = time.time()
            refresh = refresh_every > 0 and (it + 1) % refresh_every == 0
            _cg_iteration(state, B, mmv, eps, tol_sq, refresh, per_column)
            launched = it + 1
            elapsed += time.time() - t_it
            if callback is not None:
                try:
                    callback(it + 1, state.x, elapsed)
                except StopOptimizationException as e:
                    print(f"Optimization stopped from callback: {e.message}")
                    break
            # the only look at the device the loop itself takes: a chance to leave early, at the refresh cadence
            if refresh and it + 1 < max_iter and float(state.live.max()) == 0.0:
                break
        done = int(state.iterations)
        self.num_iter = max(min(done, launched) - 1, 0) if launched else None
        return state.x


class FalkonConjugateGradient(Optimizer):
    r"""Preconditioned CG for the Nystrom kernel ridge regression system (falkon/optim/conjgrad.py:206-330)

    .. math:: \tilde B^\top H \tilde B \beta = \tilde B^\top K_{nm}^\top Y / n, \qquad
              H = K_{nm}^\top K_{nm} / n + \lambda K_{mm}, \qquad \tilde B = T^{-1} A^{-1}

    with the preconditioner's factors :math:`T^\top T = K_{mm}` and :math:`A`.  Because :math:`K_{mm} = T^\top T`, the
    operator applied to :math:`\beta` is :math:`A^{-\top} [\, T^{-\top} (K_{nm}^\top K_{nm} u) / n + \lambda\, A^{-1}\beta \,]`
    with :math:`u = T^{-1} A^{-1} \beta`: four triangular solves around ONE ``dmmv`` -- the hot path of this package.

    Parameters
    ----------
    kernel
        Kernel object (``mmv`` / ``dmmv``), or a ``falkon_b200.sharded.ShardedKernelOps`` when every process holds a
        row shard of X and Y (right-hand side and every ``dmmv`` are then all-reduced, ``n`` is the global row count).
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
        self._sharded = hasattr(kernel, "mmv_t")  # ShardedKernelOps binds the kernel's options itself

    @property
    def is_weighted(self) -> bool:
        return self.weight_fn is not None

    # ---- the three products the operator is made of -------------------------------------------------
    def _gram_times(self, X, M, u):
        """K_nm^T K_nm u: one fused fdmmv (all-reduced over the ranks when sharded)."""
        if self._sharded:
            return self.kernel.dmmv(X, M, u, None)
        return self.kernel.dmmv(X, M, u, None, opt=self.params)

    def _knm_times(self, X, M, u):
        if self._sharded:
            return self.kernel.mmv(X, M, u)
        return self.kernel.mmv(X, M, u, opt=self.params)

    def _kmn_times(self, M, X, y):
        """K_mn y summed over all rows of X (all-reduced when sharded)."""
        if self._sharded:
            return self.kernel.mmv_t(M, X, y)
        return self.kernel.mmv(M, X, y, opt=self.params)

    def _operator(self, penalty, X, M, n: int, row_weights=None):
        """beta -> B~^T H B~ beta as a closure; with ``row_weights`` the Gram term is K_mn W K_nm (two products)."""
        prec = self.preconditioner

        def apply(beta: torch.Tensor) -> torch.Tensor:
            a_inv_beta = prec.invA(beta)
            u = prec.invT(a_inv_beta)
            if row_weights is None:
                g = self._gram_times(X, M, u)
            else:
                g = self._kmn_times(M, X, self._knm_times(X, M, u).mul_(row_weights))
            return prec.invAt(prec.invTt(g.div_(n)).add_(a_inv_beta, alpha=penalty))

        return apply

    # kept as named methods too: the reference exposes them and callers time or wrap them
    def falkon_mmv(self, sol, penalty, X, M, n: int):
        return self._operator(penalty, X, M, n)(sol)

    def weighted_falkon_mmv(self, sol, penalty, X, M, y_weights, n: int):
        return self._operator(penalty, X, M, n, row_weights=y_weights)(sol)

    def _check_device_status(self, *tensors):
        """A tensor-core sweep that gave up on a bounded wait stores NaN results and leaves a code in the device
        status word; surface it as an exception here rather than as NaN coefficients later."""
        from .. import _lib

        for t in tensors:
            if t is not None and t.is_cuda:
                code = _lib.tc_status(t.device)
                if code != 0:
                    raise _lib.FlkError(_lib.FLK_ERR_TIMEOUT,
                                        f"a tensor-core kernel gave up waiting on a barrier (status 0x{code:x})")
                return

    def solve(self, X, M, Y, _lambda, initial_solution, max_iter, callback=None, n: Optional[int] = None):
        """Returns beta, the solution in the preconditioned space (alpha = preconditioner.apply(beta)).
        ``n`` defaults to the number of rows of ``Y``; pass the global row count when X, Y are shards."""
        if n is None:
            n = Y.size(0)
        rhs_rows = Y / n
        row_weights = None
        if self.is_weighted:
            row_weights = self.weight_fn(Y, X, torch.arange(Y.shape[0]))
            rhs_rows.mul_(row_weights)
        rhs = self.preconditioner.apply_t(self._kmn_times(M, X, rhs_rows))
        beta = self.optimizer.solve(initial_solution, rhs, self._operator(_lambda, X, M, n, row_weights), max_iter,
                                    callback)
        self._check_device_status(beta)
        return beta

    def solve_val_rhs(self, Xtr, Xval, M, Y, _lambda, initial_solution, max_iter, callback=None):
        """Same system with the right-hand side built from a validation set (conjgrad.py:309-326)."""
        n = Xtr.size(0)
        rhs = self.preconditioner.apply_t(self._kmn_times(M, Xval, Y / n))
        beta = self.optimizer.solve(initial_solution, rhs, self._operator(_lambda, Xtr, M, n), max_iter, callback)
        self._check_device_status(beta)
        return beta
