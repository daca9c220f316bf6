"""Falkon's two-level Cholesky preconditioner, kept on the GPU.

Mathematics and method names follow falkon/preconditioner/flk_preconditioner.py:16-299:

    T = chol(K_MM + eps * M * I)            upper triangular, T^T T = K_MM (+ jitter)
    A = chol(1/M * T T^T + lambda * I)      upper triangular

and the preconditioner is  B~ = 1/sqrt(n) T^-1 A^-1.  ``invA / invAt / invT / invTt`` solve with
A, A^T, T, T^T; ``apply(v) = T^-1 A^-1 v`` and ``apply_t(v) = A^-T T^-T v``.

What differs from the reference is where the work runs.  The reference packs T and A into the two
triangles of one M x M buffer and drives cuSOLVER / its own out-of-core LAUUM and POTRF from Python
so that M x M may exceed GPU memory.  A B200 holds several M x M matrices at M = 50 000 (10 GB each
in fp32), so this class keeps T and A as two separate device tensors.  Triangular solves are the
library's (cuBLAS); the factorisations and T T^T are the library's in fp64 and, in fp32, blocked versions
whose M^3 products run as split-TF32 tensor-core GEMMs (tensor_core_la.py).  These steps are outside the
kernel-vector-product hot path.  K_MM itself comes from this package's CUDA kernel (``Kernel.__call__``
-> ``flk_fmm``), evaluated in fp64 for fp32 data when ``no_single_kernel`` is set, as in the reference.
"""
from abc import ABC, abstractmethod
from typing import Optional

import torch

from ..options import FalkonOptions
from .tensor_core_la import cholesky_lower_3xtf32, triu_times_transpose_3xtf32
from .tri_solve import BlockedTriangular

#: from this many centres on, the per-iteration triangular solves of an fp32 preconditioner go through BlockedTriangular
_BLOCKED_SOLVE_MIN_M = 8192

__all__ = ("Preconditioner", "FalkonPreconditioner")


class Preconditioner(ABC):
    """Interface of falkon/preconditioner/preconditioner.py: ``init`` then ``apply`` / ``apply_t``."""

    @abstractmethod
    def init(self, *args, **kwargs):
        ...

    @abstractmethod
    def apply(self, v: torch.Tensor) -> torch.Tensor:
        ...

    @abstractmethod
    def apply_t(self, v: torch.Tensor) -> torch.Tensor:
        ...


def _triu_times_transpose(T: torch.Tensor, block: int = 4096) -> torch.Tensor:
    """``T @ T^T`` for upper-triangular ``T`` (the LAUUM step, flk_preconditioner.py:137-143), computed
    block-wise so that only products of non-zero blocks are formed: entry block (i, j), j <= i, is
    sum over k >= i of T[i, k] T[j, k]^T.  About M^3 / 3 multiply-adds instead of the M^3 of a dense
    product; the strictly upper blocks are filled by symmetry."""
    M = T.shape[0]
    if M <= block:
        return T @ T.mT
    out = torch.empty_like(T)
    edges = list(range(0, M, block)) + [M]
    for bi in range(len(edges) - 1):
        i0, i1 = edges[bi], edges[bi + 1]
        for bj in range(bi + 1):
            j0, j1 = edges[bj], edges[bj + 1]
            # rows i0:i1 of T are zero left of column i0, so the contraction starts there
            blk = T[i0:i1, i0:] @ T[j0:j1, i0:].mT
            out[i0:i1, j0:j1] = blk
            if bj != bi:
                out[j0:j1, i0:i1] = blk.mT
    return out


def _require_init(fn):
    def wrapper(self, *args, **kwargs):
        if self.T is None or self.A is None:
            raise RuntimeError("FalkonPreconditioner is not initialized. Please run `init` before any other method.")
        return fn(self, *args, **kwargs)

    wrapper.__name__ = fn.__name__
    wrapper.__doc__ = fn.__doc__
    return wrapper


class FalkonPreconditioner(Preconditioner):
    """Approximate Cholesky preconditioner of the Nystrom kernel-ridge-regression system.

    Parameters
    ----------
    penalty
        The ridge parameter lambda (> 0).
    kernel
        Kernel object; ``kernel(X, X)`` gives K_MM.
    opt
        ``pc_epsilon_32 / pc_epsilon_64`` (jitter added to K_MM, multiplied by M as in the reference,
        flk_preconditioner.py:117) and ``no_single_kernel`` are honoured.  ``cpu_preconditioner`` /
        ``use_cpu`` are rejected: there is no CPU path in this package.  Setting the attribute
        ``opt.pc_tensor_cores = False`` (not a reference option, hence not a dataclass field) selects the library's
        fp32 Cholesky and fp32 GEMMs instead of the split-TF32 tensor-core versions.
    """

    def __init__(self, penalty: float, kernel, opt: Optional[FalkonOptions] = None):
        self.params = opt or FalkonOptions()
        if self.params.use_cpu or self.params.cpu_preconditioner:
            raise RuntimeError("falkon_b200 computes the preconditioner on the GPU only "
                               "(use_cpu / cpu_preconditioner were requested).")
        self._lambda = float(penalty)
        self.kernel = kernel
        self.T: Optional[torch.Tensor] = None
        self.A: Optional[torch.Tensor] = None
        self._t_solver: Optional[BlockedTriangular] = None
        self._a_solver: Optional[BlockedTriangular] = None

    # the reference exposes the diagonals it has to save because its two factors share a buffer
    @property
    def dT(self):
        return None if self.T is None else self.T.diagonal()

    @property
    def dA(self):
        return None if self.A is None else self.A.diagonal()

    def init(self, X: torch.Tensor, weight_vec: Optional[torch.Tensor] = None, group=None):
        """Builds T and A from the (M x D) centres ``X`` (optionally with per-centre weights for
        re-weighted least squares, flk_preconditioner.py:131-152).

        ``group``: a ``torch.distributed`` process group whose ranks all call ``init`` with the same centres.  The
        M^3 steps of the fp32 tensor-core path (two factorisations, T T^T) are then shared between the ranks
        (``tensor_core_la``: block-cyclic trailing updates with a broadcast of each panel, block products completed
        by an all-reduce); every rank ends up with the same T and A.  Other paths (fp64, library fp32) compute
        everything on every rank."""
        if weight_vec is not None and weight_vec.shape[0] != X.shape[0]:
            raise ValueError(
                f"Weights and Nystrom centers should have the same first dimension. "
                f"Found instead {weight_vec.shape[0]}, {X.shape[0]}."
            )
        if not torch.cuda.is_available():
            raise RuntimeError("falkon_b200 needs a CUDA device (B200, sm_100); none is available.")
        dev = X.device if X.is_cuda else torch.device("cuda", torch.cuda.current_device())
        with torch.inference_mode():
            Xd = X.to(dev)
            M = Xd.shape[0]
            C = self.kernel(Xd, Xd, opt=self.params)  # M x M, data dtype
            eps = self.params.pc_epsilon(C.dtype)
            C.diagonal().add_(eps * M)
            # fp32: blocked factorisation / products whose M^3 part runs on the tensor cores (tensor_core_la.py)
            tensor_cores = C.dtype == torch.float32 and getattr(self.params, "pc_tensor_cores", True)
            # T^T T = C.  Failure is reported as a status instead of a device assert.
            if tensor_cores:
                L, code = cholesky_lower_3xtf32(C, group=group)  # in place; T is its transpose, as a view
                T = L.mT
            else:
                L, info = torch.linalg.cholesky_ex(C, upper=False)
                T = L.mT
                code = int(info.item())
            if code != 0:
                raise RuntimeError(
                    f"Cholesky factorisation of K_MM failed at leading minor {code}: "
                    f"K_MM is not positive definite; increase pc_epsilon (now {eps})."
                )
            del C
            TTt = triu_times_transpose_3xtf32(T, group=group) if tensor_cores else _triu_times_transpose(T)
            if weight_vec is not None:
                s = weight_vec.to(dev, TTt.dtype).reshape(-1).sqrt()
                TTt.mul_(s.reshape(-1, 1)).mul_(s.reshape(1, -1))
            TTt.mul_(1.0 / M)
            TTt.diagonal().add_(self._lambda)
            if tensor_cores:
                L2, code = cholesky_lower_3xtf32(TTt, group=group)
                A = L2.mT
            else:
                L2, info = torch.linalg.cholesky_ex(TTt, upper=False)
                A = L2.mT
                code = int(info.item())
            if code != 0:
                raise RuntimeError(
                    f"Cholesky factorisation of 1/M T T^T + lambda I failed at leading minor {code}."
                )
            del TTt
            self.T, self.A = T, A
            # T = L^T and A = L2^T are kept as transposed views of the row-major lower factors
            self._t_solver = self._a_solver = None
            # fp32 only: multiplying with inverted diagonal blocks is not backward stable, and the fp64 factors of a
            # kernel matrix with a 1e-13 jitter are ill-conditioned enough for that to show
            if M >= _BLOCKED_SOLVE_MIN_M and L.dtype == torch.float32:
                self._t_solver = BlockedTriangular(L)
                self._a_solver = BlockedTriangular(L2)
        return self

    def to(self, device):
        if self.T is not None:
            self.T = self.T.to(device)
        if self.A is not None:
            self.A = self.A.to(device)
        if self._t_solver is not None:  # the solvers hold the lower factors the views above are taken from
            self._t_solver.to(device)
            self._a_solver.to(device)
            self.T, self.A = self._t_solver.L.mT, self._a_solver.L.mT
        return self

    @staticmethod
    def _solve(tri: torch.Tensor, v: torch.Tensor, transpose: bool) -> torch.Tensor:
        vec = v.dim() == 1
        rhs = v.reshape(-1, 1) if vec else v
        rhs = rhs.to(tri.device)
        if transpose:
            out = torch.linalg.solve_triangular(tri.mT, rhs, upper=False)
        else:
            out = torch.linalg.solve_triangular(tri, rhs, upper=True)
        return out.reshape(-1) if vec else out

    # With the block solvers: A = L2^T, so A x = v is the transposed solve with L2 and A^T x = v the plain one.
    @_require_init
    def invA(self, v: torch.Tensor) -> torch.Tensor:
        """Solves A x = v."""
        if self._a_solver is not None:
            return self._a_solver.solve_t(v)
        return self._solve(self.A, v, transpose=False)

    @_require_init
    def invAt(self, v: torch.Tensor) -> torch.Tensor:
        """Solves A^T x = v."""
        if self._a_solver is not None:
            return self._a_solver.solve(v)
        return self._solve(self.A, v, transpose=True)

    @_require_init
    def invT(self, v: torch.Tensor) -> torch.Tensor:
        """Solves T x = v."""
        if self._t_solver is not None:
            return self._t_solver.solve_t(v)
        return self._solve(self.T, v, transpose=False)

    @_require_init
    def invTt(self, v: torch.Tensor) -> torch.Tensor:
        """Solves T^T x = v."""
        if self._t_solver is not None:
            return self._t_solver.solve(v)
        return self._solve(self.T, v, transpose=True)

    @_require_init
    def apply(self, v: torch.Tensor) -> torch.Tensor:
        """T^-1 A^-1 v: maps a preconditioned solution beta back to the coefficients alpha."""
        return self.invT(self.invA(v))

    @_require_init
    def apply_t(self, v: torch.Tensor) -> torch.Tensor:
        """A^-T T^-T v: applied to the right-hand side K_nm^T y / n."""
        return self.invAt(self.invTt(v))

    def __str__(self):
        return f"FalkonPreconditioner(_lambda={self._lambda}, kernel={self.kernel})"
