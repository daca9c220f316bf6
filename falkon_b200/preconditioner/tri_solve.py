"""Triangular solves of the preconditioner at memory speed.

Every CG iteration of Falkon applies four triangular solves with the M x M factors T and A
(falkon/optim/conjgrad.py:242-256 through falkon/preconditioner/flk_preconditioner.py:166-256, where the
reference calls its TRSM wrapper, falkon/la_helpers/cuda_trsm.py:10-59).  With one or a few right-hand sides a
solve is bound by reading the triangle once (5 GB in fp32 at M = 50,000: under a millisecond on a B200), but the
library's triangular solve takes several milliseconds.  This module stores, next to a lower-triangular factor L,
the inverses of its diagonal blocks, and solves by block substitution:

    L x = b      :  x_k = inv(L_kk) (b_k - L[k, :k] x[:k])          k = 0, 1, ...        (row panels of L)
    L^T x = b    :  x_k = inv(L_kk)^T (b_k - L[k+1:, k]^T x[k+1:])   k = ..., 1, 0        (column panels of L)

Each step is one matrix-vector (or thin matrix-matrix) product over a panel of L, which runs at memory bandwidth,
and one small product with the inverted diagonal block.  Only library GEMV / GEMM calls are used.
"""
from typing import List

import torch

__all__ = ("BlockedTriangular",)


class BlockedTriangular:
    """Solver for ``L x = b`` and ``L^T x = b`` with a fixed lower-triangular ``L`` (M x M, row-major).

    ``block`` is the size of the diagonal blocks whose inverses are kept (M / block products per solve;
    extra memory M * block entries)."""

    def __init__(self, L: torch.Tensor, block: int = 2048):
        if L.dim() != 2 or L.shape[0] != L.shape[1]:
            raise ValueError("BlockedTriangular expects a square matrix")
        if not L.is_contiguous():
            raise ValueError("BlockedTriangular expects a row-major (contiguous) lower-triangular matrix")
        self.L = L
        self.M = L.shape[0]
        self.edges: List[int] = list(range(0, self.M, block)) + [self.M]
        self.dinv: List[torch.Tensor] = []
        for k0, k1 in zip(self.edges[:-1], self.edges[1:]):
            eye = torch.eye(k1 - k0, dtype=L.dtype, device=L.device)
            self.dinv.append(torch.linalg.solve_triangular(L[k0:k1, k0:k1], eye, upper=False))

    def to(self, device):
        self.L = self.L.to(device)
        self.dinv = [d.to(device) for d in self.dinv]
        return self

    def _prep(self, b: torch.Tensor):
        vec = b.dim() == 1
        rhs = b.reshape(-1, 1) if vec else b
        if rhs.shape[0] != self.M:
            raise ValueError(f"right-hand side has {rhs.shape[0]} rows, the factor has {self.M}")
        return vec, rhs.to(device=self.L.device, dtype=self.L.dtype)

    def solve(self, b: torch.Tensor) -> torch.Tensor:
        """x with ``L x = b`` (forward substitution over row panels)."""
        vec, rhs = self._prep(b)
        x = torch.empty_like(rhs)
        L = self.L
        for i, (k0, k1) in enumerate(zip(self.edges[:-1], self.edges[1:])):
            r = rhs[k0:k1]
            if k0 > 0:
                r = torch.addmm(r, L[k0:k1, :k0], x[:k0], alpha=-1.0)
            torch.mm(self.dinv[i], r, out=x[k0:k1])
        return x.reshape(-1) if vec else x

    def solve_t(self, b: torch.Tensor) -> torch.Tensor:
        """x with ``L^T x = b`` (backward substitution over column panels)."""
        vec, rhs = self._prep(b)
        x = torch.empty_like(rhs)
        L = self.L
        for i in range(len(self.edges) - 2, -1, -1):
            k0, k1 = self.edges[i], self.edges[i + 1]
            r = rhs[k0:k1]
            if k1 < self.M:
                r = torch.addmm(r, L[k1:, k0:k1].mT, x[k1:], alpha=-1.0)
            torch.mm(self.dinv[i].mT, r, out=x[k0:k1])
        return x.reshape(-1) if vec else x
