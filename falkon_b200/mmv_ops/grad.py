"""Backward pass of ``k(X1, X2) @ v`` and of ``k(X1, X2)`` for the distance kernels.

The reference differentiates by re-running each kernel block under autograd and calling
``torch.autograd.grad`` on it (``mmv_diff_run_thread``, falkon/mmv_ops/fmmv.py:405-485, and
``KernelMmFnFull.backward`` in falkon/mmv_ops/fmm.py).  For a radial kernel all of those gradients are
matrix products with one n x m block of pair weights,

    W_ij = 2 k'(D2_ij) s_ij,      s_ij = G_i . v_j  (mmv)   or   s_ij = G_ij  (kernel matrix),

which ``flk_kgrad`` (include/falkon_b200.h) evaluates in a single CUDA kernel: distance by the same norm
expansion as the forward pass, the t-long dot, the derivative of the radial profile.  With
``a = W 1``, ``b = W^T 1`` and ``X~ = X / sigma``:

    dL/dX1 = (a o X1~ - W X2~) / sigma           dL/dX2 = (b o X2~ - W^T X1~) / sigma
    dL/dsigma_k = -(1 / sigma_k) [ sum_i a_i x~_ik^2 - 2 sum_i x~_ik (W X2~)_ik + sum_j b_j c~_jk^2 ]
    dL/dv = k(X1, X2)^T G                        (the transposed product of the forward library)

-- the same expressions autograd derives from the reference's ``addmm`` expansion, so rounding behaves
alike.  Rows are processed in blocks whose weight matrix fits the GPU's L2 cache (126 MB on a B200), so the
two GEMMs that follow each ``flk_kgrad`` launch read W from L2, not from HBM.  The GEMMs themselves are
plain library products (``torch.matmul``).
"""
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import _lib

__all__ = ("kernel_backward",)

#: bytes of pair weights per row block: half of the B200's L2
_W_BLOCK_BYTES = 64 * 2**20
_MAX_ROWS_PER_CALL = 64 * 65535


def _row_block(n: int, m: int, itemsize: int) -> int:
    rows = _W_BLOCK_BYTES // max(1, m * itemsize)
    rows = max(64, (rows // 64) * 64)
    return int(min(max(n, 1), rows, _MAX_ROWS_PER_CALL))


def kernel_backward(
    kernel_id: int,
    sigma: torch.Tensor,
    X1: torch.Tensor,
    X2: torch.Tensor,
    G: torch.Tensor,
    v: Optional[torch.Tensor],
    needs: Sequence[bool],
    flags: int = 0,
) -> List[Optional[torch.Tensor]]:
    """Gradients ``[dX1, dX2, dv, dsigma]`` (``None`` where ``needs`` is False) on X1's device.

    ``G`` is the upstream gradient: n x t together with ``v`` (m x t), or n x m with ``v=None``.
    ``sigma`` is the kernel's length-scale tensor (1 or d entries, any dtype / device); its gradient is
    returned in sigma's dtype and shape.  All of X1, X2, G, v are CUDA tensors of one dtype on one device.
    """
    need_x1, need_x2, need_v, need_sigma = needs
    dev, dtype = X1.device, X1.dtype
    n, d = X1.shape
    m = X2.shape[0]
    sigma_np = sigma.detach().to(device="cpu", dtype=torch.float64).reshape(-1).numpy()
    sig = sigma.detach().to(device=dev, dtype=dtype).reshape(-1)

    grad_v = None
    if need_v and v is not None:
        grad_v = torch.empty((m, G.shape[1]), dtype=dtype, device=dev)
        _lib.call_fdmmv(kernel_id, sigma_np, X1, X2, None, G, grad_v, flags=flags & ~_lib.FLAG_FP64_MATH)
    if not (need_x1 or need_x2 or need_sigma):
        return [None, None, grad_v, None]

    X2s = X2 / sig
    need_cols = need_x2 or need_sigma
    grad_x1 = torch.empty((n, d), dtype=dtype, device=dev) if need_x1 else None
    Q = torch.zeros((m, d), dtype=dtype, device=dev) if need_cols else None
    b = torch.zeros((m,), dtype=dtype, device=dev) if need_cols else None
    sig_acc = torch.zeros((d,), dtype=dtype, device=dev) if need_sigma else None

    blk = _row_block(n, m, X1.element_size())
    W = torch.empty((min(blk, max(n, 1)), m), dtype=dtype, device=dev)
    for i0 in range(0, n, blk):
        i1 = min(n, i0 + blk)
        Wb = W[: i1 - i0]
        X1b = X1[i0:i1]
        _lib.call_kgrad(kernel_id, sigma_np, X1b, X2, G[i0:i1], v, Wb, flags=flags)
        X1s = X1b / sig
        a = Wb.sum(dim=1, keepdim=True)
        P = Wb @ X2s
        if need_x1:
            torch.addcmul(-P, a, X1s, out=grad_x1[i0:i1])
        if need_cols:
            b += Wb.sum(dim=0)
            Q.addmm_(Wb.t(), X1s)
        if need_sigma:
            sig_acc += (X1s * (a * X1s - 2.0 * P)).sum(dim=0)

    grad_x2 = None
    if need_x1:
        grad_x1 /= sig
    if need_x2:
        grad_x2 = torch.addcmul(-Q, b.unsqueeze(1), X2s)
        grad_x2 /= sig
    grad_sigma = None
    if need_sigma:
        sig_acc += (b.unsqueeze(1) * X2s * X2s).sum(dim=0)
        per_dim = -sig_acc / (sig if sig.numel() == d else sig.expand(d))
        if sigma.numel() == 1:
            per_dim = per_dim.sum().reshape(1)
        grad_sigma = per_dim.to(device=sigma.device, dtype=sigma.dtype).reshape(sigma.shape)
    return [grad_x1, grad_x2, grad_v, grad_sigma]
