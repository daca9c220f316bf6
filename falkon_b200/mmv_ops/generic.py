"""Kernel-vector products for kernels that describe themselves only through ``compute``.

The reference's extension contract (falkon/kernels/kernel.py:462-505, exercised by
falkon/tests/test_custom_kernel.py:33-98) is: implement ``compute(X1, X2, out, diag)`` and ``mmv`` / ``dmmv`` work.
The fused CUDA kernels of this package know the built-in distance kernels only (they never form the block), so a
user-defined kernel cannot use them.  For such kernels the products run the reference's own blocked algorithm
(falkon/mmv_ops/fmmv.py:358-391, :740-760) on the GPU: per row block the user's ``compute`` fills an n_blk x m block
in device memory, and the two contractions are library GEMMs.  Nothing here is on the path of the built-in kernels,
and there is still no CPU execution: operands on the host are moved to the device block by block.

The block length honours the memory budget (``max_gpu_mem`` / ``memory_slack``): the block and its side buffers take
``n_blk * (m + t + d)`` elements.
"""
from typing import Optional

import torch

__all__ = ("generic_fmmv", "generic_fdmmv")

#: cap of the kernel block (elements); a smaller memory budget lowers it, a larger one does not raise it (the
#: user's ``compute`` may need temporaries of the block's size)
_DEFAULT_BLOCK_ELEMS = 256 * 2**20


def _rows_per_block(n: int, m: int, d: int, t: int, es: int, budget: Optional[float]) -> int:
    per_row = (m + t + d) * es
    limit = _DEFAULT_BLOCK_ELEMS * es if budget is None else min(budget, _DEFAULT_BLOCK_ELEMS * es)
    rows = int(limit // max(per_row, 1))
    if rows < 1:
        raise MemoryError(f"Available memory ({limit / 2**20:.1f} MiB) cannot hold one row of the kernel block "
                          f"({per_row / 2**20:.3f} MiB)")
    return min(n, rows)


def generic_fmmv(X1, X2, v, kernel, out, dev, budget=None):
    """out[n, t] = kernel(X1, X2) @ v, block by block over the rows of X1, on ``dev``."""
    n, d = X1.shape
    m, t = v.shape
    X2d, vd = X2.to(dev), v.to(dev)
    blk = _rows_per_block(n, m, d, t, X1.element_size(), budget)
    kbuf = torch.empty((blk, m), dtype=X1.dtype, device=dev)
    for r0 in range(0, n, blk):
        r1 = min(n, r0 + blk)
        K = kernel.compute(X1[r0:r1].to(dev), X2d, kbuf[: r1 - r0], False)
        res = K @ vd
        out[r0:r1].copy_(res)
    return out


def generic_fdmmv(X1, X2, v, w, kernel, out, dev, budget=None):
    """out[m, t] = K^T (K v + w) with K = kernel(X1, X2), summed over row blocks of X1, on ``dev``."""
    n, d = X1.shape
    m = X2.shape[0]
    t = v.shape[1] if v is not None else w.shape[1]
    X2d = X2.to(dev)
    vd = None if v is None else v.to(dev)
    acc = torch.zeros((m, t), dtype=X1.dtype, device=dev)
    blk = _rows_per_block(n, m, d, t, X1.element_size(), budget)
    kbuf = torch.empty((blk, m), dtype=X1.dtype, device=dev)
    for r0 in range(0, n, blk):
        r1 = min(n, r0 + blk)
        K = kernel.compute(X1[r0:r1].to(dev), X2d, kbuf[: r1 - r0], False)
        if vd is not None:
            u = K @ vd
            if w is not None:
                u += w[r0:r1].to(dev)
        else:
            u = w[r0:r1].to(dev)
        acc.addmm_(K.mT, u)
    out.copy_(acc)
    return out
