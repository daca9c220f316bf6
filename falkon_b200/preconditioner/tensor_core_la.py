"""fp32 matrix products of the preconditioner on the tensor cores, at fp32 accuracy.

The preconditioner's cost is three M^3 / 3 steps (two Cholesky factorisations and T T^T, the reference's POTRF and
LAUUM, falkon/preconditioner/flk_preconditioner.py:119-155).  A B200 runs fp32 multiply-adds at about 70 TFLOP/s
but TF32 tensor-core products more than ten times faster, so the products here are done as three TF32 passes on an
exact split of the operands:

    x = hi + lo,   hi = x with the low 13 mantissa bits cleared (exactly a TF32 number),   lo = x - hi (exact)
    A B^T  ~=  hi(A) hi(B)^T + hi(A) lo(B)^T + lo(A) hi(B)^T          (fp32 accumulation in the tensor cores)

The dropped lo lo^T term and the rounding of lo to TF32 are both of relative size 2^-21, the same order as the
rounding of an fp32 product, which a single TF32 pass (2^-11) is far from.  What remains is the tensor cores' own
accumulation (truncating), which is kept short: see K_CHUNK.  Everything here is plain library GEMM
(``torch.mm`` with TF32 enabled for the duration of the call): these steps are outside the kernel-vector-product
hot path.  fp64 data never takes this route.
"""
from contextlib import contextmanager
from typing import Optional, Tuple

import torch

__all__ = ("split_tf32", "addmm_nt_3xtf32_", "triu_times_transpose_3xtf32", "cholesky_lower_3xtf32")


@contextmanager
def _tf32_matmul():
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        yield
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def split_tf32(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(hi, lo) with x == hi + lo exactly, hi representable in TF32 (10 explicit mantissa bits)."""
    if x.dtype != torch.float32:
        raise TypeError("split_tf32 is defined for float32 tensors")
    xc = x.contiguous()
    hi = (xc.view(torch.int32) & -8192).view(torch.float32)
    return hi, xc - hi


#: multiply-adds accumulated inside the tensor cores before the partial sum is added in ordinary fp32.  The
#: tensor cores truncate (round toward zero) when they add a product to the fp32 accumulator, a systematic
#: error that grows with the length of the accumulation; measured on K_MM of 50,000 centres the factorisation
#: residual is 1.1e-6 with the library's fp32 routine and 2.4e-6 / 4.8e-6 / 9.4e-6 with 512 / 1024 / 2048.
K_CHUNK = 512


def addmm_nt_3xtf32_(acc: torch.Tensor, a_hi, a_lo, b_hi, b_lo, alpha: float = 1.0, k_chunk: int = K_CHUNK):
    """``acc += alpha * A @ B^T`` from the split operands: for every chunk of ``k_chunk`` columns three TF32
    passes (large term first), each added to ``acc`` by the GEMM epilogue in ordinary (round-to-nearest) fp32."""
    K = a_hi.shape[1]
    with _tf32_matmul():
        for c0 in range(0, K, k_chunk):
            c = slice(c0, min(K, c0 + k_chunk))
            acc.addmm_(a_hi[:, c], b_hi[:, c].mT, alpha=alpha)
            acc.addmm_(a_hi[:, c], b_lo[:, c].mT, alpha=alpha)
            acc.addmm_(a_lo[:, c], b_hi[:, c].mT, alpha=alpha)
    return acc


def _group_info(group):
    """(rank, world, global rank of every group rank) of a torch.distributed group; (0, 1, [0]) without one."""
    if group is None:
        return 0, 1, [0]
    import torch.distributed as dist

    world = dist.get_world_size(group)
    return dist.get_rank(group), world, [dist.get_global_rank(group, r) for r in range(world)]


def _spread(costs, world):
    """Owner of every work item: largest first onto the least loaded rank (the same answer on every rank)."""
    load = [0.0] * world
    owner = [0] * len(costs)
    for idx in sorted(range(len(costs)), key=lambda i: (-costs[i], i)):
        r = min(range(world), key=lambda q: (load[q], q))
        owner[idx] = r
        load[r] += costs[idx]
    return owner


def triu_times_transpose_3xtf32(T: torch.Tensor, block: int = 4096, k_chunk: int = K_CHUNK, group=None) -> torch.Tensor:
    """``T @ T^T`` for upper-triangular fp32 ``T`` (any strides), block-wise over the non-zero blocks only
    (entry block (i, j), j <= i, is the sum over k >= i of T[i, k] T[j, k]^T), each block product by
    ``addmm_nt_3xtf32_``.  The strictly upper blocks are filled by symmetry.  The role of the reference's LAUUM
    step (falkon/preconditioner/flk_preconditioner.py:137-143).

    With a process ``group`` (every rank holding the same ``T``) the blocks are spread over the ranks by cost and the
    result is completed on every rank with one all-reduce of the M x M matrix (each entry is written by exactly one
    rank, the others contribute zeros, so the sum is exact) -- the reference spreads its LAUUM over the GPUs of a
    machine in the same spirit (falkon/ooc_ops/ooc_lauum.py:95)."""
    M = T.shape[0]
    rank, world, _ = _group_info(group)
    edges = list(range(0, M, block)) + [M]
    pairs = [(bi, bj) for bi in range(len(edges) - 1) for bj in range(bi + 1)]
    costs = [float((edges[bi + 1] - edges[bi]) * (edges[bj + 1] - edges[bj])) * (M - edges[bi]) for bi, bj in pairs]
    owner = _spread(costs, world) if world > 1 else [0] * len(pairs)
    out = (torch.zeros if world > 1 else torch.empty)((M, M), dtype=T.dtype, device=T.device)
    split_rows = {}
    for (bi, bj), who in zip(pairs, owner):
        if who != rank:
            continue
        i0, i1 = edges[bi], edges[bi + 1]
        j0, j1 = edges[bj], edges[bj + 1]
        if split_rows.get("bi") != bi:  # the split of row block bi is shared by its pairs (consecutive in the list)
            split_rows = {"bi": bi, "a": split_tf32(T[i0:i1, i0:])}
        a_hi, a_lo = split_rows["a"]
        if bj == bi:
            b_hi, b_lo = a_hi, a_lo
        else:
            b_hi, b_lo = split_tf32(T[j0:j1, i0:])
        blk = torch.zeros((i1 - i0, j1 - j0), dtype=T.dtype, device=T.device)
        addmm_nt_3xtf32_(blk, a_hi, a_lo, b_hi, b_lo, 1.0, k_chunk)
        if bj == bi:  # the two cross terms are summed in a different order on either side of the diagonal
            blk = torch.tril(blk) + torch.tril(blk, -1).mT
        out[i0:i1, j0:j1] = blk
        if bj != bi:
            out[j0:j1, i0:i1] = blk.mT
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=group)
    return out


def cholesky_lower_3xtf32(C: torch.Tensor, panel: int = 2048, trailing: int = 4096,
                          k_chunk: int = K_CHUNK, group=None) -> Tuple[torch.Tensor, int]:
    """In-place blocked (right-looking) Cholesky factorisation ``C = L L^T`` of a symmetric positive-definite fp32
    matrix; only the lower triangle of ``C`` is read.  Returns ``(L, info)``: ``L`` is ``C`` itself with the strict
    upper triangle zeroed, ``info`` is 0 on success or the order of the first leading minor that is not positive
    definite (LAPACK's convention; ``L`` is then meaningless).

    Per panel of ``panel`` columns: the diagonal block is factorised by the library (``cholesky_ex``), the rows
    below it by a library triangular solve, and the update of the trailing lower triangle -- where the
    M^3 / 3 multiply-adds are -- runs block column by block column (blocks of ``trailing`` columns at fixed
    positions) on the tensor cores (``addmm_nt_3xtf32_`` on the exactly split panel).  The role of the reference's
    POTRF step (falkon/preconditioner/flk_preconditioner.py:119-123, falkon/ooc_ops/ooc_potrf.py:19-76).

    With a process ``group`` (every rank holding the same ``C``) the block columns belong to the ranks in turn
    (block-cyclic, as the reference's multi-GPU POTRF distributes its tiles, falkon/c_ext/ops/cuda/parallel_potrf.cu:121-349):
    a rank applies the trailing updates to its own block columns only; before a panel is factorised its owner
    broadcasts the up-to-date panel columns; every rank factorises the small diagonal block itself, solves an
    equal slice of the rows below it and gathers the others' slices, so all ranks end up with the whole factor."""
    if C.dim() != 2 or C.shape[0] != C.shape[1] or C.dtype != torch.float32:
        raise ValueError("cholesky_lower_3xtf32 expects a square float32 matrix")
    M = C.shape[0]
    rank, world, global_ranks = _group_info(group)
    if world > 1:
        import torch.distributed as dist

        trailing = panel  # finer block columns spread better over the ranks
    infos, starts = [], []
    for k0 in range(0, M, panel):
        k1 = min(M, k0 + panel)
        owner = (k0 // trailing) % world
        if world > 1:
            # the owner of this block column holds its up-to-date values (rows k0..M of columns k0..k1)
            buf = C[k0:, k0:k1].contiguous() if owner == rank else torch.empty((M - k0, k1 - k0), dtype=C.dtype,
                                                                               device=C.device)
            dist.broadcast(buf, src=global_ranks[owner], group=group)
            if owner != rank:
                C[k0:, k0:k1] = buf
            del buf
        Lkk, info = torch.linalg.cholesky_ex(C[k0:k1, k0:k1])
        infos.append(info.reshape(1))
        starts.append(k0)
        C[k0:k1, k0:k1] = Lkk
        if k1 == M:
            break
        if world > 1:
            # the rows below the diagonal block are independent in A21 L11^-T: every rank solves an equal slice
            # of them and the slices are gathered (padded to equal length for the collective)
            below = M - k1
            chunk = (below + world - 1) // world
            lo, hi = min(rank * chunk, below), min((rank + 1) * chunk, below)
            mine = torch.zeros((chunk, k1 - k0), dtype=C.dtype, device=C.device)
            if hi > lo:
                mine[: hi - lo] = torch.linalg.solve_triangular(Lkk.mT, C[k1 + lo:k1 + hi, k0:k1], upper=True,
                                                                left=False)
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine, group=group)
            P = torch.cat(parts, dim=0)[:below]
            del parts, mine
        else:
            P = torch.linalg.solve_triangular(Lkk.mT, C[k1:, k0:k1], upper=True, left=False)  # A21 L11^-T
        C[k1:, k0:k1] = P
        p_hi, p_lo = split_tf32(P)
        del P
        for jb in range(k1 // trailing, (M + trailing - 1) // trailing):
            if jb % world != rank:
                continue
            j0, j1 = max(jb * trailing, k1), min(M, (jb + 1) * trailing)
            if j0 >= j1:
                continue
            rows, cols = slice(j0 - k1, None), slice(j0 - k1, j1 - k1)
            addmm_nt_3xtf32_(C[j0:, j0:j1], p_hi[rows], p_lo[rows], p_hi[cols], p_lo[cols], -1.0, k_chunk)
    codes = torch.cat(infos).cpu().tolist()  # the only host synchronisation
    info = 0
    for k0, c in zip(starts, codes):
        if c != 0:
            info = k0 + int(c)
            break
    C.tril_()
    return C, info
