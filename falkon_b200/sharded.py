"""Row-sharded kernel-vector products across GPUs: one process per GPU, ``torch.distributed``.

The products decompose over the rows of X:  K(X,C)^T (K(X,C) v + w) = sum_g K(X_g,C)^T (K(X_g,C) v + w_g).
The reference exploits this with one Python thread per GPU and a ``reduce_add`` of the per-GPU
M x T partials (falkon/mmv_ops/fmmv.py:1080-1125, falkon/utils/helpers.py:198-206).  Here every
rank owns one contiguous row shard of X (and of w / of the N x T vector of the transposed product),
C and v are replicated, each rank runs the single-GPU product on its shard, and the only exchange
is one all-reduce (NCCL over NVLink on GPUs, gloo on CPU in the tests) of the M x T result.
``K(X,C) v`` itself needs no exchange: its rows stay sharded.
"""
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

__all__ = ("shard_rows", "ShardedKernelOps")


def shard_rows(n: int, world: int, rank: int) -> Tuple[int, int]:
    """(first row, number of rows) of rank's contiguous shard; sizes differ by at most one row
    (identical GPUs; the reference weights shards by SM count, falkon/utils/helpers.py:198-206)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"invalid rank {rank} for world size {world}")
    base, rem = divmod(n, world)
    start = rank * base + min(rank, rem)
    return start, base + (1 if rank < rem else 0)


class ShardedKernelOps:
    """Distributed ``mmv`` / ``dmmv`` for a kernel object.

    ``local_mmv`` / ``local_dmmv`` default to the kernel's own (CUDA) products; the CPU tests pass
    stand-ins so that the sharding and reduction logic can run under gloo without a GPU.
    """

    def __init__(self, kernel, group=None, local_mmv: Optional[Callable] = None,
                 local_dmmv: Optional[Callable] = None):
        self.kernel = kernel
        self.group = group
        self._mmv = local_mmv if local_mmv is not None else kernel.mmv
        self._dmmv = local_dmmv if local_dmmv is not None else kernel.dmmv
        # measurement hook: when set to a list, every all-reduce of a CUDA tensor appends a (start, end) pair of
        # CUDA events recorded on the current stream around the collective
        self.collective_events = None

    @property
    def world(self) -> int:
        return dist.get_world_size(self.group) if dist.is_available() and dist.is_initialized() else 1

    def _all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return t
        if self.collective_events is not None and t.device.type == "cuda":
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            self._all_reduce_untimed(t)
            e1.record()
            self.collective_events.append((e0, e1))
            return t
        return self._all_reduce_untimed(t)

    def _all_reduce_untimed(self, t: torch.Tensor) -> torch.Tensor:
        backend = dist.get_backend(self.group)
        if backend == "nccl" and t.device.type != "cuda":
            tmp = t.to(torch.device("cuda", torch.cuda.current_device()))
            dist.all_reduce(tmp, op=dist.ReduceOp.SUM, group=self.group)
            t.copy_(tmp)
            return t
        if not t.is_contiguous():
            tmp = t.contiguous()
            dist.all_reduce(tmp, op=dist.ReduceOp.SUM, group=self.group)
            t.copy_(tmp)
            return t
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    def dmmv(self, X_shard, C, v, w_shard, out=None, opt=None):
        """sum over ranks of K(X_g,C)^T (K(X_g,C) v + w_g): every rank returns the full M x T result."""
        res = self._dmmv(X_shard, C, v, w_shard, out=out, opt=opt)
        return self._all_reduce(res)

    def mmv(self, X_shard, C, v, out=None, opt=None):
        """K(X_g, C) v: the rows of the result stay with the rank that owns the rows of X."""
        return self._mmv(X_shard, C, v, out=out, opt=opt)

    def mmv_t(self, C, X_shard, y_shard, out=None, opt=None):
        """K(C, X) y = sum over ranks of K(C, X_g) y_g (the CG right-hand side,
        falkon/optim/conjgrad.py:296): every rank returns the full M x T result."""
        res = self._mmv(C, X_shard, y_shard, out=out, opt=opt)
        return self._all_reduce(res)
