"""Host-resident operands on a machine with several GPUs, driven from ONE process.

The reference splits the rows of X1 over all visible GPUs, runs one Python thread per GPU and adds the
per-GPU partial results (``fdmmv``: falkon/mmv_ops/fmmv.py:1080-1125 with ``_start_wait_processes``,
falkon/mmv_ops/utils.py:67-87, ``PropagatingThread``, falkon/utils/threading.py:6-27, and the row split of
falkon/utils/helpers.py:198-206).  This module is the same contract on the host-buffer entry points of the
C ABI: every GPU gets a contiguous slice of rows and its own call of ``flk_fmmv_host`` / ``flk_fdmmv_host``
(which stage, compute and copy back on that device's streams; ctypes releases the GIL for the duration of
the call, so the threads really run concurrently), the m x t partials are added on the host in device order.

Programs that run one process per GPU (``torch.distributed`` initialised) never fan out from here: each rank
keeps to its own device and ``falkon_b200.sharded`` does the reduction over NCCL.
"""
import threading
from typing import Callable, List, Optional, Sequence, Tuple

import torch

from .. import _lib

__all__ = ("host_devices", "split_rows", "fmmv_host_multi", "fdmmv_host_multi")

#: below this many rows per GPU the fan-out costs more than it gains
MIN_ROWS_PER_DEVICE = 131072


def split_rows(n: int, parts: int) -> List[Tuple[int, int]]:
    """``parts`` contiguous (start, length) slices of n rows whose lengths differ by at most one
    (identical GPUs; the reference weights by SM count)."""
    base, rem = divmod(n, parts)
    out, start = [], 0
    for i in range(parts):
        length = base + (1 if i < rem else 0)
        out.append((start, length))
        start += length
    return out


def host_devices(opt, n: int, primary: torch.device) -> List[torch.device]:
    """The GPUs a host-operand call spreads over: all visible ones (or ``opt.flk_devices``, a list of
    ordinals), as many as leave MIN_ROWS_PER_DEVICE rows each; only ``primary`` inside a torch.distributed
    job."""
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        return [primary]
    wanted = getattr(opt, "flk_devices", None)
    if wanted is None:
        wanted = list(range(torch.cuda.device_count()))
    wanted = [int(i) for i in wanted]
    if not wanted:
        return [primary]
    count = max(1, min(len(wanted), n // MIN_ROWS_PER_DEVICE))
    if count == 1:
        return [primary if primary.index in wanted or primary.index is None else torch.device("cuda", wanted[0])]
    return [torch.device("cuda", i) for i in wanted[:count]]


def _run_threads(jobs: Sequence[Callable[[], None]]) -> None:
    """One thread per job; the first failure is re-raised in the caller as RuntimeError with the original
    exception as its cause (the reference's PropagatingThread contract)."""
    errors: List[Optional[BaseException]] = [None] * len(jobs)

    def runner(i):
        try:
            jobs[i]()
        except BaseException as e:  # noqa: BLE001 - propagated below
            errors[i] = e

    threads = [threading.Thread(target=runner, args=(i,), name=f"flk-gpu-{i}") for i in range(len(jobs))]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    for i, e in enumerate(errors):
        if e is not None:
            raise RuntimeError(f"Exception in GPU worker thread {i}") from e


def fmmv_host_multi(kernel_id, sigma, X1, X2, v, out, flags, devices, call=None):
    """out[n, t] = k(X1, X2) v with the rows of X1 (and of out) split over ``devices``."""
    call = call or _lib.call_fmmv
    spans = split_rows(X1.shape[0], len(devices))

    def job(dev, start, length):
        def run():
            if length > 0:
                call(kernel_id, sigma, X1[start:start + length], X2, v, out[start:start + length], flags=flags,
                     host=True, device=dev)
        return run

    _run_threads([job(dev, s, ln) for dev, (s, ln) in zip(devices, spans)])
    return out


def fdmmv_host_multi(kernel_id, sigma, X1, X2, v, w, out, flags, devices, call=None):
    """out[m, t] = sum over devices of k(X1_g, X2)^T (k(X1_g, X2) v + w_g); partials added in device order."""
    call = call or _lib.call_fdmmv
    spans = split_rows(X1.shape[0], len(devices))
    parts = [torch.zeros(out.shape, dtype=out.dtype) for _ in devices]

    def job(i, dev, start, length):
        def run():
            if length > 0:
                call(kernel_id, sigma, X1[start:start + length], X2, v,
                     None if w is None else w[start:start + length], parts[i], flags=flags, host=True, device=dev)
        return run

    _run_threads([job(i, dev, s, ln) for i, (dev, (s, ln)) in enumerate(zip(devices, spans))])
    acc = parts[0]
    for p in parts[1:]:
        acc += p
    out.copy_(acc)
    return out
