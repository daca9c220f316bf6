"""Loader (and builder) of ``libfalkon_b200.so`` and thin ctypes wrappers around its C ABI.

The library is built in-tree with nvcc for sm_100a (``build()``), and loaded with ctypes.  There
is no fallback: if the shared library is missing or fails to load, every product raises.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import re
import threading
from typing import Optional

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_HERE, "csrc")
LIB_PATH = os.environ.get("FALKON_B200_LIB") or os.path.join(_HERE, "libfalkon_b200.so")

FLK_F32, FLK_F64 = 0, 1
FLK_GAUSSIAN, FLK_LAPLACIAN, FLK_MATERN15, FLK_MATERN25 = 0, 1, 2, 3
FLAG_FORCE_SIMT, FLAG_FORCE_TC, FLAG_FP64_MATH, FLAG_NO_FOLD, FLAG_ACCUMULATE = 1, 2, 4, 8, 16
FLAG_KEEP_X1, FLAG_KEEP_X2 = 32, 64
STATIC_SCRATCH_BYTES = 64 << 20

FLK_ERR_BAD_ARG, FLK_ERR_LAYOUT, FLK_ERR_WORKSPACE = -1, -2, -3
FLK_ERR_CUDA, FLK_ERR_UNSUPPORTED, FLK_ERR_DEVICE, FLK_ERR_TIMEOUT = -4, -5, -6, -7

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared", "-Xptxas", "-v",
]
PTXAS_REPORT = LIB_PATH + ".ptxas.txt"
# The tensor-core sweeps read their accumulators with asynchronous tcgen05.ld: a register that such a load is still
# to fill must never be spilled, so the resident kernel has to compile without any spill.  It re-partitions
# registers between its warp roles and relies on being launched with exactly this many per thread:
TC_LAUNCH_REGISTERS = 80
# A few instantiations of the K-loop kernel still spill one or two 32-bit values that are stored once before the
# warp roles split (none inside a tile loop); the build tolerates up to this many bytes of spill stores / loads
# there and fails beyond (a regression guard, not an endorsement).
TCK_SPILL_ALLOWANCE = (16, 48)

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


def sources():
    return [os.path.join(_CSRC, f) for f in sorted(os.listdir(_CSRC)) if f.endswith((".cu", ".cuh"))] + [
        os.path.join(os.path.dirname(_HERE), "include", "falkon_b200.h")
    ]


def _up_to_date() -> bool:
    if not os.path.exists(LIB_PATH):
        return False
    return os.path.getmtime(LIB_PATH) >= max(os.path.getmtime(s) for s in sources())


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles csrc/flk_api.cu into libfalkon_b200.so (nvcc cross-compiles without a GPU).

    Safe when several processes (one per GPU) start at once: the build runs under an exclusive file lock,
    writes to a temporary name and is moved into place atomically, and a process that waited for the lock
    finds the library up to date and does not build again."""
    if not force and _up_to_date():
        return LIB_PATH
    import fcntl

    with open(LIB_PATH + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and _up_to_date():
                return LIB_PATH
            tmp = f"{LIB_PATH}.{os.getpid()}.tmp"
            nvcc = os.environ.get("NVCC", "nvcc")
            extra = os.environ.get("FALKON_B200_NVCC_EXTRA", "").split()  # e.g. -D tuning macros of the kernels
            cmd = [nvcc] + NVCC_FLAGS + extra + ["-o", tmp, os.path.join(_CSRC, "flk_api.cu")]
            if verbose:
                print(" ".join(cmd))
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                if os.path.exists(tmp):
                    os.remove(tmp)
                raise RuntimeError(f"nvcc failed:\n{res.stdout}\n{res.stderr}")
            table = parse_ptxas(res.stderr)
            problems = check_ptxas(table)
            with open(PTXAS_REPORT, "w") as f:
                f.write(format_ptxas(table))
            if problems:
                os.remove(tmp)
                raise RuntimeError("register check of the tensor-core kernels failed:\n" + "\n".join(problems))
            os.replace(tmp, LIB_PATH)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB_PATH


def parse_ptxas(text: str):
    """[(kernel name, registers, stack bytes, spill-store bytes, spill-load bytes)] from `ptxas -v` output."""
    import re

    pat = re.compile(
        r"Compiling entry function '(\S+)' for 'sm_100a'\s*\n.*?Function properties for \S+\s*\n"
        r"\s*(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads\s*\n"
        r".*?Used (\d+) registers", re.S)
    rows = pat.findall(text)
    if not rows:
        return []
    try:
        names = subprocess.run(["c++filt"], input="\n".join(r[0] for r in rows), capture_output=True,
                               text=True).stdout.split("\n")
    except OSError:
        names = [r[0] for r in rows]
    out = []
    for (mangled, stack, st, ld, regs), name in zip(rows, names):
        name = re.sub(r"\(.*$", "", name).replace("void ", "").strip() or mangled
        out.append((name, int(regs), int(stack), int(st), int(ld)))
    return sorted(out)


def check_ptxas(table):
    """Problems (strings) that make the build fail: any spill in the resident tensor-core kernel, a launch register
    count other than the one its register re-partitioning assumes, more than the allowance in the K-loop kernel."""
    problems = []
    seen_tc = False
    for name, regs, stack, st, ld in table:
        if "tc::kmv_tc_kernel" in name:
            seen_tc = True
            if st or ld:
                problems.append(f"{name}: {st} bytes of spill stores, {ld} of spill loads (must be 0)")
            if regs != TC_LAUNCH_REGISTERS:
                problems.append(f"{name}: launched with {regs} registers per thread, {TC_LAUNCH_REGISTERS} assumed")
        elif "tck::kmv_tck_kernel" in name and (st > TCK_SPILL_ALLOWANCE[0] or ld > TCK_SPILL_ALLOWANCE[1]):
            problems.append(f"{name}: {st} / {ld} bytes of spill stores / loads exceed the allowance")
    if table and not seen_tc:
        problems.append("no tc::kmv_tc_kernel instantiation found in the ptxas output")
    return problems


def format_ptxas(table) -> str:
    lines = ["kernel | registers | stack bytes | spill stores | spill loads", "---|---|---|---|---"]
    lines += [f"{n} | {r} | {k} | {a} | {b}" for n, r, k, a, b in table]
    return "\n".join(lines) + "\n"


_i64, _int, _vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
_dp = ctypes.POINTER(ctypes.c_double)

_MAT = [_vp, _i64, _i64, _i64]  # pointer, rows, row stride, col stride

_SIGNATURES = {
    "flk_version": (_int, []),
    "flk_last_error": (ctypes.c_char_p, []),
    "flk_status_name": (ctypes.c_char_p, [_int]),
    "flk_check_device": (_int, []),
    "flk_uses_tensor_cores": (_int, [_int, _int, _i64, _i64, _int]),
    "flk_launch_count": (_i64, []),
    "flk_square_norm": (_int, [_int, _vp, _i64, _i64, _i64, _i64, _dp, _i64, _vp, _vp]),
    "flk_fmmv_workspace_bytes": (_i64, [_int, _int, _i64, _i64, _i64, _i64, _int]),
    "flk_fdmmv_workspace_bytes": (_i64, [_int, _int, _i64, _i64, _i64, _i64, _int]),
    "flk_fmmv_host_workspace_bytes": (_i64, [_int, _int, _i64, _i64, _i64, _i64, _int]),
    "flk_fdmmv_host_workspace_bytes": (_i64, [_int, _int, _i64, _i64, _i64, _i64, _int]),
    # dtype, kernel, X1(4), X2(4), d, v ptr, t, v strides(2), out ptr + strides(3), sigma, len, ws, bytes, flags, stream
    "flk_fmmv": (_int, [_int, _int] + _MAT + _MAT + [_i64, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _dp, _i64, _vp, _i64, _int, _vp]),
    "flk_fmmv_host": (_int, [_int, _int] + _MAT + _MAT + [_i64, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _dp, _i64, _vp, _i64, _int, _vp]),
    # dtype, kernel, X1(4), X2(4), d, v(3), w(3), t, out(3), sigma, len, ws, bytes, flags, stream
    "flk_fdmmv": (_int, [_int, _int] + _MAT + _MAT + [_i64, _vp, _i64, _i64, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _dp, _i64, _vp, _i64, _int, _vp]),
    "flk_fdmmv_host": (_int, [_int, _int] + _MAT + _MAT + [_i64, _vp, _i64, _i64, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _dp, _i64, _vp, _i64, _int, _vp]),
    # dtype, kernel, X1(4), X2(4), d, v ptr, t, v strides(2), out ptr + strides(3), sigma (double), flags, stream
    "flk_fmmv_static": (_int, [_int, _int] + _MAT + _MAT + [_i64, _vp, _i64, _i64, _i64, _vp, _i64, _i64, ctypes.c_double, _int, _vp]),
    "flk_fmm_workspace_bytes": (_i64, [_int, _i64, _i64, _i64, _int]),
    # dtype, kernel, X1(4), X2(4), d, out ptr + strides(3), sigma, len, ws, bytes, flags, stream
    "flk_kgrad": (_int, [_int, _int] + _MAT + _MAT + [_i64, _vp, _i64, _i64, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _dp, _i64, _vp, _i64, _int, _vp]),
    "flk_fmm": (_int, [_int, _int] + _MAT + _MAT + [_i64, _vp, _i64, _i64, _dp, _i64, _vp, _i64, _int, _vp]),
    "flk_tc_status": (_int, [_vp, _vp, ctypes.POINTER(_int)]),
    "flk_range_flag": (_int, [_vp, _vp, ctypes.POINTER(_int)]),
    "flk_probe_mufu": (_int, [_int, _vp, ctypes.POINTER(_i64), _vp]),
    "flk_set_timing": (_int, [_int]),
    "flk_get_sweep_ms": (_int, [ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_float)]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)


def load() -> ctypes.CDLL:
    """Loads the shared library (once per process); raises if it does not exist."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: the CUDA library has not been built "
                "(run `python -c 'import __graft_entry__ as g; g.build()'` or falkon_b200._lib.build()). "
                "falkon_b200 has no CPU fallback."
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
        return lib


class FlkError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


def last_error() -> str:
    return load().flk_last_error().decode()


def raise_for_status(status: int):
    """Maps a C status code to the exception type the reference raises for the same mistake
    (ValueError for shapes / layout, RuntimeError for device problems, MemoryError for workspace)."""
    if status == 0:
        return
    msg = last_error()
    name = load().flk_status_name(status).decode()
    text = f"{name}: {msg}"
    if status in (FLK_ERR_BAD_ARG, FLK_ERR_LAYOUT):
        raise ValueError(text)
    if status == FLK_ERR_WORKSPACE:
        raise MemoryError(text)
    if status == FLK_ERR_UNSUPPORTED:
        raise NotImplementedError(text)
    raise FlkError(status, text)


# ---------------------------------------------------------------------------------------------
# workspace cache: one growing byte buffer per device, handed to the C ABI (which never allocates)
# ---------------------------------------------------------------------------------------------
_workspaces = {}

# Resident operands.  What a product prepares from X1 and X2 (operand images, scaled rows and norms, the range
# check) stays in the device's workspace after the call.  The next product on that workspace may keep it
# (FLK_FLAG_KEEP_X1 / _X2) when it is the same entry point with the same sizes, sigma, kernel and flags AND the
# operand is the same tensor, unchanged: same storage address, shape, strides, dtype and torch version counter
# (every in-place torch operation bumps the counter).  That is the pattern of a conjugate-gradient solve: the same
# X and centres in every iteration.  Tensors without a version counter (created under torch.inference_mode) are
# never kept.  The record is dropped whenever anything else touches the workspace.
_resident = {}


def _tensor_key(t: Optional[torch.Tensor]):
    if t is None:
        return None
    try:
        version = t._version
    except RuntimeError:  # inference tensors do not track versions: an in-place edit could not be noticed
        return None
    return (t.data_ptr(), tuple(t.shape), tuple(t.stride()), t.dtype, version)


def _keep_flags(dev_key, signature, key1, key2) -> int:
    rec = _resident.get(dev_key)
    if rec is None or rec[0] != signature:
        return 0
    keep = 0
    if key1 is not None and rec[1] == key1:
        keep |= FLAG_KEEP_X1
    if key2 is not None and rec[2] == key2:
        keep |= FLAG_KEEP_X2
    return keep


def forget_resident(device: Optional[torch.device] = None):
    """Drops the record of what the workspace(s) hold (a caller who edits operand memory behind torch's back --
    through a raw pointer or another library -- calls this before the next product)."""
    if device is None:
        _resident.clear()
    else:
        _resident.pop((device.type, device.index), None)


def workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    key = (device.type, device.index)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        _resident.pop(key, None)
        if buf is not None:
            del _workspaces[key]
            del buf
        buf = torch.empty(int(nbytes) + 4096, dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def release_workspaces():
    _workspaces.clear()
    _resident.clear()


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return FLK_F32
    if dtype == torch.float64:
        return FLK_F64
    raise TypeError(f"falkon_b200 supports float32 and float64 data, not {dtype}")


def _mat_args(t: Optional[torch.Tensor], with_rows: bool = True):
    if t is None:
        return [None, 0, 0, 0] if with_rows else [None, 0, 0]
    args = [ctypes.c_void_p(t.data_ptr())]
    if with_rows:
        args.append(t.shape[0])
    args += [t.stride(0), t.stride(1)]
    return args


def _sigma_args(sigma: np.ndarray):
    sigma = np.ascontiguousarray(sigma, dtype=np.float64).reshape(-1)
    return sigma, sigma.ctypes.data_as(_dp), sigma.shape[0]


def _check_operands(host: bool, **named):
    """Last line of defence before raw pointers cross the C ABI: every operand is a 2-D tensor of the expected
    shape, all share one dtype, and all live where the entry point will look for them (one CUDA device, or host
    memory for the host-buffer entry points).  A mismatch here would otherwise become an out-of-bounds access
    on the device; the reference raises a torch error for the same mistake."""
    tensors = {k: v for k, v in named.items() if v[0] is not None}
    dtype = device = None
    for name, (t, shape) in tensors.items():
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor, not {type(t).__name__}")
        if t.dim() != 2:
            raise ValueError(f"{name} must be 2-D, found {t.dim()}-D")
        if tuple(t.shape) != tuple(shape):
            raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {tuple(shape)}")
        if dtype is None:
            dtype, device = t.dtype, t.device
        if t.dtype != dtype:
            raise TypeError(f"Data types of input matrices must be equal ({name} is {t.dtype}, expected {dtype}).")
        if host:
            if t.device.type != "cpu":
                raise ValueError(f"{name} must be in host memory for the host-buffer entry points (found {t.device})")
        else:
            if t.device.type != "cuda":
                raise ValueError(f"{name} must be on a CUDA device (found {t.device})")
            if t.device != device:
                raise ValueError(f"All operands must be on the same device ({name} is on {t.device}, expected {device})")


def rows_within_budget(query, n: int, budget: Optional[float]) -> int:
    """Largest number of rows r <= n (a multiple of 512 unless r == n) whose workspace ``query(r)`` fits ``budget``
    bytes; n itself when there is no budget.  Raises MemoryError when even 512 rows do not fit, as the reference
    does when its block-size model cannot place a single block (falkon/utils/helpers.py:83-84)."""
    if budget is None or budget == float("inf") or query(n) <= budget:
        return n
    lo = 512
    if n <= lo or query(lo) > budget:
        raise MemoryError(
            f"Available memory ({budget / 2**20:.1f} MiB) is not enough for the workspace of even {min(n, lo)} rows "
            f"({query(min(n, lo)) / 2**20:.1f} MiB); raise max_gpu_mem")
    hi = n  # query(hi) > budget
    while hi - lo > 512:
        mid = (lo + hi) // 2 // 512 * 512
        if mid <= lo:
            break
        if query(mid) <= budget:
            lo = mid
        else:
            hi = mid
    # The workspace is not strictly monotonic in the row count (the sweep planner's choice of reduction chunks
    # moves the size of the partial-result buffers): make sure the shorter last chunk fits as well.
    for _ in range(32):
        last = n % lo
        if last == 0 or query(last) <= budget or lo <= 512:
            break
        lo = max(512, (lo * 15 // 16) // 512 * 512)
    return lo


def _resolve_budget(budget, need: int, device) -> Optional[float]:
    """None when the whole problem may run in one call, else the byte budget to chunk under.  ``budget`` is a number,
    None, or a callable ``budget(device) -> bytes or None`` that is only evaluated when the answer is not already
    clear: a problem whose workspace fits the buffer this package already holds on the device needs no query of
    the device's free memory (a driver call on every product would show up in short products)."""
    if budget is None:
        return None
    if callable(budget):
        limit = getattr(budget, "limit", float("inf"))
        held = _workspaces.get((device.type, device.index)) if device is not None else None
        if held is not None and need <= held.numel() and need <= limit:
            return None
        budget = budget(device)
        if budget is None:
            return None
    return None if need <= budget else float(budget)


def call_fmmv_budgeted(kernel_id, sigma, X1, X2, v, out, flags=0, host=False, device=None, budget=None):
    """``call_fmmv`` under a device-memory budget (bytes): when the workspace of the whole problem exceeds it, the
    larger operand is cut into row chunks -- rows of X1 produce independent rows of ``out``; rows of X2 (with the
    matching rows of v) are summed into ``out`` with FLK_FLAG_ACCUMULATE."""
    lib = load()
    dt = dtype_code(X1.dtype)
    n, d = X1.shape
    m = X2.shape[0]
    t = v.shape[1] if v.dim() == 2 else 1
    wsq = lib.flk_fmmv_host_workspace_bytes if host else lib.flk_fmmv_workspace_bytes
    budget = _resolve_budget(budget, wsq(dt, kernel_id, n, m, d, t, flags), device if host else X1.device)
    if budget is None:
        return call_fmmv(kernel_id, sigma, X1, X2, v, out, flags=flags, host=host, device=device)
    if n >= m:
        step = rows_within_budget(lambda r: wsq(dt, kernel_id, r, m, d, t, flags), n, budget)
        for r0 in range(0, n, step):
            call_fmmv(kernel_id, sigma, X1[r0:r0 + step], X2, v, out[r0:r0 + step], flags=flags, host=host, device=device)
        return out
    step = rows_within_budget(lambda r: wsq(dt, kernel_id, n, r, d, t, flags), m, budget)
    part = torch.empty_like(out) if host else None
    for i, r0 in enumerate(range(0, m, step)):
        if host:  # the host-buffer entry point writes host memory: sum the partial results there
            call_fmmv(kernel_id, sigma, X1, X2[r0:r0 + step], v[r0:r0 + step], out if i == 0 else part, flags=flags,
                      host=True, device=device)
            if i > 0:
                out.add_(part)
        else:
            call_fmmv(kernel_id, sigma, X1, X2[r0:r0 + step], v[r0:r0 + step], out,
                      flags=flags | (FLAG_ACCUMULATE if i > 0 else 0))
    return out


def call_fdmmv_budgeted(kernel_id, sigma, X1, X2, v, w, out, flags=0, host=False, device=None, budget=None):
    """``call_fdmmv`` under a device-memory budget (bytes): K^T (K v + w) is a sum over row blocks of X1 (the
    reference's own blocking, falkon/mmv_ops/fmmv.py:740-760), accumulated into ``out``."""
    lib = load()
    dt = dtype_code(X1.dtype)
    n, d = X1.shape
    m = X2.shape[0]
    lead = v if v is not None else w
    t = lead.shape[1] if lead is not None and lead.dim() == 2 else 1
    wsq = lib.flk_fdmmv_host_workspace_bytes if host else lib.flk_fdmmv_workspace_bytes
    budget = _resolve_budget(budget, wsq(dt, kernel_id, n, m, d, t, flags), device if host else X1.device)
    if budget is None:
        return call_fdmmv(kernel_id, sigma, X1, X2, v, w, out, flags=flags, host=host, device=device)
    step = rows_within_budget(lambda r: wsq(dt, kernel_id, r, m, d, t, flags), n, budget)
    part = torch.empty_like(out) if host else None
    for i, r0 in enumerate(range(0, n, step)):
        wc = None if w is None else w[r0:r0 + step]
        if host:
            call_fdmmv(kernel_id, sigma, X1[r0:r0 + step], X2, v, wc, out if i == 0 else part, flags=flags, host=True,
                       device=device)
            if i > 0:
                out.add_(part)
        else:
            call_fdmmv(kernel_id, sigma, X1[r0:r0 + step], X2, v, wc, out,
                       flags=flags | (FLAG_ACCUMULATE if i > 0 else 0))
    return out


def call_fmmv(kernel_id, sigma, X1, X2, v, out, flags=0, host=False, device=None):
    """out[n, t] = k(X1, X2) v through the C ABI (device pointers, or host pointers with host=True)."""
    lib = load()
    dt = dtype_code(X1.dtype)
    n, d = X1.shape
    m = X2.shape[0]
    t = v.shape[1] if v.dim() == 2 else -1
    _check_operands(host, X1=(X1, (n, d)), X2=(X2, (m, d)), v=(v, (m, t)), out=(out, (n, t)))
    dev = device if host else X1.device
    query = lib.flk_fmmv_host_workspace_bytes if host else lib.flk_fmmv_workspace_bytes
    need = query(dt, kernel_id, n, m, d, t, flags)
    if need < 0:
        raise_for_status(int(need))
    keep, sig_ptr, sig_len = _sigma_args(sigma)
    dev_key = (dev.type, dev.index)
    with torch.cuda.device(dev):
        ws = workspace(dev, need)
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        fn = lib.flk_fmmv_host if host else lib.flk_fmmv
        signature = key1 = key2 = None
        kept = 0
        if not host:
            signature = ("fmmv", dt, kernel_id, keep.tobytes(), n, m, d, t, flags, ws.data_ptr(), stream.value)
            key1, key2 = _tensor_key(X1), _tensor_key(X2)
            kept = _keep_flags(dev_key, signature, key1, key2)
        _resident.pop(dev_key, None)
        status = fn(dt, kernel_id, *_mat_args(X1), *_mat_args(X2), d,
                    ctypes.c_void_p(v.data_ptr()), t, v.stride(0), v.stride(1),
                    *_mat_args(out, with_rows=False), sig_ptr, sig_len,
                    ctypes.c_void_p(ws.data_ptr()), ws.numel(), flags | kept, stream)
        if status == 0 and signature is not None:
            _resident[dev_key] = (signature, key1, key2)
    del keep
    raise_for_status(status)
    return out


def call_fdmmv(kernel_id, sigma, X1, X2, v, w, out, flags=0, host=False, device=None):
    """out[m, t] = k(X1, X2)^T (k(X1, X2) v + w) through the C ABI."""
    lib = load()
    dt = dtype_code(X1.dtype)
    n, d = X1.shape
    m = X2.shape[0]
    if v is None and w is None:
        raise ValueError("One of v and w must be specified to run fdMMV.")
    lead = v if v is not None else w
    t = lead.shape[1] if lead.dim() == 2 else -1
    _check_operands(host, X1=(X1, (n, d)), X2=(X2, (m, d)), v=(v, (m, t)), w=(w, (n, t)), out=(out, (m, t)))
    dev = device if host else X1.device
    query = lib.flk_fdmmv_host_workspace_bytes if host else lib.flk_fdmmv_workspace_bytes
    need = query(dt, kernel_id, n, m, d, t, flags)
    if need < 0:
        raise_for_status(int(need))
    keep, sig_ptr, sig_len = _sigma_args(sigma)
    dev_key = (dev.type, dev.index)
    with torch.cuda.device(dev):
        ws = workspace(dev, need)
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        fn = lib.flk_fdmmv_host if host else lib.flk_fdmmv
        signature = key1 = key2 = None
        kept = 0
        if not host:
            signature = ("fdmmv", dt, kernel_id, keep.tobytes(), n, m, d, t, v is None, flags, ws.data_ptr(),
                         stream.value)
            key1, key2 = _tensor_key(X1), _tensor_key(X2)
            kept = _keep_flags(dev_key, signature, key1, key2)
        _resident.pop(dev_key, None)
        status = fn(dt, kernel_id, *_mat_args(X1), *_mat_args(X2), d,
                    *_mat_args(v, with_rows=False), *_mat_args(w, with_rows=False), t,
                    *_mat_args(out, with_rows=False), sig_ptr, sig_len,
                    ctypes.c_void_p(ws.data_ptr()), ws.numel(), flags | kept, stream)
        if status == 0 and signature is not None:
            _resident[dev_key] = (signature, key1, key2)
    del keep
    raise_for_status(status)
    return out


def call_fmm(kernel_id, sigma, X1, X2, out, flags=0):
    """out[n, m] = k(X1, X2) through the C ABI (device pointers)."""
    lib = load()
    dt = dtype_code(X1.dtype)
    n, d = X1.shape
    m = X2.shape[0]
    dev = X1.device
    _check_operands(False, X1=(X1, (n, d)), X2=(X2, (m, d)), out=(out, (n, m)))
    need = lib.flk_fmm_workspace_bytes(dt, n, m, d, flags)
    if need < 0:
        raise_for_status(int(need))
    keep, sig_ptr, sig_len = _sigma_args(sigma)
    with torch.cuda.device(dev):
        ws = workspace(dev, need)
        forget_resident(dev)
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        status = lib.flk_fmm(dt, kernel_id, *_mat_args(X1), *_mat_args(X2), d, *_mat_args(out, with_rows=False),
                             sig_ptr, sig_len, ctypes.c_void_p(ws.data_ptr()), ws.numel(), flags, stream)
    del keep
    raise_for_status(status)
    return out


def call_kgrad(kernel_id, sigma, X1, X2, G, v, out, flags=0):
    """out[n, m] = 2 k'(D2_ij) s_ij through the C ABI: s = G v^T (G n x t, v m x t) or, with v None, s = G (n x m)."""
    lib = load()
    dt = dtype_code(X1.dtype)
    n, d = X1.shape
    m = X2.shape[0]
    dev = X1.device
    if v is None:
        _check_operands(False, X1=(X1, (n, d)), X2=(X2, (m, d)), G=(G, (n, m)), out=(out, (n, m)))
    else:
        tg = G.shape[1] if G.dim() == 2 else -1
        _check_operands(False, X1=(X1, (n, d)), X2=(X2, (m, d)), G=(G, (n, tg)), v=(v, (m, tg)), out=(out, (n, m)))
    need = lib.flk_fmm_workspace_bytes(dt, n, m, d, flags)
    if need < 0:
        raise_for_status(int(need))
    keep, sig_ptr, sig_len = _sigma_args(sigma)
    with torch.cuda.device(dev):
        ws = workspace(dev, need)
        forget_resident(dev)
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        if v is None:
            v_args = (None, 0, 0, 0)
        else:
            v_args = (ctypes.c_void_p(v.data_ptr()), v.shape[1], v.stride(0), v.stride(1))
        status = lib.flk_kgrad(dt, kernel_id, *_mat_args(X1), *_mat_args(X2), d,
                               ctypes.c_void_p(G.data_ptr()), G.stride(0), G.stride(1), *v_args,
                               *_mat_args(out, with_rows=False), sig_ptr, sig_len,
                               ctypes.c_void_p(ws.data_ptr()), ws.numel(), flags, stream)
    del keep
    raise_for_status(status)
    return out


def call_square_norm(X, sigma=None, out=None):
    """out[n] = sum_k (X[i, k] / sigma)^2 through the C ABI (device pointers; ``sigma`` a scalar or None)."""
    lib = load()
    dt = dtype_code(X.dtype)
    if X.dim() != 2:
        raise ValueError(f"X must be 2-D, found {X.dim()}-D")
    if X.device.type != "cuda":
        raise ValueError(f"X must be on a CUDA device (found {X.device})")
    n, d = X.shape
    if out is None:
        out = torch.empty(n, dtype=X.dtype, device=X.device)
    if out.shape != (n,) or out.dtype != X.dtype or out.device != X.device or (n > 1 and out.stride(0) != 1):
        raise ValueError("out must be a dense vector of n entries with the dtype and device of X")
    if sigma is None:
        keep, sig_ptr, sig_len = None, None, 0
    else:
        keep, sig_ptr, sig_len = _sigma_args(np.atleast_1d(np.asarray(sigma, dtype=np.float64)))
    with torch.cuda.device(X.device):
        stream = ctypes.c_void_p(torch.cuda.current_stream(X.device).cuda_stream)
        status = lib.flk_square_norm(dt, ctypes.c_void_p(X.data_ptr()), n, d, X.stride(0), X.stride(1), sig_ptr,
                                     sig_len, ctypes.c_void_p(out.data_ptr()), stream)
    del keep
    raise_for_status(status)
    return out


def tc_status(device: torch.device) -> int:
    """Status word of the last tensor-core launch that used this device's cached workspace."""
    lib = load()
    key = (device.type, device.index)
    if key not in _workspaces:
        return 0
    out = ctypes.c_int(0)
    with torch.cuda.device(device):
        stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        raise_for_status(lib.flk_tc_status(ctypes.c_void_p(_workspaces[key].data_ptr()), stream, ctypes.byref(out)))
    return out.value


def range_flag(device: torch.device) -> int:
    """1 when the last tensor-core-eligible call on this device's cached workspace switched to the
    SIMT kernels because some row did not fit the fp16 operand images, else 0."""
    lib = load()
    key = (device.type, device.index)
    if key not in _workspaces:
        return 0
    out = ctypes.c_int(0)
    with torch.cuda.device(device):
        stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        raise_for_status(lib.flk_range_flag(ctypes.c_void_p(_workspaces[key].data_ptr()), stream, ctypes.byref(out)))
    return out.value


def measure_mufu_rate(device: torch.device, iters: int = 4096, reps: int = 5) -> float:
    """ex2 evaluations per second of `device`, measured with the library's probe kernel and CUDA events
    (best of `reps`; the first launch is a warm-up)."""
    lib = load()
    with torch.cuda.device(device):
        sink = torch.zeros(4, dtype=torch.float32, device=device)
        stream = torch.cuda.current_stream(device)
        ops = _i64(0)
        best = None
        for r in range(reps + 1):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            raise_for_status(lib.flk_probe_mufu(iters, ctypes.c_void_p(sink.data_ptr()), ctypes.byref(ops),
                                                ctypes.c_void_p(stream.cuda_stream)))
            e1.record(stream)
            e1.synchronize()
            ms = e0.elapsed_time(e1)
            if r > 0:
                best = ms if best is None else min(best, ms)
    return float(ops.value) / (best * 1e-3)


def set_timing(enable: bool):
    raise_for_status(load().flk_set_timing(1 if enable else 0))


def sweep_ms():
    """(sweep 1 ms, sweep 2 ms) of the most recent timed call; -1 where the sweep did not run."""
    a, b = ctypes.c_float(-1), ctypes.c_float(-1)
    raise_for_status(load().flk_get_sweep_ms(ctypes.byref(a), ctypes.byref(b)))
    return a.value, b.value


def launch_count() -> int:
    return int(load().flk_launch_count())
