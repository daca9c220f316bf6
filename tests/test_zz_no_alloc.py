"""flk_fmmv_static: the entry point for callers that cannot allocate device memory.

Some embedders (a plug-in inside an application that owns all device memory, a real-time loop that
must avoid cudaMalloc's synchronisation) have no workspace to hand to flk_fmmv.  flk_fmmv_static
uses a fixed array inside the library instead.  This test drives it through the C ABI and checks it
against the regular entry point on two calls in a row (the second, smaller call sees the first
call's leftovers in the shared array), and checks that an oversized problem is refused.

Collected last on purpose: a failure here cannot hide any other test's result under `-x`.
"""
import ctypes

import numpy as np
import pytest
import torch

from falkon_b200 import _lib

pytestmark = pytest.mark.gpu


def _mat(t):
    return [ctypes.c_void_p(t.data_ptr()), t.shape[0], t.stride(0), t.stride(1)]


def _regular(lib, dt, kid, X, C, v, sigma, flags):
    n, d = X.shape
    m, t = v.shape
    out = torch.empty(n, t, dtype=X.dtype, device=X.device)
    need = lib.flk_fmmv_workspace_bytes(dt, kid, n, m, d, t, flags)
    assert need > 0
    ws = torch.empty(need + 256, dtype=torch.uint8, device=X.device)
    base = (ws.data_ptr() + 255) // 256 * 256
    sig = (ctypes.c_double * 1)(sigma)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    st = lib.flk_fmmv(dt, kid, *_mat(X), *_mat(C), d, ctypes.c_void_p(v.data_ptr()), t, v.stride(0), v.stride(1),
                      ctypes.c_void_p(out.data_ptr()), out.stride(0), out.stride(1), sig, 1,
                      ctypes.c_void_p(base), need, flags, stream)
    assert st == 0, _lib.last_error()
    torch.cuda.synchronize()
    return out


def _static(lib, dt, kid, X, C, v, sigma, flags):
    n, d = X.shape
    m, t = v.shape
    out = torch.full((n, t), float("nan"), dtype=X.dtype, device=X.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    st = lib.flk_fmmv_static(dt, kid, *_mat(X), *_mat(C), d, ctypes.c_void_p(v.data_ptr()), t, v.stride(0),
                             v.stride(1), ctypes.c_void_p(out.data_ptr()), out.stride(0), out.stride(1),
                             ctypes.c_double(sigma), flags, stream)
    assert st == 0, _lib.last_error()
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("dtype,flags", [(torch.float32, 0), (torch.float32, 1), (torch.float64, 0)],
                         ids=["f32-tensorcore", "f32-simt", "f64-simt"])
def test_static_scratch_entry_point_matches_regular_entry_point(dtype, flags):
    lib = _lib.load()
    dt = _lib.dtype_code(dtype)
    g = torch.Generator(device="cuda").manual_seed(11)
    tol = 1e-4 if dtype == torch.float32 else 1e-10
    # first a larger problem, then a smaller one of another shape: the second call starts from a
    # scratch array full of the first call's data
    for (n, m, d, t, kid, sigma) in [(30_000, 2_500, 28, 1, _lib.FLK_GAUSSIAN, 5.0),
                                     (1_111, 333, 7, 3, _lib.FLK_MATERN25, 2.0)]:
        X = torch.randn(n, d, generator=g, device="cuda", dtype=dtype)
        C = X[:m].clone()
        v = torch.randn(m, t, generator=g, device="cuda", dtype=dtype)
        want = _regular(lib, dt, kid, X, C, v, sigma, flags)
        got = _static(lib, dt, kid, X, C, v, sigma, flags)
        assert torch.isfinite(got).all()
        err = float((got.double() - want.double()).norm() / want.double().norm())
        assert err <= tol, f"n={n} m={m} d={d} t={t}: rel-L2 {err:.3e}"


def test_static_scratch_entry_point_refuses_oversized_problems():
    lib = _lib.load()
    n, m, d, t = 400_000, 20_000, 28, 1
    assert lib.flk_fmmv_workspace_bytes(0, 0, n, m, d, t, 0) > _lib.STATIC_SCRATCH_BYTES
    X = torch.zeros(8, d, device="cuda")  # never dereferenced: the size check comes first
    v = torch.zeros(8, 1, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    st = lib.flk_fmmv_static(0, 0, ctypes.c_void_p(X.data_ptr()), n, d, 1, ctypes.c_void_p(X.data_ptr()), m, d, 1, d,
                             ctypes.c_void_p(v.data_ptr()), t, 1, 1, ctypes.c_void_p(v.data_ptr()), 1, 1,
                             ctypes.c_double(5.0), 0, stream)
    assert st == _lib.FLK_ERR_WORKSPACE
    msg = _lib.last_error()
    assert "flk_fmmv_static" in msg and "bytes" in msg
    torch.cuda.synchronize()
