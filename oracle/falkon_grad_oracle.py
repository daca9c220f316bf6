"""CPU restatement of the backward pass of Falkon's kernel products (test infrastructure only).

The reference differentiates ``k(X1, X2) @ v`` and ``k(X1, X2)`` by re-running each kernel block without
in-place output (``compute_diff``, falkon/kernels/diff_kernel.py:93-113) under autograd and calling
``torch.autograd.grad`` on it with the upstream gradient (``mmv_diff_run_thread``,
falkon/mmv_ops/fmmv.py:405-485; ``KernelMmFnFull.backward`` in falkon/mmv_ops/fmm.py).  This module restates
that on the CPU in torch operations with the same arithmetic: sigma cast to the data dtype
(falkon/kernels/distance_kernel.py:148), rows divided by sigma, squared distances by the ``addmm`` norm
expansion and the clamp at 1e-20 (:88-101), the radial profile of each kernel (:140-159, :182-204,
:228-271), then autograd.  It also provides the closed form of the pair weights
``W_ij = 2 k'(D2_ij) s_ij`` that the CUDA library's ``flk_kgrad`` computes, for the tests of the host-side
gradient algebra.

It is not part of the product: only the test-suite imports it.  Parity pinning: tests/test_grad_oracle.py
checks it against gradients computed by the reference itself (tests/golden/make_golden_grad.py ->
tests/golden/grad_*.npz).
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch

SQRT3 = math.sqrt(3.0)
SQRT5 = math.sqrt(5.0)


def _canonical(kernel: str, nu: Optional[float]):
    if kernel == "matern":
        if nu == 0.5:
            return "laplacian", None
        if nu == float("inf"):
            return "gaussian", None
        if nu not in (1.5, 2.5):
            raise ValueError("nu must be one of 0.5, 1.5, 2.5, inf")
        return "matern", nu
    if kernel not in ("gaussian", "laplacian"):
        raise ValueError(f"unknown kernel {kernel!r}")
    return kernel, None


def _sq_dist(x1: torch.Tensor, x2: torch.Tensor, sigma: torch.Tensor) -> torch.Tensor:
    s = sigma.to(dtype=x1.dtype)
    a = x1 / s
    b = x2 / s
    an = (a * a).sum(dim=1, keepdim=True)
    bn = (b * b).sum(dim=1, keepdim=True)
    d2 = torch.addmm(an, a, b.t(), alpha=-2.0, beta=1.0)
    d2 = d2 + bn.t()
    return d2.clamp_min(1e-20)


def kernel_block_diff(x1, x2, kernel: str, sigma: torch.Tensor, nu: Optional[float] = None) -> torch.Tensor:
    """Differentiable dense block k(x1, x2) (out-of-place restatement of the reference's cores)."""
    kernel, nu = _canonical(kernel, nu)
    d2 = _sq_dist(x1, x2, sigma)
    if kernel == "gaussian":
        return torch.exp(-0.5 * d2)
    r = torch.sqrt(d2)
    if kernel == "laplacian":
        return torch.exp(-r)
    if nu == 1.5:
        r = r * SQRT3
        return (1.0 + r) * torch.exp(-r)
    r = r * SQRT5
    return (d2 * (5.0 / 3.0) + r + 1.0) * torch.exp(-r)


def mmv_grads(x1, x2, v, g, kernel: str, sigma, nu: Optional[float] = None):
    """Gradients of sum(g * (k(x1, x2) @ v)) with respect to x1, x2, v and sigma (an fp64 vector of 1 or d
    entries, as the reference stores it), as numpy arrays."""
    x1, x2, v = (torch.as_tensor(a).clone().requires_grad_() for a in (x1, x2, v))
    sig = torch.as_tensor(np.atleast_1d(np.asarray(sigma, dtype=np.float64))).clone().requires_grad_()
    out = kernel_block_diff(x1, x2, kernel, sig, nu) @ v
    grads = torch.autograd.grad(out, [x1, x2, v, sig], grad_outputs=torch.as_tensor(g))
    return tuple(t.numpy() for t in grads)


def mm_grads(x1, x2, s, kernel: str, sigma, nu: Optional[float] = None):
    """Gradients of sum(s * k(x1, x2)) with respect to x1, x2 and sigma, as numpy arrays."""
    x1, x2 = (torch.as_tensor(a).clone().requires_grad_() for a in (x1, x2))
    sig = torch.as_tensor(np.atleast_1d(np.asarray(sigma, dtype=np.float64))).clone().requires_grad_()
    out = kernel_block_diff(x1, x2, kernel, sig, nu)
    grads = torch.autograd.grad(out, [x1, x2, sig], grad_outputs=torch.as_tensor(s))
    return tuple(t.numpy() for t in grads)


def pair_weights(x1, x2, upstream, v, kernel: str, sigma, nu: Optional[float] = None) -> torch.Tensor:
    """``W_ij = 2 k'(D2_ij) s_ij`` in closed form; ``s = upstream @ v^T`` (or ``upstream`` itself when ``v``
    is None); zero where the squared distance is clamped."""
    kernel, nu = _canonical(kernel, nu)
    x1, x2, upstream = (torch.as_tensor(a) for a in (x1, x2, upstream))
    sig = torch.as_tensor(np.atleast_1d(np.asarray(sigma, dtype=np.float64)))
    s = sig.to(dtype=x1.dtype)
    a, b = x1 / s, x2 / s
    raw = torch.addmm((a * a).sum(1, keepdim=True), a, b.t(), alpha=-2.0) + (b * b).sum(1, keepdim=True).t()
    d2 = raw.clamp_min(1e-20)
    r = torch.sqrt(d2)
    if kernel == "gaussian":
        w = -torch.exp(-0.5 * d2)
    elif kernel == "laplacian":
        w = -torch.exp(-r) / r
    elif nu == 1.5:
        w = -3.0 * torch.exp(-SQRT3 * r)
    else:
        w = (-5.0 / 3.0) * (1.0 + SQRT5 * r) * torch.exp(-SQRT5 * r)
    w = torch.where(raw < 1e-20, torch.zeros_like(w), w)
    pair = upstream if v is None else upstream @ torch.as_tensor(v).t()
    return w * pair
