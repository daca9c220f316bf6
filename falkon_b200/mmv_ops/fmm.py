"""``fmm``: the kernel matrix ``k(X1, X2)`` itself, on the B200.

Counterpart of the reference's function of the same name (falkon/mmv_ops/fmm.py:575-640), which the
preconditioner calls once per fit on the Nystrom centres (falkon/preconditioner/flk_preconditioner.py:89).
Same keyword signature, same output-allocation rule, and the reference's ``no_single_kernel``
behaviour: fp32 data is evaluated in fp64 and rounded once when stored (falkon/mmv_ops/fmm.py:619-622).
One call into the C ABI (``flk_fmm``); no CPU path.
"""
from typing import Dict, Optional

import torch

from .. import _lib
from ..options import BaseOptions
from .fmmv import _dense_grad, _is_sparse, _kernel_spec, _pick_device, _require_cuda, _to_dev
from .utils import check_contiguity, create_same_stride

__all__ = ("fmm", "KernelMmFn", "compute_block")


def _diag_kernel(X1, X2, kernel_id, sigma, out):
    """k(x1_i, x2_i) for paired rows: one pass of element-wise torch ops (never on a hot path)."""
    s = torch.as_tensor(sigma, dtype=torch.float64, device=X1.device)
    d2 = (((X1.double() / s) - (X2.double() / s)) ** 2).sum(dim=1).clamp_min_(1e-20)
    if kernel_id == _lib.FLK_GAUSSIAN:
        k = torch.exp(-0.5 * d2)
    elif kernel_id == _lib.FLK_LAPLACIAN:
        k = torch.exp(-torch.sqrt(d2))
    elif kernel_id == _lib.FLK_MATERN15:
        r = torch.sqrt(3.0 * d2)
        k = (1.0 + r) * torch.exp(-r)
    else:
        r = torch.sqrt(5.0 * d2)
        k = (1.0 + r + (5.0 / 3.0) * d2) * torch.exp(-r)
    out.copy_(k.to(out.dtype))
    return out


def _diag_kernel_autograd(X1, X2, kernel_id, sigma):
    """Differentiable k(x1_i, x2_i) for paired rows, as plain torch ops in the data's dtype
    (the reference's diagonal cores, falkon/kernels/distance_kernel.py:128-137, under autograd)."""
    s = sigma.to(device=X1.device, dtype=X1.dtype)
    d2 = (((X1 / s) - (X2.to(X1.device) / s)) ** 2).sum(dim=1)
    if kernel_id == _lib.FLK_GAUSSIAN:
        return torch.exp(-0.5 * d2)
    r = torch.sqrt(d2.clamp_min(1e-20))
    if kernel_id == _lib.FLK_LAPLACIAN:
        return torch.exp(-r)
    if kernel_id == _lib.FLK_MATERN15:
        r = r * 3.0**0.5
        return (1.0 + r) * torch.exp(-r)
    r = r * 5.0**0.5
    return (1.0 + r + r * r / 3.0) * torch.exp(-r)


def _fmm_forward(kernel, opt, out, diag, X1, X2):
    kernel_id, sigma = _kernel_spec(kernel)
    n, m = X1.shape[0], X2.shape[0]
    if out is None:  # created outside inference mode, as in the reference: the caller may update it in place
        out_dev = X1.device
        if diag:
            out = torch.empty((n,), dtype=X1.dtype, device=out_dev)
        else:
            out = create_same_stride((n, m), X1, X1.dtype, device=out_dev, pin_memory=out_dev.type != "cuda")
    with torch.inference_mode():
        dev = _pick_device((X1.device, X2.device, out.device))
        o_dev = out if out.device == dev else torch.empty(out.shape, dtype=out.dtype, device=dev)
        if diag:
            _diag_kernel(_to_dev(X1, dev), _to_dev(X2, dev), kernel_id, sigma, o_dev)
            if o_dev is not out:
                out.copy_(o_dev)
            return out
        _lib.call_fmm(kernel_id, sigma, _to_dev(X1, dev), _to_dev(X2, dev), o_dev, flags=_fmm_flags(X1, opt))
        if o_dev is not out:
            out.copy_(o_dev)
    return out


def _fmm_flags(X1, opt) -> int:
    if X1.dtype == torch.float32 and getattr(opt, "no_single_kernel", True):
        return _lib.FLAG_FP64_MATH
    return 0


class KernelMmFn(torch.autograd.Function):
    """``k(X1, X2)`` with a backward pass (the role of KernelMmFnFull in falkon/mmv_ops/fmm.py): gradients
    flow to X1, X2 and the kernel's ``sigma`` through the pair weights of ``flk_kgrad``."""

    @staticmethod
    def forward(ctx, kernel, opt, out, param_names, X1, X2, *params):
        if out is not None:
            ctx.mark_dirty(out)
        res = _fmm_forward(kernel, opt, out, False, X1.detach(), X2.detach())
        ctx.save_for_backward(X1, X2, *params)
        ctx.kernel, ctx.opt, ctx.param_names = kernel, opt, param_names
        return res

    @staticmethod
    def backward(ctx, grad_out):
        from .grad import kernel_backward

        X1, X2, *params = ctx.saved_tensors
        kernel_id, _ = _kernel_spec(ctx.kernel)
        dev = _pick_device((X1.device, X2.device, grad_out.device))
        sigma_idx = ctx.param_names.index("sigma") if "sigma" in ctx.param_names else None
        needs = [ctx.needs_input_grad[4], ctx.needs_input_grad[5], False,
                 sigma_idx is not None and ctx.needs_input_grad[6 + sigma_idx]]
        sigma = params[sigma_idx] if sigma_idx is not None else ctx.kernel.sigma
        with torch.no_grad():
            g = kernel_backward(kernel_id, sigma, _to_dev(X1, dev), _to_dev(X2, dev),
                                _to_dev(_dense_grad(grad_out, X1.dtype), dev), None, needs, flags=_fmm_flags(X1, ctx.opt))
        gx1 = None if g[0] is None else g[0].to(X1.device)
        gx2 = None if g[1] is None else g[1].to(X2.device)
        param_grads = [None] * len(params)
        if sigma_idx is not None:
            param_grads[sigma_idx] = g[3]
        return (None, None, None, None, gx1, gx2, *param_grads)


def fmm(
    kernel,
    opt: Optional[BaseOptions],
    out: Optional[torch.Tensor],
    diag: bool,
    X1: torch.Tensor,
    X2: torch.Tensor,
    kwargs_m1: Optional[Dict[str, torch.Tensor]] = None,
    kwargs_m2: Optional[Dict[str, torch.Tensor]] = None,
) -> torch.Tensor:
    """``k(X1, X2)`` -> (n x m), or its diagonal (n,) with ``diag=True``.  Differentiable with respect to
    X1, X2 and the kernel's ``sigma`` when any of them requires a gradient."""
    if _is_sparse(X1, X2):
        raise NotImplementedError("Sparse kernel matrices are not implemented by falkon_b200.")
    if kwargs_m1 or kwargs_m2:
        raise NotImplementedError("Distance kernels take no per-row keyword tensors (kwargs_m1 / kwargs_m2).")
    if getattr(kernel, "_flk_spec", None) is None and callable(getattr(kernel, "compute", None)):
        # a kernel that only implements `compute` (the reference's extension contract): its own code fills the block
        check_contiguity((X1, "X1"), (X2, "X2"), (out, "out"))
        _require_cuda(opt, X1, X2)
        dev = _pick_device((X1.device, X2.device) + (() if out is None else (out.device,)))
        if out is None:
            shape = (X1.shape[0],) if diag else (X1.shape[0], X2.shape[0])
            out = torch.empty(shape, dtype=X1.dtype, device=X1.device)
        o_dev = out if out.device == dev else torch.empty(out.shape, dtype=out.dtype, device=dev)
        res = kernel.compute(_to_dev(X1, dev), _to_dev(X2, dev), o_dev, diag)
        if res is not out:
            out.copy_(res)
        return out
    kernel_id, _ = _kernel_spec(kernel)
    check_contiguity((X1, "X1"), (X2, "X2"), (out, "out"))
    _require_cuda(opt, X1, X2)
    diff_params = getattr(kernel, "diff_params", {})
    if torch.is_grad_enabled() and any(t.requires_grad for t in [X1, X2] + list(diff_params.values())):
        if diag:
            res = _diag_kernel_autograd(X1, X2, kernel_id, kernel.sigma)
            if out is not None:
                raise ValueError("an `out` tensor cannot be combined with a differentiable diagonal")
            return res
        names = tuple(diff_params.keys())
        return KernelMmFn.apply(kernel, opt, out, names, X1, X2, *diff_params.values())
    return _fmm_forward(kernel, opt, out, diag, X1, X2)


class _PlainMath:
    """Options stand-in for ``compute_block``: evaluate in the dtype of the data."""

    no_single_kernel = False
    use_cpu = False


def compute_block(kernel, X1: torch.Tensor, X2: torch.Tensor, out: Optional[torch.Tensor], diag: bool) -> torch.Tensor:
    """``Kernel.compute``: the dense block (or its diagonal) into ``out``, in the data's own precision.
    Validates like ``Kernel.__call__``; differentiable like ``fmm``."""
    from ..kernels.kernel import Kernel

    X1, X2, out = Kernel._check_mm_dimensions(X1, X2, diag, out)
    return fmm(kernel, _PlainMath, out, diag, X1, X2)
