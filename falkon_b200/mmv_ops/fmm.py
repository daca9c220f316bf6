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
from .fmmv import _is_sparse, _kernel_spec, _pick_device, _require_cuda, _to_dev
from .utils import check_contiguity, create_same_stride

__all__ = ("fmm",)


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
    """``k(X1, X2)`` -> (n x m), or its diagonal (n,) with ``diag=True``."""
    if _is_sparse(X1, X2):
        raise NotImplementedError("Sparse kernel matrices are not implemented by falkon_b200.")
    if kwargs_m1 or kwargs_m2:
        raise NotImplementedError("Distance kernels take no per-row keyword tensors (kwargs_m1 / kwargs_m2).")
    kernel_id, sigma = _kernel_spec(kernel)
    params = list(getattr(kernel, "diff_params", {}).values())
    if torch.is_grad_enabled() and any(t.requires_grad for t in [X1, X2] + params):
        raise NotImplementedError(
            "falkon_b200 does not implement the backward pass of the kernel matrix; "
            "call it under torch.no_grad() / inference_mode() or detach the inputs."
        )
    check_contiguity((X1, "X1"), (X2, "X2"), (out, "out"))
    _require_cuda(opt, X1, X2)
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
        flags = 0
        if X1.dtype == torch.float32 and getattr(opt, "no_single_kernel", True):
            flags |= _lib.FLAG_FP64_MATH
        _lib.call_fmm(kernel_id, sigma, _to_dev(X1, dev), _to_dev(X2, dev), o_dev, flags=flags)
        if o_dev is not out:
            out.copy_(o_dev)
    return out
