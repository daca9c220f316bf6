"""``fmmv`` and ``fdmmv``: implicit kernel-matrix / vector products on the B200.

Drop-in for the functions of the same name in the reference (falkon/mmv_ops/fmmv.py:960-973 and
:976-1131): same positional / keyword signatures, same output-allocation rules, same exception
types.  Where the reference loops over row blocks, materialises each n_blk x m kernel block in
device memory and calls cuBLAS twice, these functions make one call into the C ABI of
``libfalkon_b200`` (include/falkon_b200.h), whose CUDA kernels keep the block in registers /
tensor memory.  There is no CPU path: ``use_cpu=True`` or a missing GPU raises.
"""
from typing import Dict, Optional

import torch

from .. import _lib
from ..options import BaseOptions
from . import multi_device
from .utils import check_contiguity, create_output_mat

__all__ = ("fmmv", "fdmmv", "KernelMmvFn")


def _kernel_spec(kernel):
    """(kernel id for the C ABI, sigma as fp64 numpy vector) of a distance-kernel object."""
    spec = getattr(kernel, "_flk_spec", None)
    if spec is None:
        raise NotImplementedError(
            f"falkon_b200 computes kernel-vector products for Gaussian, Laplacian and Matern kernels; "
            f"{type(kernel).__name__} does not describe itself to the CUDA library (no _flk_spec)."
        )
    return spec()


def _is_user_defined(kernel) -> bool:
    """A kernel that only implements ``compute`` (the reference's extension contract): its products run block by
    block through that ``compute`` on the GPU (mmv_ops/generic.py), not through the fused CUDA kernels."""
    return getattr(kernel, "_flk_spec", None) is None and callable(getattr(kernel, "compute", None))


def _generic_product(which, X1, X2, v, w, kernel, out, opt):
    from . import generic

    _require_cuda(opt, X1, X2)
    tensors = [t for t in (X1, X2, v, w) if t is not None]
    data_devs = [t.device for t in tensors]
    lead = v if v is not None else w
    rows = X1.shape[0] if which == "mmv" else X2.shape[0]
    out = create_output_mat(out, data_devs, (rows, lead.shape[1]), lead.dtype, "cuda", X1)
    with torch.inference_mode():
        dev = _pick_device(tuple(data_devs) + (out.device,))
        budget = device_budget(opt, dev)
        o_dev = out if out.device == dev else torch.empty(out.shape, dtype=out.dtype, device=dev)
        if which == "mmv":
            generic.generic_fmmv(X1, X2, v, kernel, o_dev, dev, budget)
        else:
            generic.generic_fdmmv(X1, X2, v, w, kernel, o_dev, dev, budget)
        if o_dev is not out:
            out.copy_(o_dev)
    return out


def _require_cuda(opt: Optional[BaseOptions], *tensors):
    if opt is not None and getattr(opt, "use_cpu", False):
        raise RuntimeError(
            "falkon_b200 has no CPU implementation of the kernel-vector products (use_cpu=True was requested). "
            "Use the reference package for CPU execution."
        )
    if not torch.cuda.is_available():
        raise RuntimeError("falkon_b200 needs a CUDA device (B200, sm_100); none is available.")


class _DebugTimer:
    """``opt.debug = True``: per-call timing report of a product, the role of the reference's ``TicToc`` around its
    kernel calls (falkon/utils/tictoc.py:19-63, used at falkon/optim/conjgrad.py:245).  Device times come from the
    CUDA events the library records around its sweep launches (``flk_set_timing``) and from an event pair around
    the whole call; reading them synchronises, which is why this is off unless asked for."""

    def __init__(self, opt, what: str, dev: torch.device, shape_note: str):
        self.on = bool(getattr(opt, "debug", False)) and dev.type == "cuda"
        self.what, self.dev, self.note = what, dev, shape_note

    def __enter__(self):
        if self.on:
            _lib.set_timing(True)
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e1 = torch.cuda.Event(enable_timing=True)
            self.e0.record(torch.cuda.current_stream(self.dev))
        return self

    def __exit__(self, exc_type, exc, tb):
        if not self.on:
            return False
        self.e1.record(torch.cuda.current_stream(self.dev))
        self.e1.synchronize()
        s1, s2 = _lib.sweep_ms()
        _lib.set_timing(False)
        if exc_type is None:
            sweeps = ", ".join(f"sweep {i + 1} {ms:.3f} ms" for i, ms in enumerate((s1, s2)) if ms >= 0)
            print(f"[falkon_b200] {self.what} {self.note}: {self.e0.elapsed_time(self.e1):.3f} ms on {self.dev}"
                  + (f" ({sweeps})" if sweeps else ""), flush=True)
        return False


def _is_sparse(*xs):
    return any(type(x).__name__ == "SparseTensor" or (isinstance(x, torch.Tensor) and x.is_sparse) for x in xs)


def _flags(opt) -> int:
    return int(getattr(opt, "flk_flags", 0) or 0)


def device_budget(opt, dev: torch.device) -> Optional[float]:
    """Bytes the products may take on ``dev`` for their workspace: ``min(free, max_gpu_mem) * memory_slack``, the
    reference's rule (falkon/mmv_ops/utils.py:47-57); "free" counts the cached workspace of this package as
    available, since it is what would be reused.  None when neither limit binds (max_gpu_mem = inf and no way to
    ask the device, e.g. in CPU-only tests)."""
    limit = float(getattr(opt, "max_gpu_mem", float("inf")) or float("inf")) if opt is not None else float("inf")
    slack = float(getattr(opt, "memory_slack", 0.9) or 0.9) if opt is not None else 0.9
    free = float("inf")
    if torch.cuda.is_available() and dev.type == "cuda":
        try:
            free_now, _ = torch.cuda.mem_get_info(dev)
            held = _lib._workspaces.get((dev.type, dev.index))
            cached = torch.cuda.memory_reserved(dev) - torch.cuda.memory_allocated(dev)
            free = float(free_now + cached + (held.numel() if held is not None else 0))
        except Exception:  # pragma: no cover - a device that cannot be queried imposes no limit of its own
            free = float("inf")
    budget = min(free, limit)
    return None if budget == float("inf") else budget * slack


def lazy_budget(opt):
    """``device_budget`` as a callable for the ctypes layer, which asks only when it has to; ``limit`` is the part of
    the budget that is known without asking the device."""
    def ask(dev):
        return device_budget(opt, dev)

    limit = float(getattr(opt, "max_gpu_mem", float("inf")) or float("inf")) if opt is not None else float("inf")
    slack = float(getattr(opt, "memory_slack", 0.9) or 0.9) if opt is not None else 0.9
    ask.limit = limit * slack
    return ask


def _pick_device(devs):
    cuda = [d for d in devs if d.type == "cuda"]
    if cuda:
        if any(d != cuda[0] for d in cuda):
            raise RuntimeError("All CUDA input arguments must be on the same device")
        return cuda[0]
    return torch.device("cuda", torch.cuda.current_device())


def _to_dev(t, dev):
    return None if t is None else (t if t.device == dev else t.to(dev, non_blocking=True))


def _fmmv_forward(X1, X2, v, kernel, out, opt):
    """The product itself (no autograd bookkeeping); ``v`` is 2-D here."""
    kernel_id, sigma = _kernel_spec(kernel)
    data_devs = (X1.device, X2.device, v.device)
    n, t = X1.shape[0], v.shape[1]
    # created outside inference mode, as in the reference (fmmv.py:909-912): the caller may update it in place
    out = create_output_mat(out, data_devs, (n, t), v.dtype, "cuda", X1)
    with torch.inference_mode():
        dev = _pick_device(data_devs + (out.device,))
        all_host = all(d.type == "cpu" for d in data_devs) and out.device.type == "cpu"
        if all_host:
            devices = multi_device.host_devices(opt, n, dev)
            if len(devices) > 1:
                multi_device.fmmv_host_multi(kernel_id, sigma, X1, X2, v, out, _flags(opt), devices)
            else:
                _lib.call_fmmv_budgeted(kernel_id, sigma, X1, X2, v, out, flags=_flags(opt), host=True,
                                        device=devices[0], budget=lazy_budget(opt))
        else:
            o_dev = out if out.device == dev else torch.empty(out.shape, dtype=out.dtype, device=dev)
            with _DebugTimer(opt, "fmmv", dev, f"n={n} m={X2.shape[0]} d={X1.shape[1]} t={t}"):
                _lib.call_fmmv_budgeted(kernel_id, sigma, _to_dev(X1, dev), _to_dev(X2, dev), _to_dev(v, dev), o_dev,
                                        flags=_flags(opt), budget=lazy_budget(opt))
            if o_dev is not out:
                out.copy_(o_dev)
    return out


def _dense_grad(g: torch.Tensor, dtype) -> torch.Tensor:
    """Upstream gradients may arrive expanded (stride 0) or in another dtype; the library wants real memory
    with a unit stride."""
    g = g.to(dtype)
    ok = g.dim() == 2 and (g.stride(1) == 1 or g.stride(0) == 1) and all(
        st >= 1 or sz <= 1 for st, sz in zip(g.stride(), g.shape))
    return g if ok else g.contiguous()


def _grads_to(grads, like):
    return [None if g is None else g.to(device=t.device) for g, t in zip(grads, like)]


class KernelMmvFn(torch.autograd.Function):
    """``k(X1, X2) @ v`` with a backward pass (the role of KernelMmvFnFull, falkon/mmv_ops/fmmv.py:771-957).

    Forward is the fused product; backward evaluates the pair weights with ``flk_kgrad`` block by block
    (falkon_b200/mmv_ops/grad.py).  Gradients flow to X1, X2, v and to the kernel's ``sigma``.
    """

    @staticmethod
    def forward(ctx, kernel, opt, out, param_names, X1, X2, v, *params):
        if out is not None:
            ctx.mark_dirty(out)
        res = _fmmv_forward(X1.detach(), X2.detach(), v.detach(), kernel, out, opt)
        ctx.save_for_backward(X1, X2, v, *params)
        ctx.kernel, ctx.opt, ctx.param_names = kernel, opt, param_names
        return res

    @staticmethod
    def backward(ctx, grad_out):
        from .grad import kernel_backward

        X1, X2, v, *params = ctx.saved_tensors
        kernel_id, _ = _kernel_spec(ctx.kernel)
        dev = _pick_device((X1.device, X2.device, v.device, grad_out.device))
        sigma_idx = ctx.param_names.index("sigma") if "sigma" in ctx.param_names else None
        needs = list(ctx.needs_input_grad[4:7])
        needs.append(sigma_idx is not None and ctx.needs_input_grad[7 + sigma_idx])
        sigma = params[sigma_idx] if sigma_idx is not None else ctx.kernel.sigma
        with torch.no_grad():
            g = kernel_backward(
                kernel_id, sigma, _to_dev(X1, dev), _to_dev(X2, dev),
                _to_dev(_dense_grad(grad_out, X1.dtype), dev), _to_dev(v, dev), needs, flags=_flags(ctx.opt),
            )
        gx1, gx2, gv = _grads_to(g[:3], (X1, X2, v))
        param_grads = [None] * len(params)
        if sigma_idx is not None:
            param_grads[sigma_idx] = g[3]
        return (None, None, None, None, gx1, gx2, gv, *param_grads)


def fmmv(
    X1: torch.Tensor,
    X2: torch.Tensor,
    v: torch.Tensor,
    kernel,
    out: Optional[torch.Tensor] = None,
    opt: Optional[BaseOptions] = None,
    kwargs_m1: Optional[Dict[str, torch.Tensor]] = None,
    kwargs_m2: Optional[Dict[str, torch.Tensor]] = None,
) -> torch.Tensor:
    """``k(X1, X2) @ v`` -> (n x t).  Signature of falkon/mmv_ops/fmmv.py:960-969.

    Differentiable with respect to X1, X2, v and the kernel's ``sigma`` when any of them requires a
    gradient (and gradients are enabled), like the reference's ``KernelMmvFnFull``.
    """
    if _is_sparse(X1, X2):
        raise NotImplementedError("Sparse kernel-vector products are not implemented by falkon_b200.")
    if kwargs_m1 or kwargs_m2:
        raise NotImplementedError("Distance kernels take no per-row keyword tensors (kwargs_m1 / kwargs_m2).")
    if _is_user_defined(kernel):
        check_contiguity((X1, "X1"), (X2, "X2"), (v, "v"), (out, "out"))
        return _generic_product("mmv", X1, X2, v.reshape(-1, 1) if v.dim() == 1 else v, None, kernel, out, opt)
    _kernel_spec(kernel)
    check_contiguity((X1, "X1"), (X2, "X2"), (v, "v"), (out, "out"))
    _require_cuda(opt, X1, X2, v)
    if v.dim() == 1:
        v = v.reshape(-1, 1)
    diff_params = getattr(kernel, "diff_params", {})
    if torch.is_grad_enabled() and any(t.requires_grad for t in [X1, X2, v] + list(diff_params.values())):
        names = tuple(diff_params.keys())
        return KernelMmvFn.apply(kernel, opt, out, names, X1, X2, v, *diff_params.values())
    return _fmmv_forward(X1, X2, v, kernel, out, opt)


def fdmmv(
    X1: torch.Tensor,
    X2: torch.Tensor,
    v: Optional[torch.Tensor],
    w: Optional[torch.Tensor],
    kernel,
    out: Optional[torch.Tensor] = None,
    differentiable: bool = False,
    opt: Optional[BaseOptions] = None,
    kwargs_m1: Optional[Dict[str, torch.Tensor]] = None,
    kwargs_m2: Optional[Dict[str, torch.Tensor]] = None,
) -> torch.Tensor:
    """``k(X1, X2)^T (k(X1, X2) v + w)`` -> (m x t).  Signature of falkon/mmv_ops/fmmv.py:976-987
    (also called positionally as ``(X1, X2, v, w, kernel, out, differentiable, opt)``,
    falkon/kernels/diff_kernel.py:145)."""
    if differentiable:
        raise NotImplementedError(
            "Manual D-MMV is not implemented for differentiable inputs. Try using the KeOps version instead."
        )
    if _is_sparse(X1, X2):
        raise NotImplementedError("Sparse kernel-vector products are not implemented by falkon_b200.")
    if kwargs_m1 or kwargs_m2:
        raise NotImplementedError("Distance kernels take no per-row keyword tensors (kwargs_m1 / kwargs_m2).")
    if v is None and w is None:
        raise ValueError("One of v and w must be specified to run fdMMV.")
    if _is_user_defined(kernel):
        check_contiguity((X1, "X1"), (X2, "X2"), (v, "v"), (w, "w"), (out, "out"))
        v2 = v.reshape(-1, 1) if v is not None and v.dim() == 1 else v
        w2 = w.reshape(-1, 1) if w is not None and w.dim() == 1 else w
        return _generic_product("dmmv", X1, X2, v2, w2, kernel, out, opt)
    kernel_id, sigma = _kernel_spec(kernel)
    check_contiguity((X1, "X1"), (X2, "X2"), (v, "v"), (w, "w"), (out, "out"))
    _require_cuda(opt, X1, X2)
    if v is not None and v.dim() == 1:
        v = v.reshape(-1, 1)
    if w is not None and w.dim() == 1:
        w = w.reshape(-1, 1)
    data_devs = [X1.device, X2.device]
    if v is not None:
        data_devs.append(v.device)
    if w is not None:
        data_devs.append(w.device)
    m = X2.shape[0]
    t = v.shape[1] if v is not None else w.shape[1]
    dtype = v.dtype if v is not None else w.dtype
    out = create_output_mat(out, data_devs, (m, t), dtype, "cuda", X1)
    with torch.inference_mode():
        dev = _pick_device(tuple(data_devs) + (out.device,))
        all_host = all(d.type == "cpu" for d in data_devs) and out.device.type == "cpu"
        if all_host:
            devices = multi_device.host_devices(opt, X1.shape[0], dev)
            if len(devices) > 1:
                multi_device.fdmmv_host_multi(kernel_id, sigma, X1, X2, v, w, out, _flags(opt), devices)
            else:
                _lib.call_fdmmv_budgeted(kernel_id, sigma, X1, X2, v, w, out, flags=_flags(opt), host=True,
                                         device=devices[0], budget=lazy_budget(opt))
        else:
            o_dev = out if out.device == dev else torch.empty(out.shape, dtype=out.dtype, device=dev)
            with _DebugTimer(opt, "fdmmv", dev, f"n={X1.shape[0]} m={m} d={X1.shape[1]} t={t}"):
                _lib.call_fdmmv_budgeted(kernel_id, sigma, _to_dev(X1, dev), _to_dev(X2, dev), _to_dev(v, dev),
                                         _to_dev(w, dev), o_dev, flags=_flags(opt), budget=lazy_budget(opt))
            if o_dev is not out:
                out.copy_(o_dev)
    return out
