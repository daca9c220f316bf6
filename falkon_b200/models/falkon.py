"""``Falkon``: Nystrom kernel ridge regression solved by preconditioned conjugate gradient, on the B200.

Constructor, ``fit`` / ``predict`` and the fitted attributes (``alpha_``, ``beta_``, ``ny_points_``,
``precond``, ``fit_times_``, ``val_errors_``) are those of the reference estimator
(falkon/models/falkon.py:34-320, falkon/models/model_utils.py:20-226).  The flow of ``fit`` is the
reference's: pick the centres, build the preconditioner on them, run ``maxiter`` CG iterations whose
operator is one ``dmmv`` each, map beta back with the preconditioner.

B200-first differences: the training set is moved to the GPU once and stays there for the whole fit
(10^7 x 28 fp32 is 1.1 GB of a 180 GB device; the reference re-streams row blocks from pinned host
memory in every iteration), no kernel block is ever stored (``never_store_kernel`` is implied),
and with ``group=`` every process of a ``torch.distributed`` group fits on its own row shard with
the M x T reductions done by NCCL.  There is no CPU path.
"""
import time
from typing import Any, Callable, Optional, Tuple, Union

import numpy as np
import torch

from .. import center_selection as cs
from ..optim import FalkonConjugateGradient
from ..options import FalkonOptions
from ..preconditioner import FalkonPreconditioner

__all__ = ("Falkon", "InCoreFalkon")


class Falkon:
    """Falkon kernel ridge regression solver.

    Parameters
    ----------
    kernel
        Kernel object (``falkon_b200.kernels``).
    penalty
        Ridge parameter lambda (> 0).
    M
        Number of Nystrom centres (needed unless a ``CenterSelector`` instance is given).
    center_selection
        ``"uniform"`` or a ``falkon_b200.center_selection.CenterSelector``.
    maxiter
        Number of CG iterations.
    seed
        Seed of the centre selection (``numpy.random.default_rng``) and of torch.
    error_fn, error_every
        Optional ``error_fn(y_true, y_pred)`` evaluated every ``error_every`` iterations on the
        validation set given to ``fit`` (or on the training set).
    weight_fn
        Optional ``weight_fn(Y, X, indices)`` for re-weighted least squares.
    options
        ``FalkonOptions``.
    group
        Optional ``torch.distributed`` process group: ``fit`` then expects this process's row shard of
        X and Y, and all processes must pass the same seed / centres (centres are taken from rank 0's
        shard and broadcast).
    """

    def __init__(
        self,
        kernel,
        penalty: float,
        M: Optional[int],
        center_selection: Union[str, cs.CenterSelector] = "uniform",
        maxiter: int = 20,
        seed: Optional[int] = None,
        error_fn: Optional[Callable[[torch.Tensor, torch.Tensor], Union[Any, Tuple[Any, str]]]] = None,
        error_every: Optional[int] = 1,
        weight_fn: Optional[Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor]] = None,
        options: Optional[FalkonOptions] = None,
        group=None,
    ):
        self.kernel = kernel
        self.penalty = penalty
        self.M = M
        self.maxiter = maxiter
        self.seed = seed
        if seed is not None:
            torch.manual_seed(seed)
        self.random_state_ = np.random.default_rng(seed)
        self.error_fn = error_fn
        self.error_every = error_every
        self.weight_fn = weight_fn
        self.options = options or FalkonOptions()
        if self.options.use_cpu:
            raise RuntimeError("falkon_b200 has no CPU implementation (use_cpu=True was requested).")
        self.group = group
        self.center_selection = self._init_center_selection(center_selection)
        self.alpha_ = None
        self.beta_ = None
        self.ny_points_ = None
        self.precond = None
        self.fit_times_ = None
        self.val_errors_ = None

    def _init_center_selection(self, center_selection):
        if isinstance(center_selection, str):
            if center_selection.lower() == "uniform":
                if self.M is None:
                    raise ValueError(
                        "M must be specified when no `CenterSelector` object is provided. "
                        "Specify an integer value for `M` or a `CenterSelector` object."
                    )
                return cs.UniformSelector(self.random_state_, num_centers=self.M)
            raise ValueError(f'Center selection "{center_selection}" is not valid.')
        return center_selection

    def _reset_state(self):
        self.alpha_ = None
        self.beta_ = None
        self.ny_points_ = None
        self.precond = None
        self.fit_times_ = []
        self.val_errors_ = []

    @staticmethod
    def _check_fit_inputs(X, Y, Xts, Yts):
        if X.shape[0] != Y.shape[0]:
            raise ValueError(f"X and Y must have the same number of samples (found {X.shape[0]} and {Y.shape[0]})")
        if Y.dim() == 1:
            Y = Y.reshape(-1, 1)
        if Y.dim() != 2:
            raise ValueError(f"Y is expected 1D or 2D. Found {Y.dim()}D.")
        if X.dtype != Y.dtype:
            raise TypeError(f"X and Y must have the same data-type. ({X.dtype} vs {Y.dtype})")
        if Yts is not None and Yts.dim() == 1:
            Yts = Yts.reshape(-1, 1)
        return X, Y, Xts, Yts

    def _device(self, *tensors) -> torch.device:
        if not torch.cuda.is_available():
            raise RuntimeError("falkon_b200 needs a CUDA device (B200, sm_100); none is available.")
        for t in tensors:
            if t is not None and t.is_cuda:
                return t.device
        return torch.device("cuda", torch.cuda.current_device())

    def _ops(self):
        """The object whose mmv / dmmv the solver calls: the kernel, or its sharded wrapper."""
        if self.group is None:
            return self.kernel
        from ..sharded import ShardedKernelOps

        return ShardedKernelOps(self.kernel, group=self.group)

    def _callback(self, X, Y, Xts, Yts, ny_points, precond):
        def val_cback(it, beta, train_time):
            self.fit_times_.append(self.fit_times_[0] + train_time)
            if it % self.error_every != 0:
                print(f"Iteration {it:3d} - Elapsed {self.fit_times_[-1]:.2f}s", flush=True)
                return
            err_str = "training" if Xts is None or Yts is None else "validation"
            alpha = precond.apply(beta)
            if Xts is not None and Yts is not None:
                err = self.error_fn(Yts, self._predict(Xts, ny_points, alpha))
            else:
                err = self.error_fn(Y, self._predict(X, ny_points, alpha))
            err_name = "error"
            if isinstance(err, tuple) and len(err) == 2:
                err, err_name = err
            print(f"Iteration {it:3d} - Elapsed {self.fit_times_[-1]:.2f}s - {err_str} {err_name}: {str(err)}",
                  flush=True)
            self.val_errors_.append(err)

        return val_cback

    def fit(self, X: torch.Tensor, Y: torch.Tensor, Xts: Optional[torch.Tensor] = None,
            Yts: Optional[torch.Tensor] = None, warm_start: Optional[torch.Tensor] = None):
        """Fits the model.  X: (n x d), Y: (n x t) or (n,).  ``warm_start`` is a previous ``beta_``."""
        X, Y, Xts, Yts = self._check_fit_inputs(X, Y, Xts, Yts)
        self._reset_state()
        t_s = time.time()
        dev = self._device(X, Y)
        # moved outside inference mode: ordinary tensors carry a version counter, which lets the products keep what
        # they prepared from X across the iterations of the solve (falkon_b200/_lib.py, resident operands)
        Xd, Yd = X.to(dev), Y.to(dev)
        with torch.inference_mode():
            Xts_d = None if Xts is None else Xts.to(dev)
            Yts_d = None if Yts is None else Yts.to(dev)
            if self.weight_fn is None:
                ny_points, ny_indices = self.center_selection.select(Xd, None), None
            else:
                ny_points, ny_indices = self.center_selection.select_indices(Xd, None)
            n_total = Xd.shape[0]
            ny_weight_vec = None
            if self.weight_fn is not None:
                ny_weight_vec = self.weight_fn(Yd[ny_indices], Xd[ny_indices], ny_indices)
            if self.group is not None:
                import torch.distributed as dist

                # Every rank must build the same preconditioner: the centres AND their weights are rank 0's.
                # The selector clamps the number of centres to the rows of the local shard, so the ranks first
                # agree that they all hold the same count (tensors of different shapes in one broadcast would
                # hang the collective instead of failing).
                src = dist.get_global_rank(self.group, 0)
                cnt = torch.tensor([n_total, ny_points.shape[0], -ny_points.shape[0]], dtype=torch.int64, device=dev)
                dist.all_reduce(cnt[:1], group=self.group)
                dist.all_reduce(cnt[1:], op=dist.ReduceOp.MAX, group=self.group)
                n_total = int(cnt[0].item())
                if int(cnt[1].item()) != -int(cnt[2].item()):
                    raise ValueError(
                        f"the ranks selected different numbers of centres ({-int(cnt[2].item())} to {int(cnt[1].item())}): "
                        f"every shard must hold at least M rows")
                ny_points = ny_points.contiguous()
                dist.broadcast(ny_points, src=src, group=self.group)
                if ny_weight_vec is not None:
                    ny_weight_vec = ny_weight_vec.contiguous()
                    dist.broadcast(ny_weight_vec, src=src, group=self.group)
            self.precond = FalkonPreconditioner(self.penalty, self.kernel, self.options)
            self.precond.init(ny_points, weight_vec=ny_weight_vec, group=self.group)
            self.fit_times_.append(time.time() - t_s)
            cback = None
            if self.error_fn is not None and self.error_every is not None:
                cback = self._callback(Xd, Yd, Xts_d, Yts_d, ny_points, self.precond)
            optim = FalkonConjugateGradient(self._ops(), self.precond, self.options, weight_fn=self.weight_fn)
            if warm_start is not None:
                warm_start = warm_start.to(dev).clone()
            beta = optim.solve(Xd, ny_points, Yd, self.penalty, initial_solution=warm_start,
                               max_iter=self.maxiter, callback=cback, n=n_total)
            alpha = self.precond.apply(beta)
            self.alpha_, self.beta_, self.ny_points_ = alpha, beta, ny_points
        return self

    def _predict(self, X, ny_points, alpha):
        with torch.inference_mode():
            return self.kernel.mmv(X, ny_points, alpha, opt=self.options)

    def predict(self, X: torch.Tensor) -> torch.Tensor:
        """Predictions (n x t) for the rows of X, on X's device."""
        if self.alpha_ is None or self.ny_points_ is None:
            raise RuntimeError("Falkon has not been trained. `predict` must be called after `fit`.")
        dev = self.alpha_.device
        out = self._predict(X.to(dev), self.ny_points_, self.alpha_)
        return out.to(X.device)

    def to(self, device):
        self.alpha_ = self.alpha_.to(device)
        self.ny_points_ = self.ny_points_.to(device)
        return self

    def __repr__(self):
        return (f"Falkon(kernel={self.kernel}, penalty={self.penalty}, M={self.M}, maxiter={self.maxiter}, "
                f"seed={self.seed})")


class InCoreFalkon(Falkon):
    """``Falkon`` for data that already lives on the GPU (falkon/models/incore_falkon.py:22-270).

    On a B200 the plain ``Falkon`` keeps everything on the device as well; this class only adds the
    reference's input contract: all tensors given to ``fit`` must be CUDA tensors on one device
    (``ValueError`` otherwise), and ``predict`` expects its input on the model's device.
    """

    @staticmethod
    def _same_cuda_device(*tensors) -> bool:
        devs = {t.device for t in tensors if t is not None}
        return len(devs) == 1 and next(iter(devs)).type == "cuda"

    def fit(self, X, Y, Xts=None, Yts=None, warm_start=None):
        if not self._same_cuda_device(X, Y, Xts, Yts):
            raise ValueError("All tensors for fitting InCoreFalkon must be CUDA tensors, located on the same GPU.")
        return super().fit(X, Y, Xts, Yts, warm_start)

    def predict(self, X):
        if self.alpha_ is not None and X.device != self.alpha_.device:
            raise ValueError(f"X must be on device {self.alpha_.device}")
        return super().predict(X)
