"""Generates tests/golden/grad_*.npz from the reference implementation itself (its CPU path).

Run like make_golden.py (reference on PYTHONPATH, nvcc hidden so only its CPU extension is built):

    export PATH=$(echo $PATH | tr ':' '\n' | grep -v cuda | paste -sd:)
    TORCH_EXTENSIONS_DIR=/tmp/flk_ext PYTHONPATH=<reference checkout> python tests/golden/make_golden_grad.py

For every case of grad_cases.py the reference's own differentiable ``Kernel.mmv`` and ``Kernel.__call__`` run
with ``FalkonOptions(use_cpu=True, keops_active="no")`` on inputs that require gradients; ``backward`` is
called with the seeded upstream gradients and the fixture stores the gradients with respect to X1, X2, v and
sigma (``mmv_*``) and to X1, X2 and sigma (``mm_*``).
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from grad_cases import build_grad_inputs, grad_cases  # noqa: E402

from falkon import FalkonOptions  # noqa: E402  (the reference)
from falkon.kernels import GaussianKernel, LaplacianKernel, MaternKernel  # noqa: E402


def make_kernel(case, opt):
    sigma = torch.tensor(case["sigma"], dtype=torch.float64).requires_grad_()
    if case["kernel"] == "gaussian":
        return GaussianKernel(sigma, opt=opt)
    if case["kernel"] == "laplacian":
        return LaplacianKernel(sigma, opt=opt)
    return MaternKernel(sigma, nu=float(case["nu"]), opt=opt)


def main():
    torch.set_num_threads(os.cpu_count())
    opt = FalkonOptions(use_cpu=True, keops_active="no", max_cpu_mem=2 * 2**30)
    for case in grad_cases():
        X1n, X2n, vn, Gn, Sn = build_grad_inputs(case)
        out = {}
        # k(X1, X2) @ v
        X1, X2, v = (torch.from_numpy(a).requires_grad_() for a in (X1n, X2n, vn))
        k = make_kernel(case, opt)
        res = k.mmv(X1, X2, v)
        res.backward(torch.from_numpy(Gn))
        out["mmv_out"] = res.detach().numpy()
        out["mmv_dX1"], out["mmv_dX2"], out["mmv_dv"] = (t.grad.numpy() for t in (X1, X2, v))
        out["mmv_dsigma"] = k.sigma.grad.numpy().copy()
        # k(X1, X2)
        X1, X2 = (torch.from_numpy(a).requires_grad_() for a in (X1n, X2n))
        k = make_kernel(case, opt)
        res = k(X1, X2)
        res.backward(torch.from_numpy(Sn))
        out["mm_dX1"], out["mm_dX2"] = (t.grad.numpy() for t in (X1, X2))
        out["mm_dsigma"] = k.sigma.grad.numpy().copy()
        path = os.path.join(HERE, case["name"] + ".npz")
        np.savez_compressed(path, **out)
        print(case["name"], {key: val.shape for key, val in out.items()})


if __name__ == "__main__":
    main()
