"""Generates tests/golden/fit_*.npz from the reference implementation itself (its CPU path).

Run like make_golden.py (reference on PYTHONPATH, nvcc hidden so only its CPU extension is built):

    export PATH=$(echo $PATH | tr ':' '\n' | grep -v cuda | paste -sd:)
    TORCH_EXTENSIONS_DIR=/tmp/flk_ext PYTHONPATH=<reference checkout> python tests/golden/make_golden_fit.py

For every case of fit_cases.py the reference's own ``Falkon(...).fit(X, Y)`` runs with
``FalkonOptions(use_cpu=True, keops_active="no")`` and the fixture stores: the indices of the centres
it selected, alpha_, beta_, predictions on the first 256 rows, and -- from its ``FalkonPreconditioner``
and kernel on the same centres -- K_MM on a 64 x 64 corner, ``apply`` / ``apply_t`` / ``invA`` / ``invT``
of a seeded vector.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from fit_cases import build_fit_inputs, fit_cases, weight_fn_numpy  # noqa: E402

from falkon import Falkon, FalkonOptions  # noqa: E402  (the reference)
from falkon.kernels import GaussianKernel, MaternKernel  # noqa: E402
from falkon.preconditioner import FalkonPreconditioner  # noqa: E402


def make_kernel(case, opt):
    if case["kernel"] == "gaussian":
        return GaussianKernel(case["sigma"], opt=opt)
    return MaternKernel(case["sigma"], nu=case["nu"], opt=opt)


def weight_fn(Y, X, idx):
    return torch.from_numpy(weight_fn_numpy(Y.numpy())).to(Y.dtype)


def main():
    torch.set_num_threads(os.cpu_count())
    opt = FalkonOptions(use_cpu=True, keops_active="no", max_cpu_mem=2 * 2**30)
    for case in fit_cases():
        Xn, Yn = build_fit_inputs(case)
        X, Y = torch.from_numpy(Xn), torch.from_numpy(Yn)
        k = make_kernel(case, opt)
        # the centres the uniform selector draws for this seed (recorded; the fit itself re-draws the same)
        idx = np.random.default_rng(case["seed"]).choice(case["n"], size=case["m"], replace=False)
        model = Falkon(kernel=k, penalty=case["penalty"], M=case["m"], maxiter=case["maxiter"], seed=case["seed"],
                       weight_fn=weight_fn if case["weighted"] else None, options=opt)
        model.fit(X, Y)
        C = model.ny_points_
        assert torch.equal(C, X[torch.from_numpy(idx)]), "centre selection does not follow default_rng(seed).choice"
        out = dict(center_idx=idx.astype(np.int64), alpha=model.alpha_.numpy(), beta=model.beta_.numpy(),
                   pred_head=model.predict(X[:256]).numpy())
        pc = FalkonPreconditioner(case["penalty"], k, opt)
        pc.init(C.clone())
        vr = torch.from_numpy(np.random.default_rng(9000 + case["seed"]).standard_normal((case["m"], case["t"]))
                              .astype(Xn.dtype))
        out["pc_apply"] = pc.apply(vr.clone()).numpy()
        out["pc_apply_t"] = pc.apply_t(vr.clone()).numpy()
        out["pc_invA"] = pc.invA(vr.clone()).numpy()
        out["pc_invT"] = pc.invT(vr.clone()).numpy()
        out["kmm_corner"] = k(C[:64].clone(), C[:64].clone()).numpy()
        out["knm_corner"] = k(X[:64].clone(), C[:48].clone()).numpy()
        path = os.path.join(HERE, case["name"] + ".npz")
        np.savez_compressed(path, **out)
        print(case["name"], {k_: v_.shape for k_, v_ in out.items()}, os.path.getsize(path), flush=True)


if __name__ == "__main__":
    main()
