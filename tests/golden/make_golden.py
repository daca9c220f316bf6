"""Generates tests/golden/*.npz from the reference implementation itself.

Run in the build container, where the reference source tree is mounted, with the reference on
PYTHONPATH and its CPU-only extension JIT-built (nvcc hidden from PATH so that only the CPU
operators are compiled):

    export PATH=$(echo $PATH | tr ':' '\n' | grep -v cuda | paste -sd:)
    TORCH_EXTENSIONS_DIR=/tmp/flk_ext PYTHONPATH=<reference checkout> \
        python tests/golden/make_golden.py

Every output is produced by the reference's own ``Kernel.mmv`` / ``Kernel.dmmv`` with
``FalkonOptions(use_cpu=True, keops_active="no", max_cpu_mem=256 MiB)`` on the seeded inputs
of tests/golden/cases.py.  The fixtures hold outputs only (inputs are regenerated from the
seeds); large ``mmv`` outputs are stored on a strided subset of rows.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from cases import all_cases, build_inputs  # noqa: E402

from falkon import FalkonOptions  # noqa: E402  (the reference)
from falkon.kernels import GaussianKernel, LaplacianKernel, MaternKernel  # noqa: E402

MAX_STORED_VALUES = 8192


def make_kernel(case, opt):
    sigma = torch.tensor(case["sigma"], dtype=torch.float64)
    if case["kernel"] == "gaussian":
        return GaussianKernel(sigma, opt=opt)
    if case["kernel"] == "laplacian":
        return LaplacianKernel(sigma, opt=opt)
    return MaternKernel(sigma, nu=float(case["nu"]), opt=opt)


def row_subset(nrows, ncols):
    max_rows = max(64, MAX_STORED_VALUES // ncols)
    if nrows <= max_rows:
        return np.arange(nrows)
    stride = -(-nrows // max_rows)
    return np.arange(0, nrows, stride)


def main():
    torch.set_num_threads(os.cpu_count())
    opt = FalkonOptions(use_cpu=True, keops_active="no", max_cpu_mem=256 * 2**20)
    for case in all_cases():
        inp = build_inputs(case)
        X, C, v = (torch.from_numpy(inp[k]) for k in ("X", "C", "v"))
        w = torch.from_numpy(inp["w"]) if inp["w"] is not None else None
        y = torch.from_numpy(inp["y"])
        k = make_kernel(case, opt)
        out = {}
        if "mmv" in case["ops"]:
            r = k.mmv(X, C, v).numpy()
            rows = row_subset(r.shape[0], r.shape[1])
            out["mmv_rows"] = rows
            out["mmv"] = r[rows]
        if "dmmv" in case["ops"]:
            out["dmmv"] = k.dmmv(X, C, v, w).numpy()
        if "dmmv_now" in case["ops"]:
            out["dmmv_now"] = k.dmmv(X, C, v, None).numpy()
        if "mmv_t" in case["ops"]:
            out["mmv_t"] = k.mmv(C, X, y).numpy()
        path = os.path.join(HERE, case["name"] + ".npz")
        np.savez_compressed(path, **out)
        print(case["name"], {k_: v_.shape for k_, v_ in out.items()}, os.path.getsize(path))


if __name__ == "__main__":
    main()
