"""Two-GPU run (NCCL) of the row-sharded products and of Falkon.fit on shards.  Skipped on a box with one GPU;
the sharding / reduction logic itself is covered on CPU by tests/test_sharded_gloo.py."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from falkon_b200 import Falkon
        from falkon_b200.kernels import GaussianKernel
        from falkon_b200.sharded import ShardedKernelOps, shard_rows
        from fit_cases import build_fit_inputs, fit_case_by_name

        case = fit_case_by_name("fit_c1_64")
        gold = np.load(os.path.join(ROOT, "tests", "golden", case["name"] + ".npz"))
        Xn, Yn = build_fit_inputs(case)
        n = Xn.shape[0]
        start, length = shard_rows(n, world, rank)
        Xs = torch.from_numpy(Xn[start:start + length]).to(dev)
        Ys = torch.from_numpy(Yn[start:start + length]).to(dev)
        C = torch.from_numpy(Xn[gold["center_idx"]]).to(dev)
        kernel = GaussianKernel(case["sigma"])
        # products on shards against the single-GPU product on the whole matrix
        ops = ShardedKernelOps(kernel)
        v = torch.from_numpy(np.random.default_rng(1).standard_normal((case["m"], 2))).to(dev)
        got = ops.dmmv(Xs, C, v, None)
        want = kernel.dmmv(torch.from_numpy(Xn).to(dev), C, v, None)
        e_dmmv = float((got - want).norm() / want.norm())
        # the whole fit on shards: same centres as the reference (fixed selector), alpha against its fixture
        from falkon_b200.center_selection import FixedSelector

        model = Falkon(kernel=kernel, penalty=case["penalty"], M=case["m"], maxiter=case["maxiter"],
                       center_selection=FixedSelector(C), group=dist.group.WORLD)
        model.fit(Xs, Ys)
        alpha = model.alpha_.cpu().numpy()
        e_alpha = float(np.linalg.norm(alpha - gold["alpha"]) / np.linalg.norm(gold["alpha"]))
        # fp32 preconditioner with its M^3 steps shared between the ranks against the one a single rank builds
        from falkon_b200 import FalkonOptions
        from falkon_b200.preconditioner import FalkonPreconditioner

        g = torch.Generator(device=dev).manual_seed(77)  # the same centres on every rank
        C32 = torch.randn(5000, 10, generator=g, device=dev)
        shared = FalkonPreconditioner(1e-6, GaussianKernel(3.0), FalkonOptions()).init(C32, group=dist.group.WORLD)
        alone = FalkonPreconditioner(1e-6, GaussianKernel(3.0), FalkonOptions()).init(C32)
        e_T = float((shared.T - alone.T).norm() / alone.T.norm())
        e_A = float((shared.A - alone.A).norm() / alone.A.norm())
        ret[rank] = (e_dmmv, e_alpha, e_T, e_A)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_products_and_fit_two_gpus_nccl():
    world = 2
    port = 33500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert sorted(ret.keys()) == [0, 1]
    for r in range(world):
        assert ret[r][0] <= 1e-12, ret[r]   # fp64 products: only the summation order differs
        assert ret[r][1] <= 1e-6, ret[r]    # alpha of the fit on shards = the reference's
        assert ret[r][2] <= 1e-5 and ret[r][3] <= 1e-4, ret[r]  # shared factorisations = single-rank factorisations


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_host_operands_fan_out_over_gpus_in_one_process():
    """CPU tensors in, several GPUs used from one process (the reference's default way of using a multi-GPU
    machine): same result as the one-GPU call, for both products."""
    sys.path.insert(0, ROOT)
    from falkon_b200 import _lib
    from falkon_b200.kernels import GaussianKernel
    from falkon_b200.mmv_ops import multi_device as md
    from oracle import falkon_oracle as fo

    n, m, d, t = 2 * md.MIN_ROWS_PER_DEVICE + 77, 1500, 12, 2
    g = torch.Generator().manual_seed(31)
    X = torch.randn(n, d, generator=g)
    C = X[torch.randperm(n, generator=g)[:m]].contiguous()
    v = torch.randn(m, t, generator=g)
    w = torch.randn(n, t, generator=g)
    k_one = GaussianKernel(3.0)
    k_one.params.flk_devices = [0]
    k_all = GaussianKernel(3.0)
    assert len(md.host_devices(k_all.params, n, torch.device("cuda", 0))) >= 2
    before = _lib.launch_count()
    got = k_all.dmmv(X, C, v, w)
    assert _lib.launch_count() > before
    want = k_one.dmmv(X, C, v, w)
    assert got.device.type == "cpu"
    assert fo.rel_l2(got.numpy(), want.numpy()) < 1e-5
    got = k_all.mmv(X, C, v)
    want = k_one.mmv(X, C, v)
    assert fo.rel_l2(got.numpy(), want.numpy()) < 1e-6
    # and against an fp64 evaluation on the first rows
    ref = fo.dense_fmmv_fp64(X[:512].numpy(), C.numpy(), v.numpy(), "gaussian", 3.0)
    assert fo.rel_l2(got[:512].numpy(), ref) < 1e-4
