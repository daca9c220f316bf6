"""World-size-2 gloo test of the row-sharded products (CPU; local products from the oracle)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from falkon_b200.kernels import GaussianKernel
        from falkon_b200.sharded import ShardedKernelOps, shard_rows
        from oracle import falkon_oracle as fo

        rng = np.random.default_rng(7)
        n, m, d, t = 1001, 37, 5, 2
        X = torch.from_numpy(rng.standard_normal((n, d)))
        C = X[:m].clone()
        v = torch.from_numpy(rng.standard_normal((m, t)))
        w = torch.from_numpy(rng.standard_normal((n, t)))
        start, length = shard_rows(n, world, rank)
        Xs, ws = X[start : start + length], w[start : start + length]

        def local_mmv(A, B, vec, out=None, opt=None):
            return fo.fmmv(A, B, vec, "gaussian", 2.0)

        def local_dmmv(A, B, vec, ww, out=None, opt=None):
            return fo.fdmmv(A, B, vec, ww, "gaussian", 2.0)

        ops = ShardedKernelOps(GaussianKernel(2.0), local_mmv=local_mmv, local_dmmv=local_dmmv)
        assert ops.world == world
        got = ops.dmmv(Xs, C, v, ws)
        want = fo.dense_fdmmv_fp64(X.numpy(), C.numpy(), v.numpy(), w.numpy(), "gaussian", 2.0)
        err1 = fo.rel_l2(got.numpy(), want)
        got_t = ops.mmv_t(C, Xs, ws)
        want_t = fo.dense_fmmv_fp64(C.numpy(), X.numpy(), w.numpy(), "gaussian", 2.0)
        err2 = fo.rel_l2(got_t.numpy(), want_t)
        rows = ops.mmv(Xs, C, v)
        want_rows = fo.dense_fmmv_fp64(X.numpy(), C.numpy(), v.numpy(), "gaussian", 2.0)[start : start + length]
        err3 = fo.rel_l2(rows.numpy(), want_rows)
        ret[rank] = (err1, err2, err3, length)
    finally:
        dist.destroy_process_group()


def test_sharded_products_world2_gloo():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert sorted(ret.keys()) == [0, 1]
    assert ret[0][3] + ret[1][3] == 1001
    for r in range(world):
        assert ret[r][0] < 1e-10 and ret[r][1] < 1e-10 and ret[r][2] < 1e-10, ret[r]


def _cg_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from falkon_b200.kernels import GaussianKernel
        from falkon_b200.optim import FalkonConjugateGradient
        from falkon_b200.sharded import ShardedKernelOps, shard_rows
        from oracle import falkon_fit_oracle as ffo
        from oracle import falkon_oracle as fo

        rng = np.random.default_rng(21)
        n, m, d, t = 2003, 60, 4, 2
        X = torch.from_numpy(rng.standard_normal((n, d)))
        Y = torch.from_numpy(np.sin(X.numpy() @ rng.standard_normal((d, t))))
        penalty, maxiter, seed = 1e-4, 12, 5
        alpha_ref, beta_ref, idx = ffo.falkon_fit(X, Y, "gaussian", 2.0, None, penalty, m, maxiter, seed)
        C = X[torch.from_numpy(idx)]
        start, length = shard_rows(n, world, rank)
        Xs, Ys = X[start : start + length], Y[start : start + length]

        def local_mmv(A, B, vec, out=None, opt=None):
            return fo.fmmv(A, B, vec, "gaussian", 2.0)

        def local_dmmv(A, B, vec, ww, out=None, opt=None):
            return fo.fdmmv(A, B, vec, ww, "gaussian", 2.0)

        ops = ShardedKernelOps(GaussianKernel(2.0), local_mmv=local_mmv, local_dmmv=local_dmmv)
        # the CPU oracle's preconditioner has the method names the solver calls (invA, invT, invTt, invAt, apply_t)
        pc = ffo.Preconditioner(C, "gaussian", 2.0, None, penalty)
        solver = FalkonConjugateGradient(ops, pc)
        beta = solver.solve(Xs, C, Ys, penalty, None, maxiter, n=n)
        ret[rank] = (fo.rel_l2(beta.numpy(), beta_ref.numpy()), fo.rel_l2(pc.apply(beta).numpy(), alpha_ref.numpy()))
    finally:
        dist.destroy_process_group()


def test_sharded_falkon_cg_world2_gloo():
    """The Falkon CG on two row shards (right-hand side and every dmmv all-reduced, n = global row count)
    reproduces the single-process solution."""
    world = 2
    port = 31500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_cg_worker, args=(world, port, ret), nprocs=world, join=True)
    assert sorted(ret.keys()) == [0, 1]
    for r in range(world):
        assert ret[r][0] < 1e-9 and ret[r][1] < 1e-8, ret[r]


def test_shard_rows_partition():
    sys.path.insert(0, ROOT)
    from falkon_b200.sharded import shard_rows

    for n in (0, 1, 7, 8, 1001, 10_000_000):
        for world in (1, 2, 3, 8):
            spans = [shard_rows(n, world, r) for r in range(world)]
            assert spans[0][0] == 0
            assert sum(length for _, length in spans) == n
            for (s0, l0), (s1, _) in zip(spans, spans[1:]):
                assert s0 + l0 == s1
            assert max(length for _, length in spans) - min(length for _, length in spans) <= 1
    with pytest.raises(ValueError):
        shard_rows(10, 2, 2)


def _pc_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from falkon_b200.preconditioner.tensor_core_la import cholesky_lower_3xtf32, triu_times_transpose_3xtf32

        g = torch.Generator().manual_seed(7)
        m = 700
        X = torch.randn(m, 5, generator=g)
        K = torch.exp(-0.125 * torch.cdist(X, X).pow(2)) + 0.5 * torch.eye(m)
        serial, info0 = cholesky_lower_3xtf32(K.clone(), panel=96, trailing=96, k_chunk=64)
        shared, info1 = cholesky_lower_3xtf32(K.clone(), panel=96, trailing=192, k_chunk=64, group=dist.group.WORLD)
        e_chol = float((shared - serial).abs().max() / serial.abs().max())
        T = serial.mT
        prod_serial = triu_times_transpose_3xtf32(T, block=128, k_chunk=64)
        prod_shared = triu_times_transpose_3xtf32(T, block=128, k_chunk=64, group=dist.group.WORLD)
        e_prod = float((prod_shared - prod_serial).abs().max() / prod_serial.abs().max())
        bad = K.clone()
        bad[400, 400] = -1.0
        _, info_bad = cholesky_lower_3xtf32(bad, panel=96, trailing=96, group=dist.group.WORLD)
        ret[rank] = (e_chol, e_prod, info0, info1, info_bad, bool(torch.equal(prod_shared, prod_shared.T)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_preconditioner_steps_shared_between_ranks_gloo(world):
    """The fp32 factorisation and T T^T spread over the ranks of a group give every rank the factor / product the
    single-process routine computes (same block arithmetic, only who does it changes)."""
    port = 32500 + (os.getpid() % 2000) + world
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_pc_worker, args=(world, port, ret), nprocs=world, join=True)
    assert sorted(ret.keys()) == list(range(world))
    for r in range(world):
        e_chol, e_prod, info0, info1, info_bad, sym = ret[r]
        assert e_chol < 1e-6 and e_prod < 1e-6, ret[r]
        assert info0 == 0 and info1 == 0 and info_bad == 401 and sym
