"""Benchmark of the fdmmv hot path:  out = K(X,C)^T (K(X,C) v + w).

    python bench.py --gpus N --steps K --warmup W            # this implementation
    python bench.py --impl reference --steps K --warmup W    # the reference algorithm on the host cores

Default workload (one step = one fdmmv over one batch of synthetic input): the product inside the fit of
benchmark configuration 3 -- Gaussian kernel sigma = 5, fp32, X: 10,000,000 x 28 from a two-component isotropic
Gaussian mixture (means +-0.5, unit variance), C: 50,000 rows of X, v ~ N(0,1) (M x 1), w ~ N(0,1) (N x 1).
With N GPUs the 10,000,000 rows are split evenly over the ranks (strong scaling), C and v are replicated, and
the M x 1 partial results are summed with one NCCL all-reduce per step.  `--config 2` runs benchmark
configuration 2 instead (1,000,000 rows per GPU, M = 20,000: weak scaling).

Prints ONE JSON line.  `value` is kernel pair-evaluations per second (N*M*T / time) with the inputs resident in
HBM; `e2e` is the same metric through the host-buffer entry point (pinned host inputs copied in, result copied
out, inside the timed region); `roofline` describes the dominant kernel (the tcgen05 sweep), timed live with
CUDA events on its stream, against the MUFU rate measured live; `parity` compares sampled entries of the
all-reduced result with an independent fp64 evaluation; `cpu_baseline` is the CPU oracle timed on a bounded
sample on this machine's host cores.
"""
import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np
import torch

D = 28
T = 1
SIGMA = 5.0
METRIC = "fdmmv pair-evals/s (N*M*T)"
UNIT = "pair-evals/s"
N_PER_GPU = 1_000_000  # configuration 2 (weak scaling): rows per GPU


def workload(config: int, world: int, rows: int = 0):
    """Sizes and description of the two fp32 Gaussian d = 28 workloads of the default path.
    3: the product of the fit configuration, 1e7 rows split over the GPUs (strong scaling), M = 50,000;
    2: 1e6 rows per GPU (weak scaling), M = 20,000."""
    if config == 3:
        n_total = rows or 10_000_000
        return dict(config=3, m=50_000, n_total=n_total, n_local=n_total // world, scaling="strong",
                    name=f"config3 product: fdmmv Gaussian sigma=5 fp32, N={n_total} x d=28 mixture split evenly over "
                         f"the GPUs, M=50000 sampled rows, T=1, w~N(0,1)")
    n_local = rows or N_PER_GPU
    return dict(config=2, m=20_000, n_total=n_local * world, n_local=n_local, scaling="weak",
                name=f"config2: fdmmv Gaussian sigma=5 fp32, N={n_local} per GPU x d=28 mixture, M=20000 sampled rows, "
                     f"T=1, w~N(0,1)")


def gen_shard(n, seed, device):
    g = torch.Generator(device=device).manual_seed(seed)
    z = (torch.rand(n, 1, generator=g, device=device) < 0.5).to(torch.float32)
    X = torch.randn(n, D, generator=g, device=device) + (2.0 * z - 1.0) * 0.5
    w = torch.randn(n, T, generator=g, device=device)
    return X, w


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(bf16_tflops=float(p["bf16_tflops"]), bf16_sustained=float(p.get("bf16_tflops_sustained", 0.0)),
                    hbm_gbs=float(p["hbm_gbs"]), source="measured")
    return dict(bf16_tflops=1590.0, bf16_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clock, power and clock-event (throttle) reasons through NVML from a background
    thread while the timed region runs (read-only queries; nothing is set)."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, torch_device):
        self.samples = []
        self.thread = None
        self.stop_flag = False
        self.handle = None
        self.err = None
        try:
            import pynvml

            self.nv = pynvml
            pynvml.nvmlInit()
            try:
                uuid = str(torch.cuda.get_device_properties(torch_device).uuid)
                if not uuid.startswith("GPU-"):
                    uuid = "GPU-" + uuid
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(torch_device.index or 0)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # NVML missing: report that instead of inventing numbers
            self.err = f"nvml unavailable: {e}"

    def _loop(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                sm = float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                pw = nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                try:
                    rs = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                except Exception:
                    rs = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.samples.append((sm, pw, rs))
            except Exception as e:
                self.err = str(e)
                return
            time.sleep(0.005)

    def start(self):
        if self.handle is None:
            return
        import threading

        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def stop(self):
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [self.err or "not sampled"]}
        self.stop_flag = True
        self.thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [self.err or "no samples"]}
        sm = [a for a, _, _ in self.samples]
        pw = [b for _, b, _ in self.samples]
        bits = 0
        for _, _, r in self.samples:
            bits |= r
        reasons = sorted(name for bit, name in self.REASONS.items() if bits & bit)
        return {"sm_mhz": float(np.median(sm)), "sm_min_mhz": float(min(sm)), "sm_max_mhz": self.sm_max,
                "power_w_max": float(max(pw)), "power_w_median": float(np.median(pw)), "samples": len(sm),
                "reasons": reasons}


def cpu_centres(X, g, m):
    n = X.shape[0]
    idx = torch.randperm(n, generator=g)[:m] if n >= m else torch.randint(n, (m,), generator=g)
    return X[idx].contiguous()


CPU_SAMPLE_ROWS = 200_000  # rows of the bounded CPU sample (the full workloads would take hours on the host)


def cpu_sample(wl, n_sample):
    """The first n_sample rows of the workload's generator stream on the host, with M centres and v."""
    X, w = gen_shard(n_sample, 1000 + wl["config"], "cpu")
    g = torch.Generator().manual_seed(2000 + wl["config"])
    C = cpu_centres(X, g, wl["m"])
    v = torch.randn(wl["m"], T, generator=g)
    return X, C, v, w


def cpu_fdmmv():
    """The CPU implementation that the GPU path is compared with, and what it is: the reference package itself
    (its own ``GaussianKernel.dmmv`` with ``use_cpu=True, keops_active="no"``; kind "reference") when
    oracle/build_ref.py has installed it under oracle/_ref/site, else the oracle port of the same algorithm
    (kind "port").  Returns (fdmmv(X, C, v, w) -> out, kind, description)."""
    site = os.path.join(ROOT, "oracle", "_ref", "site")
    if os.path.isdir(os.path.join(site, "falkon")) and site not in sys.path:
        sys.path.append(site)
    try:
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            from falkon import FalkonOptions as RefOptions
            from falkon.kernels import GaussianKernel as RefGaussian

        opt = RefOptions(use_cpu=True, keops_active="no", max_cpu_mem=4 * 2**30)
        k = RefGaussian(SIGMA, opt=opt)
        return (lambda X, C, v, w: k.dmmv(X, C, v, w, opt=opt)), "reference", \
            "the reference package's own GaussianKernel.dmmv (use_cpu=True, keops_active='no', max_cpu_mem=4 GiB)"
    except Exception:
        from oracle import falkon_oracle as fo

        return (lambda X, C, v, w: fo.fdmmv(X, C, v, w, "gaussian", SIGMA, max_block_elems=256 * 2**20)), "port", \
            "CPU oracle port of the reference algorithm (blocked GEMM + element-wise passes in torch CPU ops)"


def time_cpu_baseline(wl, n_sample, reps):
    """Times the CPU fdmmv on n_sample rows of the workload with all host threads.
    Returns (pair-evals/s, seconds, cores, kind, description)."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    fn, kind, what = cpu_fdmmv()
    X, C, v, w = cpu_sample(wl, n_sample)
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        fn(X, C, v, w)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return n_sample * wl["m"] * T / best, best, cores, kind, what


def base_config(wl, world):
    """The part of the JSON line's `config` that both arms share."""
    return {"workload": wl["name"], "global_rows": wl["n_total"], "centres": wl["m"], "d": D, "T": T,
            "rows_per_gpu": wl["n_local"], "n_gpus": world}


def run_reference(args):
    """The reference arm: the reference's CPU implementation of this path (see cpu_fdmmv) on all host threads.
    Every step is one fdmmv on a bounded sample of the workload:
    the first CPU_SAMPLE_ROWS rows with the workload's full M (the per-pair cost does not depend on N, so
    pair-evals/s of the sample is the figure of the full problem)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    fn, kind, what = cpu_fdmmv()
    wl = workload(args.config if args.config in (2, 3) else 3, world, 0)
    n_sample = min(args.cpu_rows, wl["n_total"])
    X, C, v, w = cpu_sample(wl, n_sample)
    for _ in range(min(args.warmup, 1)):  # one untimed pass settles the thread pool and the allocator
        fn(X, C, v, w)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn(X, C, v, w)
    dt = time.perf_counter() - t0
    value = args.steps * n_sample * wl["m"] * T / dt
    sample = (f"each step = one fdmmv on the first {n_sample} rows of the workload with all M={wl['m']} centres "
              f"(d={D}); {what}, {cores} threads; {min(args.warmup, 1)} warm-up pass")
    cfg = base_config(wl, world)
    cfg["sample"] = sample
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True,
        "scaling": wl["scaling"], "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_fit(args):
    """Benchmark configuration 3 (not the default line): the full Falkon.fit on synthetic binary regression,
    N x 28 mixture data, +-1 labels with 5 % flips, Gaussian sigma = 5, M uniform centres, lambda = 1e-7, fp32,
    20 CG iterations.  Prints one JSON line with the wall time of the fit (preconditioner included), the time
    inside the dmmv calls (the hot path) and the training accuracy."""
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a GPU (there is no CPU fallback)")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    import torch.distributed as dist

    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from falkon_b200 import Falkon, FalkonOptions, _lib
    from falkon_b200.kernels import GaussianKernel

    _lib.build()
    n_total, m = args.rows or 10_000_000, args.centres
    n = n_total // world  # rows of this rank's shard (strong scaling: the data set is fixed)
    g = torch.Generator(device=dev).manual_seed(1003 + rank)
    z = (torch.rand(n, 1, generator=g, device=dev) < 0.5).to(torch.float32)
    X = torch.randn(n, D, generator=g, device=dev) + (2.0 * z - 1.0) * 0.5
    flip = torch.rand(n, 1, generator=g, device=dev) < 0.05
    Y = torch.where(flip, -(2.0 * z - 1.0), 2.0 * z - 1.0)
    kernel = GaussianKernel(SIGMA)
    dmmv_s = [0.0]
    dmmv_calls = [0]
    orig = kernel.dmmv

    def timed_dmmv(*a, **k):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = orig(*a, **k)
        e1.record()
        e1.synchronize()
        dmmv_s[0] += e0.elapsed_time(e1) * 1e-3
        dmmv_calls[0] += 1
        return out

    # warm-up: a small fit (2048 centres, 100,000 rows, 3 iterations) takes the one-time costs of the process --
    # CUDA context, cuBLAS / cuSOLVER handles and their first-call set-up, workspace allocation -- out of the timed fit
    warm = Falkon(kernel=GaussianKernel(SIGMA), penalty=1e-7, M=2048, maxiter=3, seed=1, options=FalkonOptions(),
                  group=dist.group.WORLD if world > 1 else None)
    warm.fit(X[:100_000], Y[:100_000])
    del warm
    kernel.dmmv = timed_dmmv
    model = Falkon(kernel=kernel, penalty=1e-7, M=m, maxiter=20, seed=3, options=FalkonOptions(),
                   group=dist.group.WORLD if world > 1 else None)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    model.fit(X, Y)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    wall = time.perf_counter() - t0
    n_eval = min(n, 1_000_000)
    pred = model.predict(X[:n_eval])
    acc = float(((pred > 0) == (Y[:n_eval] > 0)).float().mean())
    iters = dmmv_calls[0]  # counted: the CG products plus the full-gradient refreshes (fewer if the CG stops early)
    if rank == 0:
        print(json.dumps({
            "workload": f"config3: Falkon.fit, N={n_total} x d={D} mixture, +-1 labels (5% flips), Gaussian sigma=5, "
                        f"M={m}, lambda=1e-7, fp32, 20 CG iterations, preconditioner included",
            "n_gpus": world, "scaling": "strong", "rows_per_gpu": n,
            "warmup": "one fit with 2048 centres on 100,000 rows (process start-up costs only)",
            "fit_wall_s": wall, "preconditioner_s": model.fit_times_[0], "dmmv_s_total": dmmv_s[0],
            "dmmv_calls": iters, "dmmv_pair_evals_per_s": iters * float(n) * world * m / dmmv_s[0],
            "train_accuracy_first_rows": acc, "accuracy_note": "labels carry 5 % flips",
            "tc_status": _lib.tc_status(dev), "range_flag": _lib.range_flag(dev),
            "peak_mem_gb": torch.cuda.max_memory_allocated(dev) / 1e9,
        }))
    if world > 1:
        dist.destroy_process_group()


def _dense_fdmmv_fp64(X, C, v, w, kind, sigma, rows_per_block=4096):
    """K^T (K v + w) in fp64 by explicit blocks of torch ops on the GPU (spot-check of the other configurations;
    explicit differences through cdist, no norm expansion)."""
    out = torch.zeros(C.shape[0], v.shape[1], dtype=torch.float64, device=X.device)
    Cs = C.double() / sigma
    for r0 in range(0, X.shape[0], rows_per_block):
        Xb = X[r0:r0 + rows_per_block].double() / sigma
        d = torch.cdist(Xb, Cs, compute_mode="donot_use_mm_for_euclid_dist")
        if kind == "gaussian":
            K = torch.exp(-0.5 * d * d)
        else:  # Matern 2.5
            r = 5.0 ** 0.5 * d
            K = (1.0 + r + r * r / 3.0) * torch.exp(-r)
        u = K @ v.double()
        if w is not None:
            u += w[r0:r0 + rows_per_block].double()
        out += K.T @ u
    return out


def run_config(args):
    """Benchmark configurations 4 and 5 as measured data points (not the default line):
    --config 4: fdmmv Gaussian sigma = 1, d = 9 Uniform[0,1), M = 100,000, w = 0, N = 10^8 sharded over the
                GPUs (12.5e6 rows per GPU at any GPU count), fp32 or fp64 (--dtype);
                with --d D (> 9) the same shape at another feature count: the fp32 path then runs the K-loop
                tensor-core kernel (30 < d <= 1024), an off-headline data point;
    --config 5: fdmmv Matern 2.5 sigma = 10, fp64, N = 2e6 x d = 128 N(0,1), M = 30,000, T = 32, w ~ N(0,1), one GPU."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a GPU (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist

    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from falkon_b200 import _lib
    from falkon_b200.kernels import GaussianKernel, MaternKernel
    from falkon_b200.sharded import ShardedKernelOps

    _lib.build()
    dtype = torch.float64 if (args.dtype == "f64" or args.config == 5) else torch.float32
    g = torch.Generator(device=dev).manual_seed(1000 + args.config * 10 + rank)
    if args.config == 4:
        n, m, d, t, kind = (args.rows or 12_500_000), 100_000, args.d or 9, 1, "gaussian"
        sigma = 1.0 if d == 9 else round(float(d) ** 0.5 / 3.0, 3)  # same typical exponent at any d
        X = torch.rand(n, d, generator=g, device=dev, dtype=dtype)
        w = None
        kernel = GaussianKernel(sigma)
        what = f"config4: fdmmv Gaussian sigma={sigma:g} {args.dtype}, N={n} per GPU x d={d} U[0,1), M=100000, T=1, w=0"
        if d != 9:
            what = "off-headline variant of " + what
    else:
        n, m, d, t, sigma, kind = (args.rows or 2_000_000), 30_000, 128, 32, 10.0, "matern25"
        X = torch.randn(n, d, generator=g, device=dev, dtype=dtype)
        w = torch.randn(n, t, generator=g, device=dev, dtype=dtype)
        kernel = MaternKernel(sigma, nu=2.5)
        what = f"config5: fdmmv Matern 2.5 sigma=10 f64, N={n} x d=128 N(0,1), M=30000, T=32, w~N(0,1)"
    g0 = torch.Generator(device=dev).manual_seed(2000 + args.config)
    C = X[torch.randperm(n, generator=g0, device=dev)[:m]].contiguous()
    v = torch.randn(m, t, generator=g0, device=dev, dtype=dtype)
    if world > 1:
        dist.broadcast(C, 0)
        dist.broadcast(v, 0)
    ops = ShardedKernelOps(kernel)
    out = torch.empty(m, t, dtype=dtype, device=dev)
    for _ in range(max(args.warmup, 1)):
        ops.dmmv(X, C, v, w, out=out)
    torch.cuda.synchronize()
    _lib.set_timing(True)
    sampler = ClockSampler(dev) if rank == 0 else None
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        ops.dmmv(X, C, v, w, out=out)
    e1.record()
    torch.cuda.synchronize()
    sweeps = _lib.sweep_ms()
    clocks = sampler.stop() if rank == 0 else None
    tmax = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    ms = float(tmax.item()) / args.steps
    # spot-check on the first rows of this rank's shard against an explicit fp64 evaluation
    ns = min(n, 8192 if args.config == 5 else 16384)
    got = kernel.dmmv(X[:ns], C, v, None if w is None else w[:ns])
    want = _dense_fdmmv_fp64(X[:ns], C, v, None if w is None else w[:ns], kind, sigma)
    err = float((got.double() - want).norm() / want.norm())
    if rank == 0:
        sm_mhz = (clocks or {}).get("sm_mhz") or 1965.0
        line = {"metric": METRIC, "value": float(n) * world * m * t / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": ms,
                "scaling": "weak",
                "dtype": "f64" if dtype == torch.float64 else "f32", "data": "synthetic",
                "config": {"workload": what, "rows_per_gpu": n, "centres": m, "d": d, "T": t,
                           "tensor_core_path": bool(_lib.load().flk_uses_tensor_cores(0 if dtype == torch.float32 else 1, 0, d, t, 0))},
                "launch_ms": {"sweep1_Kv": sweeps[0], "sweep2_KTu": sweeps[1]},
                "kernel_evals_per_s_per_gpu": 2.0 * n * m / (ms * 1e-3),
                "spot_check_rel_l2_vs_fp64": err, "spot_check_rows": ns, "clocks": clocks,
                "tc_status": _lib.tc_status(dev), "range_flag": _lib.range_flag(dev)}
        if dtype == torch.float32 and d <= 30:
            # resident tensor-core kernel: one exponential per kernel evaluation, bound by the MUFU rate
            mufu = _lib.measure_mufu_rate(dev)
            evals = float(n) * m / (0.5 * (sweeps[0] + sweeps[1]) * 1e-3)
            line["roofline"] = {"bound": "mufu", "achieved": evals / 1e9, "peak": mufu / 1e9, "unit": "Gexp/s",
                                "frac": evals / mufu, "note": "per GPU (rank 0), sweep launches only; peak = ex2 "
                                "rate measured live by the probe kernel"}
        if dtype == torch.float32 and 30 < d <= 1024:
            # K-loop tensor-core kernel: bound by the tensor pipe.  fp16 MMA flops the kernel issues per evaluation:
            # three 16-feature products per feature K-step (hi.hi, hi.lo, lo.hi) plus the K-step of the norm pieces
            peaks = load_peaks()
            flops_per_eval = 2.0 * 16.0 * (3 * ((d + 15) // 16) + 1)
            evals = float(n) * m / (0.5 * (sweeps[0] + sweeps[1]) * 1e-3)
            line["roofline"] = {"bound": "tensor", "achieved": evals * flops_per_eval / 1e12,
                                "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                "frac": evals * flops_per_eval / 1e12 / peaks["bf16_tflops"],
                                "frac_of_sustained_peak": evals * flops_per_eval / 1e12 / (peaks["bf16_sustained"] or peaks["bf16_tflops"]),
                                "peak_source": peaks["source"], "flops_per_eval": flops_per_eval,
                                "note": "per GPU (rank 0), sweep launches only; fp16 MMA flops issued against the "
                                        "measured bf16 GEMM peaks (burst / seconds-long under the power cap)"}
        if dtype == torch.float64:
            dfma_per_pair = d + (t if t > 4 else 4 + t) + 4
            peak = 148 * 64 * sm_mhz * 1e6
            line["fp64"] = {"dfma_per_kernel_eval_excluding_transcendentals": dfma_per_pair,
                            "achieved_tdfma_per_s": 2.0 * n * m * dfma_per_pair / (ms * 1e-3) / 1e12,
                            "nominal_peak_tdfma_per_s": peak / 1e12,
                            "frac": 2.0 * n * m * dfma_per_pair / (ms * 1e-3) / peak,
                            "note": "nominal 64 fp64 FMA lanes per SM x sampled clock; exp / sqrt (software, fp64) not counted"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def _fp64_reference_entries(X, w, C, v, cols, sigma, rows_per_block=8192):
    """This rank's part of  out[cols] = sum_i K(x_i, c_cols) (K(x_i, C) v + w_i)  in fp64, independent of the
    library: fp64 GEMMs and element-wise torch ops on the norm expansion, block by block over the rank's rows."""
    Cs = C.double() / sigma
    cn_half = 0.5 * (Cs * Cs).sum(dim=1)
    vd = v.double()
    acc = torch.zeros(len(cols), v.shape[1], dtype=torch.float64, device=X.device)
    for r0 in range(0, X.shape[0], rows_per_block):
        Xs = X[r0:r0 + rows_per_block].double() / sigma
        xn_half = 0.5 * (Xs * Xs).sum(dim=1, keepdim=True)
        G = torch.addmm(-xn_half, Xs, Cs.t())  # x.c - |x|^2/2
        G.sub_(cn_half).clamp_max_(0.0).exp_()  # exp(-(|x|^2 + |c|^2 - 2 x.c) / 2)
        u = G @ vd
        u += w[r0:r0 + rows_per_block].double()
        acc += G[:, cols].t() @ u
    return acc


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=0,
                    help="override the row count (config 3: total rows; 2, 4, 5: rows per GPU)")
    ap.add_argument("--simt", action="store_true", help="force the SIMT kernel (comparison runs)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-parity", action="store_true", help="skip the fp64 check of sampled outputs (profiling runs)")
    ap.add_argument("--cpu-rows", type=int, default=CPU_SAMPLE_ROWS, help="rows of the bounded CPU sample")
    ap.add_argument("--fit", action="store_true", help="run the full Falkon.fit of benchmark configuration 3 instead")
    ap.add_argument("--centres", type=int, default=50_000, help="number of Nystrom centres for --fit")
    ap.add_argument("--config", type=int, default=3, choices=[2, 3, 4, 5],
                    help="3 = the benchmark line (default): the fdmmv of the fit configuration, N = 1e7 rows split over "
                         "the GPUs, M = 50,000; 2 = 1e6 rows per GPU, M = 20,000 (weak scaling); 4 / 5 = the other "
                         "fdmmv configurations as data points")
    ap.add_argument("--dtype", default="f32", choices=["f32", "f64"], help="--config 4 only")
    ap.add_argument("--d", type=int, default=0, help="--config 4 only: feature count of an off-headline data point")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)
    if args.impl == "reference":
        return run_reference(args)
    if args.fit:
        return run_fit(args)
    if args.config in (4, 5):
        if args.steps == 20:
            args.steps = 3
        return run_config(args)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a GPU (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist

    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from falkon_b200 import FalkonOptions, _lib
    from falkon_b200.kernels import GaussianKernel
    from falkon_b200.sharded import ShardedKernelOps

    _lib.build()
    lib = _lib.load()
    if lib.flk_check_device() != 0:
        raise RuntimeError(_lib.last_error())
    wl = workload(args.config, world, args.rows)
    n, m = wl["n_local"], wl["m"]
    X, w = gen_shard(n, 1000 + wl["config"] + 100 * rank, dev)
    g = torch.Generator(device=dev).manual_seed(2000 + wl["config"])
    # centres: M rows of rank 0's shard, replicated on every rank
    idx = torch.randperm(n, generator=g, device=dev)[:m] if n >= m else torch.randint(n, (m,), generator=g, device=dev)
    C = X[idx].contiguous()
    v = torch.randn(m, T, generator=g, device=dev)
    if world > 1:
        dist.broadcast(C, 0)
        dist.broadcast(v, 0)
    opt = FalkonOptions()
    kernel = GaussianKernel(SIGMA, opt=opt)
    flags = _lib.FLAG_FORCE_SIMT if args.simt else 0
    kernel.params.flk_flags = flags
    kernel.params.flk_devices = [local_rank]  # host-operand calls stay on this rank's GPU (n_gpus is the claim)
    ops = ShardedKernelOps(kernel)
    out = torch.empty(m, T, dtype=torch.float32, device=dev)
    # L2 hygiene: configuration 3 streams 1.1 GB of X (3.8 GB of operand images) per step, far beyond the 126 MB
    # L2, so nothing of one step survives into the next; configuration 2 (0.4 GB of images per GPU) additionally
    # writes a 256 MB buffer between the timed steps.
    flush = torch.empty(256 * 2**20, dtype=torch.uint8, device=dev) if wl["config"] == 2 else None

    def step():
        ops.dmmv(X, C, v, w, out=out)

    for _ in range(max(args.warmup, 0)):
        step()
    torch.cuda.synchronize()

    # ---------------- timed region: K steps, device events per step ----------
    _lib.set_timing(True)
    ops.collective_events = []  # CUDA events around every all-reduce of the timed steps
    sampler = ClockSampler(dev) if rank == 0 else None
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    sweep_ms = []
    launches0 = _lib.launch_count()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        sampler.start()
    wall0 = time.perf_counter()
    for i in range(args.steps):
        if flush is not None:
            flush.fill_(i & 0xFF)
        starts[i].record()
        step()
        stops[i].record()
        sweep_ms.append(_lib.sweep_ms())  # waits for this step's sweeps (also paces the host)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    wall = time.perf_counter() - wall0
    launches = _lib.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    _lib.set_timing(False)
    coll_events, ops.collective_events = ops.collective_events, None
    step_ms = [s.elapsed_time(e) for s, e in zip(starts, stops)]
    dev_ms = sum(step_ms)
    coll_ms = [a.elapsed_time(b) for a, b in coll_events]
    red = torch.tensor([dev_ms, float(np.mean(coll_ms)) if coll_ms else 0.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(red, op=dist.ReduceOp.MAX)
    total_ms = float(red[0].item())
    collective_ms = float(red[1].item())
    ms_per_step = total_ms / args.steps
    pairs_per_step = float(wl["n_total"]) * m * T
    value = pairs_per_step / (ms_per_step * 1e-3)
    tc_status = _lib.tc_status(dev)

    # ---------------- parity of the all-reduced result: sampled entries against fp64 ----------------
    parity = None
    if not args.no_parity:
        gj = torch.Generator().manual_seed(77)
        cols = torch.randperm(m, generator=gj)[:16].to(dev)
        ref = _fp64_reference_entries(X, w, C, v, cols, SIGMA)
        if world > 1:
            dist.all_reduce(ref, op=dist.ReduceOp.SUM)
        got = out[cols].double()
        rel = float((got - ref).norm() / ref.norm())
        worst = float(((got - ref).abs() / ref.abs().clamp_min(1e-300)).max())
        parity = {"rel_l2": rel, "max_rel_entry": worst, "entries": int(cols.numel()), "tolerance": 1e-4,
                  "ok": bool(rel <= 1e-4),
                  "against": "fp64 GEMM + element-wise evaluation in torch of the same sampled outputs over ALL rows "
                             "of all ranks (summed across ranks), compared with the result after the all-reduce"}

    # ---------------- the single product K v of the same configuration (a data point beside the headline) ----
    fmmv_out = torch.empty(n, T, dtype=torch.float32, device=dev)
    fmmv_steps = max(3, min(args.steps, 10))
    kernel.mmv(X, C, v, out=fmmv_out)
    fe0, fe1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fmmv_ms = []
    for i in range(fmmv_steps):
        if flush is not None:
            flush.fill_(i & 0xFF)
        fe0.record()
        kernel.mmv(X, C, v, out=fmmv_out)
        fe1.record()
        fe1.synchronize()
        fmmv_ms.append(fe0.elapsed_time(fe1))
    del fmmv_out

    # ---------------- end-to-end through the host-buffer entry point (each rank its own shard) ----
    e2e = None
    if not args.no_e2e:
        Xh = X.cpu().pin_memory()
        Ch = C.cpu().pin_memory()
        vh = v.cpu().pin_memory()
        wh = w.cpu().pin_memory()
        outh = torch.empty(m, T, dtype=torch.float32).pin_memory()
        e2e_steps = max(3, min(args.steps, 5))
        ops.dmmv(Xh, Ch, vh, wh, out=outh)  # warm-up (sizes the workspace)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            ops.dmmv(Xh, Ch, vh, wh, out=outh)  # returns after the (all-reduced) result is on the host
        torch.cuda.synchronize()
        e2e_s = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
        e2e_value = pairs_per_step * e2e_steps / float(e2e_s.item())
        e2e_vs_dev = float((outh.to(dev) - out).norm() / out.norm())
        e2e = {"value": e2e_value, "unit": UNIT,
               "h2d_bytes_per_step": (Xh.numel() + Ch.numel() + vh.numel() + wh.numel()) * 4,
               "d2h_bytes_per_step": outh.numel() * 4, "steps": e2e_steps, "rel_l2_vs_device_path": e2e_vs_dev,
               "note": "per rank: its own row shard from pinned host memory through Kernel.dmmv -> flk_fdmmv_host "
                       "(copies inside the timed region, overlapped with the kernels in row chunks), then the "
                       "all-reduce; bytes are per rank"}
        del Xh, wh

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---------------- roofline of the dominant kernel ----------------
    # One launch of the sweep kernel evaluates the kernel function once for every (row, centre) pair of this
    # rank.  The unit that bounds it is the special-function unit (one exponential per evaluation, 16 MUFU
    # lanes per SM); the kernel moves part of the exponentials to the FMA pipe, so the achieved exponential
    # rate may exceed the MUFU rate.  The denominator is measured live with the library's probe kernel
    # (nothing but ex2 on every SM), the numerator is the CUDA-event duration of the sweep launches recorded by
    # the library on the launch stream.  An fdmmv that never stores K must evaluate K twice (u = K v + w has to
    # be complete before K^T u can start), so two views are given: per sweep launch (executed work) and per
    # fdmmv step with every pair counted once (algorithmic work).
    peaks = load_peaks()
    s1 = float(np.mean([a for a, _ in sweep_ms if a >= 0])) if sweep_ms else float("nan")
    s2 = float(np.mean([b for _, b in sweep_ms if b >= 0])) if sweep_ms else float("nan")
    sweep_avg_ms = 0.5 * (s1 + s2)
    pairs_per_launch = float(n) * m  # one sweep evaluates every (row, centre) pair of the rank once
    uses_tc = bool(lib.flk_uses_tensor_cores(0, 0, D, T, flags))
    sm_mhz = (clocks or {}).get("sm_mhz") or 1965.0
    evals_per_s = pairs_per_launch / (sweep_avg_ms * 1e-3)
    mufu_rate = _lib.measure_mufu_rate(dev)
    mufu_at_clock = 148 * 16 * sm_mhz * 1e6
    # tensor flops of the split-fp16 formulation per pair: 2 * (3 d + 2 * norm pieces), d = 28 -> 3 pieces
    k_used = 3 * D + 2 * 3
    tensor_tflops = evals_per_s * 2 * k_used / 1e12
    fp32_peak_tflops = 148 * 128 * 2 * sm_mhz * 1e6 / 1e12
    alg_flops_pair = 2 * D + 4 * T + 6 + 1  # algorithmic fdmmv flops per pair, each pair counted once
    # DRAM traffic of one sweep launch: 210 bytes per row of X, from the ncu capture at 400,000 rows
    # (80.9 MB read + 3.1 MB written; algorithmic 84 MB), scaled by rows (traffic is proportional to rows)
    traffic = 210.0 * n if uses_tc else None
    alg_bytes = (n * (3 * D + 6 + 6) * 2.0 + m * 96 * 2.0 + n * 4.0 + m * 4.0) if uses_tc else None
    per_gpu_pairs_per_s = value / world
    roofline = {
        "bound": "mufu" if uses_tc else "fp32",
        "kernel": "flk::tc::kmv_tc_kernel" if uses_tc else "flk::kmv_simt_kernel",
        "achieved": evals_per_s / 1e9 if uses_tc else evals_per_s * alg_flops_pair / 1e12,
        "peak": mufu_rate / 1e9 if uses_tc else fp32_peak_tflops,
        "unit": "Gexp/s" if uses_tc else "TFLOP/s",
        "frac": evals_per_s / mufu_rate if uses_tc else evals_per_s * alg_flops_pair / 1e12 / fp32_peak_tflops,
        "traffic": traffic,
        "view": "executed work of one sweep launch on rank 0 (one exponential per pair per sweep)",
        "peak_source": ("MUFU ex2 rate measured live on this GPU by flk_probe_mufu, a short burst at the boost clock "
                        f"(148 SMs x 16 lanes x the clock sampled under load = {mufu_at_clock / 1e9:.0f} Gexp/s); "
                        "the sweep is neither HBM- nor tensor-bound"
                        if uses_tc else "fp32 FMA lanes x sampled SM clock (nominal lanes)"),
        "frac_at_sampled_clock": evals_per_s / mufu_at_clock if uses_tc else None,
        "per_fdmmv": {"achieved": per_gpu_pairs_per_s / 1e9, "peak": mufu_rate / 1e9, "unit": "Gpair/s per GPU",
                      "frac": per_gpu_pairs_per_s / mufu_rate,
                      "note": "algorithmic view: every (row, centre) pair counted once per fdmmv step (the exact "
                              "K-free product evaluates it twice), whole step incl. operand preparation and all-reduce"},
        "launch_ms": {"sweep1_Kv": s1, "sweep2_KTu": s2},
        "pairs_per_launch": pairs_per_launch,
        "algorithmic_bytes_per_launch": alg_bytes,
        "tensor": {"achieved_tflops": tensor_tflops, "peak_tflops": peaks["bf16_tflops"],
                   "frac": tensor_tflops / peaks["bf16_tflops"],
                   "note": f"fp16 MMA flops of the exponent GEMM (K = {k_used} used of 96) vs {peaks['source']} bf16 peak"},
        "hbm": {"achieved_gbs": (traffic or 0.0) / (sweep_avg_ms * 1e-3) / 1e9, "peak_gbs": peaks["hbm_gbs"],
                "frac": (traffic or 0.0) / (sweep_avg_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]},
        "fp32_algorithmic": {"flops_per_pair": alg_flops_pair,
                             "achieved_tflops": per_gpu_pairs_per_s * alg_flops_pair / 1e12,
                             "peak_tflops": fp32_peak_tflops,
                             "frac": per_gpu_pairs_per_s * alg_flops_pair / 1e12 / fp32_peak_tflops,
                             "note": "north-star view: 2d + 4T + 6 + 1 flops per pair, each pair once, as if done on "
                                     "the FP32 FMA pipe (128 lanes per SM x sampled clock)"},
    }
    cpu_baseline = None
    if not args.no_cpu_baseline and world == 1:
        n_cpu = min(args.cpu_rows, wl["n_total"])
        val, secs, cores, kind, what = time_cpu_baseline(wl, n_cpu, reps=1)
        cpu_baseline = {"value": val, "unit": UNIT, "cores": cores, "kind": kind,
                        "sample": f"one fdmmv on the first {n_cpu} rows of the workload with all M={m} centres (d={D}), "
                                  f"{secs:.1f} s, {what}, {cores} threads"}
    cfg = base_config(wl, world)
    cfg.update({
        "kernel": "simt" if args.simt else "tcgen05 split-fp16 + MUFU/FMA exponential",
        "l2": ("inputs larger than L2: every step streams the rank's operand images (192 B per row per sweep)"
               if flush is None else "256 MB buffer written between timed steps"),
        "collective": "NCCL all-reduce of the M x T partial" if world > 1 else "none",
        "sample": "full workload",
    })
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": wl["scaling"], "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": cfg,
        "roofline": roofline,
        "cpu_baseline": cpu_baseline,
        "e2e": e2e,
        "parity": parity,
        "collective_ms": collective_ms,
        "ms_x_mhz": ms_per_step * sm_mhz,
        "step_ms": {"min": float(min(step_ms)), "median": float(np.median(step_ms)), "max": float(max(step_ms)),
                    "note": "per-step CUDA-event times of rank 0"},
        "fmmv": {"value": float(n) * m * T / (float(np.median(fmmv_ms)) * 1e-3), "unit": "pair-evals/s per GPU",
                 "ms_median": float(np.median(fmmv_ms)), "ms_min": float(min(fmmv_ms)), "steps": fmmv_steps,
                 "note": "K v alone (one sweep) on this rank's rows, same inputs"},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "wall_s_timed_region": wall,
        "tc_status": tc_status,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
