"""CPU tests of the in-process multi-GPU fan-out for host operands (row split, one thread per device,
ordered reduction, failure propagation), with the per-device library call replaced by the CPU oracle."""
import os
import sys
import threading

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from falkon_b200.mmv_ops import multi_device as md  # noqa: E402
from oracle import falkon_oracle as fo  # noqa: E402


def test_split_rows():
    for n in (0, 1, 5, 131072 * 3 + 1):
        for parts in (1, 2, 3, 8):
            spans = md.split_rows(n, parts)
            assert len(spans) == parts and spans[0][0] == 0
            assert sum(ln for _, ln in spans) == n
            for (s0, l0), (s1, _) in zip(spans, spans[1:]):
                assert s0 + l0 == s1
            assert max(ln for _, ln in spans) - min(ln for _, ln in spans) <= 1


def _inputs(n=1003, m=41, d=6, t=3, seed=3):
    rng = np.random.default_rng(seed)
    return tuple(torch.from_numpy(rng.standard_normal(s)) for s in ((n, d), (m, d), (m, t), (n, t)))


def test_fdmmv_fan_out_matches_single_call():
    X, C, v, w = _inputs()
    seen = []

    def call(kernel_id, sigma, X1, X2, vv, ww, out, flags=0, host=False, device=None):
        assert host and kernel_id == 0
        seen.append((device, X1.shape[0], threading.current_thread().name))
        out.copy_(fo.fdmmv(X1, X2, vv, ww, "gaussian", float(sigma[0])))

    devices = [torch.device("cuda", i) for i in range(3)]
    out = torch.empty(41, 3, dtype=torch.float64)
    md.fdmmv_host_multi(0, np.array([2.0]), X, C, v, w, out, 0, devices, call=call)
    want = fo.fdmmv(X, C, v, w, "gaussian", 2.0)
    assert fo.rel_l2(out.numpy(), want.numpy()) < 1e-13
    assert sorted(d.index for d, _, _ in seen) == [0, 1, 2]
    assert sorted(r for _, r, _ in seen) == [334, 334, 335]
    assert all(name.startswith("flk-gpu-") for _, _, name in seen)
    # w = None and v = None forms
    md.fdmmv_host_multi(0, np.array([2.0]), X, C, v, None, out, 0, devices, call=call)
    assert fo.rel_l2(out.numpy(), fo.fdmmv(X, C, v, None, "gaussian", 2.0).numpy()) < 1e-13
    md.fdmmv_host_multi(0, np.array([2.0]), X, C, None, w, out, 0, devices, call=call)
    assert fo.rel_l2(out.numpy(), fo.fdmmv(X, C, None, w, "gaussian", 2.0).numpy()) < 1e-13


def test_fmmv_fan_out_writes_row_slices():
    X, C, v, _ = _inputs(n=10, m=7)

    def call(kernel_id, sigma, X1, X2, vv, out, flags=0, host=False, device=None):
        out.copy_(fo.fmmv(X1, X2, vv, "gaussian", float(sigma[0])))

    devices = [torch.device("cuda", i) for i in range(4)]
    out = torch.full((10, 3), float("nan"), dtype=torch.float64)
    md.fmmv_host_multi(0, np.array([1.5]), X, C, v, out, 0, devices, call=call)
    assert fo.rel_l2(out.numpy(), fo.fmmv(X, C, v, "gaussian", 1.5).numpy()) < 1e-13
    # more devices than rows: empty slices are skipped
    md.fmmv_host_multi(0, np.array([1.5]), X[:2], C, v, out[:2], 0, devices, call=call)


def test_worker_failure_propagates():
    X, C, v, w = _inputs(n=64)

    def call(kernel_id, sigma, X1, X2, vv, ww, out, flags=0, host=False, device=None):
        if device.index == 1:
            raise ValueError("boom on device 1")
        out.zero_()

    out = torch.empty(41, 3, dtype=torch.float64)
    with pytest.raises(RuntimeError) as info:
        md.fdmmv_host_multi(0, np.array([2.0]), X, C, v, w, out, 0, [torch.device("cuda", i) for i in range(2)],
                            call=call)
    assert isinstance(info.value.__cause__, ValueError)


def test_host_devices_policy(monkeypatch):
    class Opt:
        flk_devices = None

    primary = torch.device("cuda", 0)
    monkeypatch.setattr(torch.cuda, "device_count", lambda: 8)
    assert md.host_devices(Opt(), 1000, primary) == [primary]                       # too few rows to split
    assert len(md.host_devices(Opt(), md.MIN_ROWS_PER_DEVICE * 3, primary)) == 3     # as many as pay off
    assert len(md.host_devices(Opt(), 10**8, primary)) == 8
    o = Opt()
    o.flk_devices = [2, 5]
    assert md.host_devices(o, 10**8, primary) == [torch.device("cuda", 2), torch.device("cuda", 5)]
    o.flk_devices = [0]
    assert md.host_devices(o, 10**8, primary) == [primary]
    monkeypatch.setattr(torch.distributed, "is_initialized", lambda: True)
    assert md.host_devices(Opt(), 10**8, primary) == [primary]                       # one process per GPU: no fan-out
