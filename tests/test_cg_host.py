"""CPU tests of the device-resident conjugate gradient (falkon_b200/optim/conjgrad.py): the masked, decision-free
iteration must produce the iterates of the textbook loop the reference runs (falkon/optim/conjgrad.py:95-186,
restated in oracle/falkon_fit_oracle.py and, with the early stop and per-column freezing, below).
"""
import pytest
import torch

from falkon_b200.optim import ConjugateGradient, StopOptimizationException
from falkon_b200.options import ConjugateGradientOptions
from oracle import falkon_fit_oracle as ffo


def _spd(m, cond, seed):
    g = torch.Generator().manual_seed(seed)
    q, _ = torch.linalg.qr(torch.randn(m, m, generator=g, dtype=torch.float64))
    ev = torch.logspace(0, -cond, m, dtype=torch.float64)
    return (q * ev) @ q.T


def _loop_with_host_decisions(B, mmv, max_iter, eps, tol, refresh_every, per_column):
    """The reference's control flow, spelled out with host-side decisions, as the yardstick."""
    X, R = torch.zeros_like(B), B.clone()
    P, rho = R.clone(), R.square().sum(0)
    live = torch.ones(B.shape[1], dtype=torch.bool)
    last = None
    for it in range(max_iter):
        last = it
        AP = mmv(P)
        alpha = torch.where(live, rho / ((P * AP).sum(0) + eps), torch.zeros_like(rho))
        X = X + P * alpha
        if refresh_every and (it + 1) % refresh_every == 0:
            R = torch.where(live, B - mmv(X), R)
        else:
            R = R - AP * alpha
        rho_new = R.square().sum(0)
        met = rho_new < tol ** 2
        if bool(met.all()):
            break
        nxt = live & ~met if per_column else live
        beta = torch.where(nxt, rho_new / (rho + eps), torch.zeros_like(rho))
        P = torch.where(nxt, P * beta + R, P)
        rho = torch.where(live, rho_new, rho)
        live = nxt
    return X, last


@pytest.mark.parametrize("per_column", [False, True])
@pytest.mark.parametrize("refresh_every", [0, 3, 10])
def test_iterates_equal_the_host_decided_loop(per_column, refresh_every):
    m, t = 60, 4
    A = _spd(m, 1.5, seed=1)  # well conditioned: rounding differences between the two loops stay at rounding level
    g = torch.Generator().manual_seed(2)
    B = torch.randn(m, t, generator=g, dtype=torch.float64)
    B[:, 1] *= 1e-9   # this column meets the tolerance at once
    B[:, 2] = A[:, 5]  # and this one after one step
    opt = ConjugateGradientOptions(cg_tolerance=1e-8, cg_full_gradient_every=refresh_every,
                                   cg_differential_convergence=per_column)
    for max_iter in (1, 7, 40, 200):
        cg = ConjugateGradient(opt)
        got = cg.solve(None, B.clone(), lambda v: A @ v, max_iter)
        want, last = _loop_with_host_decisions(B, lambda v: A @ v, max_iter, opt.cg_epsilon(torch.float64), 1e-8,
                                               refresh_every, per_column)
        # both loops stop on the tolerance 1e-8: their iterates agree to that level (bitwise equality is not expected,
        # the two accumulate in a different order)
        torch.testing.assert_close(got, want, rtol=1e-6, atol=1e-7)
        assert cg.num_iter == last, (max_iter, cg.num_iter, last)


def test_agrees_with_the_oracle_loop_and_the_dense_solve():
    m = 80
    A = _spd(m, 2.0, seed=3)
    B = torch.randn(m, 3, generator=torch.Generator().manual_seed(4), dtype=torch.float64)
    opt = ConjugateGradientOptions()  # the oracle loop runs the default options
    got = ConjugateGradient(opt).solve(None, B.clone(), lambda v: A @ v, 25)
    torch.testing.assert_close(got, ffo.conjugate_gradient(B.clone(), lambda v: A @ v, 25), rtol=1e-5, atol=1e-6)
    full = ConjugateGradient(ConjugateGradientOptions(cg_tolerance=1e-12)).solve(None, B.clone(), lambda v: A @ v, 500)
    torch.testing.assert_close(full, torch.linalg.solve(A, B), rtol=1e-5, atol=1e-6)


def test_warm_start_and_callback_stop():
    m = 40
    A = _spd(m, 1.0, seed=5)
    B = torch.randn(m, 2, generator=torch.Generator().manual_seed(6), dtype=torch.float64)
    exact = torch.linalg.solve(A, B)
    cg = ConjugateGradient(ConjugateGradientOptions(cg_tolerance=1e-9))
    got = cg.solve(exact.clone(), B.clone(), lambda v: A @ v, 50)
    assert cg.num_iter <= 1 and float((got - exact).norm() / exact.norm()) <= 1e-8
    seen = []

    def stop_at_three(it, X, elapsed):
        seen.append(it)
        if it == 3:
            raise StopOptimizationException("enough")

    cg.solve(None, B.clone(), lambda v: A @ v, 50, callback=stop_at_three)
    assert seen == [1, 2, 3]


def test_no_host_read_inside_the_loop_without_refresh(monkeypatch):
    """With cg_full_gradient_every = 0 the loop never converts a device value on the host: the only conversions are
    the final read of the iteration counter."""
    m = 30
    A = _spd(m, 1.0, seed=7)
    B = torch.randn(m, 1, generator=torch.Generator().manual_seed(8), dtype=torch.float64)
    reads = []
    real_float, real_int = torch.Tensor.__float__, torch.Tensor.__int__
    monkeypatch.setattr(torch.Tensor, "__float__", lambda self: (reads.append("float"), real_float(self))[1])
    monkeypatch.setattr(torch.Tensor, "__int__", lambda self: (reads.append("int"), real_int(self))[1])
    monkeypatch.setattr(torch.Tensor, "__bool__", lambda self: (_ for _ in ()).throw(AssertionError("host decision")))
    ConjugateGradient(ConjugateGradientOptions(cg_full_gradient_every=0)).solve(None, B, lambda v: A @ v, 30)
    assert reads == ["int"]


def test_device_timeout_status_becomes_an_exception(monkeypatch):
    """A tensor-core sweep that gave up on a bounded wait leaves a code in the device status word (and NaN in its
    results); the Falkon solver turns the word into FlkError after the solve.  The mapping is host logic: exercised
    here with a stand-in for the status read, no GPU and no hung kernel involved."""
    from falkon_b200 import _lib
    from falkon_b200.optim import FalkonConjugateGradient

    class OnDevice:  # what _check_device_status looks at: where the tensor lives
        is_cuda = True
        device = torch.device("cuda", 0)

    solver = FalkonConjugateGradient(kernel=object(), preconditioner=object())
    monkeypatch.setattr(_lib, "tc_status", lambda device: 0)
    solver._check_device_status(None, OnDevice())  # clean status: nothing happens
    monkeypatch.setattr(_lib, "tc_status", lambda device: 0x31)
    with pytest.raises(_lib.FlkError) as err:
        solver._check_device_status(OnDevice())
    assert err.value.status == _lib.FLK_ERR_TIMEOUT and "0x31" in str(err.value)
    solver._check_device_status(torch.zeros(3))  # host tensors (the gloo tests) are not asked about
