"""Integrator steps (reference: dynamis_integrator/src/csrc/*.cu) and the drift word riding on them.

* bit-exact against the C oracle (oracle/integrator_oracle.c) on random states, all five kinds;
* the analytic cases the reference's own tests use (dynamis_integrator/tests/test_verlet.py,
  test_euler.py, test_langevin.py): zero force, constant force with unit and non-unit mass, zero
  friction reducing Langevin to Verlet;
* the fused drift word equals the separate pass (dynb_drift_flag) and the oracle's word, and leaves the
  same previous-velocity buffer behind.
"""

import numpy as np
import pytest
import torch

import dynamis_b200 as D
from dynamis_b200 import integrators as I
from oracle import cpu_oracle as O

pytestmark = pytest.mark.gpu


def _state(n, seed):
    rng = np.random.default_rng(seed)
    pos = (rng.random((n, 3)) * 50.0).astype(np.float32)
    vel = rng.normal(0, 0.05, (n, 3)).astype(np.float32)
    frc = rng.normal(0, 2.0, (n, 3)).astype(np.float32)
    mass = rng.choice(np.array([1.008, 12.011, 15.999, 63.546], dtype=np.float32), n)
    noise = rng.normal(0, 1.0, (n, 3)).astype(np.float32)
    return pos, vel, frc, mass, noise


def _t(a, dev):
    return torch.as_tensor(a.copy(), device=dev)


@pytest.mark.parametrize("n", [1, 257, 100_003])
@pytest.mark.parametrize("kind", [I.EULER, I.VERLET1, I.VERLET2, I.LANGEVIN1, I.LANGEVIN2])
def test_steps_bit_exact_vs_oracle(cuda, kind, n):
    pos, vel, frc, mass, noise = _state(n, 40 + kind)
    dt, gamma, kT = 0.5, 0.01, 0.0257
    tp, tv, tf, tm, tn = (_t(a, cuda) for a in (pos, vel, frc, mass, noise))
    if kind == I.EULER:
        I.Euler.step_(tp, tv, tf, tm, dt)
    elif kind == I.VERLET1:
        I.Verlet(dt).halfstep1_(tp, tv, tf, tm, dt)
    elif kind == I.VERLET2:
        I.Verlet(dt).halfstep2_(tv, tf, tm, dt)
    elif kind == I.LANGEVIN1:
        I.Langevin(dt, gamma, kT).halfstep1_(tp, tv, tf, tm, tn, dt)
    else:
        I.Langevin(dt, gamma, kT).halfstep2_(tv, tf, tm, tn, dt)
    O.integrator_step(kind, pos, vel, frc, mass, noise, dt, gamma, kT)
    np.testing.assert_array_equal(tv.cpu().numpy(), vel)
    np.testing.assert_array_equal(tp.cpu().numpy(), pos)


@pytest.mark.parametrize("n", [1, 257, 100_003])
def test_steps_bit_exact_vs_reference_kernels(cuda, ref_ops, n):
    """The reference's own integrator kernels (compiled from its sources by oracle/build_ref.py) next to
    ours on the same state: all five steps, every float equal."""
    dt, gamma, kT = 0.5, 0.01, 0.0257
    for kind in (I.EULER, I.VERLET1, I.VERLET2, I.LANGEVIN1, I.LANGEVIN2):
        pos, vel, frc, mass, noise = _state(n, 140 + kind)
        tp, tv, tf, tm, tn = (_t(a, cuda) for a in (pos, vel, frc, mass, noise))
        rp, rv = _t(pos, cuda), _t(vel, cuda)
        if kind == I.EULER:
            I.Euler.step_(tp, tv, tf, tm, dt)
            ref_ops.euler_step(rp, rv, tf, tm, dt)
        elif kind == I.VERLET1:
            I.Verlet(dt).halfstep1_(tp, tv, tf, tm, dt)
            ref_ops.verlet_halfstep1(rp, rv, tf, tm, dt)
        elif kind == I.VERLET2:
            I.Verlet(dt).halfstep2_(tv, tf, tm, dt)
            ref_ops.verlet_halfstep2(rv, tf, tm, dt)
        elif kind == I.LANGEVIN1:
            I.Langevin(dt, gamma, kT).halfstep1_(tp, tv, tf, tm, tn, dt)
            ref_ops.langevin_halfstep1(rp, rv, tf, tm, tn, gamma, kT, dt)
        else:
            I.Langevin(dt, gamma, kT).halfstep2_(tv, tf, tm, tn, dt)
            ref_ops.langevin_halfstep2(rv, tf, tm, tn, gamma, kT, dt)
        assert torch.equal(tv, rv), f"velocities differ from the reference kernel (kind {kind})"
        assert torch.equal(tp, rp), f"positions differ from the reference kernel (kind {kind})"


def test_analytic_cases(cuda):
    mk = lambda rows: torch.tensor(rows, dtype=torch.float32, device=cuda)
    # zero force: velocity unchanged, position advances by v dt
    pos, vel, frc, mass = mk([[0, 0, 0], [0, 0, 0]]), mk([[1, 0, 0], [0, 2, 0]]), mk([[0, 0, 0], [0, 0, 0]]), mk([1, 1]).reshape(-1)
    vl = I.Verlet(0.1)
    vl.halfstep1_(pos, vel, frc, mass, 0.1)
    vl.halfstep2_(vel, frc, mass, 0.1)
    assert torch.allclose(vel, mk([[1, 0, 0], [0, 2, 0]])) and torch.allclose(pos, mk([[0.1, 0, 0], [0, 0.2, 0]]))
    # constant force F = 2 on m = 1, dt = 0.5: v_half = 0.5, x = 0.25, v = 1.0
    pos, vel, frc, mass = mk([[0, 0, 0]]), mk([[0, 0, 0]]), mk([[2, 0, 0]]), mk([1]).reshape(-1)
    vl.halfstep1_(pos, vel, frc, mass, 0.5)
    assert torch.allclose(vel, mk([[0.5, 0, 0]])) and torch.allclose(pos, mk([[0.25, 0, 0]]))
    vl.halfstep2_(vel, frc, mass, 0.5)
    assert torch.allclose(vel, mk([[1.0, 0, 0]]))
    # Euler, F = 4 on m = 2, dt = 0.25: v = 0.5, x = 0.125
    pos, vel, frc, mass = mk([[0, 0, 0]]), mk([[0, 0, 0]]), mk([[4, 0, 0]]), mk([2]).reshape(-1)
    I.Euler.step_(pos, vel, frc, mass, 0.25)
    assert torch.allclose(vel, mk([[0.5, 0, 0]])) and torch.allclose(pos, mk([[0.125, 0, 0]]))
    # Langevin with gamma = 0 is Verlet, whatever the noise
    p0, v0, f0, m0, nz = _state(1000, 9)
    a = [_t(x, cuda) for x in (p0, v0, f0, m0, nz)]
    b = [_t(x, cuda) for x in (p0, v0, f0, m0)]
    lg = I.Langevin(0.5, 0.0, 0.0257)
    lg.halfstep1_(a[0], a[1], a[2], a[3], a[4], 0.5)
    vl.halfstep1_(b[0], b[1], b[2], b[3], 0.5)
    assert torch.allclose(a[0], b[0]) and torch.allclose(a[1], b[1])
    lg.halfstep2_(a[1], a[2], a[3], a[4], 0.5)
    vl.halfstep2_(b[1], b[2], b[3], 0.5)
    assert torch.allclose(a[1], b[1])


def test_argument_checks(cuda):
    pos, vel, frc, mass, noise = (_t(a, cuda) for a in _state(8, 1))
    with pytest.raises(ValueError, match="same shape"):
        I.Euler.step_(pos, vel[:4], frc, mass, 0.1)
    with pytest.raises(ValueError, match="Mass tensor"):
        I.Euler.step_(pos, vel, frc, mass[:3], 0.1)
    with pytest.raises(ValueError, match="same device"):
        I.Euler.step_(pos, vel.cpu(), frc, mass, 0.1)
    with pytest.raises(ValueError, match="2D"):
        I.Verlet(0.1).halfstep2_(vel.reshape(-1), frc.reshape(-1), mass, 0.1)
    from dynamis_b200 import _lib
    assert _lib.lib().dynb_integrator_step(7, None, None, None, None, None, 1, 0.1, 0, 0, None, None, 0, None, None, None) != 0
    assert _lib.lib().dynb_integrator_step(2, None, vel.data_ptr(), frc.data_ptr(), mass.data_ptr(), None, 8, 0.1, 0, 0,
                                           None, None, 0.0, None, pos.data_ptr(), None) != 0  # drift on a step that moves nothing


@pytest.mark.parametrize("kind", [I.EULER, I.VERLET1, I.LANGEVIN1])
@pytest.mark.parametrize("threshold", [0.01, 0.2, 50.0])
def test_fused_drift_word(cuda, kind, threshold):
    n, dt, gamma, kT = 50_001, 0.5, 0.01, 0.0257
    pos, vel, frc, mass, noise = _state(n, 77 + kind)
    ref = pos + np.random.default_rng(5).normal(0, 0.02, pos.shape).astype(np.float32)
    pvel = vel + np.random.default_rng(6).normal(0, 0.01, vel.shape).astype(np.float32)

    def run(fused):
        tp, tv, tf, tm, tn = (_t(a, cuda) for a in (pos, vel, frc, mass, noise))
        watch = I.DriftWatch(_t(ref, cuda), _t(pvel, cuda), threshold)
        d = watch if fused else None
        if kind == I.EULER:
            I.Euler.step_(tp, tv, tf, tm, dt, drift=d)
        elif kind == I.VERLET1:
            I.Verlet(dt).halfstep1_(tp, tv, tf, tm, dt, drift=d)
        else:
            I.Langevin(dt, gamma, kT).halfstep1_(tp, tv, tf, tm, tn, dt, drift=d)
        if not fused:
            from dynamis_b200 import _lib
            _lib.check(_lib.lib().dynb_drift_flag(tp.data_ptr(), watch.ref.data_ptr(), tv.data_ptr(), watch.prev_vel.data_ptr(), n, dt,
                                                  threshold, watch.state.data_ptr(), watch.flag.data_ptr(),
                                                  torch.cuda.current_stream(cuda).cuda_stream), "drift_flag")
        return tp, tv, watch

    pa, va, wa = run(True)
    pb, vb, wb = run(False)
    assert torch.equal(pa, pb) and torch.equal(va, vb)
    assert int(wa.flag.item()) == int(wb.flag.item())
    assert torch.equal(wa.prev_vel, wb.prev_vel) and int(wa.state.abs().sum().item()) == 0
    # oracle
    O.integrator_step(kind, pos, vel, frc, mass, noise, dt, gamma, kT)
    pv = pvel.copy()
    assert int(wa.flag.item()) == O.drift_flag(pos, ref, vel, pv, dt, threshold)
    np.testing.assert_array_equal(wa.prev_vel.cpu().numpy(), pv)
