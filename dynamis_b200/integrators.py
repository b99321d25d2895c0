"""Integrator steps on the CUDA library, same interface as the reference's wrappers.

Mirrors ``dynamis_integrator`` (src/dynamis_integrator/euler.py:14-45, verlet.py:16-69,
langevin.py:14-83 and the argument checks of _data_check.py): ``Euler.step_``, ``Verlet.halfstep1_`` /
``halfstep2_``, ``Langevin.halfstep1_`` / ``halfstep2_`` update the tensors in place.  The steps that
move the positions take an optional ``drift`` argument (a :class:`DriftWatch`): the same launch then also
produces the 2-bit drift word of ``SimState.write_local_drift_flag``
(dynamis/src/dynamis/simulatorState.py:257-293), which otherwise costs a second pass over the state.
The model-driven ``step(state, model)`` loops of the reference stay in its Python layer.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import _lib

EULER, VERLET1, VERLET2, LANGEVIN1, LANGEVIN2 = range(5)


def check_devices(*args):
    devices = {a.device for a in args}
    if len(devices) > 1:
        raise ValueError(f"All input tensors must be on the same device. Found devices: {devices}")


def check_shape_2D(pos):
    if len(pos.shape) != 2:
        raise ValueError(f"Position tensor must be 2D of shape (N, D). Got: {pos.shape}")


def check_mass_shape(mass, pos):
    if mass.shape != (pos.shape[0],):
        raise ValueError("Mass tensor must have shape (N,), where N is the number of atoms. "
                         f"Got mass: {mass.shape}, expected: {(pos.shape[0],)}")


def check_shapes_match(*args):
    shapes = {a.shape for a in args}
    if len(shapes) > 1:
        raise ValueError(f"All input tensors must have the same shape. Found shapes: {shapes}")


class DriftWatch:
    """Buffers of the drift word for one rank: reference positions (set at every rebuild), the previous
    step's velocities, three state words and the flag."""

    def __init__(self, ref_positions: torch.Tensor, velocities: torch.Tensor, threshold: float):
        self.ref = ref_positions.detach().clone().contiguous()
        self.prev_vel = velocities.detach().clone().contiguous()
        self.threshold = float(threshold)
        dev = ref_positions.device
        self.state = torch.zeros(3, dtype=torch.int32, device=dev)
        self.flag = torch.zeros(1, dtype=torch.int32, device=dev)

    def rebase(self, ref_positions: torch.Tensor):
        self.ref.copy_(ref_positions)


def _launch(kind: int, pos, vel, frc, mass, noise, dt, gamma, kT, drift: Optional[DriftWatch]):
    for t in (pos, vel, frc, mass, noise):
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("integrator tensors must be CUDA tensors")
        if t.dtype != torch.float32:
            raise RuntimeError(f"integrator tensors must be float32, got {t.dtype}")
        if not t.is_contiguous():
            raise RuntimeError("integrator tensors must be contiguous")
    if vel.shape[1] != 3:
        raise RuntimeError(f"the CUDA integrators work on [N, 3] tensors, got {tuple(vel.shape)}")
    dev = vel.device
    n = vel.shape[0]
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        p = (lambda t: t.data_ptr() if t is not None else None)
        if drift is not None:
            if drift.ref.shape != vel.shape:
                raise RuntimeError("the drift watch was made for another number of atoms")
            d = (drift.ref.data_ptr(), drift.prev_vel.data_ptr(), drift.threshold, drift.state.data_ptr(), drift.flag.data_ptr())
        else:
            d = (None, None, 0.0, None, None)
        _lib.check(_lib.lib().dynb_integrator_step(kind, p(pos), p(vel), p(frc), p(mass), p(noise), n, float(dt), float(gamma),
                                                   float(kT), d[0], d[1], d[2], d[3], d[4], stream), "integrator_step")
    return drift.flag if drift is not None else None


class Euler:
    def __init__(self, dt: float) -> None:
        self.dt = dt

    @staticmethod
    def step_(pos, vel, frc, mass, dt: float, drift: Optional[DriftWatch] = None):
        check_devices(pos, vel, frc, mass)
        check_shape_2D(pos)
        check_mass_shape(mass, pos)
        check_shapes_match(pos, vel, frc)
        return _launch(EULER, pos, vel, frc, mass, None, dt, 0.0, 0.0, drift)

    def reset(self) -> None:
        pass


class Verlet:
    def __init__(self, dt: float) -> None:
        self.dt = dt
        self.prev_forces = None

    def reset(self) -> None:
        self.prev_forces = None

    def halfstep1_(self, pos, vel, frc, mass, dt: float, drift: Optional[DriftWatch] = None):
        check_devices(pos, vel, frc, mass)
        check_shape_2D(pos)
        check_mass_shape(mass, pos)
        check_shapes_match(pos, vel, frc)
        return _launch(VERLET1, pos, vel, frc, mass, None, dt, 0.0, 0.0, drift)

    def halfstep2_(self, vel, frc, mass, dt: float) -> None:
        check_devices(vel, frc, mass)
        check_shape_2D(vel)
        check_mass_shape(mass, vel)
        check_shapes_match(vel, frc)
        _launch(VERLET2, None, vel, frc, mass, None, dt, 0.0, 0.0, None)


class Langevin:
    def __init__(self, dt: float, gamma: float, kT: float) -> None:
        self.dt = dt
        self.gamma = gamma
        self.kT = kT
        self.prev_forces = None

    def reset(self) -> None:
        self.prev_forces = None

    def halfstep1_(self, pos, vel, frc, mass, noise, dt: float, drift: Optional[DriftWatch] = None):
        check_devices(pos, vel, frc, mass, noise)
        check_shape_2D(pos)
        check_mass_shape(mass, pos)
        check_shapes_match(pos, vel, frc, noise)
        return _launch(LANGEVIN1, pos, vel, frc, mass, noise, dt, self.gamma, self.kT, drift)

    def halfstep2_(self, vel, frc, mass, noise, dt: float) -> None:
        check_devices(vel, frc, mass, noise)
        check_shape_2D(vel)
        check_mass_shape(mass, vel)
        check_shapes_match(vel, frc, noise)
        _launch(LANGEVIN2, None, vel, frc, mass, noise, dt, self.gamma, self.kT, None)
