"""Seeded synthetic atom configurations with the shapes of the benchmark configs.

These stand in for the CH4-ladder and solvated-protein inputs the reference's
benchmark scripts read (benchmarks/dist_build_graph_benchmark.py:58-71), which
are datasets this package does not ship.  Everything is generated in float64
with ``numpy.random.default_rng(seed)`` and cast last; atoms are *not*
re-wrapped after the jitter, so a few lie just outside the cell and exercise
the wrap.

Every generator returns ``(pos [N,3], cell [3,3] rows = lattice vectors,
pbc [3] bool, radius)`` as numpy arrays.
"""

from __future__ import annotations

import numpy as np

_FCC_BASIS = np.array([[0.0, 0.0, 0.0], [0.5, 0.5, 0.0], [0.5, 0.0, 0.5], [0.0, 0.5, 0.5]])
_DIAMOND_BASIS = np.concatenate([_FCC_BASIS, _FCC_BASIS + 0.25])


def _lattice(nx: int, ny: int, nz: int, basis: np.ndarray) -> np.ndarray:
    """Fractional-in-conventional-cell coordinates, cell-major / basis-minor order."""
    ii, jj, kk = np.meshgrid(np.arange(nx), np.arange(ny), np.arange(nz), indexing="ij")
    cells = np.stack([ii.ravel(), jj.ravel(), kk.ravel()], axis=1).astype(np.float64)
    return (cells[:, None, :] + basis[None, :, :]).reshape(-1, 3)


def fcc_copper(ncell: int, a: float = 3.615, jitter: float = 0.1, seed: int = 1001,
               dtype=np.float32, radius: float = 6.0):
    """fcc Cu supercell of ``ncell``^3 conventional cells (4 atoms each) + Gaussian jitter.

    ``ncell=20`` is the 32,000-atom case; ``ncell=126`` the 8,001,504-atom case.
    """
    rng = np.random.default_rng(seed)
    pos = _lattice(ncell, ncell, ncell, _FCC_BASIS) * a
    pos += rng.normal(0.0, jitter, size=pos.shape)
    L = ncell * a
    cell = np.diag([L, L, L])
    return pos.astype(dtype), cell.astype(dtype), np.array([True, True, True]), float(radius)


def random_liquid(n: int, density: float = 0.1, seed: int = 1002, dtype=np.float32,
                  radius: float = 5.0):
    """``n`` atoms uniform-random in a cubic periodic box at the given number density.

    ``n=1_000_000`` gives L = 215.44 Å (the single-GPU benchmark workload);
    ``n=4_000_000`` gives L = 341.995 Å.
    """
    rng = np.random.default_rng(seed)
    L = (n / density) ** (1.0 / 3.0)
    pos = rng.random((n, 3)) * L
    cell = np.diag([L, L, L])
    return pos.astype(dtype), cell.astype(dtype), np.array([True, True, True]), float(radius)


def triclinic_silicon(nx: int = 50, ny: int = 50, nz: int = 25, a: float = 5.431,
                      jitter: float = 0.05, seed: int = 1003, dtype=np.float64,
                      radius: float = 6.0, xy: float = 0.2, xz: float = 0.1, yz: float = 0.0):
    """Diamond-lattice Si (8-atom basis) in a sheared periodic cell.

    Cell rows are a=(Lx,0,0), b=(xy*Lx,Ly,0), c=(xz*Lx,yz*Ly,Lz); positions are
    ``frac @ cell`` plus jitter.  50x50x25 cells = 500,000 atoms.
    """
    rng = np.random.default_rng(seed)
    frac = _lattice(nx, ny, nz, _DIAMOND_BASIS) / np.array([nx, ny, nz], dtype=np.float64)
    Lx, Ly, Lz = nx * a, ny * a, nz * a
    cell = np.array([[Lx, 0.0, 0.0], [xy * Lx, Ly, 0.0], [xz * Lx, yz * Ly, Lz]])
    pos = frac @ cell
    pos += rng.normal(0.0, jitter, size=pos.shape)
    return pos.astype(dtype), cell.astype(dtype), np.array([True, True, True]), float(radius)


def drift_velocities(n: int, sigma: float = 0.05, seed: int = 1005, dtype=np.float32):
    """Per-atom Gaussian displacement per step (Å/step) for the migration workload."""
    rng = np.random.default_rng(seed + 7919)
    return rng.normal(0.0, sigma, size=(n, 3)).astype(dtype)
