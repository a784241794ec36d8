"""Seeded synthetic structures with the shapes, densities and neighbour counts of the benchmark configurations:
displaced bcc / fcc supercells with random species, and batches of small random triclinic cells."""
from __future__ import annotations

import numpy as np

_BASIS = {"bcc": np.array([[0, 0, 0], [0.5, 0.5, 0.5]]),
          "fcc": np.array([[0, 0, 0], [0.5, 0.5, 0], [0.5, 0, 0.5], [0, 0.5, 0.5]]),
          "sc": np.array([[0, 0, 0]])}


def crystal(lattice, a, reps, n_species=1, sigma=0.05, seed=0):
    """Orthorhombic supercell of reps = (nx, ny, nz) conventional cells; Gaussian displacements sigma; species drawn
    uniformly from 1..n_species.  Returns types int32 [n] (1-based), positions [n, 3], cell [3, 3], pbc [3]."""
    rng = np.random.default_rng(seed)
    nx, ny, nz = reps
    g = np.stack(np.meshgrid(np.arange(nx), np.arange(ny), np.arange(nz), indexing="ij"), -1).reshape(-1, 1, 3)
    pos = ((g + _BASIS[lattice][None]) * a).reshape(-1, 3)
    pos = pos + sigma * rng.standard_normal(pos.shape)
    types = rng.integers(1, n_species + 1, size=len(pos)).astype(np.int32)
    cell = np.diag([nx * a, ny * a, nz * a]).astype(np.float64)
    return types, pos, cell, np.array([1, 1, 1], dtype=np.uint8)


def random_cell(n, density, n_species, min_sep=1.8, seed=0):
    """n atoms in a random triclinic periodic cell at `density` atoms/A^3, every pair (periodic images included) at
    least min_sep apart (rejection sampling)."""
    rng = np.random.default_rng(seed)
    vol = n / density
    L = vol ** (1.0 / 3.0)
    while True:
        cell = np.diag(L * (1.0 + 0.2 * (rng.random(3) - 0.5)))
        cell[1, 0], cell[2, 0], cell[2, 1] = 0.3 * L * (rng.random(3) - 0.5)
        cell *= (vol / abs(np.linalg.det(cell))) ** (1.0 / 3.0)
        inv = np.linalg.inv(cell)
        if (1.0 / np.linalg.norm(inv, axis=0)).min() > 2.0 * min_sep:
            break
    shifts = np.array([[i, j, k] for i in (-1, 0, 1) for j in (-1, 0, 1) for k in (-1, 0, 1)]) @ cell
    pos = np.zeros((0, 3))
    tries = 0
    while len(pos) < n:
        x = rng.random(3) @ cell
        tries += 1
        if tries > 200000:
            raise RuntimeError("random_cell: cannot place the atoms")
        if len(pos):
            d = pos[None, :, :] + shifts[:, None, :] - x
            if (d * d).sum(-1).min() < min_sep * min_sep:
                continue
        pos = np.vstack([pos, x])
    types = rng.integers(1, n_species + 1, size=n).astype(np.int32)
    return types, pos, cell, np.array([1, 1, 1], dtype=np.uint8)


def random_batch(nsys, nmin, nmax, n_species, seed=0, dmin=0.06, dmax=0.09, min_sep=1.8):
    """nsys independent periodic structures of nmin..nmax atoms (uniform): natoms [nsys], types [N], positions [N, 3],
    cells [nsys, 3, 3], pbc [nsys, 3]."""
    rng = np.random.default_rng(seed)
    natoms = rng.integers(nmin, nmax + 1, size=nsys).astype(np.int32)
    dens = dmin + (dmax - dmin) * rng.random(nsys)
    T, P, Cc = [], [], []
    for s in range(nsys):
        t, p, c, _ = random_cell(int(natoms[s]), float(dens[s]), n_species, min_sep, seed=int(rng.integers(1 << 31)))
        T.append(t)
        P.append(p)
        Cc.append(c)
    return natoms, np.concatenate(T), np.concatenate(P), np.stack(Cc), np.ones((nsys, 3), dtype=np.uint8)
