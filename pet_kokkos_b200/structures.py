"""Seeded synthetic structures with the shapes of the reference's benchmark inputs.

The reference times itself on diamond supercells and a liquid-water box
(lammps/examples/diamond_64.xyz, diamond_1728.xyz, water_648.xyz: cubic diamond
a = 3.567 A, water L = 18.6 A) and its cell-list tests build diamond supercells
in code (tests/test_cell_list.cpp:26-48).  These generators produce inputs of
the same shapes from numpy's default_rng so that every consumer (the CPU
oracle, the CUDA path, the benchmark) reads identical float64 coordinates.

A structure is a plain dict mirroring pet::System (include/pet/neighbors.hpp:15-25):
  n_atoms, atomic_numbers [N] int32, positions [N,3] float64 (Angstrom),
  cell [3,3] float64 (lattice vectors as rows), pbc [3] bool.
"""
from __future__ import annotations

import numpy as np

_DIAMOND_BASIS = np.array(
    [[0, 0, 0], [0, .5, .5], [.5, 0, .5], [.5, .5, 0],
     [.25, .25, .25], [.25, .75, .75], [.75, .25, .75], [.75, .75, .25]], dtype=np.float64)


def make_system(numbers, positions, cell, pbc=(True, True, True)):
    numbers = np.ascontiguousarray(numbers, dtype=np.int32)
    positions = np.ascontiguousarray(positions, dtype=np.float64).reshape(-1, 3)
    cell = np.ascontiguousarray(cell, dtype=np.float64).reshape(3, 3)
    return {"n_atoms": int(numbers.shape[0]), "atomic_numbers": numbers, "positions": positions,
            "cell": cell, "pbc": np.asarray(pbc, dtype=bool)}


def diamond(n: int, a: float = 3.567, shear: float = 0.0, jitter: float = 0.0, seed: int = 0, z: int = 6):
    """n^3 conventional cells of diamond, optionally sheared (c tilted toward a) and jittered.

    Atom order and fractional coordinates follow tests/test_cell_list.cpp:26-48
    (cell loops i, j, k outermost, the 8-atom basis innermost).
    """
    L = n * a
    cell = np.array([[L, 0, 0], [0, L, 0], [shear * L, 0, L]], dtype=np.float64)
    ijk = np.stack(np.meshgrid(np.arange(n), np.arange(n), np.arange(n), indexing="ij"), -1).reshape(-1, 1, 3)
    frac = ((ijk + _DIAMOND_BASIS[None, :, :]) / n).reshape(-1, 3)
    pos = frac[:, 0:1] * cell[0] + frac[:, 1:2] * cell[1] + frac[:, 2:3] * cell[2]
    if jitter > 0.0:
        pos = pos + np.random.default_rng(seed).normal(0.0, jitter, size=pos.shape)
    return make_system(np.full(len(pos), z), pos, cell)


def simple_cubic(n: int, a: float, z: int = 1):
    """n^3 simple-cubic lattice (tests/test_neighbors.cpp:21-33)."""
    g = np.stack(np.meshgrid(np.arange(n), np.arange(n), np.arange(n), indexing="ij"), -1).reshape(-1, 3)
    return make_system(np.full(len(g), z), g * float(a), np.eye(3) * n * a)


def _random_rotation(rng):
    q = rng.normal(size=4)
    q /= np.linalg.norm(q)
    w, x, y, z = q
    return np.array([[1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w)],
                     [2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w)],
                     [2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)]])


def water_box(n_mol: int = 216, L: float = 18.64, seed: int = 0, oo_min: float = 2.5):
    """n_mol rigid H2O (O-H 0.957 A, H-O-H 104.5 deg), random orientations, O-O >= oo_min (minimum image)."""
    rng = np.random.default_rng(seed)
    roh, ang = 0.957, np.deg2rad(104.5)
    mol = np.array([[0, 0, 0], [roh * np.sin(ang / 2), 0, roh * np.cos(ang / 2)],
                    [-roh * np.sin(ang / 2), 0, roh * np.cos(ang / 2)]])
    centres = np.zeros((0, 3))
    while len(centres) < n_mol:
        c = rng.uniform(0, L, size=3)
        if len(centres):
            d = centres - c
            d -= L * np.round(d / L)
            if (np.einsum("ij,ij->i", d, d) < oo_min * oo_min).any():
                continue
        centres = np.vstack([centres, c])
    pos, num = [], []
    for c in centres:
        pos.append(c + mol @ _random_rotation(rng).T)
        num += [8, 1, 1]
    return make_system(num, np.concatenate(pos), np.eye(3) * L)


def random_mixture(n_atoms: int = 64, L: float = 9.0, seed: int = 0, dmin: float = 0.9,
                   species=(6, 1, 7, 8, 14)):
    """Uniform random positions in a cubic periodic cell with a minimum-image separation of dmin."""
    rng = np.random.default_rng(seed)
    pts = np.zeros((0, 3))
    while len(pts) < n_atoms:
        c = rng.uniform(0, L, size=3)
        if len(pts):
            d = pts - c
            d -= L * np.round(d / L)
            if (np.einsum("ij,ij->i", d, d) < dmin * dmin).any():
                continue
        pts = np.vstack([pts, c])
    return make_system(rng.choice(np.asarray(species), size=n_atoms), pts, np.eye(3) * L)


def mixture_batch(n_struct: int = 512, n_atoms: int = 64, L: float = 9.0, seed: int = 0):
    return [random_mixture(n_atoms, L, seed=seed * 100003 + b) for b in range(n_struct)]


# The five workloads of the benchmark definition, by short name.
def workload(name: str, seed: int = 0):
    if name == "diamond64":
        return [diamond(2, jitter=0.05, seed=seed)]
    if name == "water648":
        return [water_box(216, 18.64, seed=seed)]
    if name == "diamond1728":
        return [diamond(6, jitter=0.05, seed=seed)]
    if name == "batch512x64":
        return mixture_batch(512, 64, 9.0, seed=seed)
    if name == "diamond13824":
        return [diamond(12, jitter=0.05, seed=seed)]
    raise KeyError(name)
