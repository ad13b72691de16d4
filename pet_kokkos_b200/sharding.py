"""Sharding a batch of independent structures across ranks (one process per GPU).

Edges never cross structures (the reference's include/pet/neighbors.hpp:75-77), so a batch
splits into contiguous runs, one per rank, with no exchange during the evaluation; only the
results are gathered.  Runs are balanced by the reference's own cost proxy, atoms times
neighbours (Calculator::memory_runs, src/calculator.cpp:326-345), estimated from the atom
count and density.
"""
from __future__ import annotations

import numpy as np

from .calculator import Results


def structure_cost(system, cutoff):
    """Atoms x expected neighbours: N * (4/3 pi rc^3) * density for a periodic cell, N * (N - 1) otherwise."""
    n = int(system["n_atoms"])
    cell = np.asarray(system.get("cell", np.zeros((3, 3))), dtype=np.float64).reshape(3, 3)
    vol = abs(np.linalg.det(cell))
    if vol < 1e-9 or not np.any(system.get("pbc", (False,) * 3)):
        return float(n * max(n - 1, 1))
    return float(n * max(1.0, 4.0 / 3.0 * np.pi * cutoff ** 3 * n / vol))


def partition(costs, world):
    """Contiguous runs [(begin, end)] of `world` parts with near-equal summed cost (order kept, runs may be empty)."""
    costs = np.asarray(costs, dtype=np.float64)
    n = len(costs)
    cum = np.concatenate([[0.0], np.cumsum(costs)])
    total = cum[-1]
    cuts = [0]
    for r in range(1, world):
        target = total * r / world
        k = int(np.searchsorted(cum, target, side="left"))
        # the boundary nearest the target
        if k > 0 and abs(cum[k - 1] - target) <= abs(cum[min(k, n)] - target):
            k -= 1
        cuts.append(min(max(k, cuts[-1]), n))
    cuts.append(n)
    return [(cuts[r], cuts[r + 1]) for r in range(world)]


def compute_sharded(calc_compute, systems, cutoff, rank, world, group=None, compute_forces=True):
    """Every rank passes the same batch; rank r evaluates its run with `calc_compute(list) -> Results`
    and all ranks return the whole batch's Results in structure order (gathered with torch.distributed)."""
    import torch.distributed as dist
    runs = partition([structure_cost(s, cutoff) for s in systems], world)
    b, e = runs[rank]
    mine = calc_compute(systems[b:e]) if e > b else None
    parts = [None] * world
    if world > 1:
        dist.all_gather_object(parts, mine, group=group)
    else:
        parts = [mine]
    parts = [p for p in parts if p is not None]
    out = Results(np.concatenate([p.energy for p in parts]), np.concatenate([p.per_atom_energy for p in parts]),
                  n_atoms=[n for p in parts for n in p.n_atoms])
    if compute_forces:
        out.forces = np.concatenate([p.forces for p in parts])
        out.virial = np.concatenate([p.virial for p in parts])
        sid, base = [], 0
        for p in parts:
            sid.append(np.asarray(p.struct_id) + base)
            base += len(p.n_atoms)
        out.struct_id = np.concatenate(sid).astype(np.int32)
    return out
