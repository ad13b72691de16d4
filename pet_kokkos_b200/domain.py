"""Centre-atom domain decomposition of one large periodic cell with ghost atoms (the reference's ghosts mode).

Each rank owns the atoms of one brick of the cell and lists, besides them, every periodic image of
any atom within `ghost_cutoff` of the brick (one cutoff per message-passing layer: the reference's
Calculator::ghost_cutoff, src/calculator.cpp:890-894).  Every listed atom is a centre, only owned
atoms count towards the energy (EdgeListView::n_local, include/pet/device_geometry.hpp:83-110); there
is no communication inside the network.  Afterwards the forces on ghosts are added onto their owners
and the energy and virial are summed over ranks (an all-reduce; NCCL when the tensors live on GPUs),
which is exact by linearity: the total energy is the sum of the ranks' owned-atom energies, so its
derivatives are the sums of theirs (the reference's tests/test_edges.cpp:117-178 checks one such domain).
"""
from __future__ import annotations

import numpy as np

from .calculator import EdgeListView


def rank_grid(world):
    """px * py * pz = world, as cubic as possible."""
    best = (world, 1, 1)
    for a in range(1, world + 1):
        if world % a:
            continue
        for b in range(1, world // a + 1):
            if (world // a) % b:
                continue
            c = world // a // b
            if max(a, b, c) - min(a, b, c) < max(best) - min(best):
                best = (a, b, c)
    return best


def _pairs_within(pos, cutoff):
    """Directed pairs (i, j), i != j, |r_j - r_i| <= cutoff, grouped by i: a binned search in numpy."""
    n = len(pos)
    lo = pos.min(0)
    cell = np.floor((pos - lo) / cutoff).astype(np.int64)
    dims = cell.max(0) + 1
    key = (cell[:, 0] * dims[1] + cell[:, 1]) * dims[2] + cell[:, 2]
    order = np.argsort(key, kind="stable")
    skey = key[order]
    start = np.searchsorted(skey, np.arange(dims.prod() + 1))
    ii, jj = [], []
    for dx in (-1, 0, 1):
        for dy in (-1, 0, 1):
            for dz in (-1, 0, 1):
                nb = cell + np.array([dx, dy, dz])
                ok = ((nb >= 0) & (nb < dims)).all(1)
                nk = (nb[:, 0] * dims[1] + nb[:, 1]) * dims[2] + nb[:, 2]
                idx = np.nonzero(ok)[0]
                cnt = start[nk[idx] + 1] - start[nk[idx]]
                rep = np.repeat(idx, cnt)
                if not len(rep):
                    continue
                offs = np.arange(cnt.sum()) - np.repeat(np.cumsum(cnt) - cnt, cnt)
                cand = order[np.repeat(start[nk[idx]], cnt) + offs]
                d = pos[cand] - pos[rep]
                m = ((d * d).sum(1) <= cutoff * cutoff) & (cand != rep)
                ii.append(rep[m]), jj.append(cand[m])
    ii, jj = np.concatenate(ii), np.concatenate(jj)
    o = np.lexsort((jj, ii))
    return ii[o], jj[o]


def local_domain(system, rank, world, cutoff, ghost_cutoff):
    """This rank's atoms: (EdgeListView, owner[n_listed] global index of each listed atom, n_local)."""
    cell = np.asarray(system["cell"], dtype=np.float64).reshape(3, 3)
    pos = np.asarray(system["positions"], dtype=np.float64)
    z = np.asarray(system["atomic_numbers"])
    inv = np.linalg.inv(cell)
    frac = pos @ inv
    frac -= np.floor(frac)
    wrapped = frac @ cell
    grid = rank_grid(world)
    coord = np.array(np.unravel_index(rank, grid))
    lo_f, hi_f = coord / np.array(grid), (coord + 1) / np.array(grid)
    owned = np.nonzero(((frac >= lo_f) & (frac < hi_f)).all(1))[0]
    # ghosts: periodic images within ghost_cutoff of the brick, measured along each lattice direction's plane spacing
    spacing = 1.0 / np.linalg.norm(inv, axis=0)           # interplanar spacing of each lattice direction
    margin = ghost_cutoff / spacing                        # the shell's thickness in fractional units
    reach = np.ceil(margin).astype(int)
    gpos, gown = [], []
    for a in range(-reach[0], reach[0] + 1):
        for b in range(-reach[1], reach[1] + 1):
            for c in range(-reach[2], reach[2] + 1):
                f = frac + np.array([a, b, c])
                inside = ((f >= lo_f - margin) & (f < hi_f + margin)).all(1)
                if (a, b, c) == (0, 0, 0):
                    inside &= ~((frac >= lo_f) & (frac < hi_f)).all(1)
                idx = np.nonzero(inside)[0]
                gpos.append(wrapped[idx] + np.array([a, b, c]) @ cell), gown.append(idx)
    lpos = np.concatenate([wrapped[owned]] + gpos)
    owner = np.concatenate([owned] + gown)
    ii, jj = _pairs_within(lpos, cutoff)
    off = np.concatenate([[0], np.cumsum(np.bincount(ii, minlength=len(lpos)))]).astype(np.int32)
    view = EdgeListView(lpos, z[owner].astype(np.int32), off, jj.astype(np.int32), n_local=len(owned))
    return view, owner, len(owned)


def fold(results, owner, n_atoms):
    """Ghost forces onto their owners; returns (energy, forces [n_atoms,3], virial [6]) of this rank's share."""
    F = np.zeros((n_atoms, 3))
    np.add.at(F, owner, results.forces)
    return float(results.energy[0]), F, np.asarray(results.virial[0], dtype=np.float64).copy()


def compute_decomposed(compute_edges, system, cutoff, ghost_cutoff, rank, world, group=None, device=None):
    """Every rank passes the same structure; returns the whole cell's (energy, forces, virial) on every rank.

    `compute_edges(view)` evaluates one rank's list (Calculator.compute_edges).  The reduction is one
    all-reduce of 1 + 3N + 6 doubles (NCCL over NVLink when `device` is a CUDA device)."""
    import torch
    import torch.distributed as dist
    view, owner, _ = local_domain(system, rank, world, cutoff, ghost_cutoff)
    e, F, W = fold(compute_edges(view), owner, system["n_atoms"])
    buf = torch.from_numpy(np.concatenate([[e], W, F.ravel()]))
    if world > 1:
        if device is not None:
            buf = buf.to(device)
        dist.all_reduce(buf, group=group)
        buf = buf.cpu()
    out = buf.numpy()
    return out[0], out[7:].reshape(-1, 3), out[1:7]
