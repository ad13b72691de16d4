"""TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's neighbour-list path.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may import
this module; the product (pet_kokkos_b200) never does.

numpy float64 throughout: Python/numpy never contract a*b+c into an FMA, so the
distance tests below reproduce the reference's un-contracted arithmetic bit for
bit when written in the reference's association order.

Parity pins: the packed list of the reference's own device search, compiled for
the host (oracle/_ref/libpet_ref.so), equals this module's to the bit -- order,
vectors, distances, partners (tests/test_reference_pin.py) -- and the reference's
own model-free tests, restated in tests/:
  tests/test_cell_list.cpp:119-157,192-212  cell list == brute force edge set,
      reproducible order, brute-force order for small structures
  tests/test_neighbors.cpp:52-128           coordination, padding, reverse map
"""
from __future__ import annotations

import math

import numpy as np

# include/pet/device_cell_list.hpp:46-47
K_CELL_LIST_MIN_ATOMS = 256
K_CELL_LIST_MIN_CHECKS = 2048


def _cross(u, v):
    return np.array([u[1] * v[2] - u[2] * v[1], u[2] * v[0] - u[0] * v[2], u[0] * v[1] - u[1] * v[0]])


def image_ranges(cell, cutoff, pbc):
    """Images to search along each lattice vector.

    include/pet/device_geometry.hpp:28-44 (image_ranges_rows) and
    src/neighbors.cpp:57-73 (image_ranges): ceil(cutoff / interplanar spacing)
    on periodic axes, zero for a degenerate cell.
    """
    a, b, c = cell[0], cell[1], cell[2]
    bc, ca, ab = _cross(b, c), _cross(c, a), _cross(a, b)
    vol = abs(a[0] * bc[0] + a[1] * bc[1] + a[2] * bc[2])
    n = [0, 0, 0]
    if vol < 1e-12:
        return n
    for d, face in enumerate((bc, ca, ab)):
        if pbc[d]:
            nf = math.sqrt(face[0] * face[0] + face[1] * face[1] + face[2] * face[2])
            n[d] = int(math.ceil(cutoff / (vol / nf)))
    return n


def brute_force_edges(system, cutoff):
    """The host search, src/neighbors.cpp:75-96: loops i, j, sa, sb, sc on unwrapped positions.

    Returns int array [E,5] (i, j, sa, sb, sc), float [E,3] vec, float [E] dist, in that loop order.
    """
    x = system["positions"]
    c = system["cell"]
    N = system["n_atoms"]
    rng = image_ranges(c, cutoff, system["pbc"])
    cutoff2 = cutoff * cutoff
    sa, sb, sc = np.meshgrid(np.arange(-rng[0], rng[0] + 1), np.arange(-rng[1], rng[1] + 1),
                             np.arange(-rng[2], rng[2] + 1), indexing="ij")
    sa, sb, sc = sa.ravel(), sb.ravel(), sc.ravel()
    # (sa*c0 + sb*c3) + sc*c6, per component, as the reference associates it
    sh = [(sa * c[0, d] + sb * c[1, d]) + sc * c[2, d] for d in range(3)]
    idx, vec, dist = [], [], []
    for i in range(N):
        # v = (x_j + shift) - x_i  for all j (rows) and images (cols)
        v = [(x[:, d][:, None] + sh[d][None, :]) - x[i, d] for d in range(3)]
        d2 = (v[0] * v[0] + v[1] * v[1]) + v[2] * v[2]
        jj, ss = np.nonzero((d2 >= 1e-24) & (d2 <= cutoff2))  # row-major: j outer, image inner
        idx.append(np.stack([np.full(len(jj), i), jj, sa[ss], sb[ss], sc[ss]], 1))
        vec.append(np.stack([v[0][jj, ss], v[1][jj, ss], v[2][jj, ss]], 1))
        dist.append(np.sqrt(d2[jj, ss]))
    if not idx:
        return np.zeros((0, 5), np.int64), np.zeros((0, 3)), np.zeros(0)
    return np.concatenate(idx), np.concatenate(vec), np.concatenate(dist)


def cell_inverse(c):
    """src/device_geometry.cpp:78-88 (pet_cellinv): adjugate over determinant, rows = lattice vectors."""
    a0, a1, a2, b0, b1, b2, c0, c1, c2 = c.ravel()
    det = a0 * (b1 * c2 - b2 * c1) - a1 * (b0 * c2 - b2 * c0) + a2 * (b0 * c1 - b1 * c0)
    inv = 1.0 / det if det != 0.0 else 0.0
    return np.array([(b1 * c2 - b2 * c1) * inv, (a2 * c1 - a1 * c2) * inv, (a1 * b2 - a2 * b1) * inv,
                     (b2 * c0 - b0 * c2) * inv, (a0 * c2 - a2 * c0) * inv, (a2 * b0 - a0 * b2) * inv,
                     (b0 * c1 - b1 * c0) * inv, (a1 * c0 - a0 * c1) * inv, (a0 * b1 - a1 * b0) * inv])


def wrap_positions(system):
    """src/device_geometry.cpp:89-104 (pet_wrap): fractional floor on periodic axes, back to Cartesian."""
    pos, c, pbc = system["positions"], system["cell"].ravel(), system["pbc"]
    cinv = cell_inverse(system["cell"])
    if not pbc.any():
        return pos.copy(), cinv
    x, y, z = pos[:, 0], pos[:, 1], pos[:, 2]
    f = []
    for d in range(3):
        fd = (x * cinv[d] + y * cinv[3 + d]) + z * cinv[6 + d]
        w = np.floor(fd) if pbc[d] else np.zeros_like(fd)
        f.append(fd - w)
    posw = np.stack([(f[0] * c[d] + f[1] * c[3 + d]) + f[2] * c[6 + d] for d in range(3)], 1)
    return posw, cinv


def grid_dims(system, cutoff):
    """Bins per axis and search reach, src/device_cell_list.cpp:125-173 (cl_grid)."""
    c = system["cell"]
    pbc = system["pbc"]
    per = bool(pbc.any())
    n = system["n_atoms"]
    per_mask = [bool(p) for p in pbc]
    rng = image_ranges(c, cutoff, per_mask)
    if n < K_CELL_LIST_MIN_ATOMS and n * (2 * rng[0] + 1) * (2 * rng[1] + 1) * (2 * rng[2] + 1) < K_CELL_LIST_MIN_CHECKS:
        return [1, 1, 1], rng
    a, b, cc = c[0], c[1], c[2]
    bc, ca, ab = _cross(b, cc), _cross(cc, a), _cross(a, b)
    vol = abs(a[0] * bc[0] + a[1] * bc[1] + a[2] * bc[2])
    area = [math.sqrt(f[0] * f[0] + f[1] * f[1] + f[2] * f[2]) for f in (bc, ca, ab)]
    nc, nr = [1, 1, 1], [0, 0, 0]
    for d in range(3):
        if per and vol > 1e-12 and area[d] > 0.0:
            perp = vol / area[d]
            k = max(int(math.floor(perp / cutoff)), 1)
            w = perp / float(k)
            nc[d] = k
            nr[d] = max(int(math.ceil(cutoff / w)), 1)
    return nc, nr


def cell_list_edges(system, cutoff):
    """The device cell-list search for one structure, in the order the reference lists edges.

    src/device_cell_list.cpp:16-49 (CellSearch::visit/edge), :180-196 (cl_assign),
    :198-240 (count/scan/fill): per centre atom, candidate bins in (da, db, dc)
    order, each bin's members by atom index; v = x_j + (shift.cell - x_i) on the
    wrapped positions; kept when 1e-24 <= |v|^2 <= cutoff^2.

    Returns (idx [E,5] int: i, j, sa, sb, sc; vec [E,3]; dist [E]).
    """
    N = system["n_atoms"]
    c = system["cell"].ravel()
    posw, cinv = wrap_positions(system)
    nc, nr = grid_dims(system, cutoff)
    per = bool(system["pbc"].any())
    ijk = np.zeros((N, 3), np.int64)
    if per:
        x, y, z = posw[:, 0], posw[:, 1], posw[:, 2]
        for d in range(3):
            f = (x * cinv[d] + y * cinv[3 + d]) + z * cinv[6 + d]
            ijk[:, d] = np.clip(np.floor(f * float(nc[d])).astype(np.int64), 0, nc[d] - 1)
    abin = (ijk[:, 0] * nc[1] + ijk[:, 1]) * nc[2] + ijk[:, 2]
    nbins = nc[0] * nc[1] * nc[2]
    order = np.argsort(abin, kind="stable")  # members by atom index within a bin
    counts = np.bincount(abin, minlength=nbins)
    start = np.concatenate([[0], np.cumsum(counts)])
    maxocc = int(counts.max()) if N else 0
    members = np.full((nbins, max(maxocc, 1)), -1, np.int64)
    for b in range(nbins):
        members[b, :counts[b]] = order[start[b]:start[b + 1]]
    cutoff2 = cutoff * cutoff
    out_i, out_o, out_j, out_s, out_v, out_d = [], [], [], [], [], []
    o = 0
    for da in range(-nr[0], nr[0] + 1):
        for db in range(-nr[1], nr[1] + 1):
            for dc in range(-nr[2], nr[2] + 1):
                t = ijk + np.array([da, db, dc])
                sh = np.stack([np.floor_divide(t[:, d], nc[d]) for d in range(3)], 1)
                tb = (np.mod(t[:, 0], nc[0]) * nc[1] + np.mod(t[:, 1], nc[1])) * nc[2] + np.mod(t[:, 2], nc[2])
                J = members[tb]  # [N, maxocc]
                valid = J >= 0
                Jc = np.where(valid, J, 0)
                v = []
                for d in range(3):
                    off = ((sh[:, 0] * c[d] + sh[:, 1] * c[3 + d]) + sh[:, 2] * c[6 + d]) - posw[:, d]
                    v.append(posw[Jc, d] + off[:, None])
                d2 = (v[0] * v[0] + v[1] * v[1]) + v[2] * v[2]
                hit = valid & (d2 >= 1e-24) & (d2 <= cutoff2)
                ii, qq = np.nonzero(hit)
                out_i.append(ii)
                out_o.append(np.full(len(ii), o))
                out_j.append(J[ii, qq])
                out_s.append(sh[ii])
                out_v.append(np.stack([v[0][ii, qq], v[1][ii, qq], v[2][ii, qq]], 1))
                out_d.append(np.sqrt(d2[ii, qq]))
                o += 1
    ii = np.concatenate(out_i)
    oo = np.concatenate(out_o)
    jj = np.concatenate(out_j)
    perm = np.lexsort((jj, oo, ii))
    idx = np.concatenate([ii[:, None], jj[:, None], np.concatenate(out_s)], 1)[perm]
    return idx, np.concatenate(out_v)[perm], np.concatenate(out_d)[perm]


def bump_cutoff_f32(d, rc, width):
    """include/pet/cutoff.hpp:17-22 (dev_bump_cutoff): the argument and transcendentals in float32."""
    x = ((d - (rc - width)) / width).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        mid = 0.5 * (1.0 + np.tanh(np.float32(1.0) / np.tan(np.float32(math.pi) * x)).astype(np.float64))
    return np.where(x <= 0, 1.0, np.where(x >= 1, 0.0, mid))


def cosine_cutoff_f32(d, rc, width):
    """include/pet/cutoff.hpp:23-26 (dev_cosine_cutoff)."""
    x = np.clip(((d - (rc - width)) / width).astype(np.float32), np.float32(0), np.float32(1))
    return 0.5 * (1.0 + np.cos(np.float32(math.pi) * x).astype(np.float64))


def bump_dcutoff_dr_f32(d, rc, width):
    """include/pet/cutoff.hpp:44-51 (dev_bump_dcutoff_dr): d(bump)/d(rc), transcendentals in float32."""
    x = ((d - (rc - width)) / width).astype(np.float32)
    ps = np.float32(math.pi) * np.clip(x, np.float32(1e-6), np.float32(1) - np.float32(1e-6))
    si = np.sin(ps)
    tt = np.tanh(np.cos(ps) / si)
    val = 0.5 * (1.0 - (tt * tt).astype(np.float64)) * ((np.float32(math.pi) / (si * si)) / np.float32(width)).astype(np.float64)
    return np.where((x <= 0) | (x >= 1), 0.0, val)


def adaptive_probes(cutoff, width_adaptive):
    """src/neighbors.cpp:23-27: from 0.5 A to the cutoff, a quarter of the taper width apart."""
    p, r = [], 0.5
    while r < cutoff - 1e-12:
        p.append(r)
        r += width_adaptive / 4.0
    return np.array(p)


SOLVER_MIN_CUTOFF_FACTOR, SOLVER_ITERS, SOLVER_DN_FLOOR = 1.0 / 16.0, 10, 1e-6  # include/pet/cutoff.hpp:53-57


def adaptive_cutoffs_solver(N, center, dist, cutoff, width, target):
    """src/device_neighbors.cpp:26-67 (solver_cutoffs): Newton-bisection for n_total(r) = target, then one
    implicit-function step. Returns (cutoff, root r, slope dn with 0 for a clamped atom), each [N]."""
    rmax, lo_bound = cutoff, cutoff * SOLVER_MIN_CUTOFF_FACTOR

    def count(r):
        n = np.bincount(center, weights=bump_cutoff_f32(dist, r[center], width), minlength=N)
        dn = np.bincount(center, weights=bump_dcutoff_dr_f32(dist, r[center], width), minlength=N)
        x = r / rmax
        return n + target * x ** 3, dn + 3.0 * target * x * x / rmax
    r_lo, r_hi, r = np.zeros(N), np.full(N, rmax), np.full(N, 0.5 * rmax)
    for _ in range(SOLVER_ITERS):
        n, dn = count(r)
        f = n - target
        r_lo, r_hi = np.where(f <= 0, r, r_lo), np.where(f <= 0, r_hi, r)
        newton = r - f / np.maximum(dn, SOLVER_DN_FLOOR)
        r = np.where((newton >= r_lo) & (newton <= r_hi), newton, 0.5 * (r_lo + r_hi))
    n, dn = count(r)
    dn_root = np.maximum(dn, SOLVER_DN_FLOOR)
    adapted = np.minimum(np.maximum(r - (n - target) / dn_root, lo_bound), rmax)
    return adapted, r, np.where((adapted > lo_bound) & (adapted < rmax), dn_root, 0.0)


def adaptive_cutoffs_grid(N, center, dist, cutoff, width, target):
    """src/device_neighbors.cpp:69-136 (grid_cutoffs): a softmax-weighted average of probe radii."""
    probes = adaptive_probes(cutoff, width)
    P = len(probes)
    if P == 0:
        return np.full(N, cutoff)
    eff = np.zeros((N, P))
    for p in range(P):
        eff[:, p] = np.bincount(center, weights=bump_cutoff_f32(dist, np.full_like(dist, probes[p]), width), minlength=N)
    x = np.arange(P) / (P - 1) if P > 1 else np.zeros(1)
    diff = eff - target + target * x ** 3
    if P == 1:
        grad = np.abs(diff) * 0.5 + 1e-12
    else:
        g = np.empty_like(diff)
        g[:, 0], g[:, -1] = diff[:, 1] - diff[:, 0], diff[:, -1] - diff[:, -2]
        g[:, 1:-1] = 0.5 * (diff[:, 2:] - diff[:, :-2])
        grad = np.maximum(np.abs(g), 1e-12)
    lw = -0.5 * (diff / grad) ** 2
    w = np.exp(lw - lw.max(1, keepdims=True))
    return (w * probes).sum(1) / w.sum(1)


def reverse_edges(idx, offsets):
    """Partner (j, i, -shift) of every edge, -1 if none (src/device_neighbors.cpp:157-176)."""
    key = {}
    for e, (i, j, a, b, c) in enumerate(idx.tolist()):
        key[(i, j, a, b, c)] = e
    return np.array([key.get((j, i, -a, -b, -c), -1) for (i, j, a, b, c) in idx.tolist()], np.int64)


def build_edges(systems, species_to_index, cutoff, width, cutoff_function="Bump", search="cells", adaptive=None):
    """Packed model edges for a batch: the reference's edge_geometry + pack_edges, no adaptive cutoff.

    src/device_neighbors.cpp:242-323 (keep d <= rc, cutoff factor, slot = number
    of the atom's kept edges before this one) and src/model.cpp:499-584
    (pack_edges: off[N+1], center, neighbour species, reverse, vec, dist, cut).
    """
    n0 = 0
    parts = []
    for b, s in enumerate(systems):
        idx, vec, dist = cell_list_edges(s, cutoff) if search == "cells" else brute_force_edges(s, cutoff)
        parts.append((idx, vec, dist, n0))
        n0 += s["n_atoms"]
    N = n0
    species = np.concatenate([np.asarray(species_to_index)[s["atomic_numbers"]] for s in systems]).astype(np.int64)
    struct_id = np.concatenate([np.full(s["n_atoms"], b) for b, s in enumerate(systems)]).astype(np.int64)
    gi = np.concatenate([p[0][:, 0] + p[3] for p in parts])
    gj = np.concatenate([p[0][:, 1] + p[3] for p in parts])
    shift = np.concatenate([p[0][:, 2:5] for p in parts])
    vec = np.concatenate([p[1] for p in parts])
    dist = np.concatenate([p[2] for p in parts])
    raw = np.concatenate([gi[:, None], gj[:, None], shift], 1)
    raw_rev = reverse_edges(raw, None)
    # Each edge's cutoff: the model's, or with an adaptive cutoff the mean of its two atoms'
    # (src/device_neighbors.cpp:243-252). adaptive = {"method": "solver"|"grid", "target": n, "width": w}.
    rc = np.full_like(dist, cutoff)
    acut = None
    if adaptive:
        if adaptive["method"] == "solver":
            acut, _, _ = adaptive_cutoffs_solver(N, gi, dist, cutoff, adaptive["width"], adaptive["target"])
        else:
            acut = adaptive_cutoffs_grid(N, gi, dist, cutoff, adaptive["width"], adaptive["target"])
        rc = 0.5 * (acut[gi] + acut[gj])
    keep = dist <= rc
    fn = bump_cutoff_f32 if cutoff_function == "Bump" else cosine_cutoff_f32
    cut = fn(dist, rc, width).astype(np.float32)
    kept_idx = np.nonzero(keep)[0]
    packed_of_raw = np.full(len(dist), -1, np.int64)
    packed_of_raw[kept_idx] = np.arange(len(kept_idx))
    center = gi[kept_idx]
    counts = np.bincount(center, minlength=N)
    off = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    rr = raw_rev[kept_idx]
    reverse = np.where(rr >= 0, packed_of_raw[np.maximum(rr, 0)], -1)
    return {
        "n_atoms": N, "n_struct": len(systems), "species": species, "struct_id": struct_id,
        "off": off, "center": center, "neighbor": gj[kept_idx], "shift": shift[kept_idx],
        "nb_species": species[gj[kept_idx]], "reverse": reverse,
        "vec": vec[kept_idx], "dist": dist[kept_idx], "cut": cut[kept_idx],
        "max_neighbors": int(max(counts.max() if N else 0, 1)),
        "raw": raw, "raw_vec": vec, "raw_dist": dist,
        "raw_center": gi, "raw_neighbor": gj, "raw_reverse": raw_rev, "kept_idx": kept_idx, "rc": rc[kept_idx],
        "atom_cutoff": acut,
    }


def build_edges_from_list(positions, species, offsets, neighbors, cutoff, width, cutoff_function="Bump", shifts=None,
                          cell=None, n_local=None):
    """Packed model edges from an engine's own full neighbour list (the reference's EdgeSession::set/step,
    src/device_geometry.cpp:410-454,712-778): v = r_j + shift.cell - r_i, kept when d <= cutoff, slots in list
    order, partner = the (j, i, -shift) entry."""
    positions = np.asarray(positions, dtype=np.float64)
    N = len(positions)
    ii = np.repeat(np.arange(N), np.diff(offsets))
    jj = np.asarray(neighbors, dtype=np.int64)
    sh = np.zeros((len(jj), 3), np.int64) if shifts is None else np.asarray(shifts, dtype=np.int64)
    vec = positions[jj] - positions[ii]
    if shifts is not None:
        vec = positions[jj] + sh @ np.asarray(cell, dtype=np.float64).reshape(3, 3) - positions[ii]
    dist = np.sqrt((vec * vec).sum(1))
    raw = np.concatenate([ii[:, None], jj[:, None], sh], 1)
    raw_rev = reverse_edges(raw, None)
    keep = dist <= cutoff
    fn = bump_cutoff_f32 if cutoff_function == "Bump" else cosine_cutoff_f32
    cut = fn(dist, np.full_like(dist, cutoff), width).astype(np.float32)
    kept = np.nonzero(keep)[0]
    packed_of_raw = np.full(len(dist), -1, np.int64)
    packed_of_raw[kept] = np.arange(len(kept))
    center = ii[kept]
    counts = np.bincount(center, minlength=N)
    rr = raw_rev[kept]
    species = np.asarray(species, dtype=np.int64)
    return {
        "n_atoms": N, "n_struct": 1, "species": species, "struct_id": np.zeros(N, np.int64),
        "off": np.concatenate([[0], np.cumsum(counts)]).astype(np.int64), "center": center, "neighbor": jj[kept],
        "shift": sh[kept], "nb_species": species[jj[kept]], "reverse": np.where(rr >= 0, packed_of_raw[np.maximum(rr, 0)], -1),
        "vec": vec[kept], "dist": dist[kept], "cut": cut[kept], "max_neighbors": int(max(counts.max() if N else 0, 1)),
        "raw": raw, "raw_vec": vec, "raw_dist": dist, "n_local": N if n_local is None or n_local < 0 else int(n_local),
    }
