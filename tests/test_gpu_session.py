"""Engine-supplied neighbour lists: set_neighbors / compute_step / compute_edges (the reference's tests/test_edges.cpp)."""
import numpy as np
import pytest

from oracle import neighbors_oracle as nbo
from pet_kokkos_b200 import EdgeListView, structures as st

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def calc(lib_path, models):
    from pet_kokkos_b200 import Calculator
    c = Calculator(*models("tiny", "feedforward", "scaled", 1))
    yield c
    c.close()


def full_list(s, cutoff, skin=0.0):
    """A full periodic list with shifts, as an engine would hand it over (pairs out to cutoff + skin)."""
    idx, _, _ = nbo.brute_force_edges(s, cutoff + skin)
    order = np.lexsort((idx[:, 4], idx[:, 3], idx[:, 2], idx[:, 1], idx[:, 0]))
    idx = idx[order]
    off = np.concatenate([[0], np.cumsum(np.bincount(idx[:, 0], minlength=s["n_atoms"]))])
    return EdgeListView(s["positions"], s["atomic_numbers"], off, idx[:, 1], idx[:, 2:5], s["cell"])


def held_to_the_reference(reference, models, view, r):
    """The same list through the reference's own compute_edges (its host build): energy, forces and virial within the
    parity bands. The device-list forms below are compared with the host list's answer to the bit; this ties that
    answer, on the very list of the test, to the reference."""
    jp, sp = models("tiny", "feedforward", "scaled", 1)
    lst = {"positions": np.asarray(view.positions), "atomic_numbers": np.asarray(view.atomic_numbers, np.int32),
           "offsets": np.asarray(view.offsets, np.int32), "neighbors": np.asarray(view.neighbors, np.int32),
           "shifts": None if view.shifts is None else np.asarray(view.shifts, np.int32), "cell": view.cell,
           "n_local": -1, "half": False}
    ref = reference.ReferenceCalculator(str(jp), str(sp)).compute_edges(lst, True, False)
    scale = max(abs(ref["energy"][0]), np.abs(ref["per_atom_energy"]).sum())
    assert abs(r.energy[0] - ref["energy"][0]) <= 1e-6 * scale
    assert np.abs(r.forces - ref["forces"]).max() <= 1e-5 * max(1.0, np.abs(ref["forces"]).max())
    assert np.abs(r.virial - ref["virial"]).max() <= 1e-5 * max(1.0, np.abs(ref["virial"]).max())


def test_shifts_list_matches_own_search(calc):
    """tests/test_edges.cpp:180-208: an engine's periodic list with shifts gives the periodic answer."""
    s = st.diamond(2, jitter=0.05, seed=0)
    ref = calc.compute(s)
    r = calc.compute_edges(full_list(s, calc.cutoff, skin=1.0))
    assert abs(r.energy[0] - ref.energy[0]) <= 1e-5 * abs(ref.energy[0])
    assert np.abs(r.forces - ref.forces).max() <= 1e-4 * max(1.0, np.abs(ref.forces).max())
    assert np.abs(r.virial - ref.virial).max() <= 1e-4 * max(1.0, np.abs(ref.virial).max())


def test_edge_gradients_fold_to_forces_and_virial(calc):
    """tests/test_edges.cpp:166-175: F_i = sum_out g - sum_in g and W = sum v (x) g, to 1e-9 of their scale."""
    s = st.diamond(2, jitter=0.05, seed=1)
    v = full_list(s, calc.cutoff, skin=0.5)
    r = calc.compute_edges(v, True, True)
    g = r.edge_gradient
    i = np.repeat(np.arange(s["n_atoms"]), np.diff(v.offsets))
    j = v.neighbors
    F = np.zeros_like(r.forces)
    np.add.at(F, i, g)
    np.add.at(F, j, -g)
    vec = s["positions"][j] + v.shifts @ s["cell"] - s["positions"][i]
    W9 = np.einsum("ea,eb->ab", vec, g)
    W = np.array([W9[0, 0], W9[1, 1], W9[2, 2], 0.5 * (W9[0, 1] + W9[1, 0]), 0.5 * (W9[0, 2] + W9[2, 0]), 0.5 * (W9[1, 2] + W9[2, 1])])
    assert np.abs(F - r.forces).max() <= 1e-9 * max(1.0, np.abs(r.forces).max())
    assert np.abs(W - r.virial[0]).max() <= 1e-9 * max(1.0, np.abs(W).max())


def test_half_list_equals_full_list(calc):
    """tests/test_edges.cpp:256-276."""
    s = st.diamond(2, jitter=0.05, seed=2)
    full = full_list(s, calc.cutoff)
    i = np.repeat(np.arange(s["n_atoms"]), np.diff(full.offsets))
    keep = (i < full.neighbors) | ((i == full.neighbors) & ([tuple(x) > (0, 0, 0) for x in full.shifts.tolist()]))
    off = np.concatenate([[0], np.cumsum(np.bincount(i[keep], minlength=s["n_atoms"]))])
    half = EdgeListView(s["positions"], s["atomic_numbers"], off, full.neighbors[keep], full.shifts[keep], s["cell"], half=True)
    a, b = calc.compute_edges(full, True, False), calc.compute_edges(half, True, False)
    assert abs(a.energy[0] - b.energy[0]) <= 1e-6 * abs(a.energy[0])
    assert np.abs(a.forces - b.forces).max() <= 1e-5 * max(1.0, np.abs(a.forces).max())


def test_ghost_domain_reproduces_the_periodic_answer(calc):
    """tests/test_edges.cpp:117-178: owned atoms plus explicit ghost images ghost_cutoff deep, no shifts;
    the energy is the periodic one and ghost forces summed onto their owners give the periodic forces."""
    s = st.diamond(2, jitter=0.05, seed=3)
    ref = calc.compute(s)
    N, L, reach = s["n_atoms"], s["cell"][0, 0], calc.ghost_cutoff
    pos, owner = [s["positions"]], [np.arange(N)]
    rng = int(np.ceil(reach / L))
    for a in range(-rng, rng + 1):
        for b in range(-rng, rng + 1):
            for c in range(-rng, rng + 1):
                if (a, b, c) == (0, 0, 0):
                    continue
                p = s["positions"] + np.array([a, b, c]) @ s["cell"]
                lo, hi = s["positions"].min(0) - reach, s["positions"].max(0) + reach
                m = ((p >= lo) & (p <= hi)).all(1)
                pos.append(p[m]), owner.append(np.arange(N)[m])
    pos, owner = np.concatenate(pos), np.concatenate(owner)
    # every atom within ghost_cutoff - cutoff of an owned atom needs its full list: list every atom's pairs
    d = pos[:, None, :] - pos[None, :, :]
    d2 = (d * d).sum(-1)
    ii, jj = np.nonzero((d2 <= calc.cutoff ** 2) & (d2 > 1e-20))
    off = np.concatenate([[0], np.cumsum(np.bincount(ii, minlength=len(pos)))])
    view = EdgeListView(pos, s["atomic_numbers"][owner], off, jj, n_local=N)
    r = calc.compute_edges(view, True, False)
    F = np.zeros((N, 3))
    np.add.at(F, owner, r.forces)
    assert abs(r.energy[0] - ref.energy[0]) <= 1e-5 * abs(ref.energy[0])
    assert np.abs(F - ref.forces).max() <= 1e-4 * max(1.0, np.abs(ref.forces).max())


def test_stepping_one_list(calc):
    """tests/test_edges.cpp:278-319: set once, step with moved positions; pairs that drift past the cutoff weigh nothing."""
    s = st.diamond(2, jitter=0.05, seed=4)
    calc.set_neighbors(full_list(s, calc.cutoff, skin=1.0))
    rng = np.random.default_rng(0)
    for _ in range(3):
        moved = dict(s)
        moved["positions"] = s["positions"] + rng.normal(0, 0.03, size=s["positions"].shape)
        r = calc.compute_step(moved["positions"], s["cell"])
        ref = calc.compute(moved)
        assert abs(r.energy[0] - ref.energy[0]) <= 1e-5 * abs(ref.energy[0])
        assert np.abs(r.forces - ref.forces).max() <= 1e-4 * max(1.0, np.abs(ref.forces).max())
    calc.set_neighbors(full_list(s, calc.cutoff, skin=1.0))


def test_no_list_set_is_an_error(lib_path, models):
    from pet_kokkos_b200 import Calculator
    c = Calculator(*models("tiny"))
    c._session_atoms = 1
    with pytest.raises(RuntimeError, match="no neighbour list set"):
        c.compute_step(np.zeros((1, 3)))
    c.close()


@pytest.mark.parametrize("world", [2, 4])
def test_domain_decomposition_on_one_gpu(calc, world):
    """The multi-GPU single-cell path with its ranks played one after another on one GPU: owned atoms plus
    ghost shells per rank, ghost forces folded onto owners, energies and virials summed (pet_kokkos_b200/domain.py).
    Tolerances are the reference's for a ghost domain (tests/test_edges.cpp:117-178)."""
    from pet_kokkos_b200 import domain
    s = st.diamond(3, jitter=0.05, seed=5)
    ref = calc.compute(s)
    e, F, W = 0.0, np.zeros((s["n_atoms"], 3)), np.zeros(6)
    for rank in range(world):
        view, owner, n_local = domain.local_domain(s, rank, world, calc.cutoff, calc.ghost_cutoff)
        pe, pF, pW = domain.fold(calc.compute_edges(view, True, False), owner, s["n_atoms"])
        e, F, W = e + pe, F + pF, W + pW
    assert abs(e - ref.energy[0]) <= 1e-5 * abs(ref.energy[0])
    assert np.abs(F - ref.forces).max() <= 1e-4 * max(1.0, np.abs(ref.forces).max())
    assert np.abs(W - ref.virial[0]).max() <= 1e-4 * max(1.0, np.abs(ref.virial).max())


@pytest.mark.parametrize("gemm", ["native", "3xtf32"])
def test_fixed_shape_stepping_equals_plain_stepping(lib_path, models, gemm):
    """Options::md_fixed_shapes (include/pet/calculator.hpp:111-116): capacities for the kept edges and the neighbour
    count, sized by the first step and kept while the atoms move, so nothing is read back and the recorded pass is
    replayed although the number of kept edges changes; a step that outgrows them is redone. Every step must give the
    bits of a calculator without fixed shapes."""
    from pet_kokkos_b200 import Calculator
    jp, sp = models("tiny", "feedforward", "scaled", 1)
    plain = Calculator(jp, sp, gemm=gemm)
    fixed = Calculator(jp, sp, gemm=gemm, md_fixed_shapes=True)
    s = st.diamond(2, jitter=0.05, seed=4)
    view = full_list(s, plain.cutoff, skin=1.0)
    plain.set_neighbors(view)
    fixed.set_neighbors(view)
    rng = np.random.default_rng(3)
    x = s["positions"].copy()
    edges = []
    for step in range(8):
        if step == 5:  # squeeze: many listed pairs come inside the cutoff at once, more than the capacity's headroom
            x = x * 0.93
            cell = s["cell"] * 0.93
        else:
            x = x + rng.normal(0, 0.02, x.shape)
            cell = s["cell"] if step < 5 else s["cell"] * 0.93
        a, b = plain.compute_step(x, cell), fixed.compute_step(x, cell)
        edges.append(plain.last_shapes()[1])
        assert (a.energy == b.energy).all() and (a.forces == b.forces).all() and (a.virial == b.virial).all(), step
    assert len(set(edges)) > 2, "the number of kept edges has to change for this test to mean anything"
    assert edges[5] > 1.05 * edges[4] + 64, "the squeeze has to outgrow the capacity"
    assert fixed.graph_replays >= 3 and plain.graph_replays == 0
    plain.close()
    fixed.close()


@pytest.mark.parametrize("fixed", [False, True])
def test_device_arrays_step_adds_into_the_engines_arrays(lib_path, models, fixed):
    """Calculator::compute_step(const DeviceArrays&, cell) (include/pet/calculator.hpp:248-259): positions read from
    and forces, per-atom energies and per-atom virials added into device arrays; only the totals come back. Checked
    against the host-array compute_step, over steps that change the number of kept edges and (with fixed shapes) one
    that outgrows the capacities and is redone without adding twice."""
    import torch
    from pet_kokkos_b200 import Calculator
    jp, sp = models("tiny", "feedforward", "scaled", 1)
    host = Calculator(jp, sp)
    dev = Calculator(jp, sp, md_fixed_shapes=fixed)
    s = st.diamond(2, jitter=0.05, seed=5)
    view = full_list(s, host.cutoff, skin=1.0)
    host.set_neighbors(view)
    dev.set_neighbors(view)
    N = s["n_atoms"]
    rng = np.random.default_rng(7)
    x = s["positions"].copy()
    for step in range(6):
        squeeze = step >= 4
        if step == 4:
            x = x * 0.93
        else:
            x = x + rng.normal(0, 0.02, x.shape)
        cell = s["cell"] * (0.93 if squeeze else 1.0)
        ref = host.compute_step(x, cell)
        d_x = torch.tensor(x, dtype=torch.float64, device="cuda")
        d_f = torch.full((N, 3), 1.5, dtype=torch.float64, device="cuda")     # "added into": start from something
        d_e = torch.full((N,), -2.0, dtype=torch.float64, device="cuda")
        d_w = torch.zeros((N, 6), dtype=torch.float64, device="cuda")
        torch.cuda.synchronize()
        energy, virial = dev.compute_step_device(d_x.data_ptr(), d_f.data_ptr(), d_e.data_ptr(), d_w.data_ptr(), -1.0, cell)
        torch.cuda.synchronize()
        assert energy == ref.energy[0] and (virial == ref.virial[0]).all()
        assert (d_f.cpu().numpy() - 1.5 == ref.forces).all() or np.abs(d_f.cpu().numpy() - 1.5 - ref.forces).max() <= 1e-12
        np.testing.assert_allclose(d_e.cpu().numpy() + 2.0, ref.per_atom_energy, rtol=0, atol=1e-12)
        np.testing.assert_allclose(d_w.cpu().numpy().sum(0), -1.0 * ref.virial[0], rtol=0,
                                   atol=1e-9 * max(1.0, np.abs(ref.virial).max()))
    host.close()
    dev.close()


@pytest.mark.parametrize("renumbered", [False, True])
@pytest.mark.parametrize("order", ["listed", "interleaved", "strided"])
def test_flat_pair_list_on_the_device_gets_what_the_host_list_does(calc, reference, models, renumbered, order):
    """tests/test_edges.cpp:709-779: the engine numbers the atoms backwards and hands the pairs over flat, in list
    order or each atom's pairs interleaved with the others'; with the renumbering the answer comes back in ours."""
    import torch
    s = st.diamond(2, jitter=0.05, seed=21)
    n = s["n_atoms"]
    v = full_list(s, calc.cutoff, skin=0.5)
    ref = calc.compute_edges(v)
    held_to_the_reference(reference, models, v, ref)
    off = np.asarray(v.offsets)
    P = int(off[-1])
    theirs = np.arange(n)[::-1].copy() if renumbered else np.arange(n)
    i = np.repeat(np.arange(n), np.diff(off))
    flat = np.column_stack([theirs[i], theirs[np.asarray(v.neighbors)], np.asarray(v.shifts)]).astype(np.int32)
    if order == "interleaved":  # round-robin over the atoms: a scattered list, each atom's pairs still in their order
        rank = np.arange(P) - off[i]
        flat = flat[np.lexsort((i, rank))]
    ren = np.empty(n, np.int32)
    ren[theirs] = np.arange(n)
    z = np.empty(n, np.int32)
    z[theirs] = s["atomic_numbers"]
    x = np.empty((n, 3))
    x[theirs] = s["positions"]
    dev = "cuda:0"
    if order == "strided":  # column-major storage: stride_pair 1, stride_col P
        t_pairs = torch.tensor(np.ascontiguousarray(flat.T), device=dev)
        strides = dict(stride_pair=1, stride_col=P)
    else:
        t_pairs = torch.tensor(flat, device=dev)
        strides = {}
    t_z, t_ren, t_x = torch.tensor(z, device=dev), torch.tensor(ren, device=dev), torch.tensor(x, device=dev)
    torch.cuda.synchronize()
    ptrs, r = calc.compute_pairs(n, P, t_pairs.data_ptr(), t_z.data_ptr(), t_x.data_ptr(), cell=s["cell"],
                                 renumber_ptr=t_ren.data_ptr() if renumbered else 0, **strides)
    assert r.energy[0] == ref.energy[0]
    assert np.array_equal(r.forces, ref.forces) and np.array_equal(r.virial, ref.virial)
    assert np.array_equal(r.per_atom_energy, ref.per_atom_energy)
    assert ptrs["energy"] and ptrs["forces"] and ptrs["virial"] and ptrs["per_atom_energy"]
    # the list stays set: a step over moved positions, on the device, in the engine's order
    moved = s["positions"] + np.random.default_rng(3).normal(0, 0.02, (n, 3))
    want = calc.compute_edges(EdgeListView(moved, v.atomic_numbers, v.offsets, v.neighbors, v.shifts, v.cell))
    xm = np.empty((n, 3))
    xm[theirs] = moved
    t_xm = torch.tensor(xm, device=dev)
    forces = torch.zeros((n, 3), dtype=torch.float64, device=dev)
    torch.cuda.synchronize()
    ptrs, r = calc.compute_pairs(n, P, t_pairs.data_ptr(), t_z.data_ptr(), t_xm.data_ptr(), cell=s["cell"],
                                 renumber_ptr=t_ren.data_ptr() if renumbered else 0, **strides)
    e, w = calc.compute_step_device(t_xm.data_ptr(), forces.data_ptr(), cell=s["cell"])
    torch.cuda.synchronize()
    assert e == want.energy[0] and np.array_equal(w, want.virial[0])
    assert np.array_equal(forces.cpu().numpy(), want.forces)


def test_flat_pair_list_errors(calc):
    """src/device_geometry.cpp:560-607: a renumbering that is no permutation, pairs naming atoms that do not exist,
    elements the model does not cover; a renumbered list takes device positions."""
    import torch
    s = st.diamond(1, jitter=0.02, seed=2)
    n = s["n_atoms"]
    v = full_list(s, calc.cutoff)
    P = int(np.asarray(v.offsets)[-1])
    i = np.repeat(np.arange(n), np.diff(v.offsets))
    flat = np.column_stack([i, np.asarray(v.neighbors), np.asarray(v.shifts)]).astype(np.int32)
    dev = "cuda:0"
    t_x = torch.tensor(s["positions"], device=dev)
    t_z = torch.tensor(np.asarray(s["atomic_numbers"], np.int32), device=dev)
    t_pairs = torch.tensor(flat, device=dev)
    bad_ren = torch.tensor(np.zeros(n, np.int32), device=dev)
    with pytest.raises(RuntimeError, match="not a permutation"):
        calc.compute_pairs(n, P, t_pairs.data_ptr(), t_z.data_ptr(), t_x.data_ptr(), cell=s["cell"], renumber_ptr=bad_ren.data_ptr())
    bad = flat.copy()
    bad[3, 1] = n + 5
    t_bad = torch.tensor(bad, device=dev)
    with pytest.raises(RuntimeError, match="1 pairs name atoms that do not exist"):
        calc.compute_pairs(n, P, t_bad.data_ptr(), t_z.data_ptr(), t_x.data_ptr(), cell=s["cell"])
    t_zbad = torch.tensor(np.full(n, 117, np.int32), device=dev)
    with pytest.raises(RuntimeError, match="elements the model does not cover"):
        calc.compute_pairs(n, P, t_pairs.data_ptr(), t_zbad.data_ptr(), t_x.data_ptr(), cell=s["cell"])
    ident = torch.tensor(np.arange(n, dtype=np.int32), device=dev)
    calc.compute_pairs(n, P, t_pairs.data_ptr(), t_z.data_ptr(), t_x.data_ptr(), cell=s["cell"], renumber_ptr=ident.data_ptr())
    with pytest.raises(RuntimeError, match="takes device positions"):
        calc.compute_step(s["positions"], s["cell"])


@pytest.mark.parametrize("layout", ["rows", "columns"])
def test_device_list_gets_the_bits_of_the_host_list(calc, reference, models, layout):
    """tests/test_edges.cpp:528-587: the engine's 2-D neighbour array in device memory (either layout, the engine's
    flag bits above the index masked off, centres listed out of order) gives what the same list gives from the host."""
    import torch
    s = st.diamond(2, jitter=0.05, seed=31)
    n = s["n_atoms"]
    # a cluster's list: no shifts, so ghosts are not needed
    c = st.make_system(s["atomic_numbers"], s["positions"], np.eye(3) * 60.0, pbc=(False, False, False))
    v = full_list(c, calc.cutoff, skin=0.4)
    calc.set_neighbors(v)
    ref = calc.compute_step(c["positions"], c["cell"])  # the host list carries (zero) shifts
    held_to_the_reference(reference, models, v, ref)
    off = np.asarray(v.offsets)
    counts = np.diff(off)
    M = int(counts.max())
    table = np.zeros((n, M), np.int32)
    for i in range(n):
        table[i, :counts[i]] = np.asarray(v.neighbors)[off[i]:off[i + 1]] | (1 << 30)  # a flag bit above the index
    dev = "cuda:0"
    ilist = np.random.default_rng(0).permutation(n).astype(np.int32)
    if layout == "rows":
        t_tab, si, sk = torch.tensor(table, device=dev), M, 1
    else:
        t_tab, si, sk = torch.tensor(np.ascontiguousarray(table.T), device=dev), 1, n
    t_il, t_nn = torch.tensor(ilist, device=dev), torch.tensor(counts.astype(np.int32), device=dev)
    t_z = torch.tensor(np.asarray(c["atomic_numbers"], np.int32), device=dev)
    torch.cuda.synchronize()
    calc.set_neighbors_device(n, n, t_il.data_ptr(), t_nn.data_ptr(), t_tab.data_ptr(), si, t_z.data_ptr(), stride_k=sk,
                              mask=(1 << 30) - 1)
    got = calc.compute_step(c["positions"])
    assert got.energy[0] == ref.energy[0] and np.array_equal(got.forces, ref.forces) and np.array_equal(got.virial, ref.virial)


def test_device_list_with_images_equals_the_periodic_list(calc):
    """Periodic images instead of ghosts (include/pet/device_geometry.hpp:109-111): every neighbour is replaced by the
    owned atom it is an image of and the lattice shift between them, which is the periodic list with shifts."""
    import torch
    s = st.diamond(2, jitter=0.05, seed=32)
    n = s["n_atoms"]
    v = full_list(s, calc.cutoff, skin=0.3)
    ref = calc.compute_edges(v, True, False)
    off, nbr, sh = np.asarray(v.offsets), np.asarray(v.neighbors), np.asarray(v.shifts)
    # one image atom per distinct (atom, shift != 0)
    keys = {}
    image_of, pos = list(range(n)), [p for p in s["positions"]]
    nb2 = np.empty_like(nbr)
    for e in range(len(nbr)):
        k = (int(nbr[e]), *map(int, sh[e]))
        if not any(k[1:]):
            nb2[e] = nbr[e]
            continue
        if k not in keys:
            keys[k] = len(image_of)
            image_of.append(k[0])
            pos.append(s["positions"][k[0]] + sh[e] @ s["cell"])
        nb2[e] = keys[k]
    na = len(image_of)
    counts = np.concatenate([np.diff(off), np.zeros(na - n, np.int64)]).astype(np.int32)
    M = int(counts.max())
    table = np.zeros((na, M), np.int32)
    for i in range(n):
        table[i, :counts[i]] = nb2[off[i]:off[i + 1]]
    z = np.asarray(s["atomic_numbers"], np.int32)[np.array(image_of)]
    dev = "cuda:0"
    t = {k: torch.tensor(a, device=dev) for k, a in dict(il=np.arange(n, dtype=np.int32), nn=counts, tab=table, z=z,
                                                           im=np.array(image_of, np.int32), x=np.array(pos)).items()}
    torch.cuda.synchronize()
    calc.set_neighbors_device(na, n, t["il"].data_ptr(), t["nn"].data_ptr(), t["tab"].data_ptr(), M, t["z"].data_ptr(),
                              n_local=n, image_of_ptr=t["im"].data_ptr(), positions_ptr=t["x"].data_ptr(), cell=s["cell"])
    got = calc.compute_step(np.array(pos), s["cell"])
    assert abs(got.energy[0] - ref.energy[0]) <= 1e-9 * abs(ref.energy[0])
    assert np.abs(got.forces[:n] - ref.forces).max() <= 1e-9 * max(1.0, np.abs(ref.forces).max())
    assert np.abs(got.forces[n:]).max() == 0.0  # the images carry no pairs and no force
    assert np.abs(got.virial - ref.virial).max() <= 1e-9 * max(1.0, np.abs(ref.virial).max())
    bad = torch.tensor(np.full(na, -1, np.int32), device=dev)
    with pytest.raises(RuntimeError, match="not an image of an owned atom"):
        calc.set_neighbors_device(na, n, t["il"].data_ptr(), t["nn"].data_ptr(), t["tab"].data_ptr(), M, t["z"].data_ptr(),
                                  n_local=n, image_of_ptr=bad.data_ptr(), positions_ptr=t["x"].data_ptr(), cell=s["cell"])


def test_recorded_passes_follow_the_list_they_were_recorded_for(tmp_path):
    """An adaptive cutoff's backward reads the raw list as well as the packed edges. Two lists of the same atoms
    with different skins keep the same edges (same packed shapes) from raw lists of different sizes: a pass
    recorded for one must not be replayed for the other."""
    from pet_kokkos_b200 import Calculator, checkpoint as ck
    jp, sp = ck.write_random_checkpoint(tmp_path / "ad", "tiny", "feedforward", seed=5, init="scaled",
                                        num_neighbors_adaptive=16.0, adaptive_cutoff_method="solver", cutoff=5.5)
    c = Calculator(jp, sp)
    s = st.diamond(2, jitter=0.08, seed=1)
    want = {}
    for skin in (0.2, 0.9):
        fresh = Calculator(jp, sp, graphs=False)
        want[skin] = fresh.compute_edges(full_list(s, fresh.cutoff, skin=skin), True, False)
        fresh.close()
    for skin in (0.2, 0.9, 0.2, 0.9):
        c.set_neighbors(full_list(s, c.cutoff, skin=skin))
        for _ in range(3):  # eager, recorded, replayed
            r = c.compute_step(s["positions"], s["cell"])
            assert r.energy[0] == want[skin].energy[0] and np.array_equal(r.forces, want[skin].forces)
            assert np.array_equal(r.virial, want[skin].virial)
    assert c.graph_replays >= 4
    c.close()
