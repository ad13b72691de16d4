"""The CPU restatement (oracle/) against the reference's own code, run live.

oracle/_ref/libpet_ref.so is peterspackman/pet-kokkos's src/*.cpp compiled for the host
(oracle/build_ref.sh). These tests hold the restatement to it on more inputs than the
committed fixtures carry: the neighbour search to the bit, the network within the parity
bands, an engine's list through compute_edges / set_neighbors + compute_step.
"""
import numpy as np
import pytest
import torch

from oracle import neighbors_oracle as nbo, pet_oracle as po
from pet_kokkos_b200 import checkpoint as ck, structures as st


def cluster(n, seed):
    s = st.water_box(n, 3.2 * n ** (1.0 / 3.0), seed=seed)
    return st.make_system(s["atomic_numbers"], s["positions"], np.eye(3) * 40.0, pbc=(False, False, False))


def slab(seed):
    s = st.diamond(2, jitter=0.05, seed=seed)
    return st.make_system(s["atomic_numbers"], s["positions"], s["cell"], pbc=(True, True, False))


STRUCTURES = {
    "diamond64": lambda: [st.diamond(2, jitter=0.05, seed=1)],
    "diamond8_many_images": lambda: [st.diamond(1, jitter=0.03, seed=2)],
    "sheared216": lambda: [st.diamond(3, shear=0.35, jitter=0.05, seed=3)],
    "diamond512_grid": lambda: [st.diamond(4, jitter=0.05, seed=4)],
    "water": lambda: [st.water_box(30, 10.0, seed=5)],
    "cluster": lambda: [cluster(10, 6)],
    "slab": lambda: [slab(7)],
    "batch": lambda: [st.diamond(2, jitter=0.05, seed=8), cluster(6, 9), st.random_mixture(40, 8.0, seed=10), slab(11)],
    "single_atom_box": lambda: [st.make_system([6], [[0.1, 0.2, 0.3]], np.eye(3) * 3.0)],
}


@pytest.mark.parametrize("name", sorted(STRUCTURES))
def test_packed_edges_equal_the_reference_device_search(reference, models, name):
    """Same kept edges in the same order, vectors and distances to the bit, same partners
    (src/device_geometry.cpp build_device_batch -> src/device_neighbors.cpp). The cutoff factor goes
    through float tanh/tan/cos of the host's libm there and numpy's here: equal within 4 float ulps."""
    jp, sp = models("tiny")
    meta, _ = ck.load_checkpoint(jp, sp)
    h = meta["hypers"]
    systems = STRUCTURES[name]()
    d = reference.ReferenceCalculator(str(jp), str(sp)).device_edges(systems)
    ed = nbo.build_edges(systems, meta["species_to_index"], h["cutoff"], h["cutoff_width"], h["cutoff_function"])
    N, M = d["N"], d["M"]
    counts = np.diff(ed["off"])
    assert N == ed["n_atoms"] and np.array_equal(d["mask"].sum(1).astype(np.int64), counts)
    if counts.sum() == 0:
        return
    assert M == ed["max_neighbors"]
    slot = np.concatenate([n * M + np.arange(c) for n, c in enumerate(counts)])
    assert np.array_equal(d["vec"].reshape(-1, 3)[slot].view(np.uint64), ed["vec"].view(np.uint64))
    assert np.array_equal(d["dist"].reshape(-1)[slot].view(np.uint64), ed["dist"].view(np.uint64))
    assert np.array_equal(d["neigh_species"].reshape(-1)[slot], ed["nb_species"])
    packed_of_slot = np.full(N * M, -1, np.int64)
    packed_of_slot[slot] = np.arange(len(slot))
    rv = d["reverse"].reshape(-1)[slot]
    assert np.array_equal(np.where(rv >= 0, packed_of_slot[np.maximum(rv, 0)], -1), ed["reverse"])
    cut_ref, cut = d["cutoff"].reshape(-1)[slot], ed["cut"].astype(np.float32)
    assert np.abs(cut_ref - cut).max() <= 4 * np.spacing(np.float32(1.0))


@pytest.mark.parametrize("name", ["diamond64", "diamond8_many_images", "cluster", "slab"])
def test_brute_force_edges_equal_the_reference_host_search(reference, name):
    """detail::build_raw_edges (src/neighbors.cpp): the same set of (i, j, shift) and the same vectors."""
    s = STRUCTURES[name]()[0]
    r = reference.host_raw_edges(s, 4.5)
    idx, vec, dist = nbo.brute_force_edges(s, 4.5)
    key = lambda i, j, sh: sorted(zip(i.tolist(), j.tolist(), map(tuple, sh.tolist())))
    assert key(r["i"], r["j"], r["shift"]) == key(idx[:, 0], idx[:, 1], idx[:, 2:5])
    order_r = np.lexsort((r["shift"][:, 2], r["shift"][:, 1], r["shift"][:, 0], r["j"], r["i"]))
    order_o = np.lexsort((idx[:, 4], idx[:, 3], idx[:, 2], idx[:, 1], idx[:, 0]))
    np.testing.assert_allclose(r["vec"][order_r], vec[order_o], rtol=0, atol=1e-12)
    np.testing.assert_allclose(r["dist"][order_r], dist[order_o], rtol=0, atol=1e-12)


def bands(a, ref):
    # the energy's scale is what was summed (a total can cancel to near zero), where the per-atom terms are at hand
    e_scale = max(np.abs(ref["energy"]).max(), np.abs(ref.get("per_atom_energy", np.zeros(1))).sum() / len(ref["energy"]))
    assert np.abs(a["energy"] - ref["energy"]).max() <= 1e-6 * e_scale
    assert np.abs(a["forces"] - ref["forces"]).max() <= 1e-5 * max(1.0, np.abs(ref["forces"]).max())
    assert np.abs(a["virial"] - ref["virial"]).max() <= 1e-5 * max(1.0, np.abs(ref["virial"]).max())


@pytest.mark.parametrize("featurizer", ["feedforward", "residual"])
@pytest.mark.parametrize("name", ["diamond64", "sheared216", "cluster", "slab", "batch"])
def test_network_matches_the_reference(reference, models, featurizer, name):
    jp, sp = models("tiny", featurizer, "scaled", 21)
    meta, tens = ck.load_checkpoint(jp, sp)
    systems = STRUCTURES[name]()
    ref = reference.ReferenceCalculator(str(jp), str(sp)).compute(systems)
    got = po.evaluate(meta, tens, systems, dtype=torch.float32)
    bands(got, ref)
    assert np.abs(got["per_atom_energy"] - ref["per_atom_energy"]).max() <= 1e-6 * np.abs(ref["energy"]).max()


def test_host_and_device_neighbour_paths_of_the_reference_agree(reference, models):
    """tests/test_device_vs_host.cpp: the reference's two list builders give the same answer; so a pin on
    one is a pin on both."""
    jp, sp = models("tiny", "feedforward", "scaled", 21)
    s = STRUCTURES["diamond64"]()
    a = reference.ReferenceCalculator(str(jp), str(sp), device_neighbors=True).compute(s)
    b = reference.ReferenceCalculator(str(jp), str(sp), device_neighbors=False).compute(s)
    bands(a, b)


def engine_list(system, cutoff, skin=0.6):
    """A full neighbour list with shifts, as an MD engine would hand over (cutoff + skin)."""
    idx, vec, dist = nbo.brute_force_edges(system, cutoff + skin)
    order = np.lexsort((idx[:, 4], idx[:, 3], idx[:, 2], idx[:, 1], idx[:, 0]))
    idx = idx[order]
    N = system["n_atoms"]
    offsets = np.concatenate([[0], np.cumsum(np.bincount(idx[:, 0], minlength=N))]).astype(np.int32)
    return {"positions": system["positions"], "atomic_numbers": system["atomic_numbers"], "offsets": offsets,
            "neighbors": idx[:, 1].astype(np.int32), "shifts": idx[:, 2:5].astype(np.int32), "cell": system["cell"],
            "n_local": -1, "half": False}


@pytest.mark.parametrize("featurizer", ["feedforward", "residual"])
def test_engine_list_and_stepping_match_the_reference(reference, models, featurizer):
    """compute_edges with edge gradients, then set_neighbors + compute_step over moved positions
    (include/pet/calculator.hpp:227-238), against the restatement on the same list."""
    jp, sp = models("tiny", featurizer, "scaled", 22)
    meta, tens = ck.load_checkpoint(jp, sp)
    h = meta["hypers"]
    s = st.diamond(2, jitter=0.05, seed=13)
    lst = engine_list(s, h["cutoff"])
    calc = reference.ReferenceCalculator(str(jp), str(sp))
    ref = calc.compute_edges(lst)
    species = np.asarray(meta["species_to_index"])[s["atomic_numbers"]]

    def restated(positions):
        ed = nbo.build_edges_from_list(positions, species, lst["offsets"], lst["neighbors"], h["cutoff"],
                                       h["cutoff_width"], h["cutoff_function"], shifts=lst["shifts"], cell=s["cell"])
        return po.evaluate(meta, tens, ed, dtype=torch.float32)

    got = restated(s["positions"])
    bands(got, ref)
    whole = reference.ReferenceCalculator(str(jp), str(sp)).compute(s)
    bands(ref, whole)  # the list path and the search path of the reference agree with each other
    rng = np.random.default_rng(5)
    moved = np.stack([s["positions"] + rng.normal(0, 0.03, s["positions"].shape) for _ in range(3)])
    steps = calc.steps(lst, moved)
    for k in range(3):
        g = restated(moved[k])
        bands(g, {"energy": steps["energy"][k:k + 1], "forces": steps["forces"][k], "virial": steps["virial"][k:k + 1]})


@pytest.mark.parametrize("method", ["solver", "grid"])
def test_adaptive_cutoff_matches_the_reference(reference, tmp_path, method):
    """The adaptive cutoff, both schemes (src/device_neighbors.cpp:26-136; backward src/forces.cpp:80-260,308-341):
    each atom's cutoff from all its raw distances, pairs kept within the mean of their atoms' cutoffs, forces and
    virial folded over the raw list. The reference implements it for the feedforward featurizer only."""
    jp, sp = ck.write_random_checkpoint(tmp_path / f"ad_{method}", "tiny", "feedforward", seed=5, init="scaled",
                                        num_neighbors_adaptive=16.0, adaptive_cutoff_method=method, cutoff=5.5)
    meta, tens = ck.load_checkpoint(jp, sp)
    systems = [st.diamond(2, jitter=0.08, seed=1), st.random_mixture(30, 8.0, seed=4), cluster(8, 3)]
    ref = reference.ReferenceCalculator(str(jp), str(sp)).compute(systems)
    got = po.evaluate(meta, tens, systems, dtype=torch.float32)
    bands(got, ref)
    ed = got["edges"]
    assert len(ed["center"]) < 0.5 * len(ed["raw"]), "the adaptive cutoff has to drop edges for this test to mean anything"
    assert got["atom_cutoff"].min() < 0.8 * got["atom_cutoff"].max()
