"""The Verlet cache of a staged batch (Options::cache_neighbors; the reference's NefCache and
tests/test_device_vs_host.cpp:93-265): pairs searched to cutoff + 1 A, kept while no pair outside could have come
inside the cutoff, their vectors taken from the positions and cells of each evaluation.

The cached pairs come in the longer search's bin order, so the network sums them in another order than the plain
search does: the two answers agree within the parity bands, not to the last bit.
"""
import numpy as np
import pytest

from pet_kokkos_b200 import checkpoint as ck, structures as st

pytestmark = pytest.mark.gpu


def make(models, cache, featurizer="feedforward"):
    from pet_kokkos_b200 import Calculator
    return Calculator(*models("tiny", featurizer, "scaled", 3), cache_neighbors=cache)


def close(a, b):
    scale = max(np.abs(b.energy).max(), 1e-3)
    assert np.abs(a.energy - b.energy).max() <= 1e-6 * scale
    assert np.abs(a.forces - b.forces).max() <= 1e-5 * max(1.0, np.abs(b.forces).max())
    assert np.abs(a.virial - b.virial).max() <= 1e-5 * max(1.0, np.abs(b.virial).max())


def cluster(n, seed):
    s = st.water_box(n, 3.2 * n ** (1.0 / 3.0), seed=seed)
    return st.make_system(s["atomic_numbers"], s["positions"], np.eye(3) * 40.0, pbc=(False, False, False))


def slab(seed):
    s = st.diamond(2, jitter=0.05, seed=seed)
    return st.make_system(s["atomic_numbers"], s["positions"], s["cell"], pbc=(True, True, False))


def batch():
    return [st.diamond(2, jitter=0.05, seed=1), cluster(8, 2), slab(3), st.random_mixture(40, 8.0, seed=4)]


def staged(calc, systems, positions=None, cells=None, first=False):
    if first:
        calc.stage(systems)
    else:
        calc.update_staged(positions, cells)
    calc.compute_staged(True)
    return calc.fetch()


@pytest.mark.parametrize("featurizer", ["feedforward", "residual"])
def test_fresh_cache_equals_the_plain_search(models, featurizer):
    plain, cached = make(models, False, featurizer), make(models, True, featurizer)
    systems = batch()
    close(staged(cached, systems, first=True), staged(plain, systems, first=True))
    assert cached.neighbor_searches == 1 and cached.neighbor_reuses == 0
    assert plain.neighbor_searches == 0
    plain.close(), cached.close()


def test_small_moves_reuse_the_pairs_and_large_ones_search_again(models):
    plain, cached = make(models, False), make(models, True)
    systems = batch()
    staged(cached, systems, first=True), staged(plain, systems, first=True)
    x0 = np.concatenate([s["positions"] for s in systems])
    rng = np.random.default_rng(0)
    x = x0.copy()
    for step in range(4):  # 0.1 A per step per atom at most: 2 d stays under the 1 A skin for four steps
        move = rng.normal(size=x.shape)
        x = x + 0.1 * move / np.linalg.norm(move, axis=1, keepdims=True)
        close(staged(cached, systems, x), staged(plain, systems, x))
    assert cached.neighbor_searches == 1 and cached.neighbor_reuses == 4
    x[5] += [0.0, 0.7, 0.0]  # one atom 0.7 A further: 2 d > 1 A
    close(staged(cached, systems, x), staged(plain, systems, x))
    assert cached.neighbor_searches == 2
    close(staged(cached, systems, x), staged(plain, systems, x))  # the new reference frame: nothing moved since
    assert cached.neighbor_searches == 2 and cached.neighbor_reuses == 5
    plain.close(), cached.close()


def test_an_atom_crossing_a_cell_face_keeps_its_pairs(models):
    """The cached shifts are in unwrapped terms (src/device_geometry.cpp:176-181)."""
    plain, cached = make(models, False), make(models, True)
    s = st.diamond(2, jitter=0.0, seed=0)
    x = s["positions"].copy()
    x[0] = [0.02, 0.02, 0.02]
    s = st.make_system(s["atomic_numbers"], x, s["cell"])
    staged(cached, [s], first=True), staged(plain, [s], first=True)
    x2 = x.copy()
    x2[0] = [-0.05, -0.04, 0.03]  # through two faces, 0.1 A away
    close(staged(cached, [s], x2), staged(plain, [s], x2))
    assert cached.neighbor_searches == 1 and cached.neighbor_reuses == 1
    plain.close(), cached.close()


def test_strain_counts_as_strain_not_as_moves(models):
    """A 1 % strain moves far atoms by more than the skin in Cartesian terms; the test takes it per cell
    (2 d + reach |D - I|_F < skin, src/device_geometry.cpp:253-261) and keeps the pairs."""
    plain, cached = make(models, False), make(models, True)
    s = st.diamond(3, jitter=0.05, seed=5)
    staged(cached, [s], first=True), staged(plain, [s], first=True)
    D = np.eye(3) + np.array([[0.01, 0.004, 0.0], [0.0, -0.008, 0.003], [0.002, 0.0, 0.006]])
    cell = s["cell"] @ D
    x = s["positions"] @ D
    assert np.abs(x - s["positions"]).max() > 0.1
    close(staged(cached, [s], x, cell[None]), staged(plain, [s], x, cell[None]))
    assert cached.neighbor_searches == 1 and cached.neighbor_reuses == 1
    big = np.eye(3) * 1.12  # reach |D - I|_F = 5.5 * 0.208 > 1 A
    close(staged(cached, [s], s["positions"] @ big, (s["cell"] @ big)[None]),
          staged(plain, [s], s["positions"] @ big, (s["cell"] @ big)[None]))
    assert cached.neighbor_searches == 2
    plain.close(), cached.close()


def test_staging_resets_the_cache(models):
    cached = make(models, True)
    s = st.diamond(2, jitter=0.05, seed=6)
    staged(cached, [s], first=True)
    staged(cached, [s], first=True)
    assert cached.neighbor_searches == 2 and cached.neighbor_reuses == 0
    cached.close()


def test_compute_on_the_same_atoms_keeps_the_cache(models):
    """An ASE-style loop: compute() on a structure whose atoms move a little each call (src/calculator.cpp:638-644)."""
    plain, cached = make(models, False), make(models, True)
    s = st.diamond(2, jitter=0.05, seed=7)
    rng = np.random.default_rng(2)
    for step in range(4):
        close(cached.compute(s), plain.compute(s))
        s = st.make_system(s["atomic_numbers"], s["positions"] + rng.normal(0, 0.02, s["positions"].shape), s["cell"])
    assert cached.neighbor_searches == 1 and cached.neighbor_reuses == 3
    other = st.make_system(np.where(np.arange(64) == 3, 14, s["atomic_numbers"]), s["positions"], s["cell"])
    close(cached.compute(other), plain.compute(other))  # another element somewhere: other atoms, a new search
    assert cached.neighbor_searches == 2
    close(cached.compute(st.diamond(1, jitter=0.02, seed=1)), plain.compute(st.diamond(1, jitter=0.02, seed=1)))
    assert cached.neighbor_searches == 3
    plain.close(), cached.close()


def test_adaptive_cutoff_over_cached_pairs(models, tmp_path):
    """Pairs past the model's cutoff weigh nothing in an atom's neighbour count, so the adaptive cutoffs come out the same."""
    from pet_kokkos_b200 import Calculator
    jp, sp = ck.write_random_checkpoint(tmp_path / "ad", "tiny", "feedforward", seed=5, init="scaled",
                                        num_neighbors_adaptive=16.0, adaptive_cutoff_method="solver", cutoff=5.5)
    plain, cached = Calculator(jp, sp), Calculator(jp, sp, cache_neighbors=True)
    systems = [st.diamond(2, jitter=0.08, seed=1), st.random_mixture(30, 8.0, seed=4)]
    close(staged(cached, systems, first=True), staged(plain, systems, first=True))
    x = np.concatenate([s["positions"] for s in systems])
    x = x + np.random.default_rng(1).normal(0, 0.03, x.shape)
    close(staged(cached, systems, x), staged(plain, systems, x))
    assert cached.neighbor_searches == 1 and cached.neighbor_reuses == 1
    plain.close(), cached.close()


def moved_systems(systems, x):
    out, at = [], 0
    for s in systems:
        n = s["n_atoms"]
        out.append(st.make_system(s["atomic_numbers"], x[at:at + n], s["cell"], pbc=tuple(s["pbc"])))
        at += n
    return out


def ref_close(r, ref):
    scale = max(np.abs(ref["energy"]).max(), 1e-3)
    assert np.abs(r.energy - ref["energy"]).max() <= 1e-6 * scale
    assert np.abs(r.forces - ref["forces"]).max() <= 1e-5 * max(1.0, np.abs(ref["forces"]).max())
    assert np.abs(r.virial - ref["virial"]).max() <= 1e-5 * max(1.0, np.abs(ref["virial"]).max())


@pytest.mark.parametrize("featurizer", ["feedforward", "residual"])
def test_cached_steps_match_the_reference_at_the_moved_positions(reference, models, featurizer):
    """The cached pairs' answers against the reference's own evaluation of the moved structures (its Calculator::compute
    on the host build), not only against this library's plain search."""
    cached = make(models, True, featurizer)
    rcalc = reference.ReferenceCalculator(*[str(p) for p in models("tiny", featurizer, "scaled", 3)])
    systems = batch()
    ref_close(staged(cached, systems, first=True), rcalc.compute(systems))
    x = np.concatenate([s["positions"] for s in systems])
    rng = np.random.default_rng(4)
    for _ in range(3):
        x = x + rng.normal(0, 0.04, x.shape)
        ref_close(staged(cached, systems, x), rcalc.compute(moved_systems(systems, x)))
    assert cached.neighbor_searches == 1 and cached.neighbor_reuses == 3
    cached.close()


def test_a_shrinking_batch_keeps_its_cached_pairs(reference, models):
    """A batched relaxation: structures finish one by one and the batch is packed to the front (the reference's
    geom.staged, include/pet/calculator.hpp:214-218; cache_reassemble, src/device_geometry.cpp:203-246). The structures
    that stay keep the positions they have on the device and their cached pairs, renumbered: no new search, and the
    answers are those of the reference for the remaining structures where they are now."""
    cached, plain = make(models, True), make(models, False)
    rcalc = reference.ReferenceCalculator(*[str(p) for p in models("tiny", "feedforward", "scaled", 3)])
    systems = batch()
    staged(cached, systems, first=True)
    x = np.concatenate([s["positions"] for s in systems])
    x = x + np.random.default_rng(5).normal(0, 0.03, x.shape)
    all4 = staged(cached, systems, x)
    assert cached.neighbor_searches == 1 and cached.neighbor_reuses == 1
    now = moved_systems(systems, x)
    # structure 1 is done; the others move on, 3 first
    keep = [3, 0, 2]
    cached.keep_staged(keep)
    cached.compute_staged(True)
    r = cached.fetch()
    kept = [now[k] for k in keep]
    ref_close(r, rcalc.compute(kept))
    close(r, plain.compute(kept))
    off = np.concatenate([[0], np.cumsum([s["n_atoms"] for s in systems])])
    for slot, k in enumerate(keep):  # and each structure's numbers are the ones it had in the whole batch
        assert abs(r.energy[slot] - all4.energy[k]) <= 1e-6 * max(abs(all4.energy[k]), 1e-3)
    assert cached.neighbor_searches == 1 and cached.neighbor_reuses == 2, "the pairs followed the structures"
    # stepping goes on in the smaller batch, and shrinking once more still needs no search
    x3 = np.concatenate([s["positions"] for s in kept])
    x3 = x3 + np.random.default_rng(6).normal(0, 0.03, x3.shape)
    ref_close(staged(cached, kept, x3), rcalc.compute(moved_systems(kept, x3)))
    cached.keep_staged([1])
    cached.compute_staged(True)
    ref_close(cached.fetch(), rcalc.compute([moved_systems(kept, x3)[1]]))
    assert cached.neighbor_searches == 1 and cached.neighbor_reuses == 4
    # without a cache the same call just restages the kept structures
    staged(plain, systems, first=True)
    plain.keep_staged([2])
    plain.compute_staged(True)
    ref_close(plain.fetch(), rcalc.compute([systems[2]]))
    with pytest.raises(ValueError):
        cached.keep_staged([0, 0])
    cached.close(), plain.close()
