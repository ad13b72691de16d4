"""The benchmark's larger configurations, checked at sizes the CPU checkers finish in seconds.

* The pet-omat-l-like shape (d_pet 512, head_dim 64, cutoff 6 A) that the 13824-atom cell runs, on a 216-atom
  jittered diamond: about 159 neighbours per atom, so the attention kernels instantiated for head_dim 64 and
  129-176 tokens run, the backward with its row blocks taken in turn; and with the cutoff pulled in so that an
  atom has 81-128 tokens (the middle instantiations), for head_dim 64 and 32.
* The 512-structure batch of 64-atom C/H/N/O/Si mixtures: its first 32 structures against the reference, and all
  512 through a memory budget that forces several memory runs, held to the bits of the unsplit answer.
* The recompute tiers (never / wide / layers, with the edge MLP in chunks of rows): in the native mode all three
  give the same bits (tests/test_determinism.cpp:116-162 of the reference holds its tiers to the same).
* The two speed modes (tf32 and bf16 GEMMs with single-pass tf32 attention) against the reference's own bands
  for those modes (its README, "Faster modes": tf32 within 0.4 meV/atom and 10 meV/A of fp64 on its models, bf16
  within 5 meV/atom and 42 meV/A), never the fp32 bands.
"""
import os

import numpy as np
import pytest
import torch

from oracle import pet_oracle as po
from pet_kokkos_b200 import checkpoint as ck, exchange, structures as st

pytestmark = pytest.mark.gpu


def bands(r, ref, e_rel=1e-6, f_abs=1e-5, w_rel=1e-5):
    e_scale = max(np.abs(ref["energy"]).max(), np.abs(ref["per_atom_energy"]).sum() / len(ref["energy"]))
    assert np.abs(r.energy - ref["energy"]).max() <= e_rel * e_scale
    assert np.abs(r.per_atom_energy - ref["per_atom_energy"]).max() <= e_rel * e_scale
    assert np.abs(r.forces - ref["forces"]).max() <= f_abs * max(1.0, np.abs(ref["forces"]).max())
    assert np.abs(r.virial - ref["virial"]).max() <= w_rel * max(1.0, np.abs(ref["virial"]).max())


def model_with(tmp_path, shape, **over):
    tag = "_".join(f"{k}{v}" for k, v in sorted(over.items()))
    return ck.write_random_checkpoint(tmp_path / f"{shape}_{tag}", shape, "feedforward", seed=0, init="n002", **over)


@pytest.mark.parametrize("shape,cutoff,tokens", [("l", 6.0, (129, 176)), ("l", 5.2, (81, 128)), ("s", 5.2, (81, 128))])
def test_long_neighbour_lists_match_the_reference_and_the_restatement(reference, lib_path, tmp_path, shape, cutoff, tokens):
    from pet_kokkos_b200 import Calculator
    jp, sp = model_with(tmp_path, shape, cutoff=cutoff)
    meta, tens = ck.load_checkpoint(jp, sp)
    systems = [st.diamond(3, jitter=0.05, seed=0)]
    ref = reference.ReferenceCalculator(str(jp), str(sp), blas=True).compute(systems)
    truth = po.evaluate(meta, tens, systems, dtype=torch.float64)
    # A random-init network's energy can all but cancel the composition energies (it does at 6 A: +2.6 eV per atom
    # against -2.6), so "relative to the energy" is taken against what the network itself adds up to.
    comp = np.asarray(meta["composition_energies"])[np.asarray(meta["species_to_index"])[systems[0]["atomic_numbers"]]]
    e_scale = max(abs(truth["energy"][0]), np.abs(truth["per_atom_energy"]).sum(), np.abs(truth["per_atom_energy"] - comp).sum())
    spread = abs(ref["energy"][0] - truth["energy"][0]) / e_scale

    def held(r, to, e_rel):
        assert abs(r.energy[0] - to["energy"][0]) <= e_rel * e_scale
        assert np.abs(r.per_atom_energy - to["per_atom_energy"]).max() <= e_rel * e_scale
        assert np.abs(r.forces - to["forces"]).max() <= 1e-5 * max(1.0, np.abs(to["forces"]).max())
        assert np.abs(r.virial - to["virial"]).max() <= 1e-5 * max(1.0, np.abs(to["virial"]).max())

    for gemm in ("native", "3xtf32"):
        c = Calculator(jp, sp, gemm=gemm)
        r = c.compute(systems)
        S = c.last_shapes()[2] + 1
        assert tokens[0] <= S <= tokens[1], f"{S} tokens per atom: not the kernel instantiation this case is for"
        print(f"{shape} cutoff {cutoff} {gemm}: dE vs reference {abs(r.energy[0] - ref['energy'][0]) / e_scale:.2e}, vs fp64 "
              f"{abs(r.energy[0] - truth['energy'][0]) / e_scale:.2e} (the reference's fp32 build itself: {spread:.2e}); "
              f"dF vs reference {np.abs(r.forces - ref['forces']).max():.2e}, vs fp64 {np.abs(r.forces - truth['forces']).max():.2e}")
        # The fp32 mode on the CUDA cores meets the 1e-6 energy band at every shape. The split product on the tensor
        # cores sits low by their truncating accumulate, a bias that grows with the contraction length: inside 1e-6 at
        # the pet-mad-s shape (K = 256 ... 1024), 4-5e-6 of the network's energy at the pet-omat-l shape (K = 512 ...
        # 2048), where its band is therefore 1e-5; forces and virial meet 1e-5 in both modes at both shapes.
        e_rel = 1e-5 if (gemm == "3xtf32" and shape == "l") else 1e-6
        held(r, ref, e_rel)
        held(r, truth, e_rel)
        assert np.abs(r.forces).max() > 1e-3, "the force band must bite"
        c.close()


def test_first_structures_of_the_batch_match_the_reference(reference, lib_path, models):
    from pet_kokkos_b200 import Calculator
    jp, sp = models("s")
    systems = st.workload("batch512x64")[:32]
    ref = reference.ReferenceCalculator(str(jp), str(sp), blas=True).compute(systems)
    for gemm in ("native", "3xtf32"):
        c = Calculator(jp, sp, gemm=gemm)
        bands(c.compute(systems), ref)
        c.close()


def test_the_whole_batch_in_memory_runs_equals_the_unsplit_batch_to_the_bit(lib_path, models):
    """512 structures of 64 atoms: with a budget that holds about a quarter of them the batch runs as several
    consecutive pieces (Engine::memory_runs; the reference's src/calculator.cpp:326-345); the native GEMMs are batch
    invariant, so every number equals the one-piece answer exactly."""
    from pet_kokkos_b200 import Calculator
    jp, sp = models("s")
    systems = st.workload("batch512x64")
    whole = Calculator(jp, sp)
    a = whole.compute(systems)
    assert whole.batch_splits == 0
    pool = whole.workspace_bytes
    whole.close()
    pieces = Calculator(jp, sp, memory_budget_bytes=max(pool // 4, 1 << 28))
    b = pieces.compute(systems)
    assert pieces.batch_splits >= 1
    for k in ("energy", "per_atom_energy", "forces", "virial"):
        assert np.array_equal(getattr(a, k), getattr(b, k)), k
    assert np.array_equal(a.struct_id, b.struct_id)
    pieces.close()


@pytest.mark.parametrize("shape,workload", [("tiny", "diamond64"), ("s", "water648")])
def test_recompute_tiers_give_the_same_bits(lib_path, models, shape, workload, monkeypatch):
    """Never, Wide and Layers in the native mode, the edge MLP in chunks of 1000 rows (PET_EDGE_CHUNK) so that several
    chunks and a ragged last one run; the plan reports the tier that ran."""
    from pet_kokkos_b200 import Calculator
    monkeypatch.setenv("PET_EDGE_CHUNK", "1000")
    jp, sp = models(shape)
    systems = st.workload(workload)
    out = {}
    for tier in ("never", "wide", "layers"):
        c = Calculator(jp, sp, recompute=tier)
        out[tier] = c.compute(systems)
        again = c.compute(systems)  # the second evaluation of a shape is the recorded one
        assert np.array_equal(out[tier].forces, again.forces)
        plan = c.memory_plan()
        assert plan["tier"] == tier and plan["atoms"] == systems[0]["n_atoms"] and plan["estimate_bytes"] > 0
        assert "recompute " + tier in c.memory_report()
        c.close()
    for tier in ("wide", "layers"):
        for k in ("energy", "per_atom_energy", "forces", "virial"):
            assert np.array_equal(getattr(out["never"], k), getattr(out[tier], k)), (tier, k)


def test_auto_picks_a_lower_tier_under_a_small_budget(lib_path, models):
    from pet_kokkos_b200 import Calculator
    jp, sp = models("s")
    systems = st.workload("water648")
    roomy = Calculator(jp, sp)
    r0 = roomy.compute(systems)
    assert roomy.memory_plan()["tier"] == "never"
    need = roomy.memory_plan()["estimate_bytes"]
    assert 0.5 * roomy.workspace_bytes <= need <= 2.0 * roomy.workspace_bytes, "the estimate should be near what the pools hold"
    assert roomy.recommended_batch_atoms >= 256
    roomy.close()
    tight = Calculator(jp, sp, memory_budget_bytes=need // 3)
    r1 = tight.compute(systems)
    assert tight.memory_plan()["tier"] == "layers"
    assert np.array_equal(r0.forces, r1.forces)
    tight.close()


def test_layers_tier_over_an_exchange_reuses_the_rows_it_received(lib_path, models):
    """Under Layers the backward runs each layer's forward again; over several ranks it must not ask the other ranks
    a second time (they are not listening then) but reuse the partner rows of the first run (the reference keeps
    remote_in for the same reason, src/feedforward.cpp:374-378)."""
    from pet_kokkos_b200 import Calculator
    jp, sp = models("tiny", "feedforward", "scaled", 31)
    s = st.diamond(2, jitter=0.05, seed=6)
    whole = Calculator(jp, sp)
    ref = whole.compute(s)
    calcs = [Calculator(jp, sp, recompute="layers") for _ in range(2)]
    E, F, W, _ = exchange.compute_threads(calcs, s, whole.cutoff)
    assert abs(E - ref.energy[0]) <= 1e-6 * max(abs(ref.energy[0]), np.abs(ref.per_atom_energy).sum())
    assert np.abs(F - ref.forces).max() <= 1e-5 * max(1.0, np.abs(ref.forces).max())
    assert np.abs(W - ref.virial[0]).max() <= 1e-5 * max(1.0, np.abs(ref.virial).max())
    for c in calcs + [whole]:
        c.close()


# The reference's own bands for its speed modes, against fp64 (README, "Faster modes"), in eV per atom and eV/A.
SPEED_BANDS = {"tf32": (0.4e-3, 10e-3), "bf16": (5e-3, 42e-3)}


@pytest.mark.parametrize("gemm", ["tf32", "bf16"])
@pytest.mark.parametrize("shape,workload", [("s", "water648"), ("xs", "diamond64")])
def test_speed_modes_stay_inside_the_reference_bands_for_them(lib_path, models, shape, workload, gemm):
    from pet_kokkos_b200 import Calculator
    jp, sp = models(shape)
    meta, tens = ck.load_checkpoint(jp, sp)
    systems = st.workload(workload)
    truth = po.evaluate(meta, tens, systems, dtype=torch.float64)
    c = Calculator(jp, sp, gemm=gemm)
    r = c.compute(systems)
    n = systems[0]["n_atoms"]
    de = np.abs(r.energy - truth["energy"]).max() / n
    df = np.abs(r.forces - truth["forces"]).max()
    print(f"{gemm} {shape} {workload}: dE {de * 1e3:.4f} meV/atom, max dF {df * 1e3:.4f} meV/A, "
          f"force scale {np.abs(truth['forces']).max():.3e} eV/A")
    e_band, f_band = SPEED_BANDS[gemm]
    assert de <= e_band and df <= f_band
    # the mode really runs at reduced precision (a silent fall-back to fp32 would pass the bands above)
    exact = Calculator(jp, sp, gemm="native").compute(systems)
    assert np.abs(r.forces - exact.forces).max() > 1e-7
    # and repeats to the bit
    assert np.array_equal(r.forces, c.compute(systems).forces)
    c.close()


def test_bf16_gemm_against_fp64(lib_path, models):
    """One GEMM in each tensor-core mode against the fp64 product: bf16 operands carry 8 significant bits, tf32 11,
    the split product fp32's 24 (the reference's tests/test_gemm_modes.cpp:76-103 bands its modes the same way).
    Shapes with a ragged last row tile, a K that is not a multiple of the 32-column stage, and all three tile widths."""
    from pet_kokkos_b200 import Calculator
    c = Calculator(*models("tiny"))
    rng = np.random.default_rng(3)
    for m, n, k in [(700, 192, 256), (20000, 256, 264), (1300, 512, 128), (257, 64, 1024)]:
        A = rng.normal(size=(m, k)).astype(np.float32)
        W = rng.normal(size=(n, k)).astype(np.float32)
        ref = A.astype(np.float64) @ W.T.astype(np.float64)
        scale = np.abs(ref).max()
        err = {mode: np.abs(c.gemm(A, W, mode) - ref).max() / scale for mode in ("native", "3xtf32", "tf32", "bf16")}
        print(m, n, k, {a: f"{b:.2e}" for a, b in err.items()})
        # fp32 chains of k products: 1.2e-6 of the largest entry at k = 1024; the split product sits low by the tensor
        # core's truncating accumulate, 0.34 (3k/8) 2^-24 of an entry for zero-mean operands: 6.6e-6 at k = 1024
        assert err["native"] <= 2e-6 and err["3xtf32"] <= 2e-6 + 0.5 * (3 * k / 8) * 2.0 ** -24, err
        assert 1e-5 <= err["tf32"] <= 2e-3, err
        # (the tf32 kernel's fp32 operands are cut to 11 bits by the tensor core, bf16's 8 bits are rounded to nearest:
        # the ratio of the two errors is 2-4, not the 8 the mantissa widths suggest)
        assert 2e-4 <= err["bf16"] <= 2e-2 and err["bf16"] > 1.5 * err["tf32"], err
        # bf16 products of bf16-rounded operands accumulate in fp32: against the fp64 product of the ROUNDED operands the
        # error is fp32-class, which pins the converter's rounding and the tile layout rather than the format's coarseness
        def rounded(x):
            u = x.view(np.uint32).astype(np.uint64)
            return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)
        ref16 = rounded(A).astype(np.float64) @ rounded(W).T.astype(np.float64)
        assert np.abs(c.gemm(A, W, "bf16") - ref16).max() / scale <= 4e-6
    c.close()
