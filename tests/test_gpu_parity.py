"""Energy, forces and virial of the CUDA path against the CPU oracle and the committed goldens.

Tolerances (the north star's): energies 1e-6 relative, forces 1e-5 eV/A, virial
1e-5 relative to the virial's scale (the reference's own path-agreement tests use
1e-5 relative, tests/test_cell_list.cpp:186-189), all against the float64 oracle;
fp32 rounding of either fp32 path is inside those bands.
"""
import copy
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import pet_oracle as po
from pet_kokkos_b200 import checkpoint as ck, structures as st

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN))
import make_golden  # noqa: E402

E_REL, F_ABS, W_REL = 1e-6, 1e-5, 1e-5


def check(r, ref, f_abs=F_ABS):
    assert np.abs(r.energy - ref["energy"]).max() <= E_REL * np.abs(ref["energy"]).max()
    assert np.abs(r.per_atom_energy - ref["per_atom_energy"]).max() <= E_REL * np.abs(ref["energy"]).max()
    assert np.abs(r.forces - ref["forces"]).max() <= f_abs
    assert np.abs(r.virial - ref["virial"]).max() <= W_REL * max(1.0, np.abs(ref["virial"]).max())


@pytest.mark.parametrize("name", sorted(make_golden.CASES))
def test_goldens(name, tmp_path, lib_path):
    from pet_kokkos_b200 import Calculator
    if "res" in name:
        pytest.importorskip("pet_kokkos_b200")
    g = np.load(GOLDEN / f"{name}.npz")
    jp, sp, meta, tens, systems = make_golden.build_case(name, tmp_path)
    assert make_golden.weights_digest(tens) == str(g["digest"])
    c = Calculator(jp, sp)
    r = c.compute(systems)
    # forces here are O(10) eV/A for the "scaled" models: the absolute band is scaled accordingly
    scale = max(1.0, np.abs(g["forces"]).max())
    check(r, {k: g[k] for k in ("energy", "per_atom_energy", "forces", "virial")}, f_abs=F_ABS * scale)
    # and against the reference's own outputs on the same files (ref_*: Calculator::compute of the reference)
    check(r, {k: g["ref_" + k] for k in ("energy", "per_atom_energy", "forces", "virial")}, f_abs=F_ABS * scale)
    assert c.last_shapes()[1] == int(g["n_edges"]) and c.last_shapes()[2] == int(g["max_neighbors"])
    c.close()


@pytest.mark.parametrize("gemm", ["native", "3xtf32"])
@pytest.mark.parametrize("shape,workload", [("xs", "diamond64"), ("s", "water648"), ("s", "diamond1728")])
def test_benchmark_configs_match_oracle(models, lib_path, shape, workload, gemm):
    """Both fp32-accurate GEMM modes (CUDA cores; 3xTF32 split on the tensor cores) meet the parity band."""
    from pet_kokkos_b200 import Calculator
    jp, sp = models(shape)
    meta, tens = ck.load_checkpoint(jp, sp)
    systems = st.workload(workload)
    ref = po.evaluate(meta, tens, systems, dtype=torch.float64)
    c = Calculator(jp, sp, gemm=gemm)
    r = c.compute(systems)
    check(r, ref)
    assert np.abs(r.forces).max() > 100 * F_ABS, "the force tolerance must bite"
    c.close()


def test_bit_identical_repeats_and_batch_independence(models, lib_path):
    """tests/test_determinism.cpp:42-63,350-380: same bits run to run, and in a batch as alone (native GEMMs)."""
    from pet_kokkos_b200 import Calculator
    c = Calculator(*models("xs"))
    a, b = st.diamond(2, jitter=0.05, seed=0), st.random_mixture(64, 9.0, seed=3)
    r1, r2 = c.compute([a, b]), c.compute([a, b])
    for k in ("energy", "forces", "virial", "per_atom_energy"):
        assert (getattr(r1, k) == getattr(r2, k)).all()
    ra, rb = c.compute(a), c.compute(b)
    assert (r1.energy == np.concatenate([ra.energy, rb.energy])).all()
    assert (r1.forces == np.concatenate([ra.forces, rb.forces])).all()
    assert (r1.virial == np.concatenate([ra.virial, rb.virial])).all()
    c.close()


@pytest.mark.parametrize("gemm", ["native", "3xtf32"])
def test_graph_replay_gives_eager_bits(models, lib_path, gemm):
    """tests/test_determinism.cpp:238-254: a replayed recording returns the bits of the eager pass."""
    from pet_kokkos_b200 import Calculator
    jp, sp = models("xs")
    systems = [st.diamond(2, jitter=0.05, seed=0), st.random_mixture(40, 9.0, seed=1)]
    eager = Calculator(jp, sp, gemm=gemm, graphs=False)
    rec = Calculator(jp, sp, gemm=gemm, graphs=True)
    want = eager.compute(systems)
    got = [rec.compute(systems) for _ in range(5)]
    assert eager.graph_replays == 0 and rec.graph_replays >= 2
    for r in got:
        for k in ("energy", "per_atom_energy", "forces", "virial"):
            assert (getattr(r, k) == getattr(want, k)).all(), k
    # other shapes in between do not disturb a recording
    rec.compute(st.diamond(1))
    again = rec.compute(systems)
    assert (again.forces == want.forces).all()
    eager.close(), rec.close()


def test_forces_match_finite_differences_on_device(models, lib_path):
    """tests/test_fd.cpp:61-112 on the CUDA path: analytic forces against central differences of its own energies."""
    from pet_kokkos_b200 import Calculator
    c = Calculator(*models("tiny", "feedforward", "n002", 2))
    s = st.diamond(2, jitter=0.05, seed=0)
    F = c.compute(s).forces
    scale = np.abs(F).max()
    h = 1e-2  # fp32 energies: a large step, as the reference's sweep starts with
    for i, comp in [(0, 0), (17, 2), (40, 1)]:
        sp, sm = copy.deepcopy(s), copy.deepcopy(s)
        sp["positions"][i, comp] += h
        sm["positions"][i, comp] -= h
        fd = -(c.compute(sp, False).energy[0] - c.compute(sm, False).energy[0]) / (2 * h)
        assert abs(fd - F[i, comp]) <= 3e-3 * scale + 1e-5
    c.close()


def test_energy_only_equals_energy_with_forces(models, lib_path):
    """tests/test_golden.cpp:188-204: the forward alone gives the same energy bits."""
    from pet_kokkos_b200 import Calculator
    c = Calculator(*models("xs"))
    s = st.diamond(2, jitter=0.05, seed=0)
    assert (c.compute(s, False).energy == c.compute(s, True).energy).all()
    c.close()


def test_full_size_properties(models, lib_path):
    """At the benchmark's size: momentum conservation and invariance under a lattice translation and an atom permutation."""
    from pet_kokkos_b200 import Calculator
    c = Calculator(*models("s"))
    s = st.workload("diamond1728")[0]
    r = c.compute(s)
    assert np.abs(r.forces.sum(0)).max() <= 1e-5 * len(r.forces) ** 0.5
    moved = copy.deepcopy(s)
    moved["positions"] = s["positions"] + s["cell"][0] * 2 - s["cell"][2]
    r2 = c.compute(moved)
    assert abs(r2.energy[0] - r.energy[0]) <= E_REL * abs(r.energy[0])
    assert np.abs(r2.forces - r.forces).max() <= F_ABS
    perm = np.random.default_rng(0).permutation(s["n_atoms"])
    ps = st.make_system(s["atomic_numbers"][perm], s["positions"][perm], s["cell"])
    r3 = c.compute(ps)
    assert abs(r3.energy[0] - r.energy[0]) <= E_REL * abs(r.energy[0])
    assert np.abs(r3.forces - r.forces[perm]).max() <= F_ABS
    c.close()


def test_tf32_mode_is_a_speed_mode_within_its_band(models, lib_path):
    """tests/test_determinism.cpp:462-568 and README accuracy table: tf32 GEMMs stay within ~1e-3 eV/atom and 0.03 eV/A."""
    from pet_kokkos_b200 import Calculator
    jp, sp = models("s")
    systems = st.workload("water648")
    a = Calculator(jp, sp, gemm="native")
    b = Calculator(jp, sp, gemm="tf32")
    ra, rb = a.compute(systems), b.compute(systems)
    n = systems[0]["n_atoms"]
    assert abs(ra.energy[0] - rb.energy[0]) / n <= 1e-3
    assert np.abs(ra.forces - rb.forces).max() <= 0.03
    assert np.abs(ra.forces - rb.forces).max() > 1e-7  # it really is a different arithmetic
    a.close(), b.close()


def test_errors_are_reported(models, lib_path):
    from pet_kokkos_b200 import Calculator
    c = Calculator(*models("tiny"))
    bad = st.make_system([200], [[0, 0, 0]], np.eye(3) * 10)
    with pytest.raises(RuntimeError, match="unsupported atomic number"):
        c.compute(bad)
    r = c.compute(st.diamond(1))  # still usable afterwards
    assert np.isfinite(r.energy).all()
    c.close()


def test_a_converted_model_with_extra_heads_loads_and_the_extras_are_ignored(models, tmp_path):
    """A converted published model carries last-layer uncertainty and non-conservative heads next to the energy
    model (tools/convert_pet.py:342-420; src/checkpoint.cpp:122-135). This path evaluates the energy model: the
    extra json sections and tensors (float64 ones among them) do not change it."""
    import json
    from pet_kokkos_b200 import Calculator, checkpoint as ck
    jp, sp = models("tiny", "feedforward", "scaled", 4)
    meta = json.loads(open(jp).read())
    tens = ck.read_safetensors(sp)
    h = meta["hypers"]
    F = 2 * h.get("num_readout_layers", 1) * h["d_head"]
    rng = np.random.default_rng(0)
    tens = dict(tens)
    tens["llpr.energy.inv_cholesky"] = rng.normal(size=(F, F))  # float64, as the converter writes it
    tens["llpr.energy.ensemble"] = rng.normal(size=(4, F)).astype(np.float32)
    tens["non_conservative.forces.node_heads.0.0.weight"] = rng.normal(size=(h["d_head"], h["d_pet"])).astype(np.float32)
    meta["uncertainty"] = {"energy": {"features": F, "multiplier": 1.5, "ensemble": 4}}
    meta["non_conservative"] = {"force": {"scale": [0.25]}, "stress": {"scale": [2.0]}}
    jp2, sp2 = tmp_path / "extras.json", tmp_path / "extras.safetensors"
    jp2.write_text(json.dumps(meta))
    ck.write_safetensors(sp2, tens, keep_f64=True)
    assert ck.read_safetensors(sp2)["llpr.energy.inv_cholesky"].dtype == np.float64
    s = st.diamond(2, jitter=0.05, seed=3)
    a, b = Calculator(jp, sp), Calculator(jp2, sp2)
    ra, rb = a.compute(s), b.compute(s)
    assert ra.energy[0] == rb.energy[0] and np.array_equal(ra.forces, rb.forces) and np.array_equal(ra.virial, rb.virial)
    a.close(), b.close()


def test_a_batch_split_to_fit_memory_gives_the_answer_of_the_whole_batch(models, lib_path):
    """tests/test_determinism.cpp:116-162: compute() runs a batch too big for the device as consecutive pieces, by
    max_batch_atoms and by a memory budget so small that every structure goes alone; the pieces come back in order,
    struct_id counted over the whole batch, each structure as the whole batch had it (the native GEMMs are
    batch-invariant and attention is per atom, so here to the bit)."""
    from pet_kokkos_b200 import Calculator
    jp, sp = models("tiny", "feedforward", "scaled", 2)
    systems = [st.diamond(2, jitter=0.05, seed=1), st.water_box(9, 7.0, seed=2), st.diamond(1, jitter=0.02, seed=3),
               st.random_mixture(30, 7.5, seed=4), st.diamond(2, jitter=0.04, seed=5), st.water_box(5, 6.0, seed=6)]
    most = max(s["n_atoms"] for s in systems)
    whole_calc = Calculator(jp, sp)
    whole = whole_calc.compute(systems)
    assert whole_calc.batch_splits == 0
    for opts, pieces in ((dict(max_batch_atoms=2 * most), None), (dict(memory_budget_bytes=1), len(systems))):
        c = Calculator(jp, sp, **opts)
        split = c.compute(systems)
        assert c.batch_splits == 1
        assert split.n_atoms == whole.n_atoms and np.array_equal(split.struct_id, whole.struct_id)
        assert np.array_equal(split.energy, whole.energy) and np.array_equal(split.per_atom_energy, whole.per_atom_energy)
        assert np.array_equal(split.forces, whole.forces) and np.array_equal(split.virial, whole.virial)
        energy_only = c.compute(systems, compute_forces=False)
        assert np.array_equal(energy_only.energy, whole.energy)
        assert c.compute(systems[:1]).energy[0] == whole.energy[0] and c.batch_splits == 2  # one structure is never split
        c.close()
    whole_calc.close()


def test_out_of_memory_is_recovered_by_smaller_pieces(models, lib_path):
    """The failure is made on the host (an allocation of the scratch pools reports out of memory once): the pools
    are released, the batch cut in half and evaluated again, and the calculator stays usable."""
    from pet_kokkos_b200 import Calculator
    jp, sp = models("tiny", "feedforward", "scaled", 2)
    systems = [st.diamond(2, jitter=0.05, seed=s) for s in range(4)]
    c = Calculator(jp, sp)
    whole = c.compute(systems)
    big = [st.diamond(3, jitter=0.05, seed=s) for s in range(4)]  # larger: the pools have to grow
    want = c.compute(big)
    c.close()
    c = Calculator(jp, sp)
    c.fail_alloc(2)
    got = c.compute(big)
    assert c.oom_recoveries == 1 and c.batch_splits == 1
    assert np.array_equal(got.energy, want.energy) and np.array_equal(got.forces, want.forces)
    assert np.array_equal(got.struct_id, want.struct_id)
    again = c.compute(systems)  # the calculator stays usable, graphs and pools rebuilt
    assert np.array_equal(again.energy, whole.energy) and np.array_equal(again.forces, whole.forces)
    one = Calculator(jp, sp)
    one.fail_alloc(1)
    r = one.compute(big[0])  # one structure cannot be cut: released pools, the same pass again
    assert one.oom_recoveries == 1 and r.energy[0] == want.energy[0]
    one.close()
    c.fail_alloc(-1)
    c.close()


def test_two_devices_in_one_process(models, lib_path):
    """pet_options.device allows calculators on several GPUs in one process: the kernels' shared-memory opt-ins, the
    tensor-core path's error word and the SM count are per device, so the second device must work as the first does
    (with process-wide caches its attention and tcgen05 launches were refused as invalid). Needs two GPUs."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from pet_kokkos_b200 import Calculator
    jp, sp = models("s")
    s = st.workload("water648")
    for gemm in ("native", "3xtf32"):
        a, b = Calculator(jp, sp, gemm=gemm, device=0), Calculator(jp, sp, gemm=gemm, device=1)
        ra, rb = a.compute(s), b.compute(s)
        rb2, ra2 = b.compute(s), a.compute(s)  # interleaved: each call makes its own device current
        for k in ("energy", "forces", "virial"):
            assert np.array_equal(getattr(ra, k), getattr(rb, k)), (gemm, k)
            assert np.array_equal(getattr(ra, k), getattr(ra2, k)) and np.array_equal(getattr(rb, k), getattr(rb2, k))
        a.close(), b.close()


def test_a_steady_loop_stops_asking_the_driver_for_free_memory(lib_path, models):
    """Under Recompute::Auto every evaluation needs a memory budget. Asking the driver for it each time (cudaMemGetInfo,
    a call into the kernel-mode driver that waits behind its other clients) held one step in ten up for 50-100 ms on a
    shared box. The answer is kept while the calculator's pools keep their size: the same shapes again ask nothing,
    after a larger structure has grown the pools the next evaluation asks again."""
    from pet_kokkos_b200 import Calculator
    c = Calculator(*models("xs", "feedforward", "n002", 0))
    small, large = st.diamond(2, jitter=0.05, seed=0), st.diamond(3, jitter=0.05, seed=0)
    ref = c.compute(small)
    c.compute(small)
    asked = c.driver_memory_queries
    assert asked >= 1
    for _ in range(5):
        r = c.compute(small)
    assert c.driver_memory_queries == asked, "same shapes, same pools: nothing to ask"
    assert np.array_equal(r.forces, ref.forces) and r.energy[0] == ref.energy[0]
    c.compute(large)  # the pools grow during this evaluation ...
    c.compute(large)  # ... so the next one finds them changed and asks again
    assert c.driver_memory_queries > asked, "the pools grew: the cached answer is stale"
    c.close()
