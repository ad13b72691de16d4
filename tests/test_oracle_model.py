"""The network oracle: self-consistency (finite differences), goldens, checkpoint format."""
import copy
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import pet_oracle as po
from pet_kokkos_b200 import checkpoint as ck, structures as st

GOLDEN = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN))
import make_golden  # noqa: E402


@pytest.mark.parametrize("featurizer", ["feedforward", "residual"])
def test_forces_match_finite_differences(models, featurizer):
    """The reference's tests/test_fd.cpp:61-112 on the float64 oracle: F = -dE/dx by central differences."""
    meta, tens = ck.load_checkpoint(*models("tiny", featurizer, "scaled", 1))
    s = st.diamond(2, jitter=0.05, seed=0)
    r = po.evaluate(meta, tens, [s], dtype=torch.float64)
    h = 3e-5
    for i, c in [(0, 0), (17, 2), (40, 1)]:
        sp, sm = copy.deepcopy(s), copy.deepcopy(s)
        sp["positions"][i, c] += h
        sm["positions"][i, c] -= h
        ep = po.evaluate(meta, tens, [sp], dtype=torch.float64, forces=False)["energy"][0]
        em = po.evaluate(meta, tens, [sm], dtype=torch.float64, forces=False)["energy"][0]
        fd = -(ep - em) / (2 * h)
        assert abs(fd - r["forces"][i, c]) <= 1e-5 * max(1.0, abs(fd))


def test_virial_matches_strain_derivative(models):
    """tests/test_fd.cpp:114-162: W_ab = dE/d(eps_ab) under x -> x (I + eps)^T, symmetrised."""
    meta, tens = ck.load_checkpoint(*models("tiny", "feedforward", "scaled", 1))
    s = st.diamond(2, jitter=0.05, seed=0)
    W = po.evaluate(meta, tens, [s], dtype=torch.float64)["virial"][0]
    eps = 1e-5
    for (a, b), voigt in [((0, 0), 0), ((1, 1), 1), ((0, 1), 3), ((1, 2), 5)]:
        def energy(sign):
            e = np.eye(3)
            e[a, b] += sign * eps / (1 if a == b else 2)
            e[b, a] += 0 if a == b else sign * eps / 2
            s2 = copy.deepcopy(s)
            s2["positions"] = s["positions"] @ e.T
            s2["cell"] = s["cell"] @ e.T
            return po.evaluate(meta, tens, [s2], dtype=torch.float64, forces=False)["energy"][0]
        fd = (energy(1) - energy(-1)) / (2 * eps)
        assert abs(fd - W[voigt]) <= 1e-5 * max(1.0, abs(fd))


def test_float32_oracle_tracks_float64(models):
    meta, tens = ck.load_checkpoint(*models("tiny", "feedforward", "n002", 2))
    systems = [st.diamond(2, jitter=0.05, seed=1), st.water_box(20, 9.0, seed=2)]
    a = po.evaluate(meta, tens, systems, dtype=torch.float32)
    b = po.evaluate(meta, tens, systems, dtype=torch.float64)
    assert np.abs(a["energy"] - b["energy"]).max() <= 1e-6 * np.abs(b["energy"]).max()
    assert np.abs(a["forces"] - b["forces"]).max() <= 1e-5


@pytest.mark.parametrize("name", sorted(make_golden.CASES))
def test_oracle_reproduces_goldens(name, tmp_path):
    g = np.load(GOLDEN / f"{name}.npz")
    jp, sp, meta, tens, systems = make_golden.build_case(name, tmp_path)
    assert make_golden.weights_digest(tens) == str(g["digest"]), "the seeded weight generator drifted"
    r = po.evaluate(meta, tens, systems, dtype=torch.float64)
    np.testing.assert_allclose(r["energy"], g["energy"], rtol=1e-10)
    np.testing.assert_allclose(r["forces"], g["forces"], atol=1e-9)
    np.testing.assert_allclose(r["virial"], g["virial"], atol=1e-8)
    assert len(r["edges"]["center"]) == int(g["n_edges"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("name", sorted(make_golden.CASES))
def test_oracle_matches_the_reference_outputs(name, dtype, tmp_path):
    """The pin: the restatement against what the reference's own Calculator::compute returned on the same
    files and structures (ref_* in the fixtures, recorded by tests/golden/make_golden.py from the reference
    compiled for the host). Bands: energy 1e-6 relative, forces 1e-5 eV/A per eV/A of force scale, virial
    1e-5 of its scale."""
    g = np.load(GOLDEN / f"{name}.npz")
    jp, sp, meta, tens, systems = make_golden.build_case(name, tmp_path)
    r = po.evaluate(meta, tens, systems, dtype=dtype)
    assert np.abs(r["energy"] - g["ref_energy"]).max() <= 1e-6 * np.abs(g["ref_energy"]).max()
    assert np.abs(r["per_atom_energy"] - g["ref_per_atom_energy"]).max() <= 1e-6 * np.abs(g["ref_energy"]).max()
    assert np.abs(r["forces"] - g["ref_forces"]).max() <= 1e-5 * max(1.0, np.abs(g["ref_forces"]).max())
    assert np.abs(r["virial"] - g["ref_virial"]).max() <= 1e-5 * max(1.0, np.abs(g["ref_virial"]).max())


def test_checkpoint_roundtrip(tmp_path):
    """The writer's files read back with the reference's layout: u64 header length, JSON index, F32 data."""
    jp, sp = ck.write_random_checkpoint(tmp_path / "m", "tiny", seed=5)
    meta, tens = ck.load_checkpoint(jp, sp)
    h = meta["hypers"]
    assert h["d_node"] == 4 * h["d_pet"] and h["head_dim"] * h["num_heads"] == h["d_pet"]
    shapes = ck.tensor_shapes(h, meta["n_species"])
    assert set(shapes) == set(tens)
    for k, v in tens.items():
        assert tuple(v.shape) == tuple(shapes[k]) and v.dtype == np.float32
    raw = Path(sp).read_bytes()
    n = int.from_bytes(raw[:8], "little")
    import json
    idx = json.loads(raw[8:8 + n])
    assert idx["edge_embedder.weight"]["dtype"] == "F32"
    assert len(raw) == 8 + n + sum(v.size * 4 for v in tens.values())
