"""The ASE calculator (the reference's python/pet_kokkos/ase.py) over a stand-in for ASE's Calculator base class:
ASE itself is not installed where these tests run, and the adapter only needs the base class's bookkeeping."""
import sys
import types

import numpy as np
import pytest

from pet_kokkos_b200 import structures as st

pytestmark = pytest.mark.gpu


@pytest.fixture()
def fake_ase(monkeypatch):
    try:
        import ase.calculators.calculator  # noqa: F401  the real one, where there is one
        return
    except ImportError:
        pass

    class Base:
        def __init__(self):
            self.results, self.atoms = {}, None

        def calculate(self, atoms=None, properties=("energy",), system_changes=()):
            if atoms is not None:
                self.atoms = atoms
            self.results = {}

    mod = types.ModuleType("ase.calculators.calculator")
    mod.Calculator, mod.all_changes = Base, ["positions", "numbers", "cell", "pbc"]
    for name in ("ase", "ase.calculators"):
        monkeypatch.setitem(sys.modules, name, types.ModuleType(name))
    monkeypatch.setitem(sys.modules, "ase.calculators.calculator", mod)
    monkeypatch.delitem(sys.modules, "pet_kokkos_b200.ase", raising=False)


class Atoms:
    """What the adapter reads of ase.Atoms."""

    def __init__(self, s):
        self.numbers, self.positions, self.pbc, self.info = s["atomic_numbers"], s["positions"], s["pbc"], {}
        self.cell = types.SimpleNamespace(array=s["cell"])

    def get_volume(self):
        return abs(np.linalg.det(self.cell.array))


def test_energy_forces_and_stress_in_ase_terms(fake_ase, models):
    from pet_kokkos_b200 import Calculator
    from pet_kokkos_b200.ase import PETCalculator
    jp, sp = models("tiny", "feedforward", "scaled", 3)
    calc = PETCalculator(jp, sp)
    direct = Calculator(jp, sp)
    s = st.diamond(2, jitter=0.05, seed=4)
    atoms = Atoms(s)
    calc.calculate(atoms, ["energy", "forces", "stress"])
    ref = direct.compute(s)
    out = calc.results
    assert abs(out["energy"] - ref.energy[0]) <= 1e-6 * abs(ref.energy[0]) and out["free_energy"] == out["energy"]
    assert np.abs(out["forces"] - ref.forces).max() <= 1e-5 and out["energies"].shape == (64,)
    w = ref.virial[0]
    want = np.array([w[0], w[1], w[2], w[5], w[4], w[3]]) / atoms.get_volume()  # yz xz xy after the diagonal
    assert np.abs(out["stress"] - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
    # a relaxation's next steps: the same atoms, moved a little, served from the cached pairs
    for k in range(3):
        atoms.positions = atoms.positions + np.random.default_rng(k).normal(0, 0.02, atoms.positions.shape)
        calc.calculate(atoms, ["energy", "forces"])
    assert calc.pet.neighbor_searches == 1 and calc.pet.neighbor_reuses == 3
    # energy alone: no backward pass, no forces in the results; a cluster has no stress
    calc.calculate(atoms, ["energy"])
    assert "forces" not in calc.results
    c = st.water_box(6, 6.0, seed=1)
    c = st.make_system(c["atomic_numbers"], c["positions"], np.eye(3) * 30.0, pbc=(False, False, False))
    calc.calculate(Atoms(c), ["energy", "forces", "stress"])
    assert "stress" not in calc.results and calc.results["forces"].shape == (c["n_atoms"], 3)
    calc.pet.close(), direct.close()
