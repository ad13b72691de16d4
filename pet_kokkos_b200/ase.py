"""ASE front end: `PETCalculator` plugs a `pet_kokkos_b200.Calculator` into `ase.Atoms`.

It answers ASE's energy / free_energy / energies / forces / stress requests from one evaluation on the GPU
(the role python/pet_kokkos/ase.py plays in the reference). Relaxations and MD call it again and again on the same
atoms, so the Verlet neighbour cache is on unless the caller turns it off.

    from pet_kokkos_b200.ase import PETCalculator
    atoms.calc = PETCalculator("models/pet-mad-s")          # path prefix, or json and safetensors paths
    energy, forces, stress = atoms.get_potential_energy(), atoms.get_forces(), atoms.get_stress()

ASE is imported here, at import time; without it this module cannot be imported.
"""
import numpy as np
from ase.calculators import calculator as _ase

from . import calculator as _native
from .structures import make_system


def virial_to_ase_stress(virial6, volume):
    """xx yy zz xy xz yz (this library's order) -> ASE's xx yy zz yz xz xy, per volume."""
    xx, yy, zz, xy, xz, yz = (float(v) for v in virial6)
    return np.array([xx, yy, zz, yz, xz, xy]) / volume


class PETCalculator(_ase.Calculator):
    implemented_properties = ["energy", "free_energy", "energies", "forces", "stress"]

    def __init__(self, model, model_weights=None, *, cache_neighbors=True, **options):
        _ase.Calculator.__init__(self)
        self.pet = _native.Calculator(model, model_weights, cache_neighbors=cache_neighbors, **options)

    def calculate(self, atoms=None, properties=("energy",), system_changes=_ase.all_changes):
        _ase.Calculator.calculate(self, atoms, properties, system_changes)
        a = self.atoms
        periodic = [bool(flag) for flag in a.pbc]
        lattice = np.array(a.cell.array, dtype=np.float64) if any(periodic) else np.zeros((3, 3))
        gradients = "forces" in properties or "stress" in properties
        out = self.pet.compute(make_system(a.numbers, a.positions, lattice, pbc=tuple(periodic)), compute_forces=gradients)
        found = {"energy": float(out.energy[0]), "energies": np.array(out.per_atom_energy)}
        found["free_energy"] = found["energy"]
        if gradients:
            found["forces"] = np.array(out.forces)
            if all(periodic):  # a stress needs a volume
                found["stress"] = virial_to_ase_stress(out.virial[0], a.get_volume())
        self.results.update(found)
