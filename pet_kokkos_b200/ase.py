"""An ASE calculator over pet_kokkos_b200.Calculator: the reference's python/pet_kokkos/ase.py.

    from pet_kokkos_b200.ase import PETCalculator
    atoms.calc = PETCalculator("models/pet-mad-s")        # a path prefix, or (json, safetensors)
    atoms.get_potential_energy(), atoms.get_forces(), atoms.get_stress()

For MD or a relaxation of the same atoms, cache_neighbors=True (the default here, as in the reference) keeps a
Verlet cache of the pairs between steps. Needs ASE, which this module imports when it is imported.
"""
import numpy as np
from ase.calculators.calculator import Calculator as _AseCalculator, all_changes

from .calculator import Calculator as _PET
from .structures import make_system

# This library's Voigt order is xx yy zz xy xz yz; ASE's is xx yy zz yz xz xy.
_TO_ASE_VOIGT = [0, 1, 2, 5, 4, 3]


class PETCalculator(_AseCalculator):
    implemented_properties = ["energy", "free_energy", "energies", "forces", "stress"]

    def __init__(self, model, model_weights=None, *, cache_neighbors=True, **options):
        super().__init__()
        self.pet = _PET(model, model_weights, cache_neighbors=cache_neighbors, **options)

    def calculate(self, atoms=None, properties=("energy",), system_changes=all_changes):
        super().calculate(atoms, properties, system_changes)
        atoms = self.atoms
        pbc = tuple(bool(p) for p in atoms.pbc)
        cell = np.asarray(atoms.cell.array, dtype=np.float64) if any(pbc) else np.zeros((3, 3))
        want_forces = any(p in properties for p in ("forces", "stress"))
        r = self.pet.compute(make_system(atoms.numbers, atoms.positions, cell, pbc=pbc), compute_forces=want_forces)
        self.results["energy"] = self.results["free_energy"] = float(r.energy[0])
        self.results["energies"] = np.array(r.per_atom_energy)
        if want_forces:
            self.results["forces"] = np.array(r.forces)
            if all(pbc):
                self.results["stress"] = np.asarray(r.virial[0])[_TO_ASE_VOIGT] / atoms.get_volume()
