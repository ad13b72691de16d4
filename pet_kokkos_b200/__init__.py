"""B200-native evaluator of PET energies, forces and virials behind the pet::Calculator interface."""
from .calculator import Calculator, EdgeListView, Results, load_library  # noqa: F401
