"""ctypes access to the reference's own evaluator, compiled for the host by build_ref.sh.

TEST INFRASTRUCTURE ONLY. `oracle/_ref/libpet_ref.so` is peterspackman/pet-kokkos's
unmodified src/*.cpp (calculator.cpp, model.cpp, feedforward.cpp, residual.cpp,
attention.cpp, ops.cpp, forces.cpp, device_geometry.cpp, device_cell_list.cpp,
device_neighbors.cpp, neighbors.cpp, checkpoint.cpp ...) built with g++ against the
host stand-in for Kokkos in oracle/kokkos_host/, behind the C entry layer in
oracle/ref_driver.cpp. It is the checker the restatement in pet_oracle.py and the CUDA
path are compared with, and the timed CPU baseline; the product never loads it.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libpet_ref.so")
# The reference's PET_HAVE_CBLAS build: same sources, GEMMs through a BLAS (the timed CPU baseline).
BLAS_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libpet_ref_blas.so")

_c_int, _c_dbl, _c_vp, _c_cp, _c_sz = ctypes.c_int, ctypes.c_double, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t


def available() -> bool:
    return os.path.exists(LIB_PATH)


def find_reference_root():
    """A checkout of the reference to compile from: $PET_REFERENCE_ROOT, else a `reference` folder beside this
    repository. None where there is none (the library then has to come prebuilt)."""
    here = os.path.dirname(os.path.abspath(__file__))
    for root in (os.environ.get("PET_REFERENCE_ROOT"), os.path.join(here, "..", "..", "reference")):
        if root and os.path.exists(os.path.join(root, "src", "calculator.cpp")):
            return os.path.abspath(root)
    return None


def build(reference_root=None, force=False) -> bool:
    """Runs build_ref.sh when a reference checkout is at hand; True if the library exists afterwards."""
    import subprocess
    root = reference_root or find_reference_root()
    if root and (force or not available()):
        script = os.path.join(os.path.dirname(os.path.abspath(__file__)), "build_ref.sh")
        subprocess.run(["bash", script, root], check=True)
    return available()


_libs = {}


def find_blas():
    """(path, symbol prefix) of an optimised BLAS with the CBLAS entries in this image: the OpenBLAS that the
    scipy wheel carries (LP64, its symbols prefixed scipy_)."""
    import glob
    import scipy
    for p in sorted(glob.glob(os.path.join(os.path.dirname(scipy.__file__), "..", "scipy.libs", "libscipy_openblas*.so"))):
        if "64_" not in os.path.basename(p):
            return os.path.abspath(p), "scipy_"
    raise RuntimeError("no BLAS with a CBLAS interface found in this image")


def _load(blas=False):
    if blas not in _libs:
        path = BLAS_LIB_PATH if blas else LIB_PATH
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is not built: run oracle/build_ref.sh <reference-root>")
        lib = ctypes.CDLL(path)
        if blas:
            bpath, prefix = find_blas()
            if lib.petref_bind_blas(bpath.encode(), prefix.encode()) != 0:
                raise RuntimeError(f"could not bind cblas_sgemm/cblas_dgemm from {bpath}")
        lib.petref_create.restype = _c_vp
        lib.petref_create.argtypes = [_c_cp, _c_cp, _c_int, _c_int, _c_cp, _c_sz]
        lib.petref_destroy.argtypes = [_c_vp]
        for name in ("petref_cutoff", "petref_ghost_cutoff", "petref_energy_scale"):
            getattr(lib, name).restype = _c_dbl
            getattr(lib, name).argtypes = [_c_vp]
        lib.petref_compute.argtypes = [_c_vp, _c_int] + [_c_vp] * 5 + [_c_int] + [_c_vp] * 4 + [_c_cp, _c_sz]
        lib.petref_compute_edges.argtypes = ([_c_vp, _c_int, _c_int] + [_c_vp] * 6 + [_c_int] * 3 + [_c_vp] * 5
                                             + [_c_cp, _c_sz])
        lib.petref_steps.argtypes = ([_c_vp, _c_int, _c_int] + [_c_vp] * 6 + [_c_int, _c_int] + [_c_vp] * 4
                                     + [_c_cp, _c_sz])
        lib.petref_device_edges.argtypes = [_c_vp, _c_int] + [_c_vp] * 13 + [_c_cp, _c_sz]
        lib.petref_host_raw_edges.argtypes = ([_c_int] + [_c_vp] * 4 + [_c_dbl, _c_int] + [_c_vp] * 6
                                              + [_c_cp, _c_sz])
        _libs[blas] = lib
    return _libs[blas]


def set_threads(n: int, blas: bool = True) -> int:
    """Gives the reference's OpenMP kernels and its BLAS `n` host threads, whatever OMP_NUM_THREADS the process
    inherited (torchrun exports OMP_NUM_THREADS=1 to its ranks), and returns the OpenMP thread count in force."""
    _load(blas)
    omp = ctypes.CDLL("libgomp.so.1")
    omp.omp_set_num_threads(int(n))
    if blas:
        path, prefix = find_blas()
        ob = ctypes.CDLL(path)
        getattr(ob, prefix + "openblas_set_num_threads")(int(n))
    return int(omp.omp_get_max_threads())


def _ptr(a):
    return None if a is None else a.ctypes.data


def _pack(systems):
    n_atoms = np.array([s["n_atoms"] for s in systems], np.int32)
    Z = np.ascontiguousarray(np.concatenate([s["atomic_numbers"] for s in systems]), np.int32)
    pos = np.ascontiguousarray(np.concatenate([s["positions"].reshape(-1, 3) for s in systems]), np.float64)
    cells = np.ascontiguousarray(np.stack([np.asarray(s["cell"], np.float64).reshape(9) for s in systems]))
    pbc = np.ascontiguousarray(np.stack([np.asarray(s["pbc"]).astype(np.int32) for s in systems]), np.int32)
    return n_atoms, Z, pos, cells, pbc


class ReferenceCalculator:
    """pet::Calculator of the reference (include/pet/calculator.hpp:174-319), on the host."""

    def __init__(self, model_json: str, model_weights: str, device_neighbors: bool = True, builtin_search: bool = True,
                 blas: bool = False):
        self._lib = _load(blas)
        err = ctypes.create_string_buffer(2048)
        self._h = self._lib.petref_create(model_json.encode(), model_weights.encode(), int(device_neighbors),
                                          int(builtin_search), err, len(err))
        if not self._h:
            raise RuntimeError(err.value.decode())

    def close(self):
        if getattr(self, "_h", None):
            self._lib.petref_destroy(self._h)
            self._h = None

    __del__ = close

    @property
    def cutoff(self):
        return self._lib.petref_cutoff(self._h)

    @property
    def ghost_cutoff(self):
        return self._lib.petref_ghost_cutoff(self._h)

    @property
    def energy_scale(self):
        return self._lib.petref_energy_scale(self._h)

    def compute(self, systems, forces: bool = True):
        """Calculator::compute on one structure or a batch (calculator.hpp:187,192)."""
        if isinstance(systems, dict):
            systems = [systems]
        n_atoms, Z, pos, cells, pbc = _pack(systems)
        B, N = len(systems), int(n_atoms.sum())
        out = {"energy": np.zeros(B), "per_atom_energy": np.zeros(N), "forces": np.zeros((N, 3)),
               "virial": np.zeros((B, 6))}
        err = ctypes.create_string_buffer(2048)
        rc = self._lib.petref_compute(self._h, B, _ptr(n_atoms), _ptr(Z), _ptr(pos), _ptr(cells), _ptr(pbc), int(forces),
                                      _ptr(out["energy"]), _ptr(out["per_atom_energy"]), _ptr(out["forces"]),
                                      _ptr(out["virial"]), err, len(err))
        if rc:
            raise RuntimeError(err.value.decode())
        return out

    @staticmethod
    def _list_args(lst):
        pos = np.ascontiguousarray(lst["positions"], np.float64)
        Z = np.ascontiguousarray(lst["atomic_numbers"], np.int32)
        off = np.ascontiguousarray(lst["offsets"], np.int32)
        nbr = np.ascontiguousarray(lst["neighbors"], np.int32)
        sh = None if lst.get("shifts") is None else np.ascontiguousarray(lst["shifts"], np.int32)
        cell = None if lst.get("cell") is None else np.ascontiguousarray(np.asarray(lst["cell"], np.float64).reshape(9))
        return pos, Z, off, nbr, sh, cell

    def compute_edges(self, lst, forces: bool = True, edge_gradients: bool = True):
        """Calculator::compute_edges (calculator.hpp:227) on an engine's own list (EdgeListView)."""
        pos, Z, off, nbr, sh, cell = self._list_args(lst)
        N, P = len(Z), len(nbr)
        out = {"energy": np.zeros(1), "per_atom_energy": np.zeros(N), "forces": np.zeros((N, 3)),
               "virial": np.zeros((1, 6)), "edge_gradient": np.zeros((P, 3))}
        err = ctypes.create_string_buffer(2048)
        rc = self._lib.petref_compute_edges(self._h, N, int(lst.get("n_local", -1)), _ptr(pos), _ptr(Z), _ptr(off),
                                            _ptr(nbr), _ptr(sh), _ptr(cell), int(bool(lst.get("half", False))),
                                            int(forces), int(edge_gradients), _ptr(out["energy"]),
                                            _ptr(out["per_atom_energy"]), _ptr(out["forces"]), _ptr(out["virial"]),
                                            _ptr(out["edge_gradient"]), err, len(err))
        if rc:
            raise RuntimeError(err.value.decode())
        return out

    def steps(self, lst, positions):
        """set_neighbors once, then compute_step per row of positions [S, N, 3] (calculator.hpp:235,238)."""
        pos, Z, off, nbr, sh, cell = self._list_args(lst)
        positions = np.ascontiguousarray(positions, np.float64)
        S, N = positions.shape[0], len(Z)
        out = {"energy": np.zeros(S), "forces": np.zeros((S, N, 3)), "virial": np.zeros((S, 6))}
        err = ctypes.create_string_buffer(2048)
        rc = self._lib.petref_steps(self._h, N, int(lst.get("n_local", -1)), _ptr(pos), _ptr(Z), _ptr(off), _ptr(nbr),
                                    _ptr(sh), _ptr(cell), int(bool(lst.get("half", False))), S, _ptr(positions),
                                    _ptr(out["energy"]), _ptr(out["forces"]), _ptr(out["virial"]), err, len(err))
        if rc:
            raise RuntimeError(err.value.decode())
        return out

    def device_edges(self, systems):
        """The packed list of the reference's device search (build_device_batch, src/device_geometry.cpp),
        slot n*M+m: vec [N,M,3], dist, mask, cutoff factor, reverse slot, neighbour species."""
        if isinstance(systems, dict):
            systems = [systems]
        n_atoms, Z, pos, cells, pbc = _pack(systems)
        B = len(systems)
        N, M = _c_int(0), _c_int(0)
        err = ctypes.create_string_buffer(2048)
        args = [self._h, B, _ptr(n_atoms), _ptr(Z), _ptr(pos), _ptr(cells), _ptr(pbc)]
        rc = self._lib.petref_device_edges(*args, ctypes.addressof(N), ctypes.addressof(M), None, None, None, None, None,
                                           None, err, len(err))
        if rc:
            raise RuntimeError(err.value.decode())
        N, M = N.value, M.value
        out = {"N": N, "M": M, "vec": np.zeros((N, M, 3)), "dist": np.zeros((N, M)), "mask": np.zeros((N, M)),
               "cutoff": np.zeros((N, M), np.float32), "reverse": np.zeros((N, M), np.int32),
               "neigh_species": np.zeros((N, M), np.int32)}
        rc = self._lib.petref_device_edges(*args, None, None, _ptr(out["vec"]), _ptr(out["dist"]), _ptr(out["mask"]),
                                           _ptr(out["cutoff"]), _ptr(out["reverse"]), _ptr(out["neigh_species"]), err,
                                           len(err))
        if rc:
            raise RuntimeError(err.value.decode())
        return out


def host_raw_edges(system, cutoff: float):
    """detail::build_raw_edges (src/neighbors.cpp): every directed edge within the cutoff, brute force over images."""
    lib = _load()
    n_atoms, Z, pos, cells, pbc = _pack([system])
    cap, count = 1 << 16, _c_int(0)
    err = ctypes.create_string_buffer(2048)
    while True:
        i, j = np.zeros(cap, np.int32), np.zeros(cap, np.int32)
        sh, vec, dist = np.zeros((cap, 3), np.int32), np.zeros((cap, 3)), np.zeros(cap)
        rc = lib.petref_host_raw_edges(int(n_atoms[0]), _ptr(Z), _ptr(pos), _ptr(cells), _ptr(pbc), float(cutoff), cap,
                                       ctypes.addressof(count), _ptr(i), _ptr(j), _ptr(sh), _ptr(vec), _ptr(dist), err,
                                       len(err))
        if rc:
            raise RuntimeError(err.value.decode())
        if count.value <= cap:
            n = count.value
            return {"i": i[:n], "j": j[:n], "shift": sh[:n], "vec": vec[:n], "dist": dist[:n]}
        cap = count.value
