"""Python face of the C ABI (include/pet_b200.h) with the reference's Calculator interface.

Mirrors pet::Calculator (the reference's include/pet/calculator.hpp:174-319) and
its Python binding (python/core.cpp:366-390): `compute`, `compute_batch`,
`set_neighbors`, `compute_step`, `compute_edges`, same argument meaning, same
units, errors raised as the matching Python exception types.  Everything runs in
the CUDA library; there is no CPU path and loading fails loudly if the library
is missing.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np

_LIB_PATH = Path(__file__).resolve().parent / "libpet_b200.so"
_lib = None

GEMM_MODES = {"native": 0, "tf32": 1, "bf16": 2, "3xtf32": 3}
RECOMPUTE_TIERS = {"auto": 0, "never": 1, "wide": 2, "layers": 3}


class PetSystem(C.Structure):
    _fields_ = [("n_atoms", C.c_int), ("atomic_numbers", C.POINTER(C.c_int)), ("positions", C.POINTER(C.c_double)),
                ("cell", C.c_double * 9), ("pbc", C.c_int * 3), ("charge", C.c_int), ("spin_multiplicity", C.c_int)]


class PetOptions(C.Structure):
    _fields_ = [("device", C.c_int), ("gemm_mode", C.c_int), ("graphs", C.c_int), ("md_fixed_shapes", C.c_int),
                ("memory_budget_bytes", C.c_size_t), ("max_batch_atoms", C.c_int), ("cache_neighbors", C.c_int),
                ("recompute", C.c_int), ("reserved", C.c_int * 6)]


class PetMemoryPlan(C.Structure):
    _fields_ = [("atoms", C.c_int), ("max_neighbors", C.c_int), ("edges", C.c_long), ("tier", C.c_int),
                ("estimate_bytes", C.c_size_t), ("budget_bytes", C.c_size_t), ("pool_bytes", C.c_size_t)]


class PetResults(C.Structure):
    _fields_ = [("energy", C.POINTER(C.c_double)), ("per_atom_energy", C.POINTER(C.c_double)),
                ("forces", C.POINTER(C.c_double)), ("virial", C.POINTER(C.c_double)),
                ("struct_id", C.POINTER(C.c_int)), ("edge_gradient", C.POINTER(C.c_double))]


# pet_exchange's callbacks: device pointers and the calculator's stream arrive as integers.
SET_LIVE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p)
EDGES_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p)


class PetExchange(C.Structure):
    _fields_ = [("user", C.c_void_p), ("set_live", SET_LIVE_FN), ("edges", EDGES_FN)]


class PetEdgeList(C.Structure):
    _fields_ = [("n_atoms", C.c_int), ("n_local", C.c_int), ("positions", C.POINTER(C.c_double)),
                ("atomic_numbers", C.POINTER(C.c_int)), ("offsets", C.POINTER(C.c_int)),
                ("neighbors", C.POINTER(C.c_int)), ("shifts", C.POINTER(C.c_int)), ("cell", C.POINTER(C.c_double)),
                ("half", C.c_int), ("exchange", C.POINTER(PetExchange))]


class PetDeviceArrays(C.Structure):
    _fields_ = [("positions", C.c_void_p), ("forces", C.c_void_p), ("per_atom_energy", C.c_void_p),
                ("per_atom_virial", C.c_void_p), ("virial_scale", C.c_double)]


class PetDeviceEdgeList(C.Structure):
    _fields_ = [("n_atoms", C.c_int), ("n_local", C.c_int), ("n_centres", C.c_int), ("ilist", C.c_void_p),
                ("numneigh", C.c_void_p), ("neighbors", C.c_void_p), ("stride_i", C.c_long), ("stride_k", C.c_long),
                ("mask", C.c_int), ("atomic_numbers", C.c_void_p), ("image_of", C.c_void_p), ("positions", C.c_void_p),
                ("cell", C.POINTER(C.c_double)), ("exchange", C.c_void_p)]


class PetPairList(C.Structure):
    _fields_ = [("n_atoms", C.c_int), ("n_local", C.c_int), ("n_pairs", C.c_int), ("pairs", C.c_void_p),
                ("stride_pair", C.c_long), ("stride_col", C.c_long), ("atomic_numbers", C.c_void_p),
                ("renumber", C.c_void_p)]


class PetDeviceResults(C.Structure):
    _fields_ = [("n_atoms", C.c_int), ("energy", C.c_void_p), ("per_atom_energy", C.c_void_p), ("forces", C.c_void_p),
                ("virial", C.c_void_p)]


class PetDeviceGeom(C.Structure):
    _fields_ = [("n_structures", C.c_int), ("n_atoms", C.c_int), ("positions", C.c_void_p), ("cells", C.c_void_p),
                ("struct_id", C.c_void_p), ("stream", C.c_void_p)]


class PetTotals(C.Structure):
    _fields_ = [("energy", C.c_double), ("virial", C.c_double * 6)]


class PetProfileEntry(C.Structure):
    _fields_ = [("name", C.c_char * 32), ("launches", C.c_int), ("ms", C.c_double), ("flops", C.c_double),
                ("bytes", C.c_double)]


class PetRawEdges(C.Structure):
    _fields_ = [("capacity", C.c_int), ("n_edges", C.c_int), ("i", C.POINTER(C.c_int)), ("j", C.POINTER(C.c_int)),
                ("shift", C.POINTER(C.c_int)), ("vec", C.POINTER(C.c_double)), ("dist", C.POINTER(C.c_double)),
                ("reverse", C.POINTER(C.c_int)), ("cutoff", C.POINTER(C.c_float))]


# Every symbol include/pet_b200.h declares, with its ctypes signature.
_P = C.POINTER
SIGNATURES = {
    "pet_calc_create": (C.c_int, [C.c_char_p, C.c_char_p, _P(PetOptions), _P(C.c_void_p)]),
    "pet_calc_destroy": (None, [C.c_void_p]),
    "pet_last_error": (C.c_char_p, [C.c_void_p]),
    "pet_compute": (C.c_int, [C.c_void_p, _P(PetSystem), C.c_int, C.c_int, _P(PetResults)]),
    "pet_stage": (C.c_int, [C.c_void_p, _P(PetSystem), C.c_int]),
    "pet_compute_staged": (C.c_int, [C.c_void_p, C.c_int]),
    "pet_fetch_results": (C.c_int, [C.c_void_p, _P(PetResults)]),
    "pet_update_staged": (C.c_int, [C.c_void_p, _P(C.c_double), _P(C.c_double)]),
    "pet_compute_edges": (C.c_int, [C.c_void_p, _P(PetEdgeList), C.c_int, C.c_int, _P(PetResults)]),
    "pet_set_neighbors": (C.c_int, [C.c_void_p, _P(PetEdgeList)]),
    "pet_compute_step": (C.c_int, [C.c_void_p, _P(C.c_double), _P(C.c_double), C.c_int, C.c_int, _P(PetResults)]),
    "pet_compute_step_device": (C.c_int, [C.c_void_p, _P(PetDeviceArrays), _P(C.c_double), _P(PetTotals)]),
    "pet_set_neighbors_device": (C.c_int, [C.c_void_p, _P(PetDeviceEdgeList)]),
    "pet_compute_pairs": (C.c_int, [C.c_void_p, _P(PetPairList), C.c_void_p, _P(C.c_double), C.c_int,
                                    _P(PetDeviceResults)]),
    "pet_neighbor_list": (C.c_int, [C.c_void_p, _P(PetSystem), C.c_int, _P(PetRawEdges)]),
    "pet_cutoff": (C.c_double, [C.c_void_p]),
    "pet_ghost_cutoff": (C.c_double, [C.c_void_p]),
    "pet_exchange_ghost_cutoff": (C.c_double, [C.c_void_p]),
    "pet_energy_scale": (C.c_double, [C.c_void_p]),
    "pet_supports": (C.c_int, [C.c_void_p, C.c_int]),
    "pet_workspace_bytes": (C.c_size_t, [C.c_void_p]),
    "pet_last_shapes": (C.c_int, [C.c_void_p, _P(C.c_int), _P(C.c_int), _P(C.c_int)]),
    "pet_nccl_last_error": (C.c_char_p, []),
    "pet_exchange_schedule": (C.c_int, [_P(C.c_int), C.c_int, C.c_int, _P(C.c_int), _P(C.c_int), _P(C.c_int)]),
    "pet_nccl_unique_id": (C.c_int, [C.c_char_p]),
    "pet_nccl_exchange_create": (C.c_int, [C.c_char_p, C.c_int, C.c_int, C.c_int, _P(C.c_int), C.c_int, _P(C.c_int), C.c_int,
                                           C.c_int, _P(C.c_void_p)]),
    "pet_nccl_exchange_destroy": (None, [C.c_void_p]),
    "pet_nccl_exchange_callbacks": (C.c_void_p, [C.c_void_p]),
    "pet_nccl_exchange_reduce": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, _P(C.c_double)]),
    "pet_nccl_exchange_timing": (C.c_int, [C.c_void_p, C.c_int, _P(C.c_double), _P(C.c_int)]),
    "pet_staged_geometry": (C.c_int, [C.c_void_p, _P(PetDeviceGeom)]),
    "pet_keep_staged": (C.c_int, [C.c_void_p, _P(C.c_int), C.c_int]),
    "pet_device_results_of": (C.c_int, [C.c_void_p, _P(PetDeviceResults), _P(C.c_void_p)]),
    "pet_memory_plan": (C.c_int, [C.c_void_p, _P(PetMemoryPlan)]),
    "pet_memory_report": (C.c_int, [C.c_void_p, C.c_char_p, C.c_size_t]),
    "pet_recommended_batch_atoms": (C.c_int, [C.c_void_p]),
    "pet_kernel_launches": (C.c_longlong, [C.c_void_p]),
    "pet_last_device_ms": (C.c_double, [C.c_void_p]),
    "pet_graph_replays": (C.c_longlong, [C.c_void_p]),
    "pet_batch_splits": (C.c_longlong, [C.c_void_p]),
    "pet_oom_recoveries": (C.c_longlong, [C.c_void_p]),
    "pet_driver_memory_queries": (C.c_longlong, [C.c_void_p]),
    "pet_debug_fail_alloc": (None, [C.c_long]),
    "pet_neighbor_searches": (C.c_longlong, [C.c_void_p]),
    "pet_neighbor_reuses": (C.c_longlong, [C.c_void_p]),
    "pet_profile": (C.c_int, [C.c_void_p, C.c_int]),
    "pet_profile_read": (C.c_int, [C.c_void_p, _P(PetProfileEntry), C.c_int, _P(C.c_int)]),
    "pet_debug_fetch": (C.c_int, [C.c_void_p, C.c_char_p, _P(C.c_float), C.c_size_t, _P(C.c_size_t)]),
    "pet_gemm_host_static": (C.c_int, [C.c_int, C.c_int, C.c_int, _P(C.c_float), _P(C.c_float), _P(C.c_float), C.c_char_p,
                                       C.c_size_t]),
    "pet_gemm_host": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _P(C.c_float), _P(C.c_float),
                                _P(C.c_float)]),
}


def model_search_dirs():
    """Where a named model is looked for, in order (the reference's model_search_dirs, src/calculator.cpp:131-150):
    $PET_MODEL_DIR (':'-separated), ./models and ., $XDG_DATA_HOME/pet/models (else ~/.local/share/pet/models)."""
    dirs = [d for d in os.environ.get("PET_MODEL_DIR", "").split(":") if d] + ["models", "."]
    if os.environ.get("XDG_DATA_HOME"):
        dirs.append(os.path.join(os.environ["XDG_DATA_HOME"], "pet", "models"))
    elif os.environ.get("HOME"):
        dirs.append(os.path.join(os.environ["HOME"], ".local", "share", "pet", "models"))
    return dirs


def resolve_model(spec):
    """A model name or a path prefix to (<spec>.json, <spec>.safetensors) (resolve_model, src/calculator.cpp:152-166).
    This library ships no default model, so an empty spec is refused."""
    if not spec:
        raise ValueError("pet: no model given (this library ships no default model)")
    if "/" in spec or os.path.exists(spec + ".json"):
        return spec + ".json", spec + ".safetensors"
    for d in model_search_dirs():
        base = os.path.join(d, spec)
        if os.path.exists(base + ".json") and os.path.exists(base + ".safetensors"):
            return base + ".json", base + ".safetensors"
    raise RuntimeError(f"pet: model '{spec}' not found in {', '.join(model_search_dirs())}")


def load_library(path=None):
    """Loads libpet_b200.so and binds every declared entry point; raises if it is absent."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = Path(path) if path else _LIB_PATH
    if not p.exists():
        raise RuntimeError(f"{p} is missing: build it with `python -m pet_kokkos_b200.build` (no CPU fallback exists)")
    lib = C.CDLL(str(p))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    if path is None:
        _lib = lib
    return lib


_ERRORS = {1: RuntimeError, 2: ValueError, 3: RuntimeError, 4: MemoryError, 5: RuntimeError}


@dataclass
class Results:
    """pet::Results (calculator.hpp:120-142)."""
    energy: np.ndarray
    per_atom_energy: np.ndarray
    forces: np.ndarray | None = None
    virial: np.ndarray | None = None
    struct_id: np.ndarray | None = None
    n_atoms: list = field(default_factory=list)
    edge_gradient: np.ndarray | None = None


def _dptr(a):
    return a.ctypes.data_as(C.POINTER(C.c_double))


def _iptr(a):
    return a.ctypes.data_as(C.POINTER(C.c_int))


class _Packed:
    """ctypes pet_system array plus the numpy arrays that back its pointers."""

    def __init__(self, systems):
        self.keep = []
        self.arr = (PetSystem * max(len(systems), 1))()
        self.n = len(systems)
        self.n_atoms = []
        for b, s in enumerate(systems):
            z = np.ascontiguousarray(s["atomic_numbers"], dtype=np.int32)
            x = np.ascontiguousarray(s["positions"], dtype=np.float64).reshape(-1, 3)
            cell = np.ascontiguousarray(s.get("cell", np.zeros((3, 3))), dtype=np.float64).reshape(9)
            pbc = s.get("pbc", (False, False, False))
            if len(z) != len(x):
                raise ValueError("atomic_numbers and positions disagree on the atom count")
            self.keep += [z, x]
            ps = self.arr[b]
            ps.n_atoms = len(z)
            ps.atomic_numbers, ps.positions = _iptr(z), _dptr(x)
            for k in range(9):
                ps.cell[k] = cell[k]
            for k in range(3):
                ps.pbc[k] = int(bool(pbc[k]))
            ps.charge, ps.spin_multiplicity = int(s.get("charge", 0)), int(s.get("spin_multiplicity", 1))
            self.n_atoms.append(len(z))
        self.total = int(sum(self.n_atoms))


@dataclass
class EdgeListView:
    """pet::EdgeListView (device_geometry.hpp:93-110): an MD engine's own neighbour list."""
    positions: np.ndarray
    atomic_numbers: np.ndarray
    offsets: np.ndarray
    neighbors: np.ndarray
    shifts: np.ndarray | None = None
    cell: np.ndarray | None = None
    half: bool = False
    n_local: int = -1
    # pet::Exchange (include/pet/exchange.hpp:19-41) for a list whose ghosts are one cutoff deep: an object with
    # set_live(live_ptr, n_live, stream) and edges(out_ptr, in_ptr, n_live, width, stream); device pointers as ints.
    exchange: object | None = None


class Calculator:
    """A loaded model on one GPU.  Reuse one across calls: it holds the scratch pools."""

    def __init__(self, model_json, model_weights=None, gemm=None, device=-1, graphs=None, md_fixed_shapes=None,
                 cache_neighbors=None, memory_budget_bytes=0, max_batch_atoms=0, recompute=None):
        self._h = None
        self._lib = load_library()
        if model_weights is None:  # a path prefix or a model's name, as the reference's resolve_model accepts
            model_json, model_weights = resolve_model(str(model_json))
        o = PetOptions()
        o.device, o.gemm_mode, o.graphs, o.md_fixed_shapes = device, -1, -1, -1
        if gemm is not None:
            o.gemm_mode = GEMM_MODES[gemm] if isinstance(gemm, str) else int(gemm)
        if graphs is not None:
            o.graphs = int(bool(graphs))
        if md_fixed_shapes is not None:  # Options::md_fixed_shapes (calculator.hpp:111-116)
            o.md_fixed_shapes = int(bool(md_fixed_shapes))
        o.memory_budget_bytes, o.max_batch_atoms = int(memory_budget_bytes), int(max_batch_atoms)
        if recompute is not None:  # Options::recompute: "auto" | "never" | "wide" | "layers"
            o.recompute = RECOMPUTE_TIERS[recompute] if isinstance(recompute, str) else int(recompute)
        if cache_neighbors:  # Options::cache_neighbors (calculator.hpp:36-40): a Verlet cache for staged batches
            o.cache_neighbors = 1
        h = C.c_void_p()
        rc = self._lib.pet_calc_create(os.fsencode(model_json), os.fsencode(model_weights), C.byref(o), C.byref(h))
        if rc:
            raise _ERRORS.get(rc, RuntimeError)(self._lib.pet_last_error(None).decode())
        self._h = h
        self._session_pairs = 0
        self._session_atoms = 0

    def close(self):
        if self._h is not None:
            self._lib.pet_calc_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc):
        if rc:
            raise _ERRORS.get(rc, RuntimeError)(self._lib.pet_last_error(self._h).decode())

    # ---- properties (calculator.hpp:272-303) ----
    @property
    def cutoff(self):
        return self._lib.pet_cutoff(self._h)

    @property
    def ghost_cutoff(self):
        return self._lib.pet_ghost_cutoff(self._h)

    @property
    def exchange_ghost_cutoff(self):
        return self._lib.pet_exchange_ghost_cutoff(self._h)

    @property
    def energy_scale(self):
        return self._lib.pet_energy_scale(self._h)

    def supports(self, z):
        return bool(self._lib.pet_supports(self._h, int(z)))

    @property
    def workspace_bytes(self):
        return self._lib.pet_workspace_bytes(self._h)

    @property
    def kernel_launches(self):
        return self._lib.pet_kernel_launches(self._h)

    @property
    def graph_replays(self):
        return self._lib.pet_graph_replays(self._h)

    @property
    def batch_splits(self):
        """Batches compute() ran as several pieces to fit memory_budget_bytes / max_batch_atoms."""
        return self._lib.pet_batch_splits(self._h)

    @property
    def oom_recoveries(self):
        """Evaluations retried after the device ran out of memory (pools released, the batch cut smaller)."""
        return self._lib.pet_oom_recoveries(self._h)

    @property
    def driver_memory_queries(self):
        """Times the calculator asked the driver for the free device memory (kept while its pools keep their size)."""
        return self._lib.pet_driver_memory_queries(self._h)

    def fail_alloc(self, k):
        """Test hook: the k-th device allocation of the scratch pools from now reports out of memory, once."""
        self._lib.pet_debug_fail_alloc(int(k))

    @property
    def neighbor_searches(self):
        """Searches run for staged batches under cache_neighbors; neighbor_reuses counts the evaluations between."""
        return self._lib.pet_neighbor_searches(self._h)

    @property
    def neighbor_reuses(self):
        return self._lib.pet_neighbor_reuses(self._h)

    @property
    def last_device_ms(self):
        return self._lib.pet_last_device_ms(self._h)

    def last_shapes(self):
        a, e, m = C.c_int(), C.c_int(), C.c_int()
        self._check(self._lib.pet_last_shapes(self._h, C.byref(a), C.byref(e), C.byref(m)))
        return a.value, e.value, m.value

    # ---- evaluation ----
    def memory_plan(self):
        """The latest evaluation's memory decision (Calculator::memory_plan): a dict with atoms, max_neighbors, edges,
        tier ("never" | "wide" | "layers"), estimate_bytes, budget_bytes, pool_bytes."""
        p = PetMemoryPlan()
        self._check(self._lib.pet_memory_plan(self._h, C.byref(p)))
        names = {v: k for k, v in RECOMPUTE_TIERS.items()}
        return {"atoms": p.atoms, "max_neighbors": p.max_neighbors, "edges": p.edges, "tier": names.get(p.tier, "?"),
                "estimate_bytes": p.estimate_bytes, "budget_bytes": p.budget_bytes, "pool_bytes": p.pool_bytes}

    def memory_report(self):
        buf = C.create_string_buffer(1024)
        self._check(self._lib.pet_memory_report(self._h, buf, len(buf)))
        return buf.value.decode()

    @property
    def recommended_batch_atoms(self):
        return int(self._lib.pet_recommended_batch_atoms(self._h))

    def _results(self, B, N, forces, n_atoms, pairs=0):
        r = Results(np.zeros(B), np.zeros(N), n_atoms=list(n_atoms))
        pr = PetResults()
        pr.energy, pr.per_atom_energy = _dptr(r.energy), _dptr(r.per_atom_energy)
        if forces:
            r.forces, r.virial = np.zeros((N, 3)), np.zeros((B, 6))
            r.struct_id = np.zeros(N, dtype=np.int32)
            pr.forces, pr.virial, pr.struct_id = _dptr(r.forces), _dptr(r.virial), _iptr(r.struct_id)
            if pairs:
                r.edge_gradient = np.zeros((pairs, 3))
                pr.edge_gradient = _dptr(r.edge_gradient)
        return r, pr

    def compute(self, systems, compute_forces=True):
        """Calculator::compute(System) / compute(vector<System>) (calculator.hpp:187,192)."""
        if isinstance(systems, dict):
            systems = [systems]
        p = _Packed(systems)
        r, pr = self._results(p.n, p.total, compute_forces, p.n_atoms)
        self._check(self._lib.pet_compute(self._h, p.arr, p.n, int(compute_forces), C.byref(pr)))
        return r

    compute_batch = compute  # the name python/core.cpp:376 exposes

    def stage(self, systems):
        """Calculator::stage (calculator.hpp:214): the batch into device memory, once."""
        p = _Packed(systems)
        self._check(self._lib.pet_stage(self._h, p.arr, p.n))
        self._staged = (p.n, p.total, p.n_atoms)

    def keep_staged(self, keep):
        """The staged batch shrinks to the structures `keep` (indices into it, in their new order); positions stay as they
        are on the device and a Verlet cache follows without searching again (pet_keep_staged)."""
        k = np.ascontiguousarray(keep, dtype=np.int32)
        B, N, n_atoms = self._staged
        self._check(self._lib.pet_keep_staged(self._h, _iptr(k), len(k)))
        kept = [n_atoms[i] for i in k]
        self._staged = (len(k), int(sum(kept)), kept)

    def update_staged(self, positions=None, cells=None):
        x = None if positions is None else np.ascontiguousarray(positions, dtype=np.float64)
        c = None if cells is None else np.ascontiguousarray(cells, dtype=np.float64)
        self._check(self._lib.pet_update_staged(self._h, None if x is None else _dptr(x), None if c is None else _dptr(c)))

    def compute_staged(self, compute_forces=True):
        """Calculator::compute_device (calculator.hpp:219): results stay on the device until fetch()."""
        self._check(self._lib.pet_compute_staged(self._h, int(compute_forces)))
        self._staged_forces = compute_forces

    def fetch(self):
        B, N, n_atoms = self._staged
        r, pr = self._results(B, N, self._staged_forces, n_atoms)
        self._check(self._lib.pet_fetch_results(self._h, C.byref(pr)))
        return r

    def _edge_list(self, v: EdgeListView):
        keep = dict(
            x=np.ascontiguousarray(v.positions, dtype=np.float64).reshape(-1, 3),
            z=np.ascontiguousarray(v.atomic_numbers, dtype=np.int32),
            off=np.ascontiguousarray(v.offsets, dtype=np.int32),
            nb=np.ascontiguousarray(v.neighbors, dtype=np.int32))
        el = PetEdgeList()
        el.n_atoms, el.n_local, el.half = len(keep["z"]), int(v.n_local), int(bool(v.half))
        el.positions, el.atomic_numbers = _dptr(keep["x"]), _iptr(keep["z"])
        el.offsets, el.neighbors = _iptr(keep["off"]), _iptr(keep["nb"])
        if v.shifts is not None:
            keep["sh"] = np.ascontiguousarray(v.shifts, dtype=np.int32).reshape(-1, 3)
            el.shifts = _iptr(keep["sh"])
        if v.cell is not None:
            keep["cell"] = np.ascontiguousarray(v.cell, dtype=np.float64).reshape(9)
            el.cell = _dptr(keep["cell"])
        if v.exchange is not None and getattr(v.exchange, "native_callbacks", None):
            # callbacks that live in the library itself (exchange.NativeNcclExchange): no Python in the pass
            el.exchange = C.cast(C.c_void_p(v.exchange.native_callbacks), _P(PetExchange))
            keep["exchange"] = v.exchange
        elif v.exchange is not None:
            ex = v.exchange

            def _guard(fn):
                def call(*a):
                    try:
                        fn(*a)
                        return 0
                    except Exception:  # an exception must not cross the C frame: fail the evaluation instead
                        import traceback
                        traceback.print_exc()
                        return 1
                return call
            cb = PetExchange(None,
                             SET_LIVE_FN(_guard(lambda user, live, n, stream: ex.set_live(live or 0, n, stream or 0))),
                             EDGES_FN(_guard(lambda user, out, inn, n, w, stream: ex.edges(out or 0, inn or 0, n, w, stream or 0))))
            keep["exchange"] = cb
            el.exchange = C.pointer(cb)
            self._exchange_keep = cb  # the library keeps the function pointers for as long as the list is set
        return el, keep

    def set_neighbors(self, view: EdgeListView):
        """Calculator::set_neighbors(const EdgeListView&) (calculator.hpp:235)."""
        el, keep = self._edge_list(view)
        self._check(self._lib.pet_set_neighbors(self._h, C.byref(el)))
        self._session_atoms, self._session_pairs = el.n_atoms, int(keep["off"][-1]) if len(keep["off"]) else 0

    def compute_step(self, positions, cell=None, compute_forces=True, edge_gradients=False):
        """Calculator::compute_step(positions, cell, forces, edge_gradients) (calculator.hpp:238)."""
        x = np.ascontiguousarray(positions, dtype=np.float64).reshape(-1, 3)
        if len(x) != self._session_atoms:
            raise ValueError("positions do not match the list set by set_neighbors")
        c = None if cell is None else np.ascontiguousarray(cell, dtype=np.float64).reshape(9)
        N = self._session_atoms
        r, pr = self._results(1, N, compute_forces, [N], self._session_pairs if edge_gradients else 0)
        self._check(self._lib.pet_compute_step(self._h, _dptr(x), None if c is None else _dptr(c), int(compute_forces),
                                               int(edge_gradients), C.byref(pr)))
        return r

    def compute_step_on_device(self, positions, cell=None, compute_forces=True):
        """compute_step with the results left on the device: nothing is copied back or waited for. device_results()
        says where they lie; an exchange's reduce() reads them there."""
        x = np.ascontiguousarray(positions, dtype=np.float64).reshape(-1, 3)
        if len(x) != self._session_atoms:
            raise ValueError("positions do not match the list set by set_neighbors")
        c = None if cell is None else np.ascontiguousarray(cell, dtype=np.float64).reshape(9)
        self._step_keep = (x, c)  # the copy to the device is asynchronous: the arrays must outlive it
        self._check(self._lib.pet_compute_step(self._h, _dptr(x), None if c is None else _dptr(c), int(compute_forces), 0, None))

    def device_results(self):
        """(PetDeviceResults with device addresses as integers, the calculator's cudaStream_t as an integer)."""
        r, s = PetDeviceResults(), C.c_void_p()
        self._check(self._lib.pet_device_results_of(self._h, C.byref(r), C.byref(s)))
        return r, s.value or 0

    def compute_edges(self, view: EdgeListView, compute_forces=True, edge_gradients=True):
        """Calculator::compute_edges (calculator.hpp:227)."""
        el, keep = self._edge_list(view)
        N, L = el.n_atoms, int(keep["off"][-1]) if len(keep["off"]) else 0
        self._session_atoms, self._session_pairs = N, L
        r, pr = self._results(1, N, compute_forces, [N], L if edge_gradients else 0)
        self._check(self._lib.pet_compute_edges(self._h, C.byref(el), int(compute_forces), int(edge_gradients), C.byref(pr)))
        return r

    def compute_step_device(self, positions_ptr, forces_ptr=0, per_atom_energy_ptr=0, per_atom_virial_ptr=0,
                            virial_scale=1.0, cell=None):
        """Calculator::compute_step(const DeviceArrays&, cell) (calculator.hpp:259): device pointers, added into."""
        a = PetDeviceArrays(positions_ptr, forces_ptr or None, per_atom_energy_ptr or None, per_atom_virial_ptr or None,
                            virial_scale)
        c = None if cell is None else np.ascontiguousarray(cell, dtype=np.float64).reshape(9)
        t = PetTotals()
        self._check(self._lib.pet_compute_step_device(self._h, C.byref(a), None if c is None else _dptr(c), C.byref(t)))
        return t.energy, np.array(list(t.virial))

    def set_neighbors_device(self, n_atoms, n_centres, ilist_ptr, numneigh_ptr, neighbors_ptr, stride_i, atomic_numbers_ptr,
                             stride_k=1, mask=0, n_local=-1, image_of_ptr=0, positions_ptr=0, cell=None):
        """Calculator::set_neighbors(const DeviceEdgeListView&) (calculator.hpp:236): an engine's full list in device
        memory (LAMMPS's KOKKOS layout). Pointers are device addresses as integers; cell is host memory."""
        c = None if cell is None else np.ascontiguousarray(cell, dtype=np.float64).reshape(9)
        v = PetDeviceEdgeList(n_atoms, n_local, n_centres, ilist_ptr or None, numneigh_ptr or None, neighbors_ptr or None,
                              stride_i, stride_k, mask, atomic_numbers_ptr or None, image_of_ptr or None, positions_ptr or None,
                              None if c is None else _dptr(c), None)
        self._check(self._lib.pet_set_neighbors_device(self._h, C.byref(v)))
        self._session_atoms, self._session_pairs = n_atoms, 0

    def compute_pairs(self, n_atoms, n_pairs, pairs_ptr, atomic_numbers_ptr, positions_ptr, cell=None, renumber_ptr=0,
                      n_local=-1, stride_pair=5, stride_col=1, compute_forces=True, fetch=True):
        """Calculator::compute_pairs(DevicePairListView, positions, cell) (calculator.hpp:260-268): an engine's flat
        pair list in device memory, set and evaluated in one call. Pointers are device addresses as integers.
        Returns the device pointers (dict) and, with fetch, the results copied to the host in the list's numbering."""
        v = PetPairList(n_atoms, n_local, n_pairs, pairs_ptr or None, stride_pair, stride_col, atomic_numbers_ptr or None,
                        renumber_ptr or None)
        c = None if cell is None else np.ascontiguousarray(cell, dtype=np.float64).reshape(9)
        d = PetDeviceResults()
        self._check(self._lib.pet_compute_pairs(self._h, C.byref(v), positions_ptr or None, None if c is None else _dptr(c),
                                                int(compute_forces), C.byref(d)))
        self._session_pairs, self._session_atoms = n_pairs, n_atoms
        dev = dict(energy=d.energy, per_atom_energy=d.per_atom_energy, forces=d.forces, virial=d.virial)
        if not fetch:
            return dev, None
        r, pr = self._results(1, n_atoms, compute_forces, [n_atoms])
        self._check(self._lib.pet_fetch_results(self._h, C.byref(pr)))
        return dev, r

    # ---- the neighbour search alone ----
    def neighbor_list(self, systems, capacity=None):
        """The device search's raw list: dict of i, j, shift, vec, dist, reverse, cutoff."""
        if isinstance(systems, dict):
            systems = [systems]
        p = _Packed(systems)
        cap = int(capacity or max(1024, p.total * 256))
        while True:
            out = dict(i=np.zeros(cap, np.int32), j=np.zeros(cap, np.int32), shift=np.zeros((cap, 3), np.int32),
                       vec=np.zeros((cap, 3)), dist=np.zeros(cap), reverse=np.zeros(cap, np.int32),
                       cutoff=np.zeros(cap, np.float32))
            re = PetRawEdges()
            re.capacity = cap
            re.i, re.j, re.shift, re.reverse = _iptr(out["i"]), _iptr(out["j"]), _iptr(out["shift"]), _iptr(out["reverse"])
            re.vec, re.dist = _dptr(out["vec"]), _dptr(out["dist"])
            re.cutoff = out["cutoff"].ctypes.data_as(C.POINTER(C.c_float))
            rc = self._lib.pet_neighbor_list(self._h, p.arr, p.n, C.byref(re))
            if rc == 2 and re.n_edges > cap:
                cap = re.n_edges
                continue
            self._check(rc)
            return {k: v[:re.n_edges] for k, v in out.items()}

    # ---- per-class device timing ----
    def profile(self, enable=True):
        self._check(self._lib.pet_profile(self._h, int(enable)))

    def profile_read(self):
        """{class: dict(launches, ms, flops, bytes)} since the last read."""
        arr = (PetProfileEntry * 16)()
        n = C.c_int()
        self._check(self._lib.pet_profile_read(self._h, arr, 16, C.byref(n)))
        return {arr[i].name.decode(): dict(launches=arr[i].launches, ms=arr[i].ms, flops=arr[i].flops, bytes=arr[i].bytes)
                for i in range(n.value)}

    # ---- testing aids ----
    def enable_taps(self):
        n = C.c_size_t()
        self._lib.pet_debug_fetch(self._h, b"", None, 0, C.byref(n))  # arms recording for the next evaluation

    def debug_fetch(self, name):
        n = C.c_size_t()
        self._check(self._lib.pet_debug_fetch(self._h, name.encode(), None, 0, C.byref(n)))
        out = np.zeros(n.value, np.float32)
        self._check(self._lib.pet_debug_fetch(self._h, name.encode(), out.ctypes.data_as(C.POINTER(C.c_float)), n.value,
                                              C.byref(n)))
        return out

    def gemm(self, A, W, mode="native", w_transposed=True):
        """C = A W^T (W [n,k]) or A W (W [k,n]) through the library's weight GEMM."""
        A = np.ascontiguousarray(A, dtype=np.float32)
        W = np.ascontiguousarray(W, dtype=np.float32)
        m, k = A.shape
        n = W.shape[0] if w_transposed else W.shape[1]
        Cm = np.zeros((m, n), np.float32)
        fp = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))
        self._check(self._lib.pet_gemm_host(self._h, GEMM_MODES[mode], int(w_transposed), m, n, k, fp(A), fp(W), fp(Cm)))
        return Cm
