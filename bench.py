#!/usr/bin/env python
"""Throughput of the energy+forces+virial hot path: atom-evaluations per second.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--gemm MODE] [--workload NAME]

One step = one evaluation (neighbour list, forward, analytic backward, force/virial
fold) of the pet-mad-s-shaped model on the 1728-atom jittered diamond cell, per
GPU.  With N > 1 (launched by torchrun, one rank per GPU) each rank evaluates its
own structure of a batch of N: the reference's batched compute shards whole
structures, edges never cross them, so there is no data-path collective; per-GPU
work is fixed (weak scaling).  `value` is measured with the structures already
staged in device memory (CUDA events, max over ranks); `e2e` goes through the
public Calculator.compute call with host arrays in and host results out.

Beside the headline the same JSON line carries `splits`: the two ways the path shards over
the GPUs of a box, both strong scaling (total work fixed as N grows).  `batch512x64`: the
512-structure batch, whole structures dealt to ranks by sharding.partition, no data-path
collective.  `diamond13824`: one 13824-atom cell (pet-omat-l shape); at N = 1 the whole cell
on one GPU (the backward re-runs each layer's forward to fit memory), at N >= 2 bricks by
centre atom with ghosts one cutoff deep, edge rows swapped at every layer and the ghost
forces reduced over NCCL.  --no-splits skips them.

--impl reference times the reference's own CPU implementation of the path on the
host cores: its unmodified sources compiled for the host (oracle/build_ref.sh, the
build with its GEMMs through a CBLAS, OpenMP threads for its kernels), through its
Calculator::compute, on the same workload, with every host core this process may use
(an inherited OMP_NUM_THREADS is overridden; the count in force is reported).  A
workload whose full size would take more than about ten minutes of CPU for the asked
steps is timed on a smaller sample of it and the line says so.  Where that library is
not built, the CPU restatement (oracle/pet_oracle.py) is timed instead and the line
says "port".
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
# The CPU arm runs OpenMP kernels and a threaded BLAS in turn: idle OpenMP threads must sleep, not spin.
os.environ.setdefault("OMP_WAIT_POLICY", "passive")

METRIC = "atom_evals_per_s"
UNIT = "atom-evals/s"
# DRAM traffic of one weight-GEMM launch per token row (atoms + kept edges), from one ncu capture:
# dram__bytes_read.sum + dram__bytes_write.sum averaged over seven consecutive k_gemm_tc launches of the water648
# workload, token-row and atom-row GEMMs as they come (50.2 MB at 25 320 rows; the capture is summarised under profiles/).
# Captured with the kernel as of commit 002f4a5; the mainloop has been re-profiled since on one 122 138-row launch
# (201 MB, 1646 B per row for a plain 256 x 256 GEMM: the same "A once, C once"), so the figure stands.
# A GEMM reads A once and writes C once, so it grows with the rows.
GEMM_DRAM_BYTES_PER_TOKEN_ROW = 50.2e6 / 25320
DTYPE_OF = {"native": "f32", "tf32": "tf32", "bf16": "bf16", "3xtf32": "f32 (3xTF32)"}
MODEL_OF = {"diamond64": "xs", "water648": "s", "diamond1728": "s", "batch512x64": "s", "diamond13824": "l"}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d.get("hbm_gbs", 6650.0), "bf16_tflops": d.get("bf16_tflops", 1590.0),
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", 1400.0), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML queries from a thread of this process
    (the same counters `nvidia-smi --query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.*` prints), every 50 ms.
    An `nvidia-smi -lms` child process was what this used first; three NVML calls from a thread are lighter.
    Reading only: nothing is set."""
    REASONS = (("hw_slowdown", "nvmlClocksEventReasonHwSlowdown"), ("hw_thermal_slowdown", "nvmlClocksEventReasonHwThermalSlowdown"),
               ("sw_thermal_slowdown", "nvmlClocksEventReasonSwThermalSlowdown"), ("sw_power_cap", "nvmlClocksEventReasonSwPowerCap"))

    def __init__(self, index):
        self.index, self.samples, self.first, self.thread, self.nvml, self.handle = index, [], 0, None, None, None
        self.stop_flag = threading.Event()

    def mark(self):
        """The timed region starts here: samples taken before it (during warm-up) are not counted."""
        self.first = len(self.samples)

    def _open(self):
        import pynvml
        pynvml.nvmlInit()
        handle = None
        try:  # the CUDA ordinal is not NVML's index when CUDA_VISIBLE_DEVICES reorders or hides devices: go by UUID
            import torch
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            handle = pynvml.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
        except Exception:
            handle = None
        if handle is None:
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
        return pynvml, handle

    def _loop(self):
        nv, h = self.nvml, self.handle
        while not self.stop_flag.is_set():
            try:
                sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                self.samples.append((float(sm), float(mx), int(mask)))
            except Exception:
                pass
            self.stop_flag.wait(0.05)

    def start(self):
        try:
            self.nvml, self.handle = self._open()
        except Exception:
            self.nvml = None
            return
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def wait_started(self, limit=5.0):
        """Until the first sample has come, or `limit` seconds."""
        t0 = time.perf_counter()
        while self.thread and not self.samples and time.perf_counter() - t0 < limit:
            time.sleep(0.02)

    def stop(self):
        if not self.thread:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["NVML unavailable"]}
        self.stop_flag.set()
        self.thread.join(timeout=2)
        taken = self.samples[self.first:]
        reasons = set()
        for _, _, mask in taken:
            for name, const in self.REASONS:
                if mask & getattr(self.nvml, const):
                    reasons.add(name)
        sm, mx = [s[0] for s in taken], [s[1] for s in taken]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "NVML, every 50 ms"}


_RESULT_FD = None


def keep_stdout_for_the_result():
    """Libraries under the GPU arm write to stdout (NCCL prints its version when its first communicator is made): from
    here on everything written to stdout goes to stderr, and emit() alone writes to the real stdout."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line):
    if _RESULT_FD is None:
        print(line, flush=True)
    else:
        sys.stdout.flush()
        os.write(_RESULT_FD, (line + "\n").encode())


def make_model(tmp, shape):
    from pet_kokkos_b200 import checkpoint as ck
    return ck.write_random_checkpoint(Path(tmp) / f"bench_{shape}", shape, seed=0, init="n002")


def rank_systems(workload, rank, world):
    """This rank's share of the step's batch: one structure per GPU (seeded per rank) for the single-cell
    workloads, a contiguous run of the 512 structures for the batch workload."""
    from pet_kokkos_b200 import structures as st
    if workload == "batch512x64":
        allb = st.workload(workload)
        per = len(allb) // world
        return allb[rank * per:(rank + 1) * per]
    return st.workload(workload, seed=rank)


def cpu_sample(workload, full):
    """The CPU arm's structures: the workload itself, or a smaller sample of it with the same model and the same
    per-atom neighbour count where the full case is too slow for the steps asked."""
    from pet_kokkos_b200 import structures as st
    if full and workload != "diamond13824":
        return st.workload(workload), "the full workload", True
    if workload in ("diamond1728", "diamond13824"):
        return ([st.diamond(3, jitter=0.05, seed=0)],
                "216-atom jittered diamond (3x3x3 cells), same model, same per-atom neighbour count", False)
    if workload == "batch512x64":
        return st.mixture_batch(8, 64, 9.0), "8 of the 512 structures", False
    return st.workload(workload), "the full workload", True


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_runner(jp, sp, threads):
    """(run(systems), kind, threads in force). "reference" is the reference's own code (oracle/_ref, its CBLAS build);
    "port" the restatement, where that library is not there."""
    from oracle import reference_lib
    if os.path.exists(reference_lib.BLAS_LIB_PATH):
        calc = reference_lib.ReferenceCalculator(str(jp), str(sp), blas=True)
        used = reference_lib.set_threads(threads)
        return (lambda systems: calc.compute(systems)), "reference", used
    import torch
    from oracle import pet_oracle as po
    from pet_kokkos_b200 import checkpoint as ck
    meta, tens = ck.load_checkpoint(jp, sp)
    torch.set_num_threads(threads)
    return (lambda systems: po.evaluate(meta, tens, systems, dtype=torch.float32)), "port", torch.get_num_threads()


def time_cpu(run, systems, steps, warmup):
    for _ in range(warmup):
        run(systems)
    t = []
    for _ in range(steps):
        t0 = time.perf_counter()
        run(systems)
        t.append(time.perf_counter() - t0)
    return t


def run_reference(args):
    """The CPU arm: rank 0 alone times the reference's path on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    with tempfile.TemporaryDirectory() as tmp:
        jp, sp = make_model(tmp, MODEL_OF[args.workload])
        run, kind, threads = cpu_runner(jp, sp, host_cores())
        # One evaluation of the small sample tells how long the full workload would take (the path's cost is
        # linear in atoms at a fixed neighbour count): the full one is timed when steps + warm-up fit ten minutes.
        small, small_what, _ = cpu_sample(args.workload, False)
        t0 = time.perf_counter()
        run(small)
        per_atom = (time.perf_counter() - t0) / sum(s["n_atoms"] for s in small)
        from pet_kokkos_b200 import structures as st
        full_atoms = sum(s["n_atoms"] for s in st.workload(args.workload)) if args.workload != "diamond13824" else 13824
        fits = per_atom * full_atoms * (args.steps + args.warmup) <= 600.0
        systems, what, same = cpu_sample(args.workload, fits)
        t = time_cpu(run, systems, args.steps, args.warmup)
        n_atoms = sum(s["n_atoms"] for s in systems)
    sec = float(np.mean(t))
    value = n_atoms / sec
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "model": f"random-init pet-mad-{MODEL_OF[args.workload]}-like", "sample": what,
                   "same_config": same, "atoms_per_step": n_atoms},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": what},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}), flush=True)


CHECKS = ROOT / "tests" / "golden" / "bench_checks.npz"


def check_against_fixture(tag, model_paths, energy, forces, virial, loose=1.0, e_loose=None):
    """Holds a sub-sample's energy, forces and virial to the reference's stored answer (tests/golden/bench_checks.npz,
    made by tests/golden/make_bench_checks.py) within the parity bands before anything is timed. Returns a short
    record for the JSON line; raises when the bands are missed."""
    e_loose = loose if e_loose is None else e_loose
    if not CHECKS.exists():
        return {"checked": False, "why": "tests/golden/bench_checks.npz is missing"}
    import hashlib
    from pet_kokkos_b200 import checkpoint as ck
    g = np.load(CHECKS)
    _, tens = ck.load_checkpoint(*model_paths)
    h = hashlib.sha256()
    for k in sorted(tens):
        h.update(k.encode()), h.update(np.ascontiguousarray(tens[k], "<f4").tobytes())
    if h.hexdigest() != str(g[f"{tag}_digest"]):
        return {"checked": False, "why": "the seeded model differs from the fixture's"}
    re, rf, rw = g[f"{tag}_energy"], g[f"{tag}_forces"], g[f"{tag}_virial"]
    # relative to what the network itself adds up to: a random-init network's energy can all but cancel the
    # composition energies (the cell's does), which would make "relative to the total" meaningless
    e_scale = max(np.abs(re).max(), np.abs(g[f"{tag}_per_atom_energy"]).sum() / len(re), float(g[f"{tag}_network_scale"]))
    de = float(np.abs(np.asarray(energy) - re).max() / e_scale)
    df = float(np.abs(np.asarray(forces) - rf).max() / max(1.0, np.abs(rf).max()))
    dw = float(np.abs(np.asarray(virial).reshape(rw.shape) - rw).max() / max(1.0, np.abs(rw).max()))
    rec = {"checked": True, "against": "the reference's CPU build on the same inputs", "rel_dE": de, "dF": df, "rel_dW": dw}
    rec["bands"] = {"rel_dE": e_loose * 1e-6, "dF": loose * 1e-5, "rel_dW": loose * 1e-5}
    if not (de <= e_loose * 1e-6 and df <= loose * 1e-5 and dw <= loose * 1e-5):
        raise RuntimeError(f"bench: the {tag} sub-sample misses the parity bands: {rec}")
    return rec


# The bands of bench.py's own checks by GEMM mode, as multiples of the fp32 bands (1e-6 / 1e-5 / 1e-5): the speed modes
# are held to the reference's bands for them (about three decimal digits), never passed off as fp32.
CHECK_LOOSE = {"native": 1.0, "3xtf32": 1.0, "tf32": 2000.0, "bf16": 20000.0}


def cell_step_fn(calc, system, rank, world, dist):
    """One evaluation of a periodic cell over `world` ranks, returning a device tensor [1 + 6 + 3 n] (energy, virial,
    forces of the WHOLE cell on every rank). One rank: the staged cell, evaluated in place. Several: bricks by centre
    atom, ghosts one cutoff deep, rows swapped at every layer (the reference's exchange mode), set once by
    set_neighbors and stepped by compute_step; ghost forces folded onto their owners and everything reduced with one
    all-reduce."""
    import torch
    from pet_kokkos_b200 import exchange
    n_total = system["n_atoms"]
    if world == 1:
        calc.stage([system])

        def step():
            calc.compute_staged(True)
            r = calc.fetch()
            return torch.from_numpy(np.concatenate([r.energy, r.virial[0], r.forces.ravel()]))
        return step, {"atoms_owned_rank0": n_total}
    domains = [exchange.exchange_domain(system, r, world, calc.cutoff) for r in range(world)]
    fields, owner, _, remote = domains[rank]
    ex = exchange.make_exchange(calc, exchange.route(domains)[rank], owner, n_total, torch.cuda.current_device())
    calc.set_neighbors(exchange.view_of(fields, ex))
    calc.cell_exchange = ex

    def step():  # host positions in; the whole cell's energy, virial and forces out on the host
        calc.compute_step_on_device(fields["positions"], None, True)
        return torch.from_numpy(ex.reduce(calc))
    return step, {"atoms_owned_rank0": int(fields["n_local"]), "atoms_listed_rank0": int(len(fields["positions"])),
                  "edges_to_ghosts_rank0": int(len(remote)), "exchange": type(ex).__name__}


def measure_cell(args, workload, rank, world, local, dist, steps, warmup, tmpdir):
    """Times the one-cell split; returns the record for the JSON line (rank 0) after checking a 512-atom cell of the
    same model through the same code path against the reference's stored answer."""
    import torch
    from pet_kokkos_b200 import Calculator, structures as st
    shape = MODEL_OF[workload]
    jp, sp = make_model(tmpdir, shape)
    calc = Calculator(jp, sp, gemm=args.gemm, device=local)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    small = st.diamond(4, jitter=0.05, seed=0)
    step, _ = cell_step_fn(calc, small, rank, world, dist)
    out = step().cpu().numpy()
    # at this shape (contractions of 512 to 2048 terms) the 3xTF32 mode's energy sits 4-5e-6 of the network's energy
    # low (the tensor core's truncating accumulate): its energy band here is 1e-5; forces and virial as everywhere
    check = check_against_fixture("cell", (jp, sp), out[:1], out[7:].reshape(-1, 3), out[1:7], CHECK_LOOSE[args.gemm],
                                  e_loose=10.0 if args.gemm == "3xtf32" else None)
    s = st.workload(workload)[0]
    n_total = s["n_atoms"]
    step, info = cell_step_fn(calc, s, rank, world, dist)
    for _ in range(warmup):
        step()
    barrier()
    launches0 = calc.kernel_launches
    dev_ms = []
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        out = step()
        dev_ms.append(calc.last_device_ms)
    barrier()
    wall = time.perf_counter() - t0
    launches = calc.kernel_launches - launches0
    n_act, n_edges, max_nb = calc.last_shapes()
    plan = calc.memory_plan()
    calc.profile(True)  # one more step with CUDA events around each kernel class (rank 0's are reported)
    step()
    calc.profile(False)
    prof = calc.profile_read()
    ex = getattr(calc, "cell_exchange", None)
    exch_ms = None
    if ex is not None:  # one more step with CUDA events around the rows in flight
        ex.timing(True)
        step()
        exch_ms = ex.timing(False)[0]
    classes = {k: {"ms_per_step": v["ms"], "tflops": v["flops"] / max(v["ms"], 1e-9) / 1e9} for k, v in prof.items()}
    if world > 1:
        t = torch.tensor([wall, float(np.sum(dev_ms))], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        wall, step_ms = [float(x) for x in t.tolist()]
    else:
        step_ms = float(np.sum(dev_ms))
    rec = {"workload": workload, "model": f"random-init pet-omat-{shape}-like", "scaling": "strong", "n_gpus": world,
           "value": n_total * steps / wall, "unit": UNIT, "steps": steps, "warmup": warmup,
           "ms_per_step": wall / steps * 1e3, "device_ms_per_step": (step_ms / steps) or None, "atoms_total": n_total,
           "kept_edges_rank0": n_edges, "max_neighbors": max_nb, "recompute": plan["tier"],
           "pool_gib_rank0": plan["pool_bytes"] / 2 ** 30, "gpu_launches": int(launches), "classes_rank0": classes,
           "non_kernel_ms_per_step": wall / steps * 1e3 - sum(v["ms"] for v in prof.values()),
           "check": check, "energy": float(out[0].item()), **info}
    if exch_ms is not None:
        rec["exchange_ms_per_step_rank0"] = exch_ms
    if ex is not None:
        ex.close()
    calc.close()
    return rec


def measure_batch(args, rank, world, local, dist, steps, warmup, tmpdir):
    """Times the 512-structure batch dealt to the ranks as contiguous runs of near-equal cost (sharding.partition): no
    data-path collective, host structures in and host results out every step; checks its first four structures
    against the reference's stored answer first."""
    import torch
    from pet_kokkos_b200 import Calculator, sharding, structures as st
    jp, sp = make_model(tmpdir, MODEL_OF["batch512x64"])
    calc = Calculator(jp, sp, gemm=args.gemm, device=local)
    systems = st.workload("batch512x64")
    r4 = calc.compute(systems[:4])
    check = check_against_fixture("batch", (jp, sp), r4.energy, r4.forces, r4.virial, CHECK_LOOSE[args.gemm])
    runs = sharding.partition([sharding.structure_cost(s, calc.cutoff) for s in systems], world)
    b, e = runs[rank]
    mine = systems[b:e]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        calc.compute(mine)
    barrier()
    t0 = time.perf_counter()
    dev_ms = 0.0
    for _ in range(steps):
        calc.compute(mine)
        dev_ms += calc.last_device_ms
    barrier()
    wall = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([wall, dev_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        wall, dev_ms = [float(x) for x in t.tolist()]
    n_total = sum(s["n_atoms"] for s in systems)
    rec = {"workload": "batch512x64", "model": "random-init pet-mad-s-like", "scaling": "strong", "n_gpus": world,
           "value": n_total * steps / wall, "unit": UNIT, "steps": steps, "warmup": warmup,
           "ms_per_step": wall / steps * 1e3, "device_ms_per_step": dev_ms / steps, "atoms_total": n_total,
           "structures_rank0": e - b if rank == 0 else None, "batch_pieces_rank0": int(calc.batch_splits),
           "sharding": "contiguous runs of near-equal atoms x neighbours per rank, no data-path collective; host in, host out",
           "check": check}
    calc.close()
    return rec


def run_one_cell(args):
    """--workload diamond13824: the one-cell split alone, as the headline line."""
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29555")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), rank=rank, world_size=world)
    tmp = tempfile.TemporaryDirectory()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    rec = measure_cell(args, args.workload, rank, world, local, dist, args.steps, args.warmup, tmp.name)
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        emit(json.dumps({
            "metric": METRIC, "value": rec["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": rec["ms_per_step"], "device_ms_per_step": rec["device_ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": DTYPE_OF[args.gemm], "data": "synthetic",
            "config": {k: rec[k] for k in rec if k not in ("value", "unit", "classes_rank0")} | {"gemm_mode": args.gemm,
                       "l2": "working set far exceeds the 126 MB L2; no flush needed"},
            "e2e": {"value": rec["value"], "unit": UNIT, "h2d_bytes_per_step": rec["atoms_total"] * 24,
                    "d2h_bytes_per_step": rec["atoms_total"] * 24 + 56, "ms_per_step": rec["ms_per_step"]},
            "gpu_launches": rec["gpu_launches"], "clocks": clocks, "roofline": None, "classes": rec["classes_rank0"],
            "cpu_baseline": None}))
    if world > 1:
        dist.destroy_process_group()


def run_ours(args):
    import torch
    import torch.distributed as dist
    from pet_kokkos_b200 import Calculator, checkpoint as ck

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(local)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    shape = MODEL_OF[args.workload]
    tmp = tempfile.TemporaryDirectory()
    jp, sp = make_model(tmp.name, shape)
    calc = Calculator(jp, sp, gemm=args.gemm, device=local)
    systems = rank_systems(args.workload, rank, world)
    n_atoms = sum(s["n_atoms"] for s in systems)

    # ---- device-resident throughput: structures staged once, evaluated in place ----
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        sampler.wait_started()
    calc.stage(systems)
    for _ in range(args.warmup):
        calc.compute_staged(True)
        calc.fetch()
    barrier()
    sampler.mark()
    launches0 = calc.kernel_launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dev_ms = []
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        calc.compute_staged(True)
        r = calc.fetch()                 # synchronizes the calculator's stream
        dev_ms.append(calc.last_device_ms)  # CUDA events on the stream the kernels were launched on
    barrier()
    wall = time.perf_counter() - t0
    launches = calc.kernel_launches - launches0
    clocks = sampler.stop() if rank == 0 else None
    step_ms = float(np.sum(dev_ms))      # device time of the K steps on this rank
    n_act, n_edges, max_nb = calc.last_shapes()

    # ---- end to end: host arrays in, host results out, every step ----
    for _ in range(min(args.warmup, 2)):
        calc.compute(systems)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        r = calc.compute(systems)
    barrier()
    e2e_wall = time.perf_counter() - t0
    B = len(systems)
    h2d = n_atoms * (24 + 4) + B * 72 + n_atoms * 8 + B * 72 + B * 36  # positions, numbers, cells; staged sid/species/cinv/grid
    d2h = B * 8 + n_atoms * 8 + n_atoms * 24 + B * 48 + n_atoms * 4

    # ---- per-class device time of two more steps (CUDA events around each class's launches) ----
    calc.profile(True)
    for _ in range(2):
        calc.compute_staged(True)
        calc.fetch()
    calc.profile(False)
    prof = calc.profile_read()

    if world > 1:
        t = torch.tensor([step_ms, wall, e2e_wall], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        step_ms, wall, e2e_wall = [float(x) for x in t.tolist()]
        a = torch.tensor([n_atoms], device="cuda", dtype=torch.float64)
        dist.all_reduce(a)
        total_atoms = int(a.item())
    else:
        total_atoms = n_atoms

    # ---- the two multi-GPU splits (every rank takes part), each checked on a sub-sample before it is timed ----
    splits = None
    line = None
    if rank == 0:
        peaks = measured_peaks()
        value = total_atoms * args.steps / wall  # barrier + synchronize on both sides, max over ranks
        top = max(prof, key=lambda k: prof[k]["ms"]) if prof else None
        roof = None
        if top:
            p = prof[top]
            per_launch_ms = p["ms"] / p["launches"]
            if top == "gemm":
                ach = p["flops"] / (p["ms"] * 1e-3) / 1e12
                roof = {"kernel": "weight GEMMs with fused epilogues", "bound": "tensor", "achieved": ach,
                        "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops_sustained"],
                        "peak_source": f"{peaks['source']} cuBLAS bf16, sustained",
                        "traffic": GEMM_DRAM_BYTES_PER_TOKEN_ROW * (n_act + n_edges),
                        "traffic_source": "ncu dram bytes per launch on water648 (capture of commit 002f4a5, summarised under profiles/), "
                                          "scaled by token rows",
                        "launches": p["launches"], "avg_launch_ms": per_launch_ms}
                # what the mode asks of the tensor cores: an fp32-accurate product is three tf32 MMAs, and tf32 runs at
                # half the bf16 rate, so the algorithmic ceiling of this mode is a sixth of the bf16 peak
                passes = {"3xtf32": 3, "tf32": 1, "bf16": 1}.get(args.gemm)
                if passes:
                    roof["mma_tflops"] = passes * ach
                    roof["mode_ceiling_frac_of_peak"] = 0.5 / passes
            else:
                ach = p["bytes"] / (p["ms"] * 1e-3) / 1e9
                roof = {"kernel": top, "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": ach / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} copy", "traffic": None,
                        "launches": p["launches"], "avg_launch_ms": per_launch_ms}
        classes = {k: {"ms_per_step": v["ms"] / 2, "share": v["ms"] / max(sum(x["ms"] for x in prof.values()), 1e-9),
                       "tflops": v["flops"] / max(v["ms"], 1e-9) / 1e9, "gbs": v["bytes"] / max(v["ms"], 1e-9) / 1e6}
                   for k, v in prof.items()}
        # the other GEMM/attention modes on the same staged structures (N = 1 only), three steps each after two:
        # native = fp32 on the CUDA cores (the default correctness mode); tf32 and bf16 = the speed modes (one
        # tensor-core pass per product, single-pass tf32 attention), each with its measured distance from native
        modes = None
        if world == 1 and not args.no_cpu:
            modes, results = {}, {args.gemm: r}
            for other in ("native", "3xtf32", "tf32", "bf16"):
                if other == args.gemm:
                    continue
                c2 = Calculator(jp, sp, gemm=other, device=local)
                c2.stage(systems)
                for _ in range(2):
                    c2.compute_staged(True)
                    c2.fetch()
                ms = []
                for _ in range(3):
                    c2.compute_staged(True)
                    results[other] = c2.fetch()
                    ms.append(c2.last_device_ms)
                modes[other] = {"device_ms_per_step": float(np.mean(ms)), "dtype": DTYPE_OF[other]}
                c2.profile(True)  # one more step with CUDA events around each kernel class
                c2.compute_staged(True)
                c2.fetch()
                c2.profile(False)
                modes[other]["classes_ms"] = {k: round(v["ms"], 3) for k, v in c2.profile_read().items()}
                c2.close()
            exact = results["native"]
            for name, res in results.items():
                d = modes.setdefault(name, {"device_ms_per_step": step_ms / args.steps, "dtype": DTYPE_OF[name]})
                d["vs_native_dE_meV_per_atom"] = float(np.abs(res.energy - exact.energy).max() / n_atoms * 1e3)
                d["vs_native_max_dF_meV_per_A"] = float(np.abs(res.forces - exact.forces).max() * 1e3)
        # the CPU arm beside it (N = 1 only): the reference's path on the host cores, on a bounded sample
        cpu = None
        if world == 1 and not args.no_cpu:
            cs, what, _ = cpu_sample(args.workload, False)  # bounded: 10-30 s of CPU work
            run, kind, threads = cpu_runner(jp, sp, host_cores())
            t = time_cpu(run, cs, 2, 1)
            na = sum(x["n_atoms"] for x in cs)
            cpu = {"value": na / float(np.mean(t)), "unit": UNIT, "cores": threads, "kind": kind, "sample": what}
        line = ({
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": wall / args.steps * 1e3, "device_ms_per_step": step_ms / args.steps,
            "device_ms_each_step_rank0": [round(float(x), 3) for x in dev_ms],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": DTYPE_OF[args.gemm],
            "data": "synthetic",
            "config": {"workload": args.workload, "model": f"random-init pet-mad-{shape}-like", "atoms_per_gpu": n_atoms,
                       "kept_edges_per_gpu": n_edges, "max_neighbors": max_nb, "gemm_mode": args.gemm,
                       "l2": "working set of saved activations (GBs) exceeds the 126 MB L2; no flush needed",
                       "sharding": "one structure per GPU, no data-path collective"},
            "e2e": {"value": total_atoms * args.steps / e2e_wall, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_wall / args.steps * 1e3},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roof, "classes": classes, "other_modes": modes,
            "cpu_baseline": cpu})
    calc.close()
    if not args.no_splits and args.workload == "diamond1728":
        splits = {}
        for name, fn in (("batch512x64", lambda: measure_batch(args, rank, world, local, dist, 3, 1, tmp.name)),
                         ("diamond13824", lambda: measure_cell(args, "diamond13824", rank, world, local, dist, 2, 1, tmp.name))):
            try:
                splits[name] = fn()
            except Exception as e:  # a split that fails must not take the headline number with it
                if world > 1:
                    raise
                splits[name] = {"failed": f"{type(e).__name__}: {e}"[:500]}
    if rank == 0:
        line["splits"] = splits
        emit(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--gemm", default=os.environ.get("PET_GEMM", "3xtf32"), choices=["native", "tf32", "bf16", "3xtf32"])
    ap.add_argument("--workload", default="diamond1728", choices=sorted(MODEL_OF))
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU arm beside the GPU number")
    ap.add_argument("--no-splits", action="store_true", help="skip the batch and one-cell splits beside the headline")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)
    keep_stdout_for_the_result()
    if args.workload == "diamond13824":
        return run_one_cell(args)
    return run_ours(args)


if __name__ == "__main__":
    main()
