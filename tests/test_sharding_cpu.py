"""Batch sharding across ranks: the host logic, exercised with two gloo ranks on CPU."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from pet_kokkos_b200 import sharding, structures as st  # noqa: E402
from pet_kokkos_b200.calculator import Results  # noqa: E402


def test_partition_is_contiguous_and_balanced():
    costs = [1, 1, 1, 1, 8, 1, 1, 1, 1]
    for world in (1, 2, 3, 4, 8, 16):
        runs = sharding.partition(costs, world)
        assert len(runs) == world and runs[0][0] == 0 and runs[-1][1] == len(costs)
        assert all(a[1] == b[0] for a, b in zip(runs, runs[1:]))
    runs = sharding.partition(np.ones(512), 8)
    assert [e - b for b, e in runs] == [64] * 8
    assert sharding.partition([], 2) == [(0, 0), (0, 0)]


def fake_compute(systems):
    """A stand-in evaluator whose answers are simple functions of the inputs (no GPU here)."""
    n_atoms = [s["n_atoms"] for s in systems]
    e = np.array([s["positions"].sum() for s in systems])
    pa = np.concatenate([s["positions"][:, 0] for s in systems])
    f = np.concatenate([s["positions"] * 2.0 for s in systems])
    w = np.stack([np.full(6, float(s["n_atoms"])) for s in systems])
    sid = np.concatenate([np.full(n, b) for b, n in enumerate(n_atoms)]).astype(np.int32)
    return Results(e, pa, f, w, sid, n_atoms)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    systems = [st.random_mixture(5 + 3 * b, 9.0, seed=b) for b in range(7)]
    out = sharding.compute_sharded(fake_compute, systems, 4.5, rank, world)
    ref = fake_compute(systems)
    ok = all(np.array_equal(getattr(out, k), getattr(ref, k)) for k in ("energy", "per_atom_energy", "forces", "virial", "struct_id"))
    q.put((rank, ok and out.n_atoms == ref.n_atoms))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_batch_equals_whole_batch(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + world
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in procs]
    got = [q.get(timeout=120) for _ in procs]
    [p.join(timeout=60) for p in procs]
    assert sorted(got) == [(r, True) for r in range(world)]
