"""Centre-atom domain decomposition with ghosts: the host logic and the reduction, with gloo ranks on CPU.

The evaluator of each rank's list is the CPU oracle here (no GPU in this test); the sum over ranks must
reproduce the single-domain periodic answer (the reference's tests/test_edges.cpp:117-178: E 1e-5, F 1e-4)."""
import os
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from oracle import neighbors_oracle as nbo, pet_oracle as po  # noqa: E402
from pet_kokkos_b200 import checkpoint as ck, domain, structures as st  # noqa: E402


def oracle_compute_edges(meta, tens):
    h = meta["hypers"]
    s2i = np.asarray(meta["species_to_index"])

    def run(view):
        ed = nbo.build_edges_from_list(view.positions, s2i[view.atomic_numbers], view.offsets, view.neighbors, h["cutoff"],
                                       h["cutoff_width"], h["cutoff_function"], n_local=view.n_local)
        r = po.evaluate(meta, tens, ed, dtype=torch.float64)
        return SimpleNamespace(energy=r["energy"], forces=r["forces"], virial=r["virial"])
    return run


def test_rank_grid_and_ownership():
    assert sorted(domain.rank_grid(8)) == [2, 2, 2] and sorted(domain.rank_grid(4)) == [1, 2, 2] and domain.rank_grid(1) == (1, 1, 1)
    s = st.diamond(3, jitter=0.05)
    for world in (2, 3, 8):
        owned = [set(domain.local_domain(s, r, world, 4.5, 9.0)[1][:domain.local_domain(s, r, world, 4.5, 9.0)[2]]) for r in range(world)]
        assert sum(len(o) for o in owned) == s["n_atoms"] and len(set().union(*owned)) == s["n_atoms"]


def _worker(rank, world, port, jp, sp, q, layers_deep):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(2)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    meta, tens = ck.load_checkpoint(jp, sp)
    s = st.diamond(2, jitter=0.05, seed=3)
    h = meta["hypers"]
    e, F, W = domain.compute_decomposed(oracle_compute_edges(meta, tens), s, h["cutoff"], layers_deep * h["cutoff"], rank, world)
    if rank == 0:
        ref = po.evaluate(meta, tens, [s], dtype=torch.float64)
        q.put((abs(e - ref["energy"][0]) / abs(ref["energy"][0]), np.abs(F - ref["forces"]).max() / np.abs(ref["forces"]).max(),
               np.abs(W - ref["virial"][0]).max() / np.abs(ref["virial"]).max()))
    dist.destroy_process_group()


@pytest.mark.parametrize("layers_deep", [2, 3])
def test_decomposed_cell_equals_periodic_cell(tmp_path, layers_deep):
    """Ghosts one cutoff per message-passing layer deep (the reference's ghost_cutoff) reproduce the periodic
    cell to the reference's own tolerance; one more cutoff (the last layer's combination also reads the
    reverse edge) makes the sum exact to rounding."""
    jp, sp = ck.write_random_checkpoint(tmp_path / "tiny", "tiny", seed=1, init="scaled")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29633 + layers_deep, jp, sp, q, layers_deep)) for r in range(2)]
    [p.start() for p in procs]
    de, df, dw = q.get(timeout=600)
    [p.join(timeout=60) for p in procs]
    if layers_deep == 2:
        assert de <= 1e-5 and df <= 1e-4 and dw <= 1e-4, (de, df, dw)
    else:
        assert de <= 1e-10 and df <= 1e-9 and dw <= 1e-9, (de, df, dw)
