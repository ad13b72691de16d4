"""Exchange-mode decomposition on the GPU: ranks played as threads of one process on one device (the reference's
ImageExchange test, tests/test_edges.cpp:385-478). Ghosts are one cutoff deep, edge rows cross at every layer, and the
sum over ranks must be the periodic single-domain answer; with the exchange muted it must not be."""
import numpy as np
import pytest

from pet_kokkos_b200 import exchange, structures as st

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("featurizer", ["feedforward", "residual"])
@pytest.mark.parametrize("n,world", [(2, 2), (3, 2), (3, 4)])
def test_exchanged_domains_reproduce_the_periodic_cell(lib_path, models, featurizer, n, world):
    from pet_kokkos_b200 import Calculator
    jp, sp = models("tiny", featurizer, "scaled", 31)
    s = st.diamond(n, jitter=0.05, seed=6)
    whole = Calculator(jp, sp)
    ref = whole.compute(s)
    assert whole.exchange_ghost_cutoff == whole.cutoff
    calcs = [Calculator(jp, sp) for _ in range(world)]
    E, F, W, hub = exchange.compute_threads(calcs, s, whole.cutoff)
    assert abs(E - ref.energy[0]) <= 1e-6 * max(abs(ref.energy[0]), np.abs(ref.per_atom_energy).sum())
    assert np.abs(F - ref.forces).max() <= 1e-5 * max(1.0, np.abs(ref.forces).max())
    assert np.abs(W - ref.virial[0]).max() <= 1e-5 * max(1.0, np.abs(ref.virial).max())
    for c in calcs + [whole]:
        c.close()


def test_muting_the_exchange_changes_the_answer(lib_path, models):
    """tests/test_edges.cpp:470-478: the rows that cross are not decoration."""
    from pet_kokkos_b200 import Calculator
    jp, sp = models("tiny", "feedforward", "scaled", 31)
    s = st.diamond(2, jitter=0.05, seed=6)
    whole = Calculator(jp, sp)
    ref = whole.compute(s)
    calcs = [Calculator(jp, sp) for _ in range(2)]
    # through compute_threads, so that a rank that raises aborts the barrier instead of leaving the other one waiting
    E, _, _, _ = exchange.compute_threads(calcs, s, whole.cutoff, mute=True)
    assert abs(E - ref.energy[0]) > 1e-4 * np.abs(ref.per_atom_energy).sum()
    for c in calcs + [whole]:
        c.close()


def test_a_callback_that_copies_on_the_legacy_stream_is_waited_for(lib_path, models):
    """An engine's `edges` callback may fill `in` with a blocking cudaMemcpy from pageable memory. That call returns once
    the rows are staged, not once they have landed, and runs on the legacy stream, which the calculator's non-blocking
    stream does not wait for by itself: one evaluation in twelve came out 2 % wrong before the library ordered its
    stream after the legacy stream when a callback returns. Thirty evaluations through such a callback must all give
    the bits of the exchange that copies on the calculator's own stream."""
    import ctypes
    from pet_kokkos_b200 import Calculator

    class LegacyStreamExchange(exchange.ThreadExchange):
        def edges(self, out_ptr, in_ptr, n_live, width, stream):
            rt = exchange._rt()
            rt.cudaStreamSynchronize(stream)
            rows = exchange._d2h(out_ptr, n_live * width, np.float32).reshape(n_live, width)
            got = np.ascontiguousarray(rows[self.src_row])  # one rank: every partner row is this rank's own
            assert rt.cudaMemcpy(ctypes.c_void_p(in_ptr), got.ctypes.data, got.nbytes, 1) == 0  # blocking, pageable, legacy stream

    c = Calculator(*models("tiny", "feedforward", "scaled", 5))
    s = st.diamond(3, jitter=0.05, seed=2)
    fields, owner, _, remote = exchange.exchange_domain(s, 0, 1, c.cutoff)
    route = exchange.route([(fields, owner, None, remote)])
    want = c.compute_edges(exchange.view_of(fields, exchange.ThreadExchange(exchange.ThreadHub(route), 0)), True, False)
    for _ in range(30):
        got = c.compute_edges(exchange.view_of(fields, LegacyStreamExchange(exchange.ThreadHub(route), 0)), True, False)
        assert got.energy[0] == want.energy[0] and np.array_equal(got.forces, want.forces)
    c.close()


@pytest.mark.parametrize("featurizer", ["feedforward", "residual"])
def test_native_exchange_on_one_rank_reproduces_the_periodic_cell(lib_path, models, featurizer):
    """The library's own exchange (csrc/nccl_exchange.cu) with a single rank: every ghost is then an image of one of
    the rank's own atoms, so all partner rows take the on-rank path (pack kernel, device copy, unpack kernel), the
    forces are folded onto their owners on the device and the one-rank NCCL communicator reduces nothing. The answer
    must be the periodic cell's; a list set once and stepped must repeat the same bits."""
    from pet_kokkos_b200 import Calculator
    jp, sp = models("tiny", featurizer, "scaled", 31)
    s = st.diamond(2, jitter=0.05, seed=6)
    calc = Calculator(jp, sp)
    ref = calc.compute(s)
    fields, owner, _, remote = exchange.exchange_domain(s, 0, 1, calc.cutoff)
    assert len(remote) > 0
    ex = exchange.NativeNcclExchange(exchange.route([(fields, owner, None, remote)])[0], owner, s["n_atoms"], 0, single=True)
    calc.set_neighbors(exchange.view_of(fields, ex))
    outs = []
    for _ in range(2):
        calc.compute_step_on_device(fields["positions"], None, True)
        outs.append(ex.reduce(calc))
    assert np.array_equal(outs[0], outs[1])
    E, W, F = outs[0][0], outs[0][1:7], outs[0][7:].reshape(-1, 3)
    assert abs(E - ref.energy[0]) <= 1e-6 * max(abs(ref.energy[0]), np.abs(ref.per_atom_energy).sum())
    assert np.abs(F - ref.forces).max() <= 1e-5 * max(1.0, np.abs(ref.forces).max())
    assert np.abs(W - ref.virial[0]).max() <= 1e-5 * max(1.0, np.abs(ref.virial).max())
    ms, calls = ex.timing(True)
    calc.compute_step_on_device(fields["positions"], None, True)
    ms, calls = ex.timing(False)
    assert calls >= 2 and ms > 0.0
    ex.close()
    calc.close()


def test_one_process_per_gpu_over_nccl():
    """The same decomposition with real ranks: torchrun, one process per GPU, rows crossing with NCCL all-to-all.
    Needs two GPUs; NVLS is switched off as for every test in which a rank could leave early."""
    import os
    import subprocess
    import sys
    import torch
    n = min(torch.cuda.device_count(), 4)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "exchange_nccl_worker.py")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29541", worker],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "EXCHANGE_NCCL_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
