"""Run under torchrun by tests/test_gpu_exchange.py: exchange-mode decomposition with one process per GPU over NCCL,
checked on every rank against the periodic single-domain answer computed on its own GPU."""
import os
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from pet_kokkos_b200 import Calculator, checkpoint as ck, exchange, structures as st  # noqa: E402


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank = dist.get_rank()
    worst = 0.0
    with tempfile.TemporaryDirectory() as tmp:
        for featurizer in ("feedforward", "residual"):
            jp, sp = ck.write_random_checkpoint(Path(tmp) / f"m_{featurizer}_{rank}", "tiny", featurizer, seed=31, init="scaled")
            calc = Calculator(jp, sp, device=local)
            s = st.diamond(3, jitter=0.05, seed=6)
            ref = calc.compute(s)
            E, F, W = exchange.compute_distributed(calc, s, calc.cutoff)
            e_scale = max(abs(ref.energy[0]), np.abs(ref.per_atom_energy).sum())
            de = abs(E - ref.energy[0]) / e_scale
            df = np.abs(F - ref.forces).max() / max(1.0, np.abs(ref.forces).max())
            dw = np.abs(W - ref.virial[0]).max() / max(1.0, np.abs(ref.virial).max())
            E3, F3, W3 = exchange.compute_distributed(calc, s, calc.cutoff, steps=3)  # a list set once, stepped
            assert abs(E3 - E) <= 1e-12 * e_scale and np.abs(F3 - F).max() == 0.0, "stepping repeats the same bits"
            print(f"rank {rank} {featurizer}: dE {de:.2e} dF {df:.2e} dW {dw:.2e}", flush=True)
            assert de <= 1e-6 and df <= 1e-5 and dw <= 1e-5, (de, df, dw)
            worst = max(worst, de, df, dw)
            # the library's own exchange (pack / ncclSend / ncclRecv / unpack on the calculator's stream, forces folded
            # and reduced on the device): the same rows cross, so the answer differs only by the order of the last sums
            En, Fn, Wn = exchange.compute_distributed(calc, s, calc.cutoff, native=True)
            assert abs(En - E) <= 1e-12 * e_scale and np.abs(Fn - F).max() <= 1e-12 * max(1.0, np.abs(F).max())
            assert np.abs(Wn - W).max() <= 1e-12 * max(1.0, np.abs(W).max())
            En3, Fn3, _ = exchange.compute_distributed(calc, s, calc.cutoff, steps=3, native=True)
            assert En3 == En and np.array_equal(Fn3, Fn), "stepping the native exchange repeats the same bits"
            print(f"rank {rank} {featurizer}: native exchange agrees", flush=True)
            calc.close()
    dist.barrier()
    if rank == 0:
        print("EXCHANGE_NCCL_OK", worst, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
