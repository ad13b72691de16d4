"""Run by tests/test_gpu_poison.py, once plain and once with the scratch pools poisoned: every kind of evaluation the
library has, its results written to one .npz for the test to compare."""
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from oracle import neighbors_oracle as nbo  # noqa: E402
from pet_kokkos_b200 import Calculator, EdgeListView, checkpoint as ck, exchange, structures as st  # noqa: E402


def main(workdir, out_path):
    out = {}

    def keep(tag, r):
        out[tag + "_e"], out[tag + "_f"], out[tag + "_w"] = np.asarray(r.energy), np.asarray(r.forces), np.asarray(r.virial)

    batch = [st.diamond(2, jitter=0.05, seed=1), st.water_box(8, 6.2, seed=2), st.diamond(1, shear=0.3), st.diamond(3, jitter=0.02, seed=3)]
    for featurizer in ("feedforward", "residual"):
        jp, sp = ck.write_random_checkpoint(Path(workdir) / featurizer, "tiny", featurizer, seed=5, init="scaled")
        for tier in ("never", "wide", "layers"):
            for mode in ("native", "3xtf32"):
                c = Calculator(jp, sp, recompute=tier, gemm=mode)
                keep(f"{featurizer}_{tier}_{mode}_batch", c.compute(batch))
                keep(f"{featurizer}_{tier}_{mode}_again", c.compute(batch[:2]))  # a smaller pass in the pools of a larger
                c.close()
        c = Calculator(jp, sp, cache_neighbors=True)
        c.stage(batch)
        c.compute_staged(True)
        keep(f"{featurizer}_staged", c.fetch())
        c.update_staged(np.concatenate([s["positions"] + 0.01 for s in batch]))
        c.compute_staged(True)
        keep(f"{featurizer}_cached", c.fetch())
        # an engine's list with shifts, stepped, with edge gradients; then one rank over an exchange
        s = st.diamond(2, jitter=0.05, seed=9)
        idx, _, _ = nbo.brute_force_edges(s, c.cutoff + 0.5)
        idx = idx[np.lexsort((idx[:, 4], idx[:, 3], idx[:, 2], idx[:, 1], idx[:, 0]))]
        off = np.concatenate([[0], np.cumsum(np.bincount(idx[:, 0], minlength=s["n_atoms"]))])
        c.set_neighbors(EdgeListView(s["positions"], s["atomic_numbers"], off, idx[:, 1], idx[:, 2:5], s["cell"]))
        r = c.compute_step(s["positions"] + 0.01, s["cell"], True, True)
        keep(f"{featurizer}_step", r)
        out[f"{featurizer}_step_g"] = np.asarray(r.edge_gradient)
        E, F, W, _ = exchange.compute_threads([c], s, c.cutoff)
        out[f"{featurizer}_exchange_e"], out[f"{featurizer}_exchange_f"], out[f"{featurizer}_exchange_w"] = np.float64(E), F, W
        c.close()
    jp, sp = ck.write_random_checkpoint(Path(workdir) / "adaptive", "tiny", "feedforward", seed=6, init="scaled",
                                        num_neighbors_adaptive=16.0, adaptive_cutoff_method="grid", cutoff=5.5)
    c = Calculator(jp, sp)
    keep("adaptive", c.compute(batch))
    c.close()
    np.savez(out_path, **out)
    print("POISON_WORKER_OK", len(out))


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
