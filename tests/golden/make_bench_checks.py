"""Regenerates tests/golden/bench_checks.npz: the reference's answers that bench.py checks itself against before it
times the two multi-GPU splits.

Run from the repository root, after oracle/build_ref.sh has compiled the reference:
    python tests/golden/make_bench_checks.py

The 512-structure batch and the 13824-atom cell are far too large for the reference's CPU build to evaluate in a
benchmark run, so bench.py checks a sub-sample of each on the very code path it is about to time:
  batch_*  the first four structures of the seeded 512-structure batch, the benchmark's pet-mad-s-shaped model;
  cell_*   a 512-atom jittered diamond (4x4x4 cells) with the benchmark's pet-omat-l-shaped model (cutoff 6 A, about
           159 neighbours per atom, as in the 13824-atom cell), evaluated by bench.py whole on one GPU or decomposed
           over the ranks exactly as the big cell is.
Outputs are Calculator::compute of the reference's CBLAS build (fp32 network, fp64 geometry). The models are the
seeded random-init checkpoints bench.py writes; their SHA-256 is stored so that a drift of the generator is caught.
"""
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))
from make_golden import weights_digest  # noqa: E402
from oracle import reference_lib as rl  # noqa: E402
from pet_kokkos_b200 import checkpoint as ck, structures as st  # noqa: E402


def main():
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        for tag, shape, systems in (("batch", "s", st.workload("batch512x64")[:4]),
                                    ("cell", "l", [st.diamond(4, jitter=0.05, seed=0)])):
            jp, sp = ck.write_random_checkpoint(Path(tmp) / f"bench_{shape}", shape, seed=0, init="n002")
            meta, tens = ck.load_checkpoint(jp, sp)
            r = rl.ReferenceCalculator(str(jp), str(sp), blas=True).compute(systems)
            out[f"{tag}_digest"] = weights_digest(tens)
            for k in ("energy", "per_atom_energy", "forces", "virial"):
                out[f"{tag}_{k}"] = np.asarray(r[k])
            # what the network itself adds up to, per structure at most: the scale its fp32 rounding is relative to
            z = np.concatenate([s["atomic_numbers"] for s in systems])
            comp = np.asarray(meta["composition_energies"])[np.asarray(meta["species_to_index"])[z]]
            out[f"{tag}_network_scale"] = float(np.abs(np.asarray(r["per_atom_energy"]) - comp).sum() / len(systems))
            print(tag, "E", r["energy"], "max |F|", np.abs(r["forces"]).max())
    np.savez_compressed(Path(__file__).resolve().parent / "bench_checks.npz", **out)


if __name__ == "__main__":
    main()
