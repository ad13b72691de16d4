"""Regenerates tests/golden/*.npz from the CPU oracle (oracle/pet_oracle.py, float64).

Run from the repository root: python tests/golden/make_golden.py
Each file holds the inputs needed to rebuild the case (model shape, seeds), a
SHA-256 of the generated weights (so a drift of the seeded generator is caught
rather than silently compared), and the oracle's float64 outputs.  The reference
itself cannot be built offline (it needs Kokkos), so these vectors pin the
restatement against regressions; they are not outputs of the reference binary.
"""
import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import neighbors_oracle as nbo, pet_oracle as po  # noqa: E402
from pet_kokkos_b200 import checkpoint as ck, structures as st  # noqa: E402

CASES = {
    # name: (shape, featurizer, init, model seed, structure builder)
    "tiny_ff_diamond64": ("tiny", "feedforward", "scaled", 1, lambda: [st.diamond(2, jitter=0.05, seed=0)]),
    "tiny_ff_batch": ("tiny", "feedforward", "n002", 2,
                      lambda: [st.diamond(2, jitter=0.05, seed=1), st.water_box(20, 9.0, seed=2),
                               st.random_mixture(30, 8.0, seed=5)]),
    "tiny_res_diamond64": ("tiny", "residual", "scaled", 3, lambda: [st.diamond(2, jitter=0.05, seed=0)]),
    "xs_ff_diamond64": ("xs", "feedforward", "n002", 0, lambda: [st.diamond(2, jitter=0.05, seed=0)]),
}


def weights_digest(tensors):
    h = hashlib.sha256()
    for k in sorted(tensors):
        h.update(k.encode())
        h.update(np.ascontiguousarray(tensors[k], dtype="<f4").tobytes())
    return h.hexdigest()


def build_case(name, tmp):
    shape, feat, init, seed, make = CASES[name]
    jp, sp = ck.write_random_checkpoint(Path(tmp) / name, shape, feat, seed=seed, init=init)
    meta, tens = ck.load_checkpoint(jp, sp)
    return jp, sp, meta, tens, make()


def main():
    import tempfile
    out = Path(__file__).resolve().parent
    with tempfile.TemporaryDirectory() as tmp:
        for name in CASES:
            jp, sp, meta, tens, systems = build_case(name, tmp)
            r = po.evaluate(meta, tens, systems, dtype=torch.float64)
            ed = r["edges"]
            np.savez_compressed(
                out / f"{name}.npz", digest=np.array(weights_digest(tens)), energy=r["energy"],
                per_atom_energy=r["per_atom_energy"], forces=r["forces"], virial=r["virial"],
                n_edges=np.array(len(ed["center"])), max_neighbors=np.array(ed["max_neighbors"]),
                edge_hash=np.array(hashlib.sha256(ed["raw"].astype("<i8").tobytes()).hexdigest()))
            print(name, r["energy"], len(ed["center"]))


if __name__ == "__main__":
    main()
