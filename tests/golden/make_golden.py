"""Regenerates tests/golden/*.npz.

Run from the repository root, after oracle/build_ref.sh has compiled the reference:
    python tests/golden/make_golden.py

Each file holds what rebuilds the case (model shape, seeds; a SHA-256 of the generated
weights, so a drift of the seeded generator is caught rather than silently compared) and
two sets of outputs on it:
  ref_*   the reference's own evaluator (peterspackman/pet-kokkos, Calculator::compute,
          fp32 network / fp64 geometry) compiled for the host into oracle/_ref/libpet_ref.so
          -- these pin both the CPU restatement and the CUDA path to the reference;
  energy, forces, ...  the CPU restatement (oracle/pet_oracle.py) in float64, the
          rounding-free answer the fp32 implementations scatter around.
The checkpoints are random-initialised in the reference's file format; the reference
reads the very files the CUDA path reads.
"""
import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import pet_oracle as po, reference_lib as rl  # noqa: E402
from pet_kokkos_b200 import checkpoint as ck, structures as st  # noqa: E402


def water_cluster(n, seed):
    """n water molecules of a seeded box, as an open (non-periodic) cluster."""
    s = st.water_box(n, 3.2 * n ** (1.0 / 3.0), seed=seed)
    return st.make_system(s["atomic_numbers"], s["positions"], np.eye(3) * 50.0, pbc=(False, False, False))


CASES = {
    # name: (shape, featurizer, init, model seed, structure builder, overrides of the hypers / energy_scale)
    "tiny_ff_diamond64": ("tiny", "feedforward", "scaled", 1, lambda: [st.diamond(2, jitter=0.05, seed=0)], {}),
    "tiny_ff_batch": ("tiny", "feedforward", "n002", 2,
                      lambda: [st.diamond(2, jitter=0.05, seed=1), st.water_box(20, 9.0, seed=2),
                               st.random_mixture(30, 8.0, seed=5)], {}),
    "tiny_res_diamond64": ("tiny", "residual", "scaled", 3, lambda: [st.diamond(2, jitter=0.05, seed=0)], {}),
    "xs_ff_diamond64": ("xs", "feedforward", "n002", 0, lambda: [st.diamond(2, jitter=0.05, seed=0)], {}),
    "tiny_ff_sheared216": ("tiny", "feedforward", "scaled", 4,
                           lambda: [st.diamond(3, shear=0.3, jitter=0.04, seed=3)], {}),
    "tiny_ff_cluster": ("tiny", "feedforward", "scaled", 5, lambda: [water_cluster(12, 4)], {}),
    "tiny_ff_cosine_scaled": ("tiny", "feedforward", "scaled", 6,
                              lambda: [st.random_mixture(40, 7.5, seed=6), st.diamond(2, jitter=0.08, seed=7)],
                              {"cutoff_function": "Cosine", "energy_scale": 2.5, "num_gnn_layers": 3}),
    "tiny_res_batch": ("tiny", "residual", "scaled", 8,
                       lambda: [st.water_box(16, 8.0, seed=8), st.random_mixture(24, 7.0, seed=9), water_cluster(5, 10)],
                       {}),
    "xs_res_water": ("xs", "residual", "scaled", 9, lambda: [st.water_box(24, 9.0, seed=11)], {}),
    "s_ff_diamond64": ("s", "feedforward", "scaled", 10, lambda: [st.diamond(2, jitter=0.05, seed=12)], {}),
}


def weights_digest(tensors):
    h = hashlib.sha256()
    for k in sorted(tensors):
        h.update(k.encode())
        h.update(np.ascontiguousarray(tensors[k], dtype="<f4").tobytes())
    return h.hexdigest()


def build_case(name, tmp):
    shape, feat, init, seed, make, over = CASES[name]
    over = dict(over)
    scale = over.pop("energy_scale", 1.0)
    jp, sp = ck.write_random_checkpoint(Path(tmp) / name, shape, feat, seed=seed, init=init, energy_scale=scale, **over)
    meta, tens = ck.load_checkpoint(jp, sp)
    return jp, sp, meta, tens, make()


def main():
    import tempfile
    out = Path(__file__).resolve().parent
    with tempfile.TemporaryDirectory() as tmp:
        for name in CASES:
            jp, sp, meta, tens, systems = build_case(name, tmp)
            r = po.evaluate(meta, tens, systems, dtype=torch.float64)
            ref = rl.ReferenceCalculator(str(jp), str(sp)).compute(systems)
            ed = r["edges"]
            np.savez_compressed(
                out / f"{name}.npz", digest=np.array(weights_digest(tens)), energy=r["energy"],
                per_atom_energy=r["per_atom_energy"], forces=r["forces"], virial=r["virial"],
                ref_energy=ref["energy"], ref_per_atom_energy=ref["per_atom_energy"], ref_forces=ref["forces"],
                ref_virial=ref["virial"],
                n_edges=np.array(len(ed["center"])), max_neighbors=np.array(ed["max_neighbors"]),
                edge_hash=np.array(hashlib.sha256(ed["raw"].astype("<i8").tobytes()).hexdigest()))
            de = np.abs(ref["energy"] - r["energy"]).max() / np.abs(r["energy"]).max()
            df = np.abs(ref["forces"] - r["forces"]).max() / max(1.0, np.abs(r["forces"]).max())
            dw = np.abs(ref["virial"] - r["virial"]).max() / max(1.0, np.abs(r["virial"]).max())
            print(f"{name}: E {r['energy']} edges {len(ed['center'])}  reference vs float64 restatement: "
                  f"dE/E {de:.2e} dF/max(1,F) {df:.2e} dW/max(1,W) {dw:.2e}")


if __name__ == "__main__":
    main()
