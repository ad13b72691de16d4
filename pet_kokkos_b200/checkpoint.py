"""Seeded random-init PET checkpoints in the reference's own on-disk format.

Format (read by the reference's src/checkpoint.cpp:12-139, written by its
tools/convert_pet.py:342-420): `<name>.json` with `hypers`, `energy_scale`,
`n_species`, `species_to_index`, `composition_energies`; `<name>.safetensors`
with a u64 little-endian header length, a JSON header
{tensor: {dtype, shape, data_offsets}} and raw little-endian F32 data.
Tensor names and shapes follow the reference's loader (src/model.cpp:180-344).

No published weights are available offline, so the benchmark and the parity
tests run on these seeded models.  `init="n002"` draws every tensor from
N(0, 0.02) as the benchmark definition says (norm weights 1 + N(0, 0.02));
`init="scaled"` draws linear weights from N(0, 1/fan_in) so activations stay
O(1) and forces come out O(0.1-1) eV/A, which makes absolute tolerances bite.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np

SHAPES = {
    # name: d_pet, heads, d_feedforward, cutoff
    "xs": dict(d_pet=128, num_heads=4, d_feedforward=256, cutoff=4.5),
    "s": dict(d_pet=256, num_heads=8, d_feedforward=512, cutoff=4.5),
    "l": dict(d_pet=512, num_heads=8, d_feedforward=1024, cutoff=6.0),
    # a tiny model for fast CPU tests
    "tiny": dict(d_pet=32, num_heads=2, d_feedforward=32, cutoff=4.5),
}


def make_hypers(shape="xs", featurizer="feedforward", num_gnn_layers=2, num_attention_layers=2, **over):
    s = dict(SHAPES[shape]) if isinstance(shape, str) else dict(shape)
    D = s["d_pet"]
    ff = featurizer == "feedforward"
    h = {
        "d_pet": D,
        "d_head": D,
        "d_node": 4 * D if ff else D,
        "d_feedforward": s["d_feedforward"],
        "num_heads": s["num_heads"],
        "head_dim": D // s["num_heads"],
        "num_attention_layers": num_attention_layers,
        "num_gnn_layers": num_gnn_layers,
        "num_readout_layers": 1 if ff else num_gnn_layers,
        "normalization": "RMSNorm" if ff else "LayerNorm",
        "activation": "SwiGLU" if ff else "SiLU",
        "transformer_type": "PreLN" if ff else "PostLN",
        "featurizer_type": featurizer,
        "attention_temperature": 1.0,
        "cutoff": s["cutoff"],
        "cutoff_width": 0.5,
        "cutoff_function": "Bump" if ff else "Cosine",
        "num_neighbors_adaptive": None,
        "adaptive_cutoff_method": "grid",
        "cutoff_width_adaptive": 0.5,
        "system_conditioning": False,
        "max_charge": 10,
        "max_spin_multiplicity": 10,
        "zbl": False,
        "long_range_enabled": False,
    }
    h.update(over)
    return h


def tensor_shapes(h, n_species):
    """{name: shape} for every tensor the loader reads (src/model.cpp:256-299)."""
    D, Dn, Dh, F = h["d_pet"], h["d_node"], h["d_head"], h["d_feedforward"]
    G, A, R = h["num_gnn_layers"], h["num_attention_layers"], h["num_readout_layers"]
    ff = h["featurizer_type"] == "feedforward"
    swiglu = h["activation"] == "SwiGLU"
    ln = h["normalization"] == "LayerNorm"
    expanded = Dn != D
    Fc = 2 * Dn
    sh = {}

    def lin(p, o, i):
        sh[p + ".weight"] = (o, i)
        sh[p + ".bias"] = (o,)

    def norm(p, d):
        sh[p + ".weight"] = (d,)
        if ln:
            sh[p + ".bias"] = (d,)

    sh["edge_embedder.weight"] = (n_species, D)
    for L in range(G):
        g = f"gnn_layers.{L}"
        lin(g + ".edge_embedder", D, 4)
        if L > 0:
            sh[g + ".neighbor_embedder.weight"] = (n_species, D)
        lin(g + ".compress.0", D, 2 * D if L == 0 else 3 * D)
        lin(g + ".compress.2", D, D)
        for a in range(A):
            t = f"{g}.trans.layers.{a}"
            lin(t + ".attention.input_linear", 3 * D, D)
            lin(t + ".attention.output_linear", D, D)
            norm(t + ".norm_attention", D)
            norm(t + ".norm_mlp", D)
            lin(t + ".mlp.w_in", 2 * F if swiglu else F, D)
            lin(t + ".mlp.w_out", D, F)
            if expanded:
                lin(t + ".center_contraction", D, Dn)
                lin(t + ".center_expansion", Dn, D)
                norm(t + ".norm_center_features", Dn)
                lin(t + ".center_mlp.w_in", 2 * Fc if swiglu else Fc, Dn)
                lin(t + ".center_mlp.w_out", Dn, Fc)
        if ff:
            sh[f"combination_norms.{L}.weight"] = (2 * D,)
            sh[f"combination_norms.{L}.bias"] = (2 * D,)
            lin(f"combination_mlps.{L}.0", 2 * D, 2 * D)
            lin(f"combination_mlps.{L}.2", D, 2 * D)
    for i in range(R):
        sh[f"node_embedders.{i}.weight"] = (n_species, Dn)
        lin(f"node_heads.energy.{i}.0", Dh, Dn)
        lin(f"node_heads.energy.{i}.2", Dh, Dh)
        lin(f"edge_heads.energy.{i}.0", Dh, D)
        lin(f"edge_heads.energy.{i}.2", Dh, Dh)
        lin(f"node_last_layers.energy.{i}.energy___0", 1, Dh)
        lin(f"edge_last_layers.energy.{i}.energy___0", 1, Dh)
    return sh


def random_tensors(h, n_species, seed=0, init="n002"):
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(h, n_species).items():
        is_norm = ".norm_" in name or name.startswith("combination_norms")
        if is_norm and name.endswith(".weight"):
            t = 1.0 + rng.normal(0.0, 0.02, size=shape)
        elif init == "n002" or len(shape) == 1:
            t = rng.normal(0.0, 0.02 if init == "n002" else 0.1, size=shape)
        elif "embedder.weight" in name or "embedders." in name:
            t = rng.normal(0.0, 1.0, size=shape)
        else:
            t = rng.normal(0.0, 1.0 / np.sqrt(shape[-1]), size=shape)
        out[name] = t.astype(np.float32)
    return out


def write_safetensors(path, tensors, keep_f64=False):
    """F32 throughout; with keep_f64, float64 arrays stay F64 (a converted model's statistics are stored so)."""
    header, off = {}, 0
    wide = lambda v: keep_f64 and np.asarray(v).dtype == np.float64
    for k, v in tensors.items():
        n = v.size * (8 if wide(v) else 4)
        header[k] = {"dtype": "F64" if wide(v) else "F32", "shape": list(v.shape), "data_offsets": [off, off + n]}
        off += n
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for v in tensors.values():
            f.write(np.ascontiguousarray(v, dtype="<f8" if wide(v) else "<f4").tobytes())


def read_safetensors(path):
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for k, e in header.items():
        if k == "__metadata__":
            continue
        b, e_ = e["data_offsets"]
        dt = {"F32": "<f4", "F64": "<f8"}[e["dtype"]]
        out[k] = np.frombuffer(data[b:e_], dtype=dt).reshape(e["shape"]).copy()
    return out


def write_random_checkpoint(prefix, shape="xs", featurizer="feedforward", seed=0, init="n002",
                            n_species=85, energy_scale=1.0, **hyper_over):
    """Write `<prefix>.json` and `<prefix>.safetensors`; returns (json_path, safetensors_path).

    species_to_index maps atomic number Z in 1..n_species to Z-1.  Composition
    energies are seeded and eV-scale per atom so that "relative energy error" is
    measured against a realistic total energy.
    """
    prefix = Path(prefix)
    prefix.parent.mkdir(parents=True, exist_ok=True)
    h = make_hypers(shape, featurizer, **hyper_over)
    rng = np.random.default_rng(seed + 7919)
    meta = {
        "format_version": 1,
        "architecture": "pet",
        "source_model": f"random-init {shape} seed {seed} init {init}",
        "target": "energy",
        "hypers": h,
        "length_unit": "angstrom",
        "energy_unit": "eV",
        "energy_scale": float(energy_scale),
        "n_species": n_species,
        "atomic_types": list(range(1, n_species + 1)),
        "species_to_index": [-1] + list(range(n_species)),
        "composition_energies": [float(x) for x in -rng.uniform(1.0, 12.0, size=n_species)],
    }
    jp, sp = Path(str(prefix) + ".json"), Path(str(prefix) + ".safetensors")
    jp.write_text(json.dumps(meta, indent=2))
    write_safetensors(sp, random_tensors(h, n_species, seed, init))
    return str(jp), str(sp)


def load_checkpoint(json_path, weights_path):
    meta = json.loads(Path(json_path).read_text())
    return meta, read_safetensors(weights_path)
