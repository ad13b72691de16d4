"""TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's PET energy/forces/virial pass.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import
this module; the product (pet_kokkos_b200) never does.

The forward is restated op by op from the reference (citations on each
function).  Forces and the virial come from the per-edge gradient g = dE/dv,
obtained here by reverse-mode differentiation of that forward (torch autograd
on CPU) rather than by the reference's hand-written backward: an independent
derivation of the same quantity, folded exactly as the reference folds it
(src/forces.cpp:50-70, src/model.cpp:983-993).  dtype=float32 reproduces the
reference's mixed precision (fp32 network, fp64 geometry and sums);
dtype=float64 is the rounding-free truth both fp32 paths are compared against.

PARITY PINNED against the reference's own code: its unmodified sources are
compiled for the host (oracle/build_ref.sh -> oracle/_ref/libpet_ref.so, g++
against the Kokkos stand-in in oracle/kokkos_host/) and this restatement is held
to that library's Calculator::compute, compute_edges and set_neighbors +
compute_step outputs -- live in tests/test_reference_pin.py, and through the ref_*
arrays of the committed fixtures (tests/golden/*.npz, written by
tests/golden/make_golden.py from that library) where the library is not present.
The reference's golden files (tests/golden/pet-*.json) need published weights
that are not available offline; random-initialised checkpoints in the
reference's file format, read by both sides, take their place.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from . import neighbors_oracle as nbo

RMS_EPS = 1.1920928955078125e-07  # src/ops.hpp:195
LN_EPS = 1e-5                     # src/ops.hpp:196


class Weights:
    """Loads and folds weights as src/model.cpp:180-344 does."""

    def __init__(self, meta, tensors, dtype=torch.float32):
        self.h = meta["hypers"]
        self.meta = meta
        self.dtype = dtype
        self.t = {k: torch.from_numpy(np.asarray(v, np.float64)) for k, v in tensors.items()}
        self.folded = {}
        for L in range(self.h["num_gnn_layers"]):
            self._fold_compress(L)

    def __call__(self, name):
        if name in self.folded:
            return self.folded[name].to(self.dtype)
        # weights are stored as float32 on the device whatever the fold's precision
        return self.t[name].to(torch.float32).to(self.dtype)

    def _fold_compress(self, L):
        """CompressFold, src/model.cpp:233-254, in double then rounded to float32."""
        g = f"gnn_layers.{L}"
        W, b0 = self.t[g + ".compress.0.weight"], self.t[g + ".compress.0.bias"]
        We, be = self.t[g + ".edge_embedder.weight"], self.t[g + ".edge_embedder.bias"]
        T = self.t["edge_embedder.weight" if L == 0 else g + ".neighbor_embedder.weight"]
        D = W.shape[0]
        f32 = lambda x: x.to(torch.float32)
        self.folded[g + ".compress.0@x4"] = f32(W[:, :D] @ We)            # [D,4]
        self.folded[g + ".compress.0@b"] = f32(b0 + W[:, :D] @ be)         # [D]
        self.folded[g + ".compress.0@tab"] = f32(T @ W[:, D:2 * D].T)      # [ns,D]
        if L > 0:
            self.folded[g + ".compress.0@in"] = f32(W[:, 2 * D:3 * D])    # [D,D]


def linear(x, W, b=None):
    """out = in W^T + b (src/ops.cpp:26)."""
    y = x @ W.T
    return y if b is None else y + b


def silu(x):
    return x * torch.sigmoid(x)


def rmsnorm(x, w):
    """src/ops.hpp:381-401 with bias empty: x * w / sqrt(mean(x^2) + 2^-23)."""
    inv = 1.0 / torch.sqrt((x * x).mean(-1, keepdim=True) + RMS_EPS)
    return x * inv * w


def layernorm(x, w, b):
    """src/ops.hpp:381-401 with a bias: two-pass variance, eps 1e-5."""
    mu = x.mean(-1, keepdim=True)
    xc = x - mu
    inv = 1.0 / torch.sqrt((xc * xc).mean(-1, keepdim=True) + LN_EPS)
    return xc * inv * w + b


def swiglu_mlp(x, w_in, b_in, w_out, b_out):
    """src/ops.cpp:248-279: pre = x W_in^T + b_in, rows [v ; g]; h = v * sigmoid(g); out = h W_out^T + b_out."""
    pre = linear(x, w_in, b_in)
    F = pre.shape[-1] // 2
    h = pre[..., :F] * torch.sigmoid(pre[..., F:])
    return linear(h, w_out, b_out)


def bump_cutoff_t(d, rc, width, dtype):
    """include/pet/cutoff.hpp:17-22, differentiable; transcendentals in the network's dtype."""
    x = ((d - (rc - width)) / width).to(dtype)
    xs = x.clamp(1e-6, 1 - 1e-6)
    mid = 0.5 * (1.0 + torch.tanh(1.0 / torch.tan(math.pi * xs)))
    return torch.where(x <= 0, torch.ones_like(mid), torch.where(x >= 1, torch.zeros_like(mid), mid))


def cosine_cutoff_t(d, rc, width, dtype):
    """include/pet/cutoff.hpp:23-26."""
    x = ((d - (rc - width)) / width).to(dtype).clamp(0.0, 1.0)
    return 0.5 * (1.0 + torch.cos(math.pi * x))


def bump_dcutoff_dr_t(d, rc, width, dtype):
    """include/pet/cutoff.hpp:44-51, the slope the solver root-finds with (not differentiated)."""
    x = ((d - (rc - width)) / width).to(dtype)
    ps = math.pi * x.clamp(1e-6, 1 - 1e-6)
    si = torch.sin(ps)
    tt = torch.tanh(torch.cos(ps) / si)
    val = 0.5 * (1.0 - (tt * tt).double()) * ((math.pi / (si * si)) / width).double()
    return torch.where((x <= 0) | (x >= 1), torch.zeros_like(val), val)


def adaptive_cutoffs_t(h, N, center, dist, dtype):
    """Each atom's adaptive cutoff as a differentiable function of ALL its raw distances.

    Solver (src/device_neighbors.cpp:26-67): the iterations run without gradient; the last line, one
    implicit-function step cutoff = r - (n_total(r) - target) / dn with r and dn held constant, carries it
    (src/forces.cpp:93-110). Grid (src/device_neighbors.cpp:69-136; backward src/forces.cpp:111-196): differentiated
    as written. Both taper the neighbour count with the bump whatever the model's own cutoff function."""
    rmax, width, target = h["cutoff"], h["cutoff_width_adaptive"], float(h["num_neighbors_adaptive"])
    c = torch.from_numpy(np.asarray(center))
    bump = lambda d, r: bump_cutoff_t(d, r, width, dtype).double()
    if h["adaptive_cutoff_method"] == "solver":
        lo_bound = rmax * nbo.SOLVER_MIN_CUTOFF_FACTOR

        def count(r, d):
            n = torch.zeros(N, dtype=torch.float64).index_add(0, c, bump(d, r[c]))
            dn = torch.zeros(N, dtype=torch.float64).index_add(0, c, bump_dcutoff_dr_t(d, r[c], width, dtype))
            x = r / rmax
            return n + target * x ** 3, dn + 3.0 * target * x * x / rmax
        with torch.no_grad():
            dd = dist.detach()
            r_lo, r_hi = torch.zeros(N, dtype=torch.float64), torch.full((N,), rmax, dtype=torch.float64)
            r = torch.full((N,), 0.5 * rmax, dtype=torch.float64)
            for _ in range(nbo.SOLVER_ITERS):
                n, dn = count(r, dd)
                f = n - target
                r_lo, r_hi = torch.where(f <= 0, r, r_lo), torch.where(f <= 0, r_hi, r)
                newton = r - f / dn.clamp(min=nbo.SOLVER_DN_FLOOR)
                r = torch.where((newton >= r_lo) & (newton <= r_hi), newton, 0.5 * (r_lo + r_hi))
            _, dn = count(r, dd)
            dn_root = dn.clamp(min=nbo.SOLVER_DN_FLOOR)
        n = torch.zeros(N, dtype=torch.float64).index_add(0, c, bump(dist, r[c])) + target * (r / rmax) ** 3
        return (r - (n - target) / dn_root).clamp(lo_bound, rmax)
    probes = torch.from_numpy(nbo.adaptive_probes(rmax, width))
    P = len(probes)
    if P == 0:
        return torch.full((N,), rmax, dtype=torch.float64)
    eff = torch.stack([torch.zeros(N, dtype=torch.float64).index_add(0, c, bump(dist, torch.full_like(dist, float(probes[p]))))
                       for p in range(P)], 1)
    x = torch.arange(P, dtype=torch.float64) / (P - 1) if P > 1 else torch.zeros(1, dtype=torch.float64)
    diff = eff - target + target * x ** 3
    if P == 1:
        grad = diff.abs() * 0.5 + 1e-12
    else:
        g = torch.cat([(diff[:, 1] - diff[:, 0])[:, None], 0.5 * (diff[:, 2:] - diff[:, :-2]), (diff[:, -1] - diff[:, -2])[:, None]], 1)
        grad = g.abs().clamp(min=1e-12)
    w = torch.softmax(-0.5 * (diff / grad) ** 2, 1)
    return (w * probes).sum(1)


def attention(qkv, cf, tok_index, tok_valid, N, H, hd, temperature):
    """Per-atom multi-head attention with the log-cutoff key bias.

    src/attention.cpp:207-266 (Forward): for atom n, head h, query slot sq over
    key slots s < count(n): score = sc * q.k + log(cf[n,s]); keys with cf <= 0
    are skipped; a query on an edge with cf <= 0 outputs zero.  tok_index [N,S]
    maps (atom, slot) to a token row, tok_valid marks real slots.
    Returns merged [T, D].
    """
    T, D3 = qkv.shape
    D = D3 // 3
    S = tok_index.shape[1]
    sc = 1.0 / (math.sqrt(hd) * temperature)
    g = qkv[tok_index.clamp(min=0)]                                  # [N,S,3D]
    q = g[..., :D].reshape(N, S, H, hd).permute(0, 2, 1, 3)
    k = g[..., D:2 * D].reshape(N, S, H, hd).permute(0, 2, 1, 3)
    v = g[..., 2 * D:].reshape(N, S, H, hd).permute(0, 2, 1, 3)
    live = tok_valid & (cf > 0)                                       # [N,S]
    bias = torch.where(live, torch.log(cf.clamp(min=1e-38)), torch.full_like(cf, -float("inf")))
    s = sc * (q @ k.transpose(-1, -2)) + bias[:, None, None, :]
    p = torch.softmax(s, dim=-1)
    o = (p @ v).permute(0, 2, 1, 3).reshape(N, S, D)
    o = torch.where(live[..., None], o, torch.zeros_like(o))         # dead queries give zero
    merged = torch.zeros(T, D, dtype=qkv.dtype)
    rows = tok_index[tok_valid]
    merged[rows] = o[tok_valid]
    return merged


def token_index(off, N):
    """Tokens (src/ops.hpp:31-37): slot 0 is row n, slot s is row N + off(n) + s - 1."""
    cnt = (off[1:] - off[:-1]).astype(np.int64)
    S = int(cnt.max() if N else 0) + 1
    idx = np.full((N, S), -1, np.int64)
    idx[:, 0] = np.arange(N)
    ar = np.arange(S - 1)[None, :]
    m = ar < cnt[:, None]
    idx[:, 1:][m] = (N + off[:-1, None] + ar)[m]
    return idx


def forward_feedforward(W: Weights, ed, vec, want=None, rc=None):
    """The feedforward featurizer's energy: src/feedforward.cpp:34-197 (ff_layer) and :338-394 (ff_pass).

    ed: packed edges from neighbors_oracle.build_edges; vec: [E,3] float64 tensor
    (the differentiable input).  Returns per-atom energies (float64) and a dict
    of named intermediates when `want` is a dict.
    """
    h, dt = W.h, W.dtype
    N, E = ed["n_atoms"], len(ed["center"])
    D, Dn, H, hd = h["d_pet"], h["d_node"], h["num_heads"], h["head_dim"]
    G, A = h["num_gnn_layers"], h["num_attention_layers"]
    species = torch.from_numpy(ed["species"])
    nb_species = torch.from_numpy(ed["nb_species"])
    rev = torch.from_numpy(ed["reverse"])
    off = ed["off"]
    keep = lambda k, v: want.__setitem__(k, v.detach().clone()) if want is not None else None

    dist = torch.sqrt((vec * vec).sum(-1))
    fn = bump_cutoff_t if h["cutoff_function"] == "Bump" else cosine_cutoff_t
    cut = fn(dist, h["cutoff"] if rc is None else rc, h["cutoff_width"], dt)   # [E] network dtype; rc: per-edge cutoffs
    tok_index = torch.from_numpy(token_index(off, N))
    tok_valid = tok_index >= 0
    S = tok_index.shape[1]
    cf = torch.zeros(N, S, dtype=dt)
    cf[:, 0] = 1.0
    ecol = torch.from_numpy(np.arange(E) - off[ed["center"]] + 1)
    cf = cf.index_put((torch.from_numpy(ed["center"]), ecol), cut)   # src/device_neighbors.cpp:319-323
    x4 = torch.cat([vec, dist[:, None]], 1).to(dt)                    # (v, |v|) cast to the network type

    node = W("node_embedders.0.weight")[species]                      # src/feedforward.cpp:351-353
    input_edge = W("edge_embedder.weight")[nb_species]
    for L in range(G):
        g = f"gnn_layers.{L}"
        # compress (src/ops.cpp:326-365)
        z = W(g + ".compress.0@b") + W(g + ".compress.0@tab")[nb_species] + x4 @ W(g + ".compress.0@x4").T
        if L > 0:
            z = z + input_edge @ W(g + ".compress.0@in").T
        cpre = silu(z)
        et = linear(cpre, W(g + ".compress.2.weight"), W(g + ".compress.2.bias"))
        keep(f"et{L}", et)
        node_cur, edge_cur = node, et
        for a in range(A):
            t = f"{g}.trans.layers.{a}"
            input_node = linear(node_cur, W(t + ".center_contraction.weight"), W(t + ".center_contraction.bias"))
            tokens = torch.cat([input_node, edge_cur], 0)
            attn_in = rmsnorm(tokens, W(t + ".norm_attention.weight"))
            qkv = linear(attn_in, W(t + ".attention.input_linear.weight"), W(t + ".attention.input_linear.bias"))
            merged = attention(qkv, cf, tok_index, tok_valid, N, H, hd, h["attention_temperature"])
            keep(f"merged{L}_{a}", merged)
            attn_out = linear(merged, W(t + ".attention.output_linear.weight"), W(t + ".attention.output_linear.bias"))
            node_exp = linear(attn_out[:N], W(t + ".center_expansion.weight"), W(t + ".center_expansion.bias"))
            eps = attn_out[N:] + edge_cur
            edge_norm = rmsnorm(eps, W(t + ".norm_mlp.weight"))
            node_res = node_cur + node_exp
            node_norm = rmsnorm(node_res, W(t + ".norm_center_features.weight"))
            node_next = node_res + swiglu_mlp(node_norm, W(t + ".center_mlp.w_in.weight"), W(t + ".center_mlp.w_in.bias"),
                                              W(t + ".center_mlp.w_out.weight"), W(t + ".center_mlp.w_out.bias"))
            edge_next = eps + swiglu_mlp(edge_norm, W(t + ".mlp.w_in.weight"), W(t + ".mlp.w_in.bias"),
                                         W(t + ".mlp.w_out.weight"), W(t + ".mlp.w_out.bias"))
            node_cur, edge_cur = node_next, edge_next
            keep(f"node{L}_{a}", node_cur)
            keep(f"edge{L}_{a}", edge_cur)
        node = node_cur
        out_edge = edge_cur
        input_edge = input_edge + out_edge                              # src/feedforward.cpp:182-193
        partner = torch.where((rev >= 0)[:, None], out_edge[rev.clamp(min=0)], torch.zeros_like(out_edge))
        comb = layernorm(torch.cat([out_edge, partner], 1), W(f"combination_norms.{L}.weight"),
                         W(f"combination_norms.{L}.bias"))
        cph = silu(linear(comb, W(f"combination_mlps.{L}.0.weight"), W(f"combination_mlps.{L}.0.bias")))
        input_edge = input_edge + linear(cph, W(f"combination_mlps.{L}.2.weight"), W(f"combination_mlps.{L}.2.bias"))
        keep(f"input_edge{L}", input_edge)

    # readout (src/model.cpp:656-691; src/ops.cpp:406-425)
    def head(x, p, last):
        x = silu(linear(x, W(p + ".0.weight"), W(p + ".0.bias")))
        x = silu(linear(x, W(p + ".2.weight"), W(p + ".2.bias")))
        return linear(x, W(last + ".weight"), W(last + ".bias"))
    node_pred = head(node, "node_heads.energy.0", "node_last_layers.energy.0.energy___0")[:, 0]
    edge_pred = head(input_edge, "edge_heads.energy.0", "edge_last_layers.energy.0.energy___0")[:, 0]
    keep("node_pred", node_pred)
    keep("edge_pred", edge_pred)
    contrib = cut.double() * edge_pred.double()
    net = node_pred.double().index_add(0, torch.from_numpy(ed["center"]), contrib)
    net = net.to(dt)                                                   # "Net(s)": rounded to the network type
    comp = torch.tensor(W.meta["composition_energies"], dtype=torch.float64)
    per_atom = W.meta["energy_scale"] * net.double() + comp[species]
    return per_atom


def forward_residual(W: Weights, ed, vec, want=None, rc=None):
    """The residual featurizer: src/residual.cpp:13-62 (residual_layer) and :64-133 (residual_pass forward)."""
    h, dt = W.h, W.dtype
    N, E = ed["n_atoms"], len(ed["center"])
    D, H, hd = h["d_pet"], h["num_heads"], h["head_dim"]
    G, A = h["num_gnn_layers"], h["num_attention_layers"]
    species = torch.from_numpy(ed["species"])
    nb_species = torch.from_numpy(ed["nb_species"])
    rev = torch.from_numpy(ed["reverse"])
    off = ed["off"]
    center = torch.from_numpy(ed["center"])
    dist = torch.sqrt((vec * vec).sum(-1))
    fn = bump_cutoff_t if h["cutoff_function"] == "Bump" else cosine_cutoff_t
    cut = fn(dist, h["cutoff"] if rc is None else rc, h["cutoff_width"], dt)
    tok_index = torch.from_numpy(token_index(off, N))
    tok_valid = tok_index >= 0
    S = tok_index.shape[1]
    cf = torch.zeros(N, S, dtype=dt)
    cf[:, 0] = 1.0
    ecol = torch.from_numpy(np.arange(E) - off[ed["center"]] + 1)
    cf = cf.index_put((center, ecol), cut)
    x4 = torch.cat([vec, dist[:, None]], 1).to(dt)

    def ln(x, key):
        return layernorm(x, W(key + ".weight"), W(key + ".bias"))

    def head(x, i, side):
        p, last = f"{side}_heads.energy.{i}", f"{side}_last_layers.energy.{i}.energy___0"
        x = silu(linear(x, W(p + ".0.weight"), W(p + ".0.bias")))
        x = silu(linear(x, W(p + ".2.weight"), W(p + ".2.bias")))
        return linear(x, W(last + ".weight"), W(last + ".bias"))[:, 0]

    input_edge = W("edge_embedder.weight")[nb_species]
    net = torch.zeros(N, dtype=dt)
    keep = lambda k, v: want.__setitem__(k, v.detach().clone()) if want is not None else None
    for L in range(G):
        g = f"gnn_layers.{L}"
        z = W(g + ".compress.0@b") + W(g + ".compress.0@tab")[nb_species] + x4 @ W(g + ".compress.0@x4").T
        if L > 0:
            z = z + input_edge @ W(g + ".compress.0@in").T
        et = linear(silu(z), W(g + ".compress.2.weight"), W(g + ".compress.2.bias"))
        tokens = torch.cat([W(f"node_embedders.{L}.weight")[species], et], 0)
        for a in range(A):
            t = f"{g}.trans.layers.{a}"
            qkv = linear(tokens, W(t + ".attention.input_linear.weight"), W(t + ".attention.input_linear.bias"))
            merged = attention(qkv, cf, tok_index, tok_valid, N, H, hd, h["attention_temperature"])
            s1 = linear(merged, W(t + ".attention.output_linear.weight"), W(t + ".attention.output_linear.bias")) + tokens
            tok_a = ln(s1, t + ".norm_attention")
            s2 = linear(silu(linear(tok_a, W(t + ".mlp.w_in.weight"), W(t + ".mlp.w_in.bias"))),
                        W(t + ".mlp.w_out.weight"), W(t + ".mlp.w_out.bias")) + tok_a
            tokens = ln(s2, t + ".norm_mlp")
        node_feat, edge_feat = tokens[:N], tokens[N:]
        keep(f"tokens{L}", tokens)
        node_pred, edge_pred = head(node_feat, L, "node"), head(edge_feat, L, "edge")
        keep(f"node_pred{L}", node_pred)
        keep(f"edge_pred{L}", edge_pred)
        s = node_pred.double().index_add(0, center, cut.double() * edge_pred.double())
        net = (net.double() + s).to(dt) if L > 0 else s.to(dt)        # readout_accumulate(acc = i > 0)
        keep(f"net{L}", net)
        if L + 1 < G:                                                  # src/residual.cpp:123-132
            partner = torch.where((rev >= 0)[:, None], edge_feat[rev.clamp(min=0)], torch.zeros_like(edge_feat))
            input_edge = 0.5 * (input_edge + partner)
    comp = torch.tensor(W.meta["composition_energies"], dtype=torch.float64)
    return W.meta["energy_scale"] * net.double() + comp[species]


def _evaluate_adaptive(h, W, fwd, ed, dtype, forces, want):
    """With an adaptive cutoff every raw edge's distance shapes its atom's cutoff, so the differentiable input is the
    raw list, kept or not, and forces and virial are folded over it (src/forces.cpp:80-260,308-341)."""
    N, B = ed["n_atoms"], ed["n_struct"]
    raw_vec = torch.from_numpy(ed["raw_vec"]).clone().requires_grad_(forces)
    kept = torch.from_numpy(ed["kept_idx"])
    ri, rj = torch.from_numpy(ed["raw_center"]), torch.from_numpy(ed["raw_neighbor"])
    with torch.set_grad_enabled(forces):
        raw_dist = torch.sqrt((raw_vec * raw_vec).sum(-1))
        acut = adaptive_cutoffs_t(h, N, ed["raw_center"], raw_dist, dtype)
        rc = 0.5 * (acut[ri] + acut[rj])[kept]
        per_atom = fwd(W, ed, raw_vec[kept], want, rc=rc)
        sid = torch.from_numpy(ed["struct_id"])
        energy = torch.zeros(B, dtype=torch.float64).index_add(0, sid, per_atom)
        out = {"energy": energy.detach().numpy(), "per_atom_energy": per_atom.detach().numpy(), "edges": ed,
               "atom_cutoff": acut.detach().numpy()}
        if not forces:
            return out
        (g,) = torch.autograd.grad(per_atom.sum(), raw_vec)
    g = g.double()
    rev = torch.from_numpy(ed["raw_reverse"])
    back = torch.where((rev >= 0)[:, None], g[rev.clamp(min=0)], torch.zeros_like(g))
    F = torch.zeros(N, 3, dtype=torch.float64).index_add(0, ri, g - back)
    w9 = (raw_vec.detach()[:, :, None] * g[:, None, :]).reshape(-1, 9)
    W9 = torch.zeros(B, 9, dtype=torch.float64).index_add(0, sid[ri], w9)
    voigt = torch.stack([W9[:, 0], W9[:, 4], W9[:, 8], 0.5 * (W9[:, 1] + W9[:, 3]), 0.5 * (W9[:, 2] + W9[:, 6]),
                         0.5 * (W9[:, 5] + W9[:, 7])], 1)
    out.update(forces=F.numpy(), virial=voigt.numpy(), edge_gradient=g.numpy())
    return out


def evaluate(meta, tensors, systems, dtype=torch.float32, forces=True, want=None, search="cells", threads=None):
    """Energy, per-atom energy, forces [N,3], virial [B,6] (Voigt xx yy zz xy xz yz) for a batch.

    Folds as the reference does: F_i = scale-included sum_k (g_k - g_rev(k))
    (src/forces.cpp:50-70), W_b = sum v (x) g, symmetrised to Voigt
    (src/model.cpp:983-993).
    """
    if threads:
        torch.set_num_threads(threads)
    h = meta["hypers"]
    if isinstance(systems, dict) and "off" in systems:  # packed edges made elsewhere (an engine's own list)
        ed = systems
    else:
        adaptive = None
        if h.get("num_neighbors_adaptive"):
            adaptive = {"method": h["adaptive_cutoff_method"], "target": float(h["num_neighbors_adaptive"]),
                        "width": h["cutoff_width_adaptive"]}
        ed = nbo.build_edges(systems, meta["species_to_index"], h["cutoff"], h["cutoff_width"], h["cutoff_function"],
                             search=search, adaptive=adaptive)
    W = Weights(meta, tensors, dtype)
    fwd = forward_feedforward if h["featurizer_type"] == "feedforward" else forward_residual
    if ed.get("atom_cutoff") is not None:
        return _evaluate_adaptive(h, W, fwd, ed, dtype, forces, want)
    vec = torch.from_numpy(ed["vec"]).clone().requires_grad_(forces)
    with torch.set_grad_enabled(forces):
        per_atom = fwd(W, ed, vec, want)
        N, B = ed["n_atoms"], ed["n_struct"]
        if ed.get("n_local", N) < N:  # ghosts shape the energy but are not in it (src/ops.cpp:420-425)
            per_atom = per_atom * (torch.arange(N) < ed["n_local"])
        sid = torch.from_numpy(ed["struct_id"])
        energy = torch.zeros(B, dtype=torch.float64).index_add(0, sid, per_atom)
        out = {"energy": energy.detach().numpy(), "per_atom_energy": per_atom.detach().numpy(), "edges": ed}
        if not forces:
            return out
        (g,) = torch.autograd.grad(per_atom.sum(), vec)
    g = g.double()
    center, rev = torch.from_numpy(ed["center"]), torch.from_numpy(ed["reverse"])
    back = torch.where((rev >= 0)[:, None], g[rev.clamp(min=0)], torch.zeros_like(g))
    F = torch.zeros(N, 3, dtype=torch.float64).index_add(0, center, g - back)
    w9 = (vec.detach()[:, :, None] * g[:, None, :]).reshape(-1, 9)
    W9 = torch.zeros(B, 9, dtype=torch.float64).index_add(0, sid[center], w9)
    voigt = torch.stack([W9[:, 0], W9[:, 4], W9[:, 8], 0.5 * (W9[:, 1] + W9[:, 3]), 0.5 * (W9[:, 2] + W9[:, 6]),
                         0.5 * (W9[:, 5] + W9[:, 7])], 1)
    out.update(forces=F.numpy(), virial=voigt.numpy(), edge_gradient=g.numpy())
    return out
