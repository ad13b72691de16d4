// The network's non-GEMM passes: lookups, norms (forward and backward, with the
// gathers and residual sums that ride along), compress.0's folded terms, the
// readout's ordered sums and the geometry end of the backward. Each names the
// reference pass it stands for.
#pragma once

#include "common.h"
#include "neighbors.h"

namespace petb {

// out(r,:) = table(idx(r),:)   (gather, src/ops.cpp:109-114)
void gather_rows(Stream& st, float* out, const float* table, const int* idx, int R, int D);

// Layer 0's compress.0: pre = b + tab[species] + wx.(v,|v|); out = silu(pre)  (compress_fwd without a GEMM, src/ops.cpp:326-365)
void compress0(Stream& st, float* out, float* pre, const float* b, const float* tab, const float* wx, const PackedEdges& pk,
               int D);

// out = norm(in [+ add, stored back into in]); RMSNorm when bias is null, else LayerNorm  (norm_rows, src/ops.hpp:381-401)
void norm_fwd(Stream& st, float* out, float* in, const float* add, const float* w, const float* bias, int R, int D);

// Partner rows that live on another rank (an exchanged list): edge k's partner row is rows[of[k]] when its local
// partner is missing and of[k] >= 0. All null without an exchange.
struct RemoteRows {
  const int* of = nullptr;      // [E] live index of a packed edge, or -1
  const float* rows = nullptr;  // [n_live, D]
};

// out(l, :) = src(live_packed[l], col0 : col0 + D), src rows ld floats apart: the rows an exchange sends.
void gather_live(Stream& st, float* out, const float* src, int ld, int col0, const int* live_packed, int n_live, int D);

// The combination norm with its gather: row k of the input is [oe(k) | oe(rev k), the remote partner's row, or 0];
// ie(k) += oe(k) on the way  (src/feedforward.cpp:182-193)
void concat_norm_fwd(Stream& st, float* out, const float* oe, const int* rev, float* ie, const float* w, const float* bias,
                     int E, int D, RemoteRows remote = {});

// in_adj = g for rows < acc_row0, in_adj += g for the rest; g the norm's input adjoint
// (norm_rows_bwd, src/ops.hpp:404-436). `also`, unless null, receives a copy of the result.
void norm_bwd(Stream& st, float* in_adj, const float* out_adj, const float* in, const float* w, bool layernorm, int R, int D,
              int acc_row0, float* also = nullptr);

// edge_adj(k) = ie_adj(k) + g(k)[:D] + g(rev k)[D:], g from out_adj [E,2D]  (concat_norm_bwd, src/ops.cpp:191-244)
// With an exchange: `remote` holds the partner rows the forward read, `remote_adj` the partners' adjoints of this
// rank's rows (what concat_norm_remote_bwd computed on the other side).
void concat_norm_bwd(Stream& st, float* edge_adj, const float* out_adj, const float* oe, const int* rev, const float* ie_adj,
                     const float* w, int E, int D, RemoteRows remote = {}, const float* remote_adj = nullptr);
// send(l, :) = the adjoint of the partner row that live edge l read: g(live_packed[l])[D:]  (src/feedforward.cpp:246-255)
void concat_norm_remote_bwd(Stream& st, float* send, const float* out_adj, const float* oe, const float* w,
                            const int* live_packed, int n_live, int D, RemoteRows remote);

// x4_adj(k,c) += sum_d g(k,d) wx(d,c)  (the reduction of compress_bwd, src/ops.cpp:373-401)
void compress_geometry_bwd(Stream& st, float* x4_adj, const float* g, const float* wx, int E, int D);

// net(n) = float(node_pred(n) + sum_k double(cut k) * double(edge_pred k)); per_atom(n) = scale*net + comp[species]
// (readout_accumulate + assemble_energy, src/ops.cpp:406-425). acc: add onto net first.
void readout_energy(Stream& st, float* net, double* per_atom, const float* node_pred, const float* edge_pred,
                    const PackedEdges& pk, const double* composition, double scale, bool acc, bool assemble);

// out(r,j) = seed(r) * w(j) * silu'(pre(r,j)); seed is 1 for rows < n_one when cut is null, else cut(r) for rows
// whose centre is owned  (the seeds of readout_bwd fused with its first linear_silu_bwd, src/model.cpp:749-778)
void readout_seed_bwd(Stream& st, float* out, const float* w, const float* pre, const float* cut, const int* center,
                      int n_local, int R, int Dh);

// cf_adj(k) += (sum_h cfh(N+k,h)) / cut(k)  (attn_bwd_cf, src/attention.cpp:1829-1838; only edge slots carry a gradient)
void cutoff_share(Stream& st, float* cf_adj, const float* cfh, const float* cut, int N, int E, int H);

// a += b, elementwise
void add_inplace(Stream& st, float* a, const float* b, size_t n);
// input_edge(k) = 0.5 (input_edge(k) + oe(rev k) or 0)  (re_msg, src/residual.cpp:123-132)
void message_average(Stream& st, float* ie, const float* oe, const int* rev, int E, int D, RemoteRows remote = {});
// With an exchange, `remote_adj` holds the partners' ie_adj_in rows (src/residual.cpp:189).
void message_average_bwd(Stream& st, float* ie_adj_out, float* oe_adj, const float* ie_adj_in, const int* rev, int E, int D,
                         RemoteRows remote_adj = {});

struct ForceOut {
  double* edge_grad = nullptr;  // [E,3]
  double* forces = nullptr;     // [n_atoms,3]
  double* vir_atom = nullptr;   // [n_atoms,9]
  double* vir9 = nullptr;       // [B,9]
  double* vir6 = nullptr;       // [B,6]
  double* energy = nullptr;     // [B]
  // With an adaptive cutoff: the radial gradient it puts on every raw edge, scale included (dE/dv += gmag v).
  double* adaptive_gmag = nullptr;  // [E_raw]
};
// dE/dv per edge, the per-atom fold, and each structure's ordered sums
// (forces_and_virial, fold_edge_gradients, sum_by_structure: src/forces.cpp:50-70,287-302,345-411; Voigt: src/model.cpp:983-993)
void forces_and_virial(Stream& st, Arena& arena, ForceOut& out, const PackedEdges& pk, const float* x4_adj, const float* cutoff_adj,
                       const float* cf_adj, const CutoffSpec& cs, double scale);
// The adaptive cutoff's share of forces and virial (adaptive.cu): pc_adj [E] is each kept edge's pair-cutoff adjoint.
void adaptive_backward(Stream& st, Arena& arena, const PackedEdges& pk, const CutoffSpec& cs, const double* pc_adj, double scale,
                       double* forces, double* vir_atom, double** gmag_out);
// energy(b) = ordered sum of per_atom over the structure's atoms
void structure_energy(Stream& st, double* energy, const double* per_atom, const int* soff, int B);

}  // namespace petb
