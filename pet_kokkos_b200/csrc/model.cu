// The PET network: see model.h.
#include "model.h"

#include <algorithm>
#include <cmath>
#include <cstring>

#include "../../include/pet_b200.h"
#include "attention.h"
#include "gemm.h"

namespace petb {

using Taps = std::map<std::string, std::pair<const float*, size_t>>;

// ---- weights -----------------------------------------------------------------
//
// A checkpoint tensor is uploaded once as it is stored (doubles) and every layout the kernels read is made from it
// on the device: both orientations in fp32, the low parts of their 3xTF32 split, and bf16 copies of both. The
// SwiGLU row pairing and the fold of compress.0 are index maps and short fp64 sums over the uploaded tensors, so
// the host never loops over a weight.

namespace {

// Row a of the prepared matrix comes from this row of the stored one. A SwiGLU input layer is stored as [v ; g]
// (F value rows, then F gate rows) and read as (v_0, g_0, v_1, g_1, ...) so that a gate pair meets in one GEMM
// thread's run of columns (the reference does the same at load, src/model.cpp:211-222).
__device__ __forceinline__ int stored_row(int a, int rows, int paired) { return paired ? (a & 1) * (rows / 2) + (a >> 1) : a; }

__device__ __forceinline__ uint16_t bf16_bits(float x) {  // round to nearest even; weights are finite
  const uint32_t u = __float_as_uint(x);
  return uint16_t((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
// x minus its leading 11 significant bits, with half of the last bit the tensor core keeps added so that its
// truncation of this part rounds.
__device__ __forceinline__ float tf32_low_part(float x) {
  return __uint_as_float(__float_as_uint(x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u)) + 0x1000u);
}

// src [rows, ld] doubles (the first `cols` columns of each row) -> [w | wt | w_lo | wt_lo] floats, then bf16 w, wt.
__global__ void k_weight_layouts(const double* src, int ld, int rows, int cols, int paired, float* out, uint16_t* out16) {
  const size_t n = size_t(rows) * cols, i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int a = int(i / cols), b = int(i % cols);
  const float v = float(src[size_t(stored_row(a, rows, paired)) * ld + b]);
  const size_t t = size_t(b) * rows + a;
  out[i] = v, out[n + t] = v;
  out[2 * n + i] = out[3 * n + t] = tf32_low_part(v);
  out16[i] = out16[n + t] = bf16_bits(v);
}
__global__ void k_weight_vector(const double* src, int len, int paired, float* out) {
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a < len) out[a] = float(src[stored_row(a, len, paired)]);
}

// compress.0 acts on [edge embedding of (v, |v|) | species embedding | input_edge]; the first two blocks are linear
// in four numbers and in a table row, so their products with compress.0 are formed once, in fp64 with every product
// and sum rounded on its own, in column order (the reference's fold, src/model.cpp:233-254, gives the same bits):
//   wx[d, c]  = sum_j W[d, j] We[j, c]        b[d] = b0[d] + sum_j W[d, j] be[j]
//   tab[s, d] = sum_j T[s, j] W[d, D + j]
__global__ void k_fold_geometry(const double* W, int K, const double* We, const double* be, const double* b0, int D, double* wx,
                                double* b) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  double x[4] = {0.0, 0.0, 0.0, 0.0}, bias = b0[d];
  for (int j = 0; j < D; ++j) {
    const double w = W[size_t(d) * K + j];
    for (int c = 0; c < 4; ++c) x[c] = __dadd_rn(x[c], __dmul_rn(w, We[j * 4 + c]));
    bias = __dadd_rn(bias, __dmul_rn(w, be[j]));
  }
  for (int c = 0; c < 4; ++c) wx[d * 4 + c] = x[c];
  b[d] = bias;
}
__global__ void k_fold_species(const double* W, int K, const double* T, int ns, int D, double* tab) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= ns * D) return;
  const int s = i / D, d = i % D;
  double acc = 0.0;
  for (int j = 0; j < D; ++j) acc = __dadd_rn(acc, __dmul_rn(T[size_t(s) * D + j], W[size_t(d) * K + D + j]));
  tab[i] = acc;
}

// A tensor's doubles on the device for the duration of the load.
struct Staged {
  double* p = nullptr;
  int rows = 0, cols = 0;
  explicit Staged(const Tensor& t) {
    rows = t.shape.empty() ? 1 : int(t.dim(0));
    cols = t.shape.size() > 1 ? int(t.dim(1)) : 1;
    alloc(t.data.size());
    PETB_CUDA(cudaMemcpy(p, t.data.data(), t.data.size() * sizeof(double), cudaMemcpyHostToDevice));
  }
  explicit Staged(size_t n) { alloc(n); }
  ~Staged() { cudaFree(p); }
  Staged(const Staged&) = delete;
  void alloc(size_t n) { PETB_CUDA(cudaMalloc(&p, (n ? n : 1) * sizeof(double))); }
};

// What the network reads from a checkpoint, as (tensor name, how it is prepared).
enum class Prep { Matrix, Vector, PairedMatrix, PairedVector, CompressFold };
struct PlanItem {
  std::string name;
  Prep prep;
  int layer = 0;
};

std::vector<PlanItem> weight_plan(const Hypers& h) {
  std::vector<PlanItem> plan;
  const bool ff = h.feedforward, paired = h.swiglu;
  auto dense = [&](const std::string& stem, bool pair_rows = false) {
    plan.push_back({stem + ".weight", pair_rows ? Prep::PairedMatrix : Prep::Matrix});
    plan.push_back({stem + ".bias", pair_rows ? Prep::PairedVector : Prep::Vector});
  };
  auto norm = [&](const std::string& stem) {
    plan.push_back({stem + ".weight", Prep::Vector});
    if (h.layernorm) plan.push_back({stem + ".bias", Prep::Vector});
  };
  plan.push_back({"edge_embedder.weight", Prep::Matrix});
  for (int L = 0; L < h.num_gnn_layers; ++L) {
    const std::string layer = "gnn_layers." + std::to_string(L);
    plan.push_back({layer + ".compress.0", Prep::CompressFold, L});
    dense(layer + ".compress.2");
    for (int a = 0; a < h.num_attention_layers; ++a) {
      const std::string block = layer + ".trans.layers." + std::to_string(a);
      for (const char* part : {".attention.input_linear", ".attention.output_linear", ".mlp.w_out"}) dense(block + part);
      dense(block + ".mlp.w_in", paired);
      norm(block + ".norm_attention"), norm(block + ".norm_mlp");
      if (!h.expanded_node()) continue;
      for (const char* part : {".center_contraction", ".center_expansion", ".center_mlp.w_out"}) dense(block + part);
      dense(block + ".center_mlp.w_in", paired);
      norm(block + ".norm_center_features");
    }
    if (ff) {
      const std::string n = "combination_norms." + std::to_string(L), m = "combination_mlps." + std::to_string(L);
      plan.push_back({n + ".weight", Prep::Vector}), plan.push_back({n + ".bias", Prep::Vector});
      dense(m + ".0"), dense(m + ".2");
    }
  }
  for (int i = 0; i < h.num_readout_layers; ++i) {
    const std::string r = std::to_string(i);
    plan.push_back({"node_embedders." + r + ".weight", Prep::Matrix});
    for (const char* side : {"node", "edge"}) {
      dense(std::string(side) + "_heads.energy." + r + ".0"), dense(std::string(side) + "_heads.energy." + r + ".2");
      dense(std::string(side) + "_last_layers.energy." + r + ".energy___0");
    }
  }
  return plan;
}

}  // namespace

void Model::put_mat(const std::string& name, const double* src, int ld, int rows, int cols, bool paired) {
  const size_t n = size_t(rows) * cols;
  float* dev = nullptr;
  PETB_CUDA(cudaMalloc(&dev, (4 * n + n + 8) * sizeof(float)));  // four fp32 layouts, then two bf16 ones (2n halves)
  owned_.push_back(dev);
  uint16_t* dev16 = reinterpret_cast<uint16_t*>(dev + 4 * n);
  if (n) k_weight_layouts<<<cdiv((long long) n, 256), 256>>>(src, ld, rows, cols, paired ? 1 : 0, dev, dev16);
  PETB_CUDA(cudaGetLastError());
  Mat m;
  m.w = dev, m.wt = dev + n, m.rows = rows, m.cols = cols, m.lo_off = 2 * n, m.w16 = dev16, m.wt16 = dev16 + n;
  mat_[name] = m;
}

void Model::put_vec(const std::string& name, const double* src, int len, bool paired) {
  float* dev = nullptr;
  PETB_CUDA(cudaMalloc(&dev, (len > 0 ? len : 1) * sizeof(float)));
  owned_.push_back(dev);
  if (len) k_weight_vector<<<cdiv(len, 256), 256>>>(src, len, paired ? 1 : 0, dev);
  PETB_CUDA(cudaGetLastError());
  vec_[name] = dev;
}

const Mat& Model::mat(const std::string& name) const {
  auto it = mat_.find(name);
  if (it == mat_.end()) throw Error(1, "model: missing matrix '" + name + "'");
  return it->second;
}
const float* Model::vec(const std::string& name) const {
  auto it = vec_.find(name);
  if (it == vec_.end()) throw Error(1, "model: missing vector '" + name + "'");
  return it->second;
}

// compress.0 of layer L -> "@x4" [D,4], "@b" [D], "@tab" [n_species, D] and, past the first layer, "@in" [D,D] (the
// block that still multiplies input_edge). At layer 0 the species block is the edge embedder's table itself.
void Model::fold_compress(const Checkpoint& ck, const std::string& c0, int L) {
  const std::string layer = "gnn_layers." + std::to_string(L);
  const Staged W(ck.at(c0 + ".weight")), b0(ck.at(c0 + ".bias"));
  const Staged We(ck.at(layer + ".edge_embedder.weight")), be(ck.at(layer + ".edge_embedder.bias"));
  const Staged T(ck.at(L == 0 ? "edge_embedder.weight" : layer + ".neighbor_embedder.weight"));
  const int D = W.rows, K = W.cols, ns = T.rows;
  if (K != (L == 0 ? 2 : 3) * D || T.cols != D || We.rows != D || We.cols != 4)
    throw Error(1, "model: '" + c0 + "' does not have the shape of a compress layer");
  const size_t nx = size_t(D) * 4, nb = size_t(D), nt = size_t(ns) * D;
  const Staged wx(nx), b(nb), tab(nt);
  k_fold_geometry<<<cdiv(D, 128), 128>>>(W.p, K, We.p, be.p, b0.p, D, wx.p, b.p);
  k_fold_species<<<cdiv((long long) ns * D, 128), 128>>>(W.p, K, T.p, ns, D, tab.p);
  PETB_CUDA(cudaGetLastError());
  put_mat(c0 + "@x4", wx.p, 4, D, 4, false);
  put_vec(c0 + "@b", b.p, D, false);
  put_mat(c0 + "@tab", tab.p, D, ns, D, false);
  if (L > 0) put_mat(c0 + "@in", W.p + 2 * D, K, D, D, false);
  PETB_CUDA(cudaDeviceSynchronize());  // the staged tensors are freed on return
}

Model::Model(const Checkpoint& ck) : h_(ck.hypers), scale_(ck.energy_scale) {
  const bool ff = h_.feedforward, ln = h_.layernorm, expanded = h_.expanded_node(), swiglu = h_.swiglu;

  // The two families the reference implements (src/model.cpp:314-334); anything else is refused by name.
  if (ff && (!h_.preln || ln || !swiglu || !expanded))
    throw Error(1, "model: the feedforward featurizer needs PreLN + RMSNorm + SwiGLU with d_node != d_pet");
  if (!ff && (h_.preln || !ln || swiglu || expanded))
    throw Error(1, "model: the residual featurizer needs PostLN + LayerNorm + SiLU with d_node == d_pet");
  if (h_.num_attention_layers < 1) throw Error(1, "model: num_attention_layers must be >= 1");
  if (h_.head_dim * h_.num_heads != h_.d_pet) throw Error(1, "model: num_heads * head_dim must equal d_pet");
  if (h_.d_pet % 4 || h_.d_node % 4 || h_.d_head % 4 || h_.d_feedforward % 4)
    throw Error(1, "model: layer widths must be multiples of 4");

  for (const PlanItem& it : weight_plan(h_)) {
    if (it.prep == Prep::CompressFold) {
      fold_compress(ck, it.name, it.layer);
      continue;
    }
    const Tensor& t = ck.at(it.name);
    const bool matrix = it.prep == Prep::Matrix || it.prep == Prep::PairedMatrix;
    const bool paired = it.prep == Prep::PairedMatrix || it.prep == Prep::PairedVector;
    if (matrix && t.shape.size() != 2) throw Error(1, "model: expected a 2-D tensor '" + it.name + "'");
    const Staged dev(t);
    if (matrix) put_mat(it.name, dev.p, dev.cols, dev.rows, dev.cols, paired);
    else put_vec(it.name, dev.p, int(t.numel()), paired);
    PETB_CUDA(cudaDeviceSynchronize());
  }
  const size_t ns = ck.composition_energies.size();
  PETB_CUDA(cudaMalloc(&comp_, (ns ? ns : 1) * sizeof(double)));
  PETB_CUDA(cudaMemcpy(comp_, ck.composition_energies.data(), ns * sizeof(double), cudaMemcpyHostToDevice));
  if (h_.adaptive() && !h_.adaptive_solver) {  // from 0.5 A to the cutoff, a quarter of the taper width apart
    std::vector<double> probes;
    for (double r = 0.5; r < h_.cutoff - 1e-12; r += h_.cutoff_width_adaptive / 4.0) probes.push_back(r);
    n_probes_ = int(probes.size());
    PETB_CUDA(cudaMalloc(&probes_, (probes.size() ? probes.size() : 1) * sizeof(double)));
    PETB_CUDA(cudaMemcpy(probes_, probes.data(), probes.size() * sizeof(double), cudaMemcpyHostToDevice));
  }
  // a blocking copy from pageable memory returns once staged: fence, since the evaluations run on a stream that
  // does not wait for the legacy one
  PETB_CUDA(cudaDeviceSynchronize());
}

Model::~Model() {
  for (void* p : owned_) cudaFree(p);
  cudaFree(comp_);
  cudaFree(probes_);
}

// ---- the GEMM calls, by role ------------------------------------------------------

namespace {

// The attention mode that goes with a GEMM mode unless PET_ATTN names one (native | tf32x3 | tf32), as the reference's
// Options::attention / PET_ATTN (include/pet/calculator.hpp:46-49): Native with native GEMMs, TF32x3 with 3xTF32 GEMMs,
// and the single-pass TF32 form with the tf32 and bf16 speed modes.
int attention_mode_for(int gemm_mode) {
  static const int forced = [] {
    const char* e = std::getenv("PET_ATTN");
    if (!e) return -1;
    const std::string v(e);
    return v == "native" ? int(ATTN_NATIVE) : (v == "tf32x3" || v == "3xtf32") ? int(ATTN_TF32X3) : v == "tf32" ? int(ATTN_TF32) : -1;
  }();
  if (forced >= 0) return forced;
  return gemm_mode == GEMM_NATIVE ? ATTN_NATIVE : gemm_mode == GEMM_TF32X3 ? ATTN_TF32X3 : ATTN_TF32;
}

struct Gemms {
  Stream& st;
  Arena& tmp;
  int mode;

  // out[M, W.rows] = in[M, W.cols] . W^T + bias (+ res for rows >= res_row0)
  void linear(float* out, const float* in, const Mat& W, const float* bias, int M, const float* res = nullptr,
              int res_row0 = 0) const {
    GemmArgs a;
    a.A = in, a.lda = W.cols, a.B = W.w, a.ldb = W.cols, a.b_lo_offset = W.lo_off, a.B16 = W.w16, a.C = out, a.ldc = W.rows;
    a.M = M, a.N = W.rows, a.K = W.cols, a.bias = bias, a.res = res, a.ldr = W.rows, a.res_row0 = res_row0;
    gemm(st, tmp, a, mode);
  }
  // out = silu(pre), pre = in . W^T + bias, kept when `pre` is given
  void linear_silu(float* out, float* pre, const float* in, const Mat& W, const float* bias, int M) const {
    GemmArgs a;
    a.A = in, a.lda = W.cols, a.B = W.w, a.ldb = W.cols, a.b_lo_offset = W.lo_off, a.B16 = W.w16, a.C = out, a.ldc = W.rows;
    a.M = M, a.N = W.rows, a.K = W.cols, a.bias = bias, a.pre = pre, a.ldp = W.rows, a.epi = EPI_SILU;
    gemm(st, tmp, a, mode);
  }
  // pre[M, 2F] = in . W^T + bias (interleaved v, g); h[M, F] = v * sigmoid(g)
  void swiglu_in(float* h, float* pre, const float* in, const Mat& W, const float* bias, int M) const {
    GemmArgs a;
    a.A = in, a.lda = W.cols, a.B = W.w, a.ldb = W.cols, a.b_lo_offset = W.lo_off, a.B16 = W.w16, a.C = h, a.ldc = W.rows / 2;
    a.M = M, a.N = W.rows, a.K = W.cols, a.bias = bias, a.pre = pre, a.ldp = W.rows, a.epi = EPI_SWIGLU;
    gemm(st, tmp, a, mode);
  }
  // in_adj[M, W.cols] (+)= out_adj[M, W.rows] . W
  void linear_bwd(float* in_adj, const float* out_adj, const Mat& W, int M, bool acc) const {
    GemmArgs a;
    a.A = out_adj, a.lda = W.rows, a.B = W.wt, a.ldb = W.rows, a.b_lo_offset = W.lo_off, a.B16 = W.wt16, a.C = in_adj, a.ldc = W.cols;
    a.M = M, a.N = W.cols, a.K = W.rows, a.res = acc ? in_adj : nullptr, a.ldr = W.cols;
    gemm(st, tmp, a, mode);
  }
  // grad[M, W.cols] = (out_adj . W) * silu'(pre)
  void linear_silu_bwd(float* grad, const float* out_adj, const Mat& W, const float* pre, int M) const {
    GemmArgs a;
    a.A = out_adj, a.lda = W.rows, a.B = W.wt, a.ldb = W.rows, a.b_lo_offset = W.lo_off, a.B16 = W.wt16, a.C = grad, a.ldc = W.cols;
    a.M = M, a.N = W.cols, a.K = W.rows, a.pre = const_cast<float*>(pre), a.ldp = W.cols, a.epi = EPI_SILU_BWD;
    gemm(st, tmp, a, mode);
  }
  // pre_adj[M, 2F] from h_adj = out_adj . W_out and the saved pre
  void swiglu_out_bwd(float* pre_adj, const float* out_adj, const Mat& w_out, const float* pre, int M) const {
    GemmArgs a;
    a.A = out_adj, a.lda = w_out.rows, a.B = w_out.wt, a.ldb = w_out.rows, a.b_lo_offset = w_out.lo_off, a.B16 = w_out.wt16, a.C = pre_adj, a.ldc = 2 * w_out.cols;
    a.M = M, a.N = w_out.cols, a.K = w_out.rows, a.pre = const_cast<float*>(pre), a.ldp = 2 * w_out.cols;
    a.epi = EPI_SWIGLU_BWD;
    gemm(st, tmp, a, mode);
  }
};

// One swap of rows with the other ranks (Exchange::edges, include/pet/exchange.hpp:36-40): out[n_live, width] goes to
// the ranks that own the ghosts, in[n_live, width] comes back with the partner edges' rows. Every rank calls it the same
// number of times, with or without live edges of its own.
void exchange_rows(Stream& st, const PackedEdges& pk, const float* out, float* in, int width) {
  const pet_exchange* ex = static_cast<const pet_exchange*>(pk.exchange);
  if (!ex || !ex->edges) throw Error(3, "pet: an exchanged list without an edges() callback");
  if (ex->edges(ex->user, out, in, pk.n_live, width, static_cast<void*>(st.s)) != 0)
    throw Error(1, "pet: the exchange's edges() failed");
  order_after_legacy_stream(st);
}

struct Scope {
  Arena& a;
  Arena::Mark m;
  explicit Scope(Arena& ar) : a(ar), m(ar.mark()) {}
  ~Scope() { a.rewind(m); }
};

void tap(Taps* taps, const std::string& name, const float* p, size_t n) {
  if (taps) (*taps)[name] = {p, n};
}

}  // namespace

// ---- the tail shared by both featurizers ------------------------------------------

PassOut Model::finish(Stream& st, Arena& save, const PackedEdges& pk, bool grad, float* x4_adj, const float* cutoff_adj,
                      float* cf_adj, double* per_atom) {
  PassOut out;
  out.per_atom = per_atom;
  out.f.energy = save.alloc<double>(pk.B);
  structure_energy(st, out.f.energy, per_atom, pk.soff, pk.B);
  if (!grad) return out;
  out.has_forces = true;
  out.f.edge_grad = save.alloc<double>(3 * size_t(pk.E > 0 ? pk.E : 1));
  out.f.forces = save.alloc<double>(3 * size_t(pk.n_atoms));
  out.f.vir_atom = save.alloc<double>(9 * size_t(pk.n_atoms));
  out.f.vir9 = save.alloc<double>(9 * size_t(pk.B));
  out.f.vir6 = save.alloc<double>(6 * size_t(pk.B));
  forces_and_virial(st, save, out.f, pk, x4_adj, cutoff_adj, cf_adj, cutoff_spec(), scale_);
  return out;
}

PassOut Model::run(Stream& st, Arena& save, Arena& tmp, const PackedEdges& pk, bool grad, int mode, Taps* taps,
                   const RunOptions& opt) {
  if (h_.feedforward) return run_feedforward(st, save, tmp, pk, grad, mode, taps, opt);
  last_tier_ = RECOMPUTE_NEVER, last_estimate_ = 0;
  return run_residual(st, save, tmp, pk, grad, mode, taps);
}

// ---- the feedforward featurizer ---------------------------------------------------
//
// How much of the forward the backward keeps (the reference's Recompute tiers, include/pet/config.hpp:19-24,
// src/feedforward.cpp:355-420): Never keeps every saved activation; Wide drops the two widest per block (the
// attention's qkv [T,3D] and the edge MLP's pre-activation [E,2F]) and rebuilds them in the backward with one norm and
// one GEMM each; Layers also keeps only each layer's inputs and re-runs one layer's forward at a time in the
// backward. Under Wide and Layers the edge MLP runs a chunk of edge rows at a time, forward and backward, so its wide
// temporaries are a chunk's. A row's GEMM result does not depend on which rows share its launch, so in the native
// mode every tier gives the bits of Never.

int Model::edge_chunk_rows(int E) {
  if (const char* c = std::getenv("PET_EDGE_CHUNK"))
    if (std::atoi(c) > 0) return std::atoi(c);
  const int eighth = (E + 7) / 8;
  return eighth > 65536 ? eighth : 65536;  // an eighth of the edges, never so few rows that the GEMMs run short
}

// Bytes the two pools hold at their fullest during one feedforward evaluation with forces under a tier: the sums of
// what run_feedforward takes from `save` and the largest of its scopes of `tmp`, from the shapes; 3 % and a few MiB on
// top for the pools' 256-byte rounding and the small per-atom and per-structure arrays of the force fold.
MemoryNeed Model::memory_need(int tier, int N, int E, int n_live) const {
  MemoryNeed need;
  if (!h_.feedforward) return need;
  const double D = h_.d_pet, H = h_.num_heads, F = h_.d_feedforward, Dn = h_.d_node, Dh = h_.d_head;
  const double G = h_.num_gnn_layers, A = h_.num_attention_layers;
  const double n = N, e = E, T = n + e, live = n_live;
  const bool keep = tier == RECOMPUTE_NEVER, relayer = tier == RECOMPUTE_LAYERS;
  const double c = keep ? e : std::min(e, double(edge_chunk_rows(E)));
  // save: what lives for the whole pass
  double save = (G + 1) * n * Dn + e * D + G * live * D + (relayer ? G * e * D : 0.0);
  const double block = T * (2 * D + 2 * H) + n * (Dn + 4 * Dn + Dn) + (keep ? T * 3 * D + e * 2 * F : 0.0);
  const double layer = (A + 1) * T * D + e * 3 * D + A * block + (relayer ? n * Dn : 0.0);
  save += (relayer ? 1.0 : G) * layer;
  save += 2 * n * Dh + 2 * e * Dh + 2 * n + e + 2 * n;              // readout
  save += 5 * e + n * Dn + e * D + T * D + 6 * e + 30 * n;          // adjoints, edge gradients (doubles), forces, virials
  // tmp: the fullest scope
  const double attention_bwd = T * (5 * D + H) + (keep ? 0.0 : T * 4 * D);
  const double attention_fwd = T * D + (keep ? 0.0 : T * 3 * D);
  const double edge_mlp = c * (2 * F + D) + (keep ? c * F : c * (2 * F + D));
  const double combination = e * 4 * D + 2 * live * D;
  const double heads = 2 * n * Dh + 2 * e * Dh;
  double tmp = std::max(std::max(attention_bwd, attention_fwd), std::max(std::max(edge_mlp, combination), heads));
  tmp = std::max(tmp, n * 5 * Dn);
  need.save = size_t(save * 4.0 * 1.03) + (size_t(8) << 20);
  need.tmp = size_t(tmp * 4.0 * 1.03) + (size_t(8) << 20);
  return need;
}

size_t Model::memory_estimate(int tier, int N, int E) const {
  const MemoryNeed need = memory_need(tier, N, E, 0);
  return need.save + need.tmp;
}

int Model::choose_tier(const RunOptions& o, int N, int E) const {
  if (o.recompute != RECOMPUTE_AUTO) return o.recompute;
  for (int tier = std::max(int(RECOMPUTE_NEVER), o.tier_floor); tier < RECOMPUTE_LAYERS; ++tier)
    if (o.budget == 0 || memory_estimate(tier, N, E) <= o.budget) return tier;
  return RECOMPUTE_LAYERS;
}

PassOut Model::run_feedforward(Stream& st, Arena& save, Arena& tmp, const PackedEdges& pk, bool grad, int mode, Taps* taps,
                               const RunOptions& opt) {
  const int N = pk.N, E = pk.E, T = N + E, S = pk.M + 1;
  const int D = h_.d_pet, Dn = h_.d_node, Dh = h_.d_head, H = h_.num_heads, hd = h_.head_dim;
  const int G = h_.num_gnn_layers, A = h_.num_attention_layers;
  const Gemms gm{st, tmp, mode};
  const float sc = float(1.0 / (std::sqrt(double(hd)) * h_.attention_temperature));
  const size_t Ea = E > 0 ? E : 1, Ta = T > 0 ? T : 1, Na = N > 0 ? N : 1;

  // taps name buffers that a recompute would overwrite or never keep: a tapped pass keeps everything
  const int tier = (taps || !grad) ? int(RECOMPUTE_NEVER) : choose_tier(opt, N, E);
  last_tier_ = tier, last_estimate_ = memory_estimate(tier, N, E);
  const bool keep_wide = tier == RECOMPUTE_NEVER, relayer = grad && tier == RECOMPUTE_LAYERS;
  const int chunk = keep_wide ? 0 : edge_chunk_rows(E);

  struct Block {
    float *tok, *qkv, *merged, *ml, *eps, *node_res, *pre_c, *pre_e;
  };
  struct Layer {
    float *cpre, *cph_pre, *out_edge;
    std::vector<Block> blk;
  };
  auto attention_args = [&](const Block& b, const float* qkv) {
    AttnArgs at;
    at.N = N, at.H = H, at.hd = hd, at.S = S, at.sc = sc, at.off = pk.off, at.cut = pk.cut;
    at.mode = attention_mode_for(mode);
    at.pairs = pk.pairs, at.T = T;
    at.qkv = qkv, at.merged = b.merged, at.ml = b.ml;
    return at;
  };
  // qkv = W_in . norm(tokens) + b
  auto make_qkv = [&](float* qkv, const std::string& tl, float* tok) {
    Scope s(tmp);
    float* attn_in = tmp.alloc<float>(Ta * D);
    norm_fwd(st, attn_in, tok, nullptr, vec(tl + ".norm_attention.weight"), nullptr, T, D);
    gm.linear(qkv, attn_in, mat(tl + ".attention.input_linear.weight"), vec(tl + ".attention.input_linear.bias"), T);
  };
  // The edge MLP's first half on rows [r0, r0 + nr): pre = W_in . norm(eps) + b and, with `he`, v * sigmoid(g).
  auto edge_mlp_in = [&](float* he, float* pre, const float* eps_rows, const std::string& tl, int nr) {
    float* edge_norm = tmp.alloc<float>(size_t(nr) * D);
    norm_fwd(st, edge_norm, const_cast<float*>(eps_rows), nullptr, vec(tl + ".norm_mlp.weight"), nullptr, nr, D);
    gm.swiglu_in(he, pre, edge_norm, mat(tl + ".mlp.w_in.weight"), vec(tl + ".mlp.w_in.bias"), nr);
  };

  // One message-passing layer forward: node_in [N,Dn] -> node_out, input_edge [E,D] updated in place, saves in `sl`
  // (from `save`; the wide ones only with keep). `remote_in` [n_live, D] holds the partner rows of an exchanged list:
  // asked for from the other ranks when `ask`, else the rows a first run of this layer received.
  auto layer_forward = [&](int L, const float* node_in, float* node_out, float* input_edge, Layer& sl, bool keep,
                           float* remote_in, bool ask) {
    const std::string g = "gnn_layers." + std::to_string(L), ls = std::to_string(L), c0 = g + ".compress.0";
    sl.blk.resize(A);
    // Token buffers: block a's tokens are [input_node ; edge_cur]; its edge output is written
    // straight into the edge rows of block a+1's, the last one's being the layer's out_edge.
    std::vector<float*> tokbuf(A + 1);
    for (int a = 0; a <= A; ++a) tokbuf[a] = save.alloc<float>(Ta * D);
    sl.cpre = save.alloc<float>(Ea * D);
    {
      Scope s0(tmp);
      float* cact = tmp.alloc<float>(Ea * D);
      if (L == 0) {
        compress0(st, cact, sl.cpre, vec(c0 + "@b"), mat(c0 + "@tab").w, mat(c0 + "@x4").w, pk, D);
      } else {
        const Mat& wi = mat(c0 + "@in");
        GemmArgs a;
        a.A = input_edge, a.lda = D, a.B = wi.w, a.ldb = D, a.b_lo_offset = wi.lo_off, a.B16 = wi.w16, a.C = cact, a.ldc = D;
        a.M = E, a.N = D, a.K = D;
        a.bias = vec(c0 + "@b"), a.pre = sl.cpre, a.ldp = D, a.tab = mat(c0 + "@tab").w, a.sp = pk.species;
        a.wx = mat(c0 + "@x4").w, a.vec = pk.vec, a.dist = pk.dist, a.epi = EPI_COMPRESS;
        gemm(st, tmp, a, mode);
      }
      gm.linear(tokbuf[0] + size_t(N) * D, cact, mat(g + ".compress.2.weight"), vec(g + ".compress.2.bias"), E);
    }
    tap(taps, "et" + ls, tokbuf[0] + size_t(N) * D, size_t(E) * D);

    const float* node_cur = node_in;
    for (int a = 0; a < A; ++a) {
      const std::string tl = g + ".trans.layers." + std::to_string(a), tag = ls + "_" + std::to_string(a);
      Block& b = sl.blk[a];
      const Mat &w_cin = mat(tl + ".center_mlp.w_in.weight"), &w_ein = mat(tl + ".mlp.w_in.weight");
      b.tok = tokbuf[a];
      b.merged = save.alloc<float>(Ta * D);
      b.ml = save.alloc<float>(Ta * H * 2);
      b.eps = save.alloc<float>(Ta * D);  // rows < N: the attention output's atom rows; rows >= N: eps
      b.node_res = save.alloc<float>(Na * Dn);
      b.pre_c = save.alloc<float>(Na * w_cin.rows);
      b.qkv = keep ? save.alloc<float>(Ta * 3 * D) : nullptr;
      b.pre_e = keep ? save.alloc<float>(Ea * w_ein.rows) : nullptr;
      float* node_next = a + 1 == A ? node_out : save.alloc<float>(Na * Dn);
      float* edge_next = tokbuf[a + 1] + size_t(N) * D;

      gm.linear(b.tok, node_cur, mat(tl + ".center_contraction.weight"), vec(tl + ".center_contraction.bias"), N);
      {
        Scope s1(tmp);
        float* qkv = keep ? b.qkv : tmp.alloc<float>(Ta * 3 * D);
        make_qkv(qkv, tl, b.tok);
        attention_forward(st, attention_args(b, qkv));
      }
      tap(taps, "merged" + tag, b.merged, size_t(T) * D);
      // attn_out = merged W_out^T + b; its edge rows take the residual: eps = attn_out + edge_cur.
      gm.linear(b.eps, b.merged, mat(tl + ".attention.output_linear.weight"), vec(tl + ".attention.output_linear.bias"), T,
                b.tok, N);
      // node_res = node_cur + expansion(atom rows of attn_out)
      gm.linear(b.node_res, b.eps, mat(tl + ".center_expansion.weight"), vec(tl + ".center_expansion.bias"), N, node_cur, 0);
      {
        Scope s2(tmp);
        float* node_norm = tmp.alloc<float>(Na * Dn);
        float* hc = tmp.alloc<float>(Na * (w_cin.rows / 2));
        norm_fwd(st, node_norm, b.node_res, nullptr, vec(tl + ".norm_center_features.weight"), nullptr, N, Dn);
        gm.swiglu_in(hc, b.pre_c, node_norm, w_cin, vec(tl + ".center_mlp.w_in.bias"), N);
        gm.linear(node_next, hc, mat(tl + ".center_mlp.w_out.weight"), vec(tl + ".center_mlp.w_out.bias"), N, b.node_res, 0);
      }
      const int rows = keep || chunk <= 0 ? (E > 0 ? E : 1) : chunk;
      for (int r0 = 0; r0 < E; r0 += rows) {
        const int nr = std::min(rows, E - r0);
        Scope s3(tmp);
        float* eps_rows = b.eps + (size_t(N) + r0) * D;
        float* he = tmp.alloc<float>(size_t(nr) * (w_ein.rows / 2));
        float* pre = keep ? b.pre_e + size_t(r0) * w_ein.rows : tmp.alloc<float>(size_t(nr) * w_ein.rows);
        edge_mlp_in(he, pre, eps_rows, tl, nr);
        gm.linear(edge_next + size_t(r0) * D, he, mat(tl + ".mlp.w_out.weight"), vec(tl + ".mlp.w_out.bias"), nr, eps_rows, 0);
      }
      node_cur = node_next;
      tap(taps, "node" + tag, node_cur, size_t(N) * Dn);
      tap(taps, "edge" + tag, edge_next, size_t(E) * D);
    }
    sl.out_edge = tokbuf[A] + size_t(N) * D;
    sl.cph_pre = save.alloc<float>(Ea * 2 * D);
    {
      Scope s4(tmp);
      float* comb = tmp.alloc<float>(Ea * 2 * D);
      float* cph = tmp.alloc<float>(Ea * 2 * D);
      RemoteRows remote;
      if (pk.exchange) {  // edges to ghosts read their partners' rows from the ghosts' ranks (src/feedforward.cpp:171-179)
        if (ask) {
          float* send = tmp.alloc<float>(size_t(pk.n_live > 0 ? pk.n_live : 1) * D);
          gather_live(st, send, sl.out_edge, D, 0, pk.live_packed, pk.n_live, D);
          exchange_rows(st, pk, send, remote_in, D);
        }
        remote = RemoteRows{pk.remote_of, remote_in};
      }
      concat_norm_fwd(st, comb, sl.out_edge, pk.reverse, input_edge, vec("combination_norms." + ls + ".weight"),
                      vec("combination_norms." + ls + ".bias"), E, D, remote);
      gm.linear_silu(cph, sl.cph_pre, comb, mat("combination_mlps." + ls + ".0.weight"), vec("combination_mlps." + ls + ".0.bias"), E);
      gm.linear(input_edge, cph, mat("combination_mlps." + ls + ".2.weight"), vec("combination_mlps." + ls + ".2.bias"), E,
                input_edge, 0);
    }
    tap(taps, "input_edge" + ls, input_edge, size_t(E) * D);
  };

  // ---- forward ----
  std::vector<Layer> sav(G);
  std::vector<float*> node_at(G + 1), ie_at(G, nullptr), remote_in(G, nullptr);
  for (int L = 0; L <= G; ++L) node_at[L] = save.alloc<float>(Na * Dn);  // the nodes entering layer L; [G]: the readout's
  float* input_edge = save.alloc<float>(Ea * D);
  if (pk.exchange)
    for (int L = 0; L < G; ++L) remote_in[L] = save.alloc<float>(size_t(pk.n_live > 0 ? pk.n_live : 1) * D);
  if (relayer)
    for (int L = 0; L < G; ++L) ie_at[L] = save.alloc<float>(Ea * D);  // input_edge as it entered layer L
  gather_rows(st, node_at[0], mat("node_embedders.0.weight").w, pk.atom_species, N, Dn);
  gather_rows(st, input_edge, mat("edge_embedder.weight").w, pk.species, E, D);
  for (int L = 0; L < G; ++L) {
    if (relayer) {
      PETB_CUDA(cudaMemcpyAsync(ie_at[L], input_edge, sizeof(float) * size_t(E) * D, cudaMemcpyDeviceToDevice, st.s));
      Scope layer_saves(save);  // nothing of the layer is kept: the backward runs it again
      layer_forward(L, node_at[L], node_at[L + 1], input_edge, sav[L], false, remote_in[L], true);
    } else {
      layer_forward(L, node_at[L], node_at[L + 1], input_edge, sav[L], grad && keep_wide, remote_in[L], true);
    }
  }
  float* node = node_at[G];

  // ---- readout (src/model.cpp:656-691) ----
  float* nh0_pre = save.alloc<float>(Na * Dh);
  float* nh1_pre = save.alloc<float>(Na * Dh);
  float* eh0_pre = save.alloc<float>(Ea * Dh);
  float* eh1_pre = save.alloc<float>(Ea * Dh);
  float* node_pred = save.alloc<float>(Na);
  float* edge_pred = save.alloc<float>(Ea);
  float* net = save.alloc<float>(Na);
  double* per_atom = save.alloc<double>(pk.n_atoms > 0 ? pk.n_atoms : 1);
  {
    Scope s5(tmp);
    float* nh0 = tmp.alloc<float>(Na * Dh);
    float* nh1 = tmp.alloc<float>(Na * Dh);
    float* eh0 = tmp.alloc<float>(Ea * Dh);
    float* eh1 = tmp.alloc<float>(Ea * Dh);
    gm.linear_silu(nh0, nh0_pre, node, mat("node_heads.energy.0.0.weight"), vec("node_heads.energy.0.0.bias"), N);
    gm.linear_silu(nh1, nh1_pre, nh0, mat("node_heads.energy.0.2.weight"), vec("node_heads.energy.0.2.bias"), N);
    gemv_rows(st, nh1, Dh, mat("node_last_layers.energy.0.energy___0.weight").w, vec("node_last_layers.energy.0.energy___0.bias"),
              node_pred, N, Dh);
    gm.linear_silu(eh0, eh0_pre, input_edge, mat("edge_heads.energy.0.0.weight"), vec("edge_heads.energy.0.0.bias"), E);
    gm.linear_silu(eh1, eh1_pre, eh0, mat("edge_heads.energy.0.2.weight"), vec("edge_heads.energy.0.2.bias"), E);
    gemv_rows(st, eh1, Dh, mat("edge_last_layers.energy.0.energy___0.weight").w, vec("edge_last_layers.energy.0.energy___0.bias"),
              edge_pred, E, Dh);
  }
  tap(taps, "node_pred", node_pred, N);
  tap(taps, "edge_pred", edge_pred, E);
  PETB_CUDA(cudaMemsetAsync(per_atom, 0, sizeof(double) * size_t(pk.n_atoms > 0 ? pk.n_atoms : 1), st.s));
  readout_energy(st, net, per_atom, node_pred, edge_pred, pk, comp_, scale_, false, true);
  if (!grad) return finish(st, save, pk, false, nullptr, nullptr, nullptr, per_atom);

  // ---- backward (src/model.cpp:749-778, src/feedforward.cpp:199-336) ----
  float* x4_adj = save.alloc<float>(Ea * 4);
  float* cf_adj = save.alloc<float>(Ea);
  PETB_CUDA(cudaMemsetAsync(x4_adj, 0, sizeof(float) * Ea * 4, st.s));
  PETB_CUDA(cudaMemsetAsync(cf_adj, 0, sizeof(float) * Ea, st.s));
  float* node_adj = save.alloc<float>(Na * Dn);
  float* ie_adj = save.alloc<float>(Ea * D);
  float* tok_adj = save.alloc<float>(Ta * D);
  float* edge_adj = tok_adj + size_t(N) * D;
  {
    Scope s6(tmp);
    float* nh1_adj = tmp.alloc<float>(Na * Dh);
    float* nh0_adj = tmp.alloc<float>(Na * Dh);
    float* eh1_adj = tmp.alloc<float>(Ea * Dh);
    float* eh0_adj = tmp.alloc<float>(Ea * Dh);
    readout_seed_bwd(st, nh1_adj, mat("node_last_layers.energy.0.energy___0.weight").w, nh1_pre, nullptr, nullptr, pk.n_local, N, Dh);
    gm.linear_silu_bwd(nh0_adj, nh1_adj, mat("node_heads.energy.0.2.weight"), nh0_pre, N);
    gm.linear_bwd(node_adj, nh0_adj, mat("node_heads.energy.0.0.weight"), N, false);
    readout_seed_bwd(st, eh1_adj, mat("edge_last_layers.energy.0.energy___0.weight").w, eh1_pre, pk.cut, pk.center, pk.n_local, E, Dh);
    gm.linear_silu_bwd(eh0_adj, eh1_adj, mat("edge_heads.energy.0.2.weight"), eh0_pre, E);
    gm.linear_bwd(ie_adj, eh0_adj, mat("edge_heads.energy.0.0.weight"), E, false);
  }
  for (int L = G - 1; L >= 0; --L) {
    const std::string g = "gnn_layers." + std::to_string(L), ls = std::to_string(L), c0 = g + ".compress.0";
    Scope relayered(save);  // under Layers: this layer's saves, made again below and dropped after its backward
    Layer again;
    if (relayer) {
      float* scratch_node = save.alloc<float>(Na * Dn);
      layer_forward(L, node_at[L], scratch_node, ie_at[L], again, false, remote_in[L], false);
    }
    const Layer& sl = relayer ? again : sav[L];
    {
      Scope s7(tmp);
      float* cph_adj = tmp.alloc<float>(Ea * 2 * D);
      float* cnorm_adj = tmp.alloc<float>(Ea * 2 * D);
      gm.linear_silu_bwd(cph_adj, ie_adj, mat("combination_mlps." + ls + ".2.weight"), sl.cph_pre, E);
      gm.linear_bwd(cnorm_adj, cph_adj, mat("combination_mlps." + ls + ".0.weight"), E, false);
      RemoteRows remote;
      float* remote_adj = nullptr;
      if (pk.exchange) {  // the partner's rank wants the adjoint of the row this edge read (src/feedforward.cpp:241-255)
        const size_t La = size_t(pk.n_live > 0 ? pk.n_live : 1) * D;
        float* send = tmp.alloc<float>(La);
        remote_adj = tmp.alloc<float>(La);
        remote = RemoteRows{pk.remote_of, remote_in[L]};
        concat_norm_remote_bwd(st, send, cnorm_adj, sl.out_edge, vec("combination_norms." + ls + ".weight"), pk.live_packed,
                               pk.n_live, D, remote);
        exchange_rows(st, pk, send, remote_adj, D);
      }
      concat_norm_bwd(st, edge_adj, cnorm_adj, sl.out_edge, pk.reverse, ie_adj, vec("combination_norms." + ls + ".weight"), E, D,
                      remote, remote_adj);
    }
    for (int a = A - 1; a >= 0; --a) {
      const std::string tl = g + ".trans.layers." + std::to_string(a);
      const Block& b = sl.blk[a];
      const Mat &w_cin = mat(tl + ".center_mlp.w_in.weight"), &w_ein = mat(tl + ".mlp.w_in.weight");
      // the two MLPs: afterwards edge_adj and node_adj are eps's and node_res's
      const int rows = b.pre_e || chunk <= 0 ? (E > 0 ? E : 1) : chunk;
      for (int r0 = 0; r0 < E; r0 += rows) {
        const int nr = std::min(rows, E - r0);
        Scope s8(tmp);
        const float* eps_rows = b.eps + (size_t(N) + r0) * D;
        float* adj_rows = edge_adj + size_t(r0) * D;
        const float* pre = b.pre_e ? b.pre_e + size_t(r0) * w_ein.rows : nullptr;
        if (!pre) {  // the pre-activation was not kept: these rows' again
          float* again_pre = tmp.alloc<float>(size_t(nr) * w_ein.rows);
          edge_mlp_in(nullptr, again_pre, eps_rows, tl, nr);
          pre = again_pre;
        }
        float* pre_adj = tmp.alloc<float>(size_t(nr) * w_ein.rows);
        float* enorm_adj = tmp.alloc<float>(size_t(nr) * D);
        gm.swiglu_out_bwd(pre_adj, adj_rows, mat(tl + ".mlp.w_out.weight"), pre, nr);
        gm.linear_bwd(enorm_adj, pre_adj, w_ein, nr, false);
        norm_bwd(st, adj_rows, enorm_adj, eps_rows, vec(tl + ".norm_mlp.weight"), false, nr, D, 0);
      }
      {
        Scope s9(tmp);
        float* prec_adj = tmp.alloc<float>(Na * w_cin.rows);
        float* cnorm_adj = tmp.alloc<float>(Na * Dn);
        gm.swiglu_out_bwd(prec_adj, node_adj, mat(tl + ".center_mlp.w_out.weight"), b.pre_c, N);
        gm.linear_bwd(cnorm_adj, prec_adj, w_cin, N, false);
        norm_bwd(st, node_adj, cnorm_adj, b.node_res, vec(tl + ".norm_center_features.weight"), false, N, Dn, 0);
      }
      {  // attention: the output adjoint is [expansion's input adjoint ; eps adjoint] = tok_adj
        Scope s10(tmp);
        float* dmerged = tmp.alloc<float>(Ta * D);
        float* qkv_adj = tmp.alloc<float>(Ta * 3 * D);
        float* cfh = tmp.alloc<float>(Ta * H);
        float* attn_in_adj = tmp.alloc<float>(Ta * D);
        const float* qkv = b.qkv;
        if (!qkv) {
          float* again_qkv = tmp.alloc<float>(Ta * 3 * D);
          make_qkv(again_qkv, tl, b.tok);
          qkv = again_qkv;
        }
        gm.linear_bwd(tok_adj, node_adj, mat(tl + ".center_expansion.weight"), N, false);
        gm.linear_bwd(dmerged, tok_adj, mat(tl + ".attention.output_linear.weight"), T, false);
        AttnArgs at = attention_args(b, qkv);
        at.dmerged = dmerged, at.qkv_adj = qkv_adj, at.cfh = cfh;
        attention_backward(st, at);
        cutoff_share(st, cf_adj, cfh, pk.cut, N, E, H);
        gm.linear_bwd(attn_in_adj, qkv_adj, mat(tl + ".attention.input_linear.weight"), T, false);
        // through the norm, back to where the tokens came from: atom rows to the contraction's
        // output adjoint (written), edge rows onto the edge residual (accumulated)
        norm_bwd(st, tok_adj, attn_in_adj, b.tok, vec(tl + ".norm_attention.weight"), false, T, D, N);
      }
      gm.linear_bwd(node_adj, tok_adj, mat(tl + ".center_contraction.weight"), N, true);
    }
    {  // edge_adj is now et's
      Scope s11(tmp);
      float* gz = tmp.alloc<float>(Ea * D);
      gm.linear_silu_bwd(gz, edge_adj, mat(g + ".compress.2.weight"), sl.cpre, E);
      compress_geometry_bwd(st, x4_adj, gz, mat(c0 + "@x4").w, E, D);
      if (L > 0) gm.linear_bwd(ie_adj, gz, mat(c0 + "@in"), E, true);
    }
  }
  tap(taps, "x4_adj", x4_adj, size_t(E) * 4);
  tap(taps, "cf_adj", cf_adj, E);
  return finish(st, save, pk, true, x4_adj, edge_pred, cf_adj, per_atom);
}

// ---- the residual featurizer ------------------------------------------------------

// Per GNN layer L: tokens = [node_embedders.L[species] ; compress(input_edge, geometry, species)];
// A PostLN blocks  tokens = LN(t + mlp(t)), t = LN(tokens + attention(tokens));  every layer is read
// out and the readouts summed; between layers input_edge = 0.5 (input_edge + out_edge of the reverse
// edge)  (src/residual.cpp:13-133 forward, :135-249 backward).
PassOut Model::run_residual(Stream& st, Arena& save, Arena& tmp, const PackedEdges& pk, bool grad, int mode, Taps* taps) {
  const int N = pk.N, E = pk.E, T = N + E, S = pk.M + 1;
  const int D = h_.d_pet, Dh = h_.d_head, H = h_.num_heads, hd = h_.head_dim;
  const int G = h_.num_gnn_layers, A = h_.num_attention_layers;
  const Gemms gm{st, tmp, mode};
  const float sc = float(1.0 / (std::sqrt(double(hd)) * h_.attention_temperature));
  const size_t Ea = E > 0 ? E : 1, Ta = T > 0 ? T : 1, Na = N > 0 ? N : 1;

  struct Block {
    float *qkv, *merged, *ml, *s1, *s2, *pre;
  };
  struct Layer {
    float *cpre, *tokens;
    float *nh0_pre, *nh1_pre, *eh0_pre, *eh1_pre, *edge_pred;
    std::vector<Block> blk;
  };
  std::vector<Layer> sav(G);

  float* input_edge = save.alloc<float>(Ea * D);
  gather_rows(st, input_edge, mat("edge_embedder.weight").w, pk.species, E, D);
  float* net = save.alloc<float>(Na);
  float* node_pred = save.alloc<float>(Na);
  double* per_atom = save.alloc<double>(pk.n_atoms > 0 ? pk.n_atoms : 1);
  PETB_CUDA(cudaMemsetAsync(per_atom, 0, sizeof(double) * size_t(pk.n_atoms > 0 ? pk.n_atoms : 1), st.s));

  for (int L = 0; L < G; ++L) {
    const std::string g = "gnn_layers." + std::to_string(L), ls = std::to_string(L), c0 = g + ".compress.0";
    Layer& sl = sav[L];
    sl.blk.resize(A);
    sl.tokens = save.alloc<float>(Ta * D);
    sl.cpre = save.alloc<float>(Ea * D);
    float* tokens = sl.tokens;
    gather_rows(st, tokens, mat("node_embedders." + ls + ".weight").w, pk.atom_species, N, D);
    {
      Scope s0(tmp);
      float* cact = tmp.alloc<float>(Ea * D);
      if (L == 0) {
        compress0(st, cact, sl.cpre, vec(c0 + "@b"), mat(c0 + "@tab").w, mat(c0 + "@x4").w, pk, D);
      } else {
        const Mat& wi = mat(c0 + "@in");
        GemmArgs a;
        a.A = input_edge, a.lda = D, a.B = wi.w, a.ldb = D, a.b_lo_offset = wi.lo_off, a.B16 = wi.w16, a.C = cact, a.ldc = D, a.M = E, a.N = D, a.K = D;
        a.bias = vec(c0 + "@b"), a.pre = sl.cpre, a.ldp = D, a.tab = mat(c0 + "@tab").w, a.sp = pk.species;
        a.wx = mat(c0 + "@x4").w, a.vec = pk.vec, a.dist = pk.dist, a.epi = EPI_COMPRESS;
        gemm(st, tmp, a, mode);
      }
      gm.linear(tokens + size_t(N) * D, cact, mat(g + ".compress.2.weight"), vec(g + ".compress.2.bias"), E);
    }
    for (int a = 0; a < A; ++a) {
      const std::string tl = g + ".trans.layers." + std::to_string(a);
      Block& b = sl.blk[a];
      const Mat& w_in = mat(tl + ".mlp.w_in.weight");
      b.qkv = save.alloc<float>(Ta * 3 * D);
      b.merged = save.alloc<float>(Ta * D);
      b.ml = save.alloc<float>(Ta * H * 2);
      b.s1 = save.alloc<float>(Ta * D);
      b.s2 = save.alloc<float>(Ta * D);
      b.pre = save.alloc<float>(Ta * w_in.rows);
      gm.linear(b.qkv, tokens, mat(tl + ".attention.input_linear.weight"), vec(tl + ".attention.input_linear.bias"), T);
      AttnArgs at;
      at.N = N, at.H = H, at.hd = hd, at.S = S, at.sc = sc, at.off = pk.off, at.cut = pk.cut;
      at.mode = attention_mode_for(mode);
      at.pairs = pk.pairs, at.T = T;
      at.qkv = b.qkv, at.merged = b.merged, at.ml = b.ml;
      attention_forward(st, at);
      // s1 = attention(tokens) + tokens
      gm.linear(b.s1, b.merged, mat(tl + ".attention.output_linear.weight"), vec(tl + ".attention.output_linear.bias"), T,
                tokens, 0);
      Scope s1(tmp);
      float* tok_a = tmp.alloc<float>(Ta * D);
      float* hmid = tmp.alloc<float>(Ta * w_in.rows);
      norm_fwd(st, tok_a, b.s1, nullptr, vec(tl + ".norm_attention.weight"), vec(tl + ".norm_attention.bias"), T, D);
      gm.linear_silu(hmid, b.pre, tok_a, w_in, vec(tl + ".mlp.w_in.bias"), T);
      // s2 = mlp(tok_a) + tok_a; tokens = LN(s2)
      gm.linear(b.s2, hmid, mat(tl + ".mlp.w_out.weight"), vec(tl + ".mlp.w_out.bias"), T, tok_a, 0);
      norm_fwd(st, tokens, b.s2, nullptr, vec(tl + ".norm_mlp.weight"), vec(tl + ".norm_mlp.bias"), T, D);
    }
    tap(taps, "tokens" + ls, tokens, size_t(T) * D);
    // this layer's readout, summed onto the earlier layers' (src/model.cpp:656-691)
    sl.nh0_pre = save.alloc<float>(Na * Dh), sl.nh1_pre = save.alloc<float>(Na * Dh);
    sl.eh0_pre = save.alloc<float>(Ea * Dh), sl.eh1_pre = save.alloc<float>(Ea * Dh);
    sl.edge_pred = save.alloc<float>(Ea);
    {
      Scope s2(tmp);
      float* nh0 = tmp.alloc<float>(Na * Dh);
      float* nh1 = tmp.alloc<float>(Na * Dh);
      float* eh0 = tmp.alloc<float>(Ea * Dh);
      float* eh1 = tmp.alloc<float>(Ea * Dh);
      const std::string nh = "node_heads.energy." + ls, eh = "edge_heads.energy." + ls;
      const std::string nl = "node_last_layers.energy." + ls + ".energy___0", el = "edge_last_layers.energy." + ls + ".energy___0";
      gm.linear_silu(nh0, sl.nh0_pre, tokens, mat(nh + ".0.weight"), vec(nh + ".0.bias"), N);
      gm.linear_silu(nh1, sl.nh1_pre, nh0, mat(nh + ".2.weight"), vec(nh + ".2.bias"), N);
      gemv_rows(st, nh1, Dh, mat(nl + ".weight").w, vec(nl + ".bias"), node_pred, N, Dh);
      gm.linear_silu(eh0, sl.eh0_pre, tokens + size_t(N) * D, mat(eh + ".0.weight"), vec(eh + ".0.bias"), E);
      gm.linear_silu(eh1, sl.eh1_pre, eh0, mat(eh + ".2.weight"), vec(eh + ".2.bias"), E);
      gemv_rows(st, eh1, Dh, mat(el + ".weight").w, vec(el + ".bias"), sl.edge_pred, E, Dh);
      readout_energy(st, net, per_atom, node_pred, sl.edge_pred, pk, comp_, scale_, L > 0, L + 1 == G);
      tap(taps, "node_pred" + ls, node_pred, N);
      tap(taps, "edge_pred" + ls, sl.edge_pred, E);
      tap(taps, "net" + ls, net, N);
    }
    if (L + 1 < G) {
      RemoteRows remote;
      if (pk.exchange) {  // src/residual.cpp:123-132
        const size_t La = size_t(pk.n_live > 0 ? pk.n_live : 1) * D;
        float* send = tmp.alloc<float>(La);
        float* recv = tmp.alloc<float>(La);
        gather_live(st, send, tokens + size_t(N) * D, D, 0, pk.live_packed, pk.n_live, D);
        exchange_rows(st, pk, send, recv, D);
        remote = RemoteRows{pk.remote_of, recv};
      }
      message_average(st, input_edge, tokens + size_t(N) * D, pk.reverse, E, D, remote);
    }
  }
  if (!grad) return finish(st, save, pk, false, nullptr, nullptr, nullptr, per_atom);

  // ---- backward ----
  float* x4_adj = save.alloc<float>(Ea * 4);
  float* cf_adj = save.alloc<float>(Ea);
  float* cutoff_adj = save.alloc<float>(Ea);  // sum over layers of the edge predictions
  PETB_CUDA(cudaMemsetAsync(x4_adj, 0, sizeof(float) * Ea * 4, st.s));
  PETB_CUDA(cudaMemsetAsync(cf_adj, 0, sizeof(float) * Ea, st.s));
  PETB_CUDA(cudaMemcpyAsync(cutoff_adj, sav[0].edge_pred, sizeof(float) * Ea, cudaMemcpyDeviceToDevice, st.s));
  for (int L = 1; L < G; ++L) add_inplace(st, cutoff_adj, sav[L].edge_pred, size_t(E));
  float* ie_a = save.alloc<float>(Ea * D);
  float* ie_b = save.alloc<float>(Ea * D);
  float* ie_adj = ie_a;  // adjoint of the next layer's input_edge
  for (int L = G - 1; L >= 0; --L) {
    const std::string g = "gnn_layers." + std::to_string(L), ls = std::to_string(L), c0 = g + ".compress.0";
    const Layer& sl = sav[L];
    Scope layer_scope(tmp);
    float* tokens_adj = tmp.alloc<float>(Ta * D);
    float* alt = tmp.alloc<float>(Ta * D);
    {  // the readout's adjoint of this layer's tokens
      Scope s3(tmp);
      float* nh1_adj = tmp.alloc<float>(Na * Dh);
      float* nh0_adj = tmp.alloc<float>(Na * Dh);
      float* eh1_adj = tmp.alloc<float>(Ea * Dh);
      float* eh0_adj = tmp.alloc<float>(Ea * Dh);
      const std::string nh = "node_heads.energy." + ls, eh = "edge_heads.energy." + ls;
      const std::string nl = "node_last_layers.energy." + ls + ".energy___0", el = "edge_last_layers.energy." + ls + ".energy___0";
      readout_seed_bwd(st, nh1_adj, mat(nl + ".weight").w, sl.nh1_pre, nullptr, nullptr, pk.n_local, N, Dh);
      gm.linear_silu_bwd(nh0_adj, nh1_adj, mat(nh + ".2.weight"), sl.nh0_pre, N);
      gm.linear_bwd(tokens_adj, nh0_adj, mat(nh + ".0.weight"), N, false);
      readout_seed_bwd(st, eh1_adj, mat(el + ".weight").w, sl.eh1_pre, pk.cut, pk.center, pk.n_local, E, Dh);
      gm.linear_silu_bwd(eh0_adj, eh1_adj, mat(eh + ".2.weight"), sl.eh0_pre, E);
      gm.linear_bwd(tokens_adj + size_t(N) * D, eh0_adj, mat(eh + ".0.weight"), E, false);
    }
    float* ie_next = ie_adj == ie_a ? ie_b : ie_a;
    if (L + 1 < G) {
      RemoteRows remote;
      if (pk.exchange) {  // src/residual.cpp:189
        const size_t La = size_t(pk.n_live > 0 ? pk.n_live : 1) * D;
        float* send = tmp.alloc<float>(La);
        float* recv = tmp.alloc<float>(La);
        gather_live(st, send, ie_adj, D, 0, pk.live_packed, pk.n_live, D);
        exchange_rows(st, pk, send, recv, D);
        remote = RemoteRows{pk.remote_of, recv};
      }
      message_average_bwd(st, ie_next, tokens_adj + size_t(N) * D, ie_adj, pk.reverse, E, D, remote);
    }
    else PETB_CUDA(cudaMemsetAsync(ie_next, 0, sizeof(float) * Ea * D, st.s));
    for (int a = A - 1; a >= 0; --a) {
      const std::string tl = g + ".trans.layers." + std::to_string(a);
      const Block& b = sl.blk[a];
      const Mat& w_in = mat(tl + ".mlp.w_in.weight");
      Scope s4(tmp);
      float* s2_adj = tmp.alloc<float>(Ta * D);
      float* tok_a_adj = tmp.alloc<float>(Ta * D);
      // tokens_out = LN(s2), s2 = tok_a + mlp(tok_a)
      norm_bwd(st, s2_adj, tokens_adj, b.s2, vec(tl + ".norm_mlp.weight"), true, T, D, T, tok_a_adj);
      {
        Scope s5(tmp);
        float* h_adj = tmp.alloc<float>(Ta * w_in.rows);
        gm.linear_silu_bwd(h_adj, s2_adj, mat(tl + ".mlp.w_out.weight"), b.pre, T);
        gm.linear_bwd(tok_a_adj, h_adj, w_in, T, true);
      }
      // tok_a = LN(s1), s1 = tokens_in + attention(tokens_in)
      float* s1_adj = alt;
      norm_bwd(st, s1_adj, tok_a_adj, b.s1, vec(tl + ".norm_attention.weight"), true, T, D, T);
      {
        Scope s6(tmp);
        float* dmerged = tmp.alloc<float>(Ta * D);
        float* qkv_adj = tmp.alloc<float>(Ta * 3 * D);
        float* cfh = tmp.alloc<float>(Ta * H);
        gm.linear_bwd(dmerged, s1_adj, mat(tl + ".attention.output_linear.weight"), T, false);
        AttnArgs at;
        at.N = N, at.H = H, at.hd = hd, at.S = S, at.sc = sc, at.off = pk.off, at.cut = pk.cut;
      at.mode = attention_mode_for(mode);
        at.pairs = pk.pairs, at.T = T;
        at.qkv = b.qkv, at.merged = b.merged, at.ml = b.ml, at.dmerged = dmerged, at.qkv_adj = qkv_adj, at.cfh = cfh;
        attention_backward(st, at);
        cutoff_share(st, cf_adj, cfh, pk.cut, N, E, H);
        gm.linear_bwd(s1_adj, qkv_adj, mat(tl + ".attention.input_linear.weight"), T, true);
      }
      alt = tokens_adj;
      tokens_adj = s1_adj;
    }
    {  // tokens = [node_L ; et]: only et depends on the geometry
      Scope s7(tmp);
      float* gz = tmp.alloc<float>(Ea * D);
      gm.linear_silu_bwd(gz, tokens_adj + size_t(N) * D, mat(g + ".compress.2.weight"), sl.cpre, E);
      compress_geometry_bwd(st, x4_adj, gz, mat(c0 + "@x4").w, E, D);
      if (L > 0) gm.linear_bwd(ie_next, gz, mat(c0 + "@in"), E, true);
    }
    ie_adj = ie_next;
  }
  return finish(st, save, pk, true, x4_adj, cutoff_adj, cf_adj, per_atom);
}

}  // namespace petb
