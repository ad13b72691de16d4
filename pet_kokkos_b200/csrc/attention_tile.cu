// Attention as small dense products in shared memory: the register-tiled form used whenever an
// atom's tokens, and the S x S tables of the backward, fit a CTA's shared memory.
//
// One CTA per (atom, head). Q, K, V (and dO) slices are staged once with a pitch of head_dim + 4
// floats, so threads that read different rows hit different banks; each thread then owns 4 x 4
// register tiles whose rows and columns are strided by ceil(cnt / 4), which keeps the 16-byte
// shared loads of a quarter-warp on distinct bank groups. Forward: scores = sc Q K^T + log cf into
// an S x S table, a warp per query row for the softmax (max, sum, 1/sum saved as in the streaming
// kernel), then O = P V. Backward, with nothing recomputed (the reference's "Pairs" form,
// src/attention.cpp:1699-1812): A = exp(score - m) / l and dS = A (dO V^T - dO.O) into two tables,
// then dQ = sc dS K, dK = sc dS^T Q, dV = A^T dO and each key's column sum of dS. Every sum has one
// owner and a fixed order. Same arithmetic as attention.cu up to the order of the sums.
#include <cstdlib>

#include "attention.h"

namespace petb {

namespace {

constexpr float kOff = -1e30f;
__device__ __forceinline__ bool is_off(float lc) { return lc < -1e29f; }
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float dot4(const float4& a, const float4& b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }
__device__ __forceinline__ void fma4(float4& acc, float s, const float4& v) {
  acc.x = fmaf(s, v.x, acc.x), acc.y = fmaf(s, v.y, acc.y), acc.z = fmaf(s, v.z, acc.z), acc.w = fmaf(s, v.w, acc.w);
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct Layout {
  int S4, P, SP;  // padded rows, row pitch of the staged slices, row pitch of the S x S tables
};
__host__ __device__ inline Layout layout(int S, int HD) {
  Layout l;
  l.S4 = (S + 3) / 4 * 4;
  l.P = HD + 4;
  l.SP = l.S4 + 4;  // a multiple of 4 floats whose quarter is odd: 16-byte row reads of consecutive rows spread over the banks
  if ((l.SP / 4) % 2 == 0) l.SP += 4;
  return l;
}

// Columns [col, col + HD) of the atom's token rows of src into dst [S4][P]; rows past cnt are zero.
template <int HD>
__device__ __forceinline__ void stage(float* dst, const float* src, size_t ld, int col, int n, int N, int e0, int cnt, int rows,
                                      int P) {
  constexpr int Q = HD / 4;
  for (int t = threadIdx.x; t < rows * Q; t += blockDim.x) {
    const int r = t / Q, c = (t % Q) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < cnt) {
      const size_t row = r == 0 ? size_t(n) : size_t(N) + e0 + r - 1;
      v = ld4(src + row * ld + col + c);
    }
    *reinterpret_cast<float4*>(dst + r * P + c) = v;
  }
}

// Tiles of the S x S phase as (qi, ki) pairs: a warp takes a 4 x 8 block of tiles, lane = 8 lq + lk,
// so its 16-byte loads touch 4 distinct Q rows and 8 distinct K rows (one shared-memory wavefront each).
struct TileIter {
  int QS, bq_n, bk_n, total;
  __device__ TileIter(int qs) : QS(qs), bq_n((qs + 3) / 4), bk_n((qs + 7) / 8), total(bq_n * bk_n) {}
  // block `wb` (one per warp iteration): this lane's tile, false if it lies outside the table
  __device__ bool tile(int wb, int lane, int& qi, int& ki) const {
    qi = (wb / bk_n) * 4 + (lane >> 3);
    ki = (wb % bk_n) * 8 + (lane & 7);
    return qi < QS && ki < QS;
  }
};

template <int HD>
__global__ void __launch_bounds__(192) k_attn_fwd_tile(AttnArgs p) {
  extern __shared__ __align__(16) float smem[];
  const Layout L = layout(p.S, HD);
  const int n = blockIdx.x / p.H, h = blockIdx.x % p.H, D = p.H * HD;
  const int e0 = p.off[n], cnt = p.off[n + 1] - e0 + 1;
  const int QS = (cnt + 3) / 4, rows = 4 * QS;
  float* sq = smem;
  float* sk = sq + L.S4 * L.P;
  float* sv = sk + L.S4 * L.P;
  float* sp = sv + L.S4 * L.P;  // [S4][SP] scores, then probabilities
  float* slc = sp + L.S4 * L.SP;
  stage<HD>(sq, p.qkv, 3 * size_t(D), h * HD, n, p.N, e0, cnt, rows, L.P);
  stage<HD>(sk, p.qkv, 3 * size_t(D), D + h * HD, n, p.N, e0, cnt, rows, L.P);
  stage<HD>(sv, p.qkv, 3 * size_t(D), 2 * D + h * HD, n, p.N, e0, cnt, rows, L.P);
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    const float cf = r == 0 ? 1.0f : (r < cnt ? p.cut[e0 + r - 1] : 0.f);
    slc[r] = cf > 0.f ? __logf(cf) : kOff;
  }
  __syncthreads();
  // scores: 4 x 4 tiles, queries {qi + a QS}, keys {ki + b QS}
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const TileIter it(QS);
  for (int wb = warp; wb < it.total; wb += nw) {
    int qi, ki;
    if (!it.tile(wb, lane, qi, ki)) continue;
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
#pragma unroll
    for (int d = 0; d < HD; d += 4) {
      float4 qv[4], kv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) qv[j] = ld4(sq + (qi + j * QS) * L.P + d), kv[j] = ld4(sk + (ki + j * QS) * L.P + d);
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] += dot4(qv[a], kv[b]);
    }
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int k = ki + b * QS;
        const float lc = slc[k];
        sp[(qi + a * QS) * L.SP + k] = is_off(lc) ? kOff : acc[a][b] * p.sc + lc;
      }
  }
  __syncthreads();
  // softmax, a warp per query row; the keys past cnt (up to the padded width) are zeroed for the product below
  for (int q = warp; q < cnt; q += nw) {
    float* row = sp + q * L.SP;
    const size_t grow = q == 0 ? size_t(n) : size_t(p.N) + e0 + q - 1;
    const bool dead = q > 0 && is_off(slc[q]);  // a query on an edge at its cutoff
    float mx = kOff;
    for (int k = lane; k < cnt; k += 32) mx = fmaxf(mx, row[k]);
    mx = warp_max(mx);
    float l = 0.f;
    for (int k = lane; k < cnt; k += 32) {
      const float s = row[k];
      const float e = is_off(s) ? 0.f : __expf(s - mx);
      row[k] = e;
      l += e;
    }
    l = warp_sum(l);
    const float invl = (!dead && l > 0.f) ? 1.0f / l : 0.f;
    for (int k = lane; k < rows; k += 32) row[k] = k < cnt ? row[k] * invl : 0.f;
    if (lane == 0 && p.ml) {
      p.ml[(grow * p.H + h) * 2] = dead ? kOff : mx;
      p.ml[(grow * p.H + h) * 2 + 1] = invl;
    }
  }
  __syncthreads();
  // O = P V: 4 consecutive query rows x 4 dims per thread, four keys per step (16-byte loads of P and V)
  constexpr int DQ = HD / 4;
  for (int t = threadIdx.x; t < QS * DQ; t += blockDim.x) {
    const int q0 = (t / DQ) * 4, d = (t % DQ) * 4;
    float4 acc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < rows; k += 4) {
      float4 pj[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) pj[j] = ld4(sp + (q0 + j) * L.SP + k);
      const float4 v0 = ld4(sv + k * L.P + d), v1 = ld4(sv + (k + 1) * L.P + d), v2 = ld4(sv + (k + 2) * L.P + d),
                   v3 = ld4(sv + (k + 3) * L.P + d);
#pragma unroll
      for (int j = 0; j < 4; ++j) fma4(acc[j], pj[j].x, v0), fma4(acc[j], pj[j].y, v1), fma4(acc[j], pj[j].z, v2), fma4(acc[j], pj[j].w, v3);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int q = q0 + j;
      if (q < cnt) {
        const size_t grow = q == 0 ? size_t(n) : size_t(p.N) + e0 + q - 1;
        *reinterpret_cast<float4*>(p.merged + grow * D + h * HD + d) = acc[j];
      }
    }
  }
}

template <int HD>
__global__ void __launch_bounds__(192) k_attn_bwd_tile(AttnArgs p) {
  extern __shared__ __align__(16) float smem[];
  const Layout L = layout(p.S, HD);
  const int n = blockIdx.x / p.H, h = blockIdx.x % p.H, D = p.H * HD;
  const int e0 = p.off[n], cnt = p.off[n + 1] - e0 + 1;
  const int QS = (cnt + 3) / 4, rows = 4 * QS;
  float* sq = smem;
  float* sk = sq + L.S4 * L.P;
  float* sv = sk + L.S4 * L.P;
  float* sg = sv + L.S4 * L.P;
  float* sA = sg + L.S4 * L.P;     // [S4][SP] softmax weights
  float* sdS = sA + L.S4 * L.SP;   // [S4][SP] score adjoints before the scale
  float* slc = sdS + L.S4 * L.SP;
  float* sm = slc + L.S4;
  float* sl = sm + L.S4;
  float* sd = sl + L.S4;
  stage<HD>(sq, p.qkv, 3 * size_t(D), h * HD, n, p.N, e0, cnt, rows, L.P);
  stage<HD>(sk, p.qkv, 3 * size_t(D), D + h * HD, n, p.N, e0, cnt, rows, L.P);
  stage<HD>(sv, p.qkv, 3 * size_t(D), 2 * D + h * HD, n, p.N, e0, cnt, rows, L.P);
  stage<HD>(sg, p.dmerged, size_t(D), h * HD, n, p.N, e0, cnt, rows, L.P);
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    float lc = kOff, m = 0.f, il = 0.f;
    if (r < cnt) {
      const size_t row = r == 0 ? size_t(n) : size_t(p.N) + e0 + r - 1;
      const float cf = r == 0 ? 1.0f : p.cut[e0 + r - 1];
      lc = cf > 0.f ? __logf(cf) : kOff;
      m = p.ml[(row * p.H + h) * 2], il = p.ml[(row * p.H + h) * 2 + 1];
    }
    slc[r] = lc, sm[r] = m, sl[r] = il;
  }
  __syncthreads();
  // Dq = dO . O, a warp per query row (O from global memory)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int q = warp; q < rows; q += nw) {
    float s = 0.f;
    if (q < cnt) {
      const size_t grow = q == 0 ? size_t(n) : size_t(p.N) + e0 + q - 1;
      for (int d = lane; d < HD; d += 32) s += p.merged[grow * D + h * HD + d] * sg[q * L.P + d];
    }
    s = warp_sum(s);
    if (lane == 0) sd[q] = s;
  }
  __syncthreads();
  // A and dS tables: scores and dO V^T in one sweep of the head dimension
  const TileIter it(QS);
  for (int wb = warp; wb < it.total; wb += nw) {
    int qi, ki;
    if (!it.tile(wb, lane, qi, ki)) continue;
    float as[4][4], ap[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) as[a][b] = 0.f, ap[a][b] = 0.f;
#pragma unroll 2
    for (int d = 0; d < HD; d += 4) {
      float4 qv[4], kv[4], gv[4], vv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        qv[j] = ld4(sq + (qi + j * QS) * L.P + d), kv[j] = ld4(sk + (ki + j * QS) * L.P + d);
        gv[j] = ld4(sg + (qi + j * QS) * L.P + d), vv[j] = ld4(sv + (ki + j * QS) * L.P + d);
      }
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) as[a][b] += dot4(qv[a], kv[b]), ap[a][b] += dot4(gv[a], vv[b]);
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int q = qi + a * QS;
      const float m = sm[q], il = sl[q], dq = sd[q];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int k = ki + b * QS;
        const float lc = slc[k];
        const float A = (il > 0.f && !is_off(lc)) ? __expf(as[a][b] * p.sc + lc - m) * il : 0.f;
        sA[q * L.SP + k] = A;
        sdS[q * L.SP + k] = A * (ap[a][b] - dq);
      }
    }
  }
  __syncthreads();
  // dQ = sc dS K,  dK = sc dS^T Q,  dV = A^T dO: 4 consecutive rows x 4 dims per thread, the three products as one tile list
  constexpr int DQ = HD / 4;
  const int per = QS * DQ;
  for (int t = threadIdx.x; t < 3 * per; t += blockDim.x) {
    const int which = t / per, u = t % per;
    const int r0 = (u / DQ) * 4, d = (u % DQ) * 4;
    float4 acc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (which == 0) {  // rows are queries; four keys per step
      for (int k = 0; k < rows; k += 4) {
        float4 sj[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) sj[j] = ld4(sdS + (r0 + j) * L.SP + k);
        const float4 k0 = ld4(sk + k * L.P + d), k1 = ld4(sk + (k + 1) * L.P + d), k2 = ld4(sk + (k + 2) * L.P + d),
                     k3 = ld4(sk + (k + 3) * L.P + d);
#pragma unroll
        for (int j = 0; j < 4; ++j) fma4(acc[j], sj[j].x, k0), fma4(acc[j], sj[j].y, k1), fma4(acc[j], sj[j].z, k2), fma4(acc[j], sj[j].w, k3);
      }
    } else {  // rows are keys: a table column group per query
      const float* tab = which == 1 ? sdS : sA;
      const float* src = which == 1 ? sq : sg;
      for (int q = 0; q < cnt; ++q) {
        const float4 x = ld4(src + q * L.P + d);
        const float4 w = ld4(tab + q * L.SP + r0);
        fma4(acc[0], w.x, x), fma4(acc[1], w.y, x), fma4(acc[2], w.z, x), fma4(acc[3], w.w, x);
      }
    }
    const float scale = which == 2 ? 1.0f : p.sc;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = r0 + j;
      if (r < cnt) {
        const size_t grow = r == 0 ? size_t(n) : size_t(p.N) + e0 + r - 1;
        *reinterpret_cast<float4*>(p.qkv_adj + grow * 3 * D + which * D + h * HD + d) =
            make_float4(acc[j].x * scale, acc[j].y * scale, acc[j].z * scale, acc[j].w * scale);
      }
    }
  }
  // each key's dS summed over its queries: the cutoff factor's share from this head
  for (int k = threadIdx.x; k < cnt; k += blockDim.x) {
    float s = 0.f;
    for (int q = 0; q < cnt; ++q) s += sdS[q * L.SP + k];
    const size_t grow = k == 0 ? size_t(n) : size_t(p.N) + e0 + k - 1;
    p.cfh[grow * p.H + h] = s;
  }
}

bool enabled() {
  static const bool on = [] {
    const char* e = std::getenv("PET_ATTN_TILED");
    return !(e && e[0] == '0');
  }();
  return on;
}

constexpr size_t kMaxBytes = 112 * 1024;  // two CTAs per SM

size_t fwd_bytes(int S, int HD) {
  const Layout l = layout(S, HD);
  return sizeof(float) * (3 * size_t(l.S4) * l.P + size_t(l.S4) * l.SP + l.S4);
}
size_t bwd_bytes(int S, int HD) {
  const Layout l = layout(S, HD);
  return sizeof(float) * (4 * size_t(l.S4) * l.P + 2 * size_t(l.S4) * l.SP + 4 * size_t(l.S4));
}

template <class K>
void launch(Stream& st, K kernel, const AttnArgs& p, size_t bytes, SmemOptIn& opted) {
  opt_in_shared_memory(kernel, bytes, opted);
  kernel<<<p.N * p.H, 192, bytes, st.s>>>(p);
  PETB_LAUNCH_CHECK(st);
}

template <int HD>
void fwd_hd(Stream& st, const AttnArgs& p) {
  static SmemOptIn opted;
  launch(st, k_attn_fwd_tile<HD>, p, fwd_bytes(p.S, HD), opted);
}
template <int HD>
void bwd_hd(Stream& st, const AttnArgs& p) {
  static SmemOptIn opted;
  launch(st, k_attn_bwd_tile<HD>, p, bwd_bytes(p.S, HD), opted);
}

}  // namespace

// True if the tiled kernel took the pass; false leaves it to the streaming kernel.
bool attention_forward_tiled(Stream& st, const AttnArgs& p) {
  if (!enabled() || fwd_bytes(p.S, p.hd) > kMaxBytes) return false;
  switch (p.hd) {
    case 16: fwd_hd<16>(st, p); return true;
    case 32: fwd_hd<32>(st, p); return true;
    case 48: fwd_hd<48>(st, p); return true;
    case 64: fwd_hd<64>(st, p); return true;
    default: return false;
  }
}

bool attention_backward_tiled(Stream& st, const AttnArgs& p) {
  if (!enabled() || bwd_bytes(p.S, p.hd) > kMaxBytes) return false;
  switch (p.hd) {
    case 16: bwd_hd<16>(st, p); return true;
    case 32: bwd_hd<32>(st, p); return true;
    case 48: bwd_hd<48>(st, p); return true;
    case 64: bwd_hd<64>(st, p); return true;
    default: return false;
  }
}

}  // namespace petb
