// The network's non-GEMM passes: see ops.h.
#include "ops.h"

#include "epilogue.cuh"

namespace petb {

namespace {

constexpr float kRmsEps = 1.1920928955078125e-07f;  // the reference's kRmsNormEps (src/ops.hpp:195)
constexpr float kLnEps = 1e-5f;                     // kLayerNormEps (:196)
constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
  return v;
}

__global__ void k_gather_rows(float* __restrict__ out, const float* __restrict__ table, const int* __restrict__ idx, int R,
                              int D4) {
  const size_t t = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= size_t(R) * D4) return;
  const int r = int(t / D4), q = int(t % D4);
  reinterpret_cast<float4*>(out)[t] = reinterpret_cast<const float4*>(table)[size_t(idx[r]) * D4 + q];
}

__global__ void k_compress0(GemmArgs p) {
  const size_t t = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int D4 = p.N / 4;
  if (t >= size_t(p.M) * D4) return;
  const float zero[4] = {0.f, 0.f, 0.f, 0.f};
  epilogue_run4<EPI_COMPRESS>(p, int(t / D4), int(t % D4) * 4, zero);
}

// One warp per row. x = in (+ add, stored back); out = (x - mu) inv w + b.
__global__ void __launch_bounds__(256) k_norm_fwd(float* __restrict__ out, float* __restrict__ in, const float* __restrict__ add,
                                                  const float* __restrict__ w, const float* __restrict__ bias, int R, int D) {
  const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (r >= R) return;
  float* x = in + size_t(r) * D;
  const bool ln = bias != nullptr;
  if (add) {
    const float* a = add + size_t(r) * D;
    for (int d = lane; d < D; d += 32) x[d] += a[d];
  }
  float mu = 0.f;
  if (ln) {
    float s = 0.f;
    for (int d = lane; d < D; d += 32) s += x[d];
    mu = warp_sum(s) / D;
  }
  float v = 0.f;
  for (int d = lane; d < D; d += 32) {
    const float c = x[d] - mu;
    v += c * c;
  }
  v = warp_sum(v);
  const float inv = 1.0f / sqrtf(v / D + (ln ? kLnEps : kRmsEps));
  float* o = out + size_t(r) * D;
  for (int d = lane; d < D; d += 32) o[d] = (x[d] - mu) * inv * w[d] + (ln ? bias[d] : 0.f);
}

// Edge q's partner row: its reverse edge's, the row another rank sent for it, or none.
__device__ __forceinline__ const float* partner_row(const float* oe, const int* rev, const RemoteRows& rm, int q, int D) {
  const int r = rev[q];
  if (r >= 0) return oe + size_t(r) * D;
  if (rm.of) {
    const int l = rm.of[q];
    if (l >= 0) return rm.rows + size_t(l) * D;
  }
  return nullptr;
}

__global__ void k_gather_live(float* __restrict__ out, const float* __restrict__ src, int ld, int col0,
                              const int* __restrict__ live_packed, int n_live, int D4) {
  const size_t t = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= size_t(n_live) * D4) return;
  const int l = int(t / D4), q = int(t % D4), k = live_packed[l];
  reinterpret_cast<float4*>(out)[t] = k >= 0 ? ld4(src + size_t(k) * ld + col0 + 4 * q) : make_float4(0.f, 0.f, 0.f, 0.f);
}

// The same with each lane holding NV runs of four consecutive values in registers (D = 128 NV): the row is read
// once, 16 bytes at a time, for the statistics and for the output.
template <int NV>
__global__ void __launch_bounds__(256) k_norm_fwd_v(float* __restrict__ out, float* __restrict__ in, const float* __restrict__ add,
                                                    const float* __restrict__ w, const float* __restrict__ bias, int R) {
  constexpr int D = 128 * NV;
  const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (r >= R) return;
  float* x = in + size_t(r) * D;
  const bool ln = bias != nullptr;
  float4 v[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) v[i] = ld4(x + 128 * i + 4 * lane);
  if (add) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const float4 a = ld4(add + size_t(r) * D + 128 * i + 4 * lane);
      v[i].x += a.x, v[i].y += a.y, v[i].z += a.z, v[i].w += a.w;
      st4(x + 128 * i + 4 * lane, v[i]);
    }
  }
  float mu = 0.f;
  if (ln) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    mu = warp_sum(s) / D;
  }
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const float a = v[i].x - mu, b = v[i].y - mu, c = v[i].z - mu, d = v[i].w - mu;
    q += (a * a + b * b) + (c * c + d * d);
  }
  q = warp_sum(q);
  const float inv = 1.0f / sqrtf(q / D + (ln ? kLnEps : kRmsEps));
  float* o = out + size_t(r) * D;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const float4 ww = ld4(w + 128 * i + 4 * lane);
    float4 y = make_float4((v[i].x - mu) * inv * ww.x, (v[i].y - mu) * inv * ww.y, (v[i].z - mu) * inv * ww.z,
                           (v[i].w - mu) * inv * ww.w);
    if (ln) {
      const float4 bb = ld4(bias + 128 * i + 4 * lane);
      y.x += bb.x, y.y += bb.y, y.z += bb.z, y.w += bb.w;
    }
    st4(o + 128 * i + 4 * lane, y);
  }
}

__global__ void __launch_bounds__(256) k_concat_norm_fwd(float* __restrict__ out, const float* __restrict__ oe,
                                                         const int* __restrict__ rev, float* __restrict__ ie,
                                                         const float* __restrict__ w, const float* __restrict__ bias, int E,
                                                         int D, RemoteRows rm) {
  const int k = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (k >= E) return;
  const int W = 2 * D;
  const float* a = oe + size_t(k) * D;
  const float* b = partner_row(oe, rev, rm, k, D);
  float s = 0.f;
  for (int d = lane; d < D; d += 32) {
    const float v = a[d];
    ie[size_t(k) * D + d] += v;
    s += v + (b ? b[d] : 0.f);
  }
  const float mu = warp_sum(s) / W;
  float v = 0.f;
  for (int d = lane; d < D; d += 32) {
    const float c0 = a[d] - mu, c1 = (b ? b[d] : 0.f) - mu;
    v += c0 * c0 + c1 * c1;
  }
  v = warp_sum(v);
  const float inv = 1.0f / sqrtf(v / W + kLnEps);
  float* o = out + size_t(k) * W;
  for (int d = lane; d < D; d += 32) {
    o[d] = (a[d] - mu) * inv * w[d] + bias[d];
    o[D + d] = ((b ? b[d] : 0.f) - mu) * inv * w[D + d] + bias[D + d];
  }
}

struct RowStats {
  float mu, inv, mg, mgx;
};

__global__ void __launch_bounds__(256) k_norm_bwd(float* __restrict__ in_adj, const float* __restrict__ out_adj,
                                                  const float* __restrict__ in, const float* __restrict__ w, bool ln, int R, int D,
                                                  int acc_row0, float* __restrict__ also) {
  const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (r >= R) return;
  const float* x = in + size_t(r) * D;
  const float* ga = out_adj + size_t(r) * D;
  float mu = 0.f;
  if (ln) {
    float s = 0.f;
    for (int d = lane; d < D; d += 32) s += x[d];
    mu = warp_sum(s) / D;
  }
  float sq = 0.f, sg = 0.f, sgx = 0.f;
  for (int d = lane; d < D; d += 32) {
    const float c = x[d] - mu, gw = ga[d] * w[d];
    sq += c * c, sg += gw, sgx += gw * c;
  }
  sq = warp_sum(sq), sg = warp_sum(sg), sgx = warp_sum(sgx);
  const float inv = 1.0f / sqrtf(sq / D + (ln ? kLnEps : kRmsEps));
  const float mg = ln ? sg / D : 0.f, mgx = sgx * inv / D;
  float* o = in_adj + size_t(r) * D;
  const bool acc = r >= acc_row0;
  for (int d = lane; d < D; d += 32) {
    const float g = inv * (ga[d] * w[d] - mg - (x[d] - mu) * inv * mgx);
    const float v = acc ? o[d] + g : g;
    o[d] = v;
    if (also) also[size_t(r) * D + d] = v;
  }
}

template <int NV>
__global__ void __launch_bounds__(256) k_norm_bwd_v(float* __restrict__ in_adj, const float* __restrict__ out_adj,
                                                    const float* __restrict__ in, const float* __restrict__ w, bool ln, int R,
                                                    int acc_row0, float* __restrict__ also) {
  constexpr int D = 128 * NV;
  const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (r >= R) return;
  float4 x[NV], gw[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    x[i] = ld4(in + size_t(r) * D + 128 * i + 4 * lane);
    const float4 g = ld4(out_adj + size_t(r) * D + 128 * i + 4 * lane), ww = ld4(w + 128 * i + 4 * lane);
    gw[i] = make_float4(g.x * ww.x, g.y * ww.y, g.z * ww.z, g.w * ww.w);
  }
  float mu = 0.f;
  if (ln) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) s += (x[i].x + x[i].y) + (x[i].z + x[i].w);
    mu = warp_sum(s) / D;
  }
  float sq = 0.f, sg = 0.f, sgx = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    x[i].x -= mu, x[i].y -= mu, x[i].z -= mu, x[i].w -= mu;
    sq += (x[i].x * x[i].x + x[i].y * x[i].y) + (x[i].z * x[i].z + x[i].w * x[i].w);
    sg += (gw[i].x + gw[i].y) + (gw[i].z + gw[i].w);
    sgx += (gw[i].x * x[i].x + gw[i].y * x[i].y) + (gw[i].z * x[i].z + gw[i].w * x[i].w);
  }
  sq = warp_sum(sq), sg = warp_sum(sg), sgx = warp_sum(sgx);
  const float inv = 1.0f / sqrtf(sq / D + (ln ? kLnEps : kRmsEps));
  const float mg = ln ? sg / D : 0.f, mgx = sgx * inv / D;
  float* o = in_adj + size_t(r) * D;
  const bool acc = r >= acc_row0;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    float4 g = make_float4(inv * (gw[i].x - mg - x[i].x * inv * mgx), inv * (gw[i].y - mg - x[i].y * inv * mgx),
                           inv * (gw[i].z - mg - x[i].z * inv * mgx), inv * (gw[i].w - mg - x[i].w * inv * mgx));
    if (acc) {
      const float4 old = ld4(o + 128 * i + 4 * lane);
      g.x += old.x, g.y += old.y, g.z += old.z, g.w += old.w;
    }
    st4(o + 128 * i + 4 * lane, g);
    if (also) st4(also + size_t(r) * D + 128 * i + 4 * lane, g);
  }
}

// The statistics of row q of the concat [oe(q) | partner(q) or 0] and of its adjoint.
__device__ __forceinline__ RowStats concat_stats(const float* oe, const float* b, const float* out_adj, const float* w, int q,
                                                 int D, int lane) {
  const int W = 2 * D;
  const float* a = oe + size_t(q) * D;
  const float* ga = out_adj + size_t(q) * W;
  float s = 0.f;
  for (int d = lane; d < D; d += 32) s += a[d] + (b ? b[d] : 0.f);
  const float mu = warp_sum(s) / W;
  float sq = 0.f, sg = 0.f, sgx = 0.f;
  for (int d = lane; d < D; d += 32) {
    const float c0 = a[d] - mu, c1 = (b ? b[d] : 0.f) - mu;
    const float g0 = ga[d] * w[d], g1 = ga[D + d] * w[D + d];
    sq += c0 * c0 + c1 * c1, sg += g0 + g1, sgx += g0 * c0 + g1 * c1;
  }
  sq = warp_sum(sq), sg = warp_sum(sg), sgx = warp_sum(sgx);
  const float inv = 1.0f / sqrtf(sq / W + kLnEps);
  return RowStats{mu, inv, sg / W, sgx * inv / W};
}

__global__ void __launch_bounds__(256) k_concat_norm_bwd(float* __restrict__ edge_adj, const float* __restrict__ out_adj,
                                                         const float* __restrict__ oe, const int* __restrict__ rev,
                                                         const float* __restrict__ ie_adj, const float* __restrict__ w, int E,
                                                         int D, RemoteRows rm, const float* __restrict__ remote_adj) {
  const int k = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (k >= E) return;
  const int W = 2 * D, r = rev[k];
  const RowStats sk = concat_stats(oe, partner_row(oe, rev, rm, k, D), out_adj, w, k, D, lane);
  RowStats sr = sk;
  const float* xr2 = nullptr;  // the second half of row r: its partner's row
  if (r >= 0) {
    xr2 = partner_row(oe, rev, rm, r, D);
    sr = concat_stats(oe, xr2, out_adj, w, r, D, lane);
  }
  // An edge to another rank's atom: that rank computed the adjoint of the row it read from here.
  const float* far = (r < 0 && rm.of && remote_adj && rm.of[k] >= 0) ? remote_adj + size_t(rm.of[k]) * D : nullptr;
  for (int d = lane; d < D; d += 32) {
    const float gk = sk.inv * (out_adj[size_t(k) * W + d] * w[d] - sk.mg - (oe[size_t(k) * D + d] - sk.mu) * sk.inv * sk.mgx);
    float back = 0.f;
    if (r >= 0) {
      const float x = (xr2 ? xr2[d] : 0.f) - sr.mu;
      back = sr.inv * (out_adj[size_t(r) * W + D + d] * w[D + d] - sr.mg - x * sr.inv * sr.mgx);
    } else if (far) {
      back = far[d];
    }
    edge_adj[size_t(k) * D + d] = ie_adj[size_t(k) * D + d] + gk + back;
  }
}

// The same, one warp per PAIR of partner rows (single-rank lists only). Row k's concat is [oe(k) | oe(r)] and row r's is
// [oe(r) | oe(k)]: the same numbers, so one mean and one variance serve both, and each row is read once for the two
// outputs. The warp of the larger index of a pair leaves; a row without a partner is a pair with a zero half.
template <int NV>
__global__ void __launch_bounds__(256) k_concat_norm_bwd_pair(float* __restrict__ edge_adj, const float* __restrict__ out_adj,
                                                              const float* __restrict__ oe, const int* __restrict__ rev,
                                                              const float* __restrict__ ie_adj, const float* __restrict__ w,
                                                              int E) {
  constexpr int D = 128 * NV, W = 2 * D;
  const int k = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (k >= E) return;
  const int r = rev[k];
  const bool mutual = r >= 0 && rev[r] == k;
  if (mutual && r < k) return;
  if (r >= 0 && !mutual) {
    // A list whose partner map is not an involution: this row alone, partner's statistics from its own partner.
    const RemoteRows none{};
    const RowStats sk = concat_stats(oe, oe + size_t(r) * D, out_adj, w, k, D, lane);
    const float* xr2 = partner_row(oe, rev, none, r, D);
    const RowStats sr = concat_stats(oe, xr2, out_adj, w, r, D, lane);
    for (int d = lane; d < D; d += 32) {
      const float gk = sk.inv * (out_adj[size_t(k) * W + d] * w[d] - sk.mg - (oe[size_t(k) * D + d] - sk.mu) * sk.inv * sk.mgx);
      const float x = (xr2 ? xr2[d] : 0.f) - sr.mu;
      const float back = sr.inv * (out_adj[size_t(r) * W + D + d] * w[D + d] - sr.mg - x * sr.inv * sr.mgx);
      edge_adj[size_t(k) * D + d] = ie_adj[size_t(k) * D + d] + gk + back;
    }
    return;
  }
  float4 a[NV], b[NV], g0[NV], g1[NV], h0[NV], h1[NV];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = 128 * i + 4 * lane;
    a[i] = ld4(oe + size_t(k) * D + c);
    b[i] = mutual ? ld4(oe + size_t(r) * D + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 w0 = ld4(w + c), w1 = ld4(w + D + c);
    const float4 p = ld4(out_adj + size_t(k) * W + c), q = ld4(out_adj + size_t(k) * W + D + c);
    g0[i] = make_float4(p.x * w0.x, p.y * w0.y, p.z * w0.z, p.w * w0.w);
    g1[i] = make_float4(q.x * w1.x, q.y * w1.y, q.z * w1.z, q.w * w1.w);
    if (mutual) {
      const float4 t = ld4(out_adj + size_t(r) * W + c), u = ld4(out_adj + size_t(r) * W + D + c);
      h0[i] = make_float4(t.x * w0.x, t.y * w0.y, t.z * w0.z, t.w * w0.w);
      h1[i] = make_float4(u.x * w1.x, u.y * w1.y, u.z * w1.z, u.w * w1.w);
    } else {
      h0[i] = h1[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    s += ((a[i].x + b[i].x) + (a[i].y + b[i].y)) + ((a[i].z + b[i].z) + (a[i].w + b[i].w));
  }
  const float mu = warp_sum(s) / W;
  float sq = 0.f, sgk = 0.f, sgxk = 0.f, sgr = 0.f, sgxr = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    a[i].x -= mu, a[i].y -= mu, a[i].z -= mu, a[i].w -= mu;
    b[i].x -= mu, b[i].y -= mu, b[i].z -= mu, b[i].w -= mu;
    sq += ((a[i].x * a[i].x + b[i].x * b[i].x) + (a[i].y * a[i].y + b[i].y * b[i].y)) +
          ((a[i].z * a[i].z + b[i].z * b[i].z) + (a[i].w * a[i].w + b[i].w * b[i].w));
    sgk += ((g0[i].x + g1[i].x) + (g0[i].y + g1[i].y)) + ((g0[i].z + g1[i].z) + (g0[i].w + g1[i].w));
    sgxk += ((g0[i].x * a[i].x + g1[i].x * b[i].x) + (g0[i].y * a[i].y + g1[i].y * b[i].y)) +
            ((g0[i].z * a[i].z + g1[i].z * b[i].z) + (g0[i].w * a[i].w + g1[i].w * b[i].w));
    sgr += ((h0[i].x + h1[i].x) + (h0[i].y + h1[i].y)) + ((h0[i].z + h1[i].z) + (h0[i].w + h1[i].w));
    sgxr += ((h0[i].x * b[i].x + h1[i].x * a[i].x) + (h0[i].y * b[i].y + h1[i].y * a[i].y)) +
            ((h0[i].z * b[i].z + h1[i].z * a[i].z) + (h0[i].w * b[i].w + h1[i].w * a[i].w));
  }
  sq = warp_sum(sq), sgk = warp_sum(sgk), sgxk = warp_sum(sgxk), sgr = warp_sum(sgr), sgxr = warp_sum(sgxr);
  const float inv = 1.0f / sqrtf(sq / W + kLnEps);
  const float mgk = sgk / W, mgxk = sgxk * inv / W, mgr = sgr / W, mgxr = sgxr * inv / W;
  // input adjoint of a concat row's element with centred value x and weighted output adjoint g, for row k's / r's statistics
  auto in_k = [&](float g, float x) { return inv * (g - mgk - x * inv * mgxk); };
  auto in_r = [&](float g, float x) { return inv * (g - mgr - x * inv * mgxr); };
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = 128 * i + 4 * lane;
    float4 o = ld4(ie_adj + size_t(k) * D + c);
    o.x += in_k(g0[i].x, a[i].x), o.y += in_k(g0[i].y, a[i].y), o.z += in_k(g0[i].z, a[i].z), o.w += in_k(g0[i].w, a[i].w);
    if (mutual) {
      o.x += in_r(h1[i].x, a[i].x), o.y += in_r(h1[i].y, a[i].y), o.z += in_r(h1[i].z, a[i].z), o.w += in_r(h1[i].w, a[i].w);
      float4 t = ld4(ie_adj + size_t(r) * D + c);
      t.x += in_r(h0[i].x, b[i].x) + in_k(g1[i].x, b[i].x), t.y += in_r(h0[i].y, b[i].y) + in_k(g1[i].y, b[i].y);
      t.z += in_r(h0[i].z, b[i].z) + in_k(g1[i].z, b[i].z), t.w += in_r(h0[i].w, b[i].w) + in_k(g1[i].w, b[i].w);
      st4(edge_adj + size_t(r) * D + c, t);
    }
    st4(edge_adj + size_t(k) * D + c, o);
  }
}

// send(l, :) = the second half of the norm's input adjoint on live edge l's row: what its partner's rank adds.
__global__ void __launch_bounds__(256) k_concat_norm_remote_bwd(float* __restrict__ send, const float* __restrict__ out_adj,
                                                                const float* __restrict__ oe, const float* __restrict__ w,
                                                                const int* __restrict__ live_packed, int n_live, int D,
                                                                RemoteRows rm) {
  const int l = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (l >= n_live) return;
  const int k = live_packed[l], W = 2 * D;
  if (k < 0) {
    for (int d = lane; d < D; d += 32) send[size_t(l) * D + d] = 0.f;
    return;
  }
  const float* b = rm.rows + size_t(l) * D;
  const RowStats sk = concat_stats(oe, b, out_adj, w, k, D, lane);
  for (int d = lane; d < D; d += 32)
    send[size_t(l) * D + d] = sk.inv * (out_adj[size_t(k) * W + D + d] * w[D + d] - sk.mg - (b[d] - sk.mu) * sk.inv * sk.mgx);
}

__global__ void __launch_bounds__(256) k_compress_geometry_bwd(float* __restrict__ x4_adj, const float* __restrict__ g,
                                                               const float* __restrict__ wx, int E, int D) {
  const int k = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (k >= E) return;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  for (int d = lane; d < D; d += 32) {
    const float gd = g[size_t(k) * D + d];
    const float4 ww = ld4(wx + 4 * d);
    a0 += gd * ww.x, a1 += gd * ww.y, a2 += gd * ww.z, a3 += gd * ww.w;
  }
  a0 = warp_sum(a0), a1 = warp_sum(a1), a2 = warp_sum(a2), a3 = warp_sum(a3);
  if (lane == 0) {
    float4 v = ld4(x4_adj + 4 * size_t(k));
    v.x += a0, v.y += a1, v.z += a2, v.w += a3;
    st4(x4_adj + 4 * size_t(k), v);
  }
}

__global__ void k_readout_energy(float* __restrict__ net, double* __restrict__ per_atom, const float* __restrict__ node_pred,
                                 const float* __restrict__ edge_pred, PackedEdges pk, const double* __restrict__ comp,
                                 double scale, bool acc, bool assemble) {
  const int n = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (n >= pk.N) return;
  double s = 0.0;
  for (int k = pk.off[n] + lane; k < pk.off[n + 1]; k += 32) s += (double) pk.cut[k] * (double) edge_pred[k];
  s = warp_sum(s);
  if (lane == 0) {
    s += (double) node_pred[n];
    const float v = acc ? (float) ((double) net[n] + s) : (float) s;
    net[n] = v;
    if (assemble) per_atom[n] = n < pk.n_local ? scale * (double) v + comp[pk.atom_species[n]] : 0.0;
  }
}

__global__ void k_readout_seed_bwd(float* __restrict__ out, const float* __restrict__ w, const float* __restrict__ pre,
                                   const float* __restrict__ cut, const int* __restrict__ center, int n_local, int R, int Dh4) {
  const size_t t = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= size_t(R) * Dh4) return;
  const int r = int(t / Dh4), q = int(t % Dh4);
  float seed;
  if (cut) seed = center[r] < n_local ? cut[r] : 0.f;
  else seed = r < n_local ? 1.f : 0.f;
  const float4 x = reinterpret_cast<const float4*>(pre)[t], ww = reinterpret_cast<const float4*>(w)[q];
  reinterpret_cast<float4*>(out)[t] = make_float4(seed * ww.x * dsilu_f(x.x), seed * ww.y * dsilu_f(x.y),
                                                  seed * ww.z * dsilu_f(x.z), seed * ww.w * dsilu_f(x.w));
}

__global__ void k_cutoff_share(float* __restrict__ cf_adj, const float* __restrict__ cfh, const float* __restrict__ cut, int N,
                               int E, int H) {
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= E) return;
  const float cf = cut[k];
  if (cf <= 0.f) return;
  float total = 0.f;
  for (int h = 0; h < H; ++h) total += cfh[size_t(N + k) * H + h];
  cf_adj[k] += total / cf;
}

__global__ void k_add_inplace(float* __restrict__ a, const float* __restrict__ b, size_t n) {
  const size_t t = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t < n) a[t] += b[t];
}

__global__ void k_message_average(float* __restrict__ ie, const float* __restrict__ oe, const int* __restrict__ rev, int E,
                                  int D4, RemoteRows rm) {
  const size_t t = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= size_t(E) * D4) return;
  const int k = int(t / D4), q = int(t % D4);
  float4 x = reinterpret_cast<float4*>(ie)[t];
  const float* pr = partner_row(oe, rev, rm, k, 4 * D4);
  const float4 y = pr ? ld4(pr + 4 * q) : make_float4(0, 0, 0, 0);
  reinterpret_cast<float4*>(ie)[t] = make_float4(0.5f * (x.x + y.x), 0.5f * (x.y + y.y), 0.5f * (x.z + y.z), 0.5f * (x.w + y.w));
}

// The adjoint of message_average: ie_adj_out(k) = 0.5 ie_adj_in(k); oe_adj(k) += 0.5 ie_adj_in(rev k).
__global__ void k_message_average_bwd(float* __restrict__ ie_out, float* __restrict__ oe_adj, const float* __restrict__ ie_in,
                                      const int* __restrict__ rev, int E, int D4, RemoteRows rm) {
  const size_t t = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= size_t(E) * D4) return;
  const int k = int(t / D4), q = int(t % D4);
  const float4 x = reinterpret_cast<const float4*>(ie_in)[t];
  float4 o = reinterpret_cast<float4*>(oe_adj)[t];
  const float* pr = partner_row(ie_in, rev, rm, k, 4 * D4);  // the partner edge's adjoint row, here or from its rank
  if (pr) {
    const float4 y = ld4(pr + 4 * q);
    o.x += 0.5f * y.x, o.y += 0.5f * y.y, o.z += 0.5f * y.z, o.w += 0.5f * y.w;
  }
  reinterpret_cast<float4*>(oe_adj)[t] = o;
  reinterpret_cast<float4*>(ie_out)[t] = make_float4(0.5f * x.x, 0.5f * x.y, 0.5f * x.z, 0.5f * x.w);
}

// The smooth cutoff's derivative in the distance, in float like the factor itself
// (bump_ddist / cosine_ddist, src/forces.cpp:22-35).
__device__ inline double cutoff_ddist(double d, double rc, double w, int kind) {
  const float pi = (float) 3.14159265358979323846;
  const float x = (float) ((d - (rc - w)) / w);
  if (x <= 0.f || x >= 1.f) return 0.0;
  if (kind == 0) {
    const float si = sinf(pi * x);
    const float t = tanhf(cosf(pi * x) / si);
    const float du = (-pi / (si * si)) / (float) w;
    return 0.5 * (1.0 - (double) (t * t)) * (double) du;
  }
  return 0.5 * (double) (-pi * sinf(pi * x)) / w;
}

// pc_adj, unless null, receives the adjoint of the edge's own cutoff (an adaptive cutoff): the factor depends on
// d - rc, so it is minus the distance's share (src/forces.cpp:372-377).
__global__ void k_edge_grad(double* __restrict__ grad, PackedEdges pk, const float* __restrict__ x4_adj,
                            const float* __restrict__ cutoff_adj, const float* __restrict__ cf_adj, CutoffSpec cs,
                            double* __restrict__ pc_adj) {
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= pk.E) return;
  if (pc_adj && k >= pk.off[pk.N]) {  // a capacity's dead row
    pc_adj[k] = 0.0;
    for (int c = 0; c < 3; ++c) grad[3 * size_t(k) + c] = 0.0;
    return;
  }
  const bool own = pk.center[k] < pk.n_local;
  const double cutoff_total = (own ? (double) cutoff_adj[k] : 0.0) + (double) cf_adj[k];
  const double d = pk.dist[k];
  const double dcut_dd = cutoff_ddist(d, pk.rc ? pk.rc[k] : cs.cutoff, cs.width, cs.kind);
  if (pc_adj) pc_adj[k] = -cutoff_total * dcut_dd;
  const double dist_adj = (double) x4_adj[4 * size_t(k) + 3] + cutoff_total * dcut_dd;
  const double invd = d > 0.0 ? 1.0 / d : 0.0;
  for (int c = 0; c < 3; ++c) grad[3 * size_t(k) + c] = (double) x4_adj[4 * size_t(k) + c] + dist_adj * pk.vec[3 * size_t(k) + c] * invd;
}

// One warp per atom: F(i) = scale sum_k [g(k) - g(rev k)], W(i) = scale sum_k v (x) g, lanes striding
// the atom's edges and combining in a fixed tree.
__global__ void __launch_bounds__(256) k_fold_forces(ForceOut out, PackedEdges pk, double scale) {
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (i >= pk.n_atoms) return;
  double f[3] = {0, 0, 0}, w[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
  if (i < pk.N)
    for (int k = pk.off[i] + lane; k < pk.off[i + 1]; k += 32) {
      const double* g = out.edge_grad + 3 * size_t(k);
      const double* v = pk.vec + 3 * size_t(k);
      const int r = pk.reverse[k];
      for (int c = 0; c < 3; ++c) f[c] += g[c] - (r >= 0 ? out.edge_grad[3 * size_t(r) + c] : 0.0);
      for (int a = 0; a < 3; ++a)
        for (int b = 0; b < 3; ++b) w[a * 3 + b] += v[a] * g[b];
    }
  for (int c = 0; c < 3; ++c) f[c] = warp_sum(f[c]);
  for (int t = 0; t < 9; ++t) w[t] = warp_sum(w[t]);
  if (lane == 0) {
    for (int c = 0; c < 3; ++c) out.forces[3 * size_t(i) + c] = scale * f[c];
    for (int t = 0; t < 9; ++t) out.vir_atom[9 * size_t(i) + t] = scale * w[t];
  }
}

// One warp per (structure, component): lane l sums every 32nd atom from the l-th, then a fixed tree.
__global__ void k_struct_sum(double* __restrict__ out, const double* __restrict__ x, const int* __restrict__ soff, int B, int T) {
  const int u = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (u >= B * T) return;
  const int b = u / T, t = u % T;
  double s = 0.0;
  for (int a = soff[b] + lane; a < soff[b + 1]; a += 32) s += x[size_t(a) * T + t];
  s = warp_sum(s);
  if (lane == 0) out[u] = s;
}

__global__ void k_voigt(double* __restrict__ w6, const double* __restrict__ w9, int B) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const double* w = w9 + 9 * b;
  double* o = w6 + 6 * b;
  o[0] = w[0], o[1] = w[4], o[2] = w[8];
  o[3] = 0.5 * (w[1] + w[3]), o[4] = 0.5 * (w[2] + w[6]), o[5] = 0.5 * (w[5] + w[7]);
}

inline unsigned blocks_for(size_t n, int per) { return (unsigned) ((n + per - 1) / per); }

}  // namespace

void gather_rows(Stream& st, float* out, const float* table, const int* idx, int R, int D) {
  if (R == 0) return;
  const ProfScope ps(st, PC_GATHER, 0.0, 8.0 * double(R) * D);
  k_gather_rows<<<blocks_for(size_t(R) * (D / 4), 256), 256, 0, st.s>>>(out, table, idx, R, D / 4);
  PETB_LAUNCH_CHECK(st);
}

void compress0(Stream& st, float* out, float* pre, const float* b, const float* tab, const float* wx, const PackedEdges& pk,
               int D) {
  if (pk.E == 0) return;
  const ProfScope ps(st, PC_ELEMENTWISE, 12.0 * double(pk.E) * D, 8.0 * double(pk.E) * D);
  GemmArgs p;
  p.M = pk.E, p.N = D, p.C = out, p.ldc = D, p.pre = pre, p.ldp = D, p.bias = b, p.tab = tab, p.wx = wx, p.sp = pk.species;
  p.vec = pk.vec, p.dist = pk.dist, p.epi = EPI_COMPRESS;
  k_compress0<<<blocks_for(size_t(pk.E) * (D / 4), 256), 256, 0, st.s>>>(p);
  PETB_LAUNCH_CHECK(st);
}

void norm_fwd(Stream& st, float* out, float* in, const float* add, const float* w, const float* bias, int R, int D) {
  if (R == 0) return;
  const ProfScope ps(st, PC_NORM, 6.0 * double(R) * D, (add ? 16.0 : 8.0) * double(R) * D);
  const unsigned blocks = blocks_for(size_t(R) * 32, 256);
  switch (D) {  // whole rows in registers for the usual widths
    case 128: k_norm_fwd_v<1><<<blocks, 256, 0, st.s>>>(out, in, add, w, bias, R); break;
    case 256: k_norm_fwd_v<2><<<blocks, 256, 0, st.s>>>(out, in, add, w, bias, R); break;
    case 512: k_norm_fwd_v<4><<<blocks, 256, 0, st.s>>>(out, in, add, w, bias, R); break;
    case 1024: k_norm_fwd_v<8><<<blocks, 256, 0, st.s>>>(out, in, add, w, bias, R); break;
    default: k_norm_fwd<<<blocks, 256, 0, st.s>>>(out, in, add, w, bias, R, D);
  }
  PETB_LAUNCH_CHECK(st);
}

void gather_live(Stream& st, float* out, const float* src, int ld, int col0, const int* live_packed, int n_live, int D) {
  if (n_live == 0) return;
  const ProfScope ps(st, PC_GATHER, 0.0, 8.0 * double(n_live) * D);
  k_gather_live<<<blocks_for(size_t(n_live) * (D / 4), 256), 256, 0, st.s>>>(out, src, ld, col0, live_packed, n_live, D / 4);
  PETB_LAUNCH_CHECK(st);
}

void concat_norm_fwd(Stream& st, float* out, const float* oe, const int* rev, float* ie, const float* w, const float* bias,
                     int E, int D, RemoteRows remote) {
  if (E == 0) return;
  const ProfScope ps(st, PC_NORM, 12.0 * double(E) * D, 24.0 * double(E) * D);
  k_concat_norm_fwd<<<blocks_for(size_t(E) * 32, 256), 256, 0, st.s>>>(out, oe, rev, ie, w, bias, E, D, remote);
  PETB_LAUNCH_CHECK(st);
}

void norm_bwd(Stream& st, float* in_adj, const float* out_adj, const float* in, const float* w, bool layernorm, int R, int D,
              int acc_row0, float* also) {
  if (R == 0) return;
  const ProfScope ps(st, PC_NORM, 10.0 * double(R) * D, (acc_row0 < R ? 16.0 : 12.0) * double(R) * D);
  const unsigned blocks = blocks_for(size_t(R) * 32, 256);
  switch (D) {
    case 128: k_norm_bwd_v<1><<<blocks, 256, 0, st.s>>>(in_adj, out_adj, in, w, layernorm, R, acc_row0, also); break;
    case 256: k_norm_bwd_v<2><<<blocks, 256, 0, st.s>>>(in_adj, out_adj, in, w, layernorm, R, acc_row0, also); break;
    case 512: k_norm_bwd_v<4><<<blocks, 256, 0, st.s>>>(in_adj, out_adj, in, w, layernorm, R, acc_row0, also); break;
    case 1024: k_norm_bwd_v<8><<<blocks, 256, 0, st.s>>>(in_adj, out_adj, in, w, layernorm, R, acc_row0, also); break;
    default: k_norm_bwd<<<blocks, 256, 0, st.s>>>(in_adj, out_adj, in, w, layernorm, R, D, acc_row0, also);
  }
  PETB_LAUNCH_CHECK(st);
}

void concat_norm_bwd(Stream& st, float* edge_adj, const float* out_adj, const float* oe, const int* rev, const float* ie_adj,
                     const float* w, int E, int D, RemoteRows remote, const float* remote_adj) {
  if (E == 0) return;
  const ProfScope ps(st, PC_NORM, 20.0 * double(E) * D, 24.0 * double(E) * D);
  const auto grid = blocks_for(size_t(E) * 32, 256);
  const bool one_rank = !remote.of && !remote_adj;
  if (one_rank && D == 128)
    k_concat_norm_bwd_pair<1><<<grid, 256, 0, st.s>>>(edge_adj, out_adj, oe, rev, ie_adj, w, E);
  else if (one_rank && D == 256)
    k_concat_norm_bwd_pair<2><<<grid, 256, 0, st.s>>>(edge_adj, out_adj, oe, rev, ie_adj, w, E);
  else if (one_rank && D == 512)
    k_concat_norm_bwd_pair<4><<<grid, 256, 0, st.s>>>(edge_adj, out_adj, oe, rev, ie_adj, w, E);
  else
    k_concat_norm_bwd<<<grid, 256, 0, st.s>>>(edge_adj, out_adj, oe, rev, ie_adj, w, E, D, remote, remote_adj);
  PETB_LAUNCH_CHECK(st);
}

void concat_norm_remote_bwd(Stream& st, float* send, const float* out_adj, const float* oe, const float* w,
                            const int* live_packed, int n_live, int D, RemoteRows remote) {
  if (n_live == 0) return;
  const ProfScope ps(st, PC_NORM, 20.0 * double(n_live) * D, 16.0 * double(n_live) * D);
  k_concat_norm_remote_bwd<<<blocks_for(size_t(n_live) * 32, 256), 256, 0, st.s>>>(send, out_adj, oe, w, live_packed, n_live, D,
                                                                                  remote);
  PETB_LAUNCH_CHECK(st);
}

void compress_geometry_bwd(Stream& st, float* x4_adj, const float* g, const float* wx, int E, int D) {
  if (E == 0) return;
  const ProfScope ps(st, PC_ELEMENTWISE, 8.0 * double(E) * D, 4.0 * double(E) * D);
  k_compress_geometry_bwd<<<blocks_for(size_t(E) * 32, 256), 256, 0, st.s>>>(x4_adj, g, wx, E, D);
  PETB_LAUNCH_CHECK(st);
}

void readout_energy(Stream& st, float* net, double* per_atom, const float* node_pred, const float* edge_pred,
                    const PackedEdges& pk, const double* composition, double scale, bool acc, bool assemble) {
  if (pk.N == 0) return;
  const ProfScope ps(st, PC_GATHER, 2.0 * pk.E, 8.0 * double(pk.E) + 16.0 * pk.N);
  k_readout_energy<<<blocks_for(size_t(pk.N) * 32, 256), 256, 0, st.s>>>(net, per_atom, node_pred, edge_pred, pk, composition,
                                                                        scale, acc, assemble);
  PETB_LAUNCH_CHECK(st);
}

void readout_seed_bwd(Stream& st, float* out, const float* w, const float* pre, const float* cut, const int* center,
                      int n_local, int R, int Dh) {
  if (R == 0) return;
  const ProfScope ps(st, PC_ELEMENTWISE, 8.0 * double(R) * Dh, 8.0 * double(R) * Dh);
  k_readout_seed_bwd<<<blocks_for(size_t(R) * (Dh / 4), 256), 256, 0, st.s>>>(out, w, pre, cut, center, n_local, R, Dh / 4);
  PETB_LAUNCH_CHECK(st);
}

void cutoff_share(Stream& st, float* cf_adj, const float* cfh, const float* cut, int N, int E, int H) {
  if (E == 0) return;
  const ProfScope ps(st, PC_ELEMENTWISE, double(E) * H, 4.0 * double(E) * (H + 2));
  k_cutoff_share<<<blocks_for(E, 256), 256, 0, st.s>>>(cf_adj, cfh, cut, N, E, H);
  PETB_LAUNCH_CHECK(st);
}

void add_inplace(Stream& st, float* a, const float* b, size_t n) {
  if (n == 0) return;
  const ProfScope ps(st, PC_ELEMENTWISE, double(n), 12.0 * double(n));
  k_add_inplace<<<blocks_for(n, 256), 256, 0, st.s>>>(a, b, n);
  PETB_LAUNCH_CHECK(st);
}

void message_average(Stream& st, float* ie, const float* oe, const int* rev, int E, int D, RemoteRows remote) {
  if (E == 0) return;
  const ProfScope ps(st, PC_GATHER, 2.0 * double(E) * D, 12.0 * double(E) * D);
  k_message_average<<<blocks_for(size_t(E) * (D / 4), 256), 256, 0, st.s>>>(ie, oe, rev, E, D / 4, remote);
  PETB_LAUNCH_CHECK(st);
}

void message_average_bwd(Stream& st, float* ie_adj_out, float* oe_adj, const float* ie_adj_in, const int* rev, int E, int D,
                         RemoteRows remote_adj) {
  if (E == 0) return;
  const ProfScope ps(st, PC_GATHER, 2.0 * double(E) * D, 20.0 * double(E) * D);
  k_message_average_bwd<<<blocks_for(size_t(E) * (D / 4), 256), 256, 0, st.s>>>(ie_adj_out, oe_adj, ie_adj_in, rev, E, D / 4,
                                                                              remote_adj);
  PETB_LAUNCH_CHECK(st);
}

void forces_and_virial(Stream& st, Arena& arena, ForceOut& out, const PackedEdges& pk, const float* x4_adj, const float* cutoff_adj,
                       const float* cf_adj, const CutoffSpec& cs, double scale) {
  const ProfScope ps(st, PC_FORCES, 40.0 * pk.E, 100.0 * double(pk.E) + 96.0 * pk.n_atoms);
  double* pc_adj = pk.adaptive.acut ? arena.alloc<double>(pk.E > 0 ? pk.E : 1) : nullptr;
  if (pk.E > 0) {
    k_edge_grad<<<blocks_for(pk.E, 256), 256, 0, st.s>>>(out.edge_grad, pk, x4_adj, cutoff_adj, cf_adj, cs, pc_adj);
    PETB_LAUNCH_CHECK(st);
  }
  if (pk.n_atoms > 0) {
    k_fold_forces<<<blocks_for(size_t(pk.n_atoms) * 32, 256), 256, 0, st.s>>>(out, pk, scale);
    PETB_LAUNCH_CHECK(st);
  }
  // the adaptive cutoff's share, folded over the raw list, before the per-structure sums
  if (pc_adj) adaptive_backward(st, arena, pk, cs, pc_adj, scale, out.forces, out.vir_atom, &out.adaptive_gmag);
  k_struct_sum<<<blocks_for(size_t(pk.B) * 9 * 32, 256), 256, 0, st.s>>>(out.vir9, out.vir_atom, pk.soff, pk.B, 9);
  PETB_LAUNCH_CHECK(st);
  k_voigt<<<blocks_for(pk.B, 128), 128, 0, st.s>>>(out.vir6, out.vir9, pk.B);
  PETB_LAUNCH_CHECK(st);
}

void structure_energy(Stream& st, double* energy, const double* per_atom, const int* soff, int B) {
  const ProfScope ps(st, PC_FORCES, 0.0, 8.0 * B);
  k_struct_sum<<<blocks_for(size_t(B) * 32, 256), 256, 0, st.s>>>(energy, per_atom, soff, B, 1);
  PETB_LAUNCH_CHECK(st);
}

}  // namespace petb
