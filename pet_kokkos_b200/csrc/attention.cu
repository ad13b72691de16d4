// Multi-head attention over each atom's tokens, forward and backward.
//
// Atom n's tokens are its own row n and one row N + k per kept edge k in
// [off(n), off(n+1)) (the reference's Tokens, src/ops.hpp:31-37). Per head, query q
// attends to key k with weight softmax_k(sc q.k + log cf_k), cf the key's smooth
// cutoff factor (1 for the atom's own token); a key with cf <= 0 is left out and a
// query on such an edge gives zero (src/attention.cpp:1-8,207-266). The backward
// recomputes the weights from each query's saved max and 1/sum and never stores
// anything S x S (src/attention.cpp:1560-1697); every sum has one owner and a
// fixed order, so results repeat to the bit.
//
// One block per (atom, head): the head's slices of the atom's K, V (and Q, dO in
// the backward) rows are staged once in shared memory with 16-byte loads, then a
// thread per token walks them (all threads read the same shared row: a broadcast).
#include "attention.h"

namespace petb {

bool attention_forward_tiled(Stream& st, const AttnArgs& p);   // attention_tile.cu
bool attention_backward_tiled(Stream& st, const AttnArgs& p);
bool attention_forward_mma(Stream& st, const AttnArgs& p);  // attention_mma.cu
bool attention_backward_mma(Stream& st, const AttnArgs& p);

namespace {

constexpr float kOff = -1e30f;
__device__ __forceinline__ bool is_off(float lc) { return lc < -1e29f; }
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }

template <int HD>
__device__ __forceinline__ float dot_row(const float* row, const float* reg) {
  float s = 0.f;
#pragma unroll
  for (int d = 0; d < HD; d += 4) {
    const float4 x = ld4(row + d);
    s += x.x * reg[d] + x.y * reg[d + 1] + x.z * reg[d + 2] + x.w * reg[d + 3];
  }
  return s;
}
template <int HD>
__device__ __forceinline__ void load_row(float* reg, const float* row) {
#pragma unroll
  for (int d = 0; d < HD; d += 4) {
    const float4 x = ld4(row + d);
    reg[d] = x.x, reg[d + 1] = x.y, reg[d + 2] = x.z, reg[d + 3] = x.w;
  }
}
// acc = acc * c + p * row
template <int HD>
__device__ __forceinline__ void axpby_row(float* acc, float c, float p, const float* row) {
#pragma unroll
  for (int d = 0; d < HD; d += 4) {
    const float4 x = ld4(row + d);
    acc[d] = acc[d] * c + p * x.x, acc[d + 1] = acc[d + 1] * c + p * x.y;
    acc[d + 2] = acc[d + 2] * c + p * x.z, acc[d + 3] = acc[d + 3] * c + p * x.w;
  }
}

// Columns [col, col + HD) of the atom's token rows of src (row stride ld) into dst [cnt][HD].
template <int HD>
__device__ __forceinline__ void stage(float* dst, const float* src, size_t ld, int col, int n, int N, int e0, int cnt) {
  constexpr int Q = HD / 4;
  for (int t = threadIdx.x; t < cnt * Q; t += blockDim.x) {
    const int r = t / Q, c = (t % Q) * 4;
    const size_t row = r == 0 ? size_t(n) : size_t(N) + e0 + r - 1;
    *reinterpret_cast<float4*>(dst + r * HD + c) = ld4(src + row * ld + col + c);
  }
}

template <int HD>
__global__ void __launch_bounds__(256) k_attn_fwd(AttnArgs p) {
  extern __shared__ __align__(16) float smem[];
  const int n = blockIdx.x / p.H, h = blockIdx.x % p.H, D = p.H * HD;
  const int e0 = p.off[n], cnt = p.off[n + 1] - e0 + 1;
  float* sk = smem;
  float* sv = sk + size_t(p.S) * HD;
  float* slc = sv + size_t(p.S) * HD;
  stage<HD>(sk, p.qkv, 3 * size_t(D), D + h * HD, n, p.N, e0, cnt);
  stage<HD>(sv, p.qkv, 3 * size_t(D), 2 * D + h * HD, n, p.N, e0, cnt);
  for (int r = threadIdx.x; r < cnt; r += blockDim.x) {
    const float cf = r == 0 ? 1.0f : p.cut[e0 + r - 1];
    slc[r] = cf > 0.f ? __logf(cf) : kOff;
  }
  __syncthreads();
  for (int sq = threadIdx.x; sq < cnt; sq += blockDim.x) {
    const size_t row = sq == 0 ? size_t(n) : size_t(p.N) + e0 + sq - 1;
    float* o = p.merged + row * D + h * HD;
    float* ml = p.ml ? p.ml + (row * p.H + h) * 2 : nullptr;
    if (sq > 0 && is_off(slc[sq])) {  // a query on an edge at its cutoff
#pragma unroll
      for (int d = 0; d < HD; ++d) o[d] = 0.f;
      if (ml) ml[0] = kOff, ml[1] = 0.f;
      continue;
    }
    float q[HD], acc[HD];
    load_row<HD>(q, p.qkv + row * 3 * D + h * HD);
#pragma unroll
    for (int d = 0; d < HD; ++d) acc[d] = 0.f;
    float mx = kOff, l = 0.f;
    for (int k = 0; k < cnt; ++k) {
      const float lc = slc[k];
      if (is_off(lc)) continue;
      const float s = dot_row<HD>(sk + k * HD, q) * p.sc + lc;
      const float nm = s > mx ? s : mx;
      const float c = __expf(mx - nm), w = __expf(s - nm);
      l = l * c + w;
      axpby_row<HD>(acc, c, w, sv + k * HD);
      mx = nm;
    }
    const float invl = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int d = 0; d < HD; d += 4)
      *reinterpret_cast<float4*>(o + d) = make_float4(acc[d] * invl, acc[d + 1] * invl, acc[d + 2] * invl, acc[d + 3] * invl);
    if (ml) ml[0] = mx, ml[1] = invl;
  }
}

template <int HD>
__global__ void __launch_bounds__(256) k_attn_bwd(AttnArgs p) {
  extern __shared__ __align__(16) float smem[];
  const int n = blockIdx.x / p.H, h = blockIdx.x % p.H, D = p.H * HD;
  const int e0 = p.off[n], cnt = p.off[n + 1] - e0 + 1;
  const size_t SH = size_t(p.S) * HD;
  float* sq_ = smem;
  float* sk = sq_ + SH;
  float* sv = sk + SH;
  float* sg = sv + SH;
  float* sm = sg + SH;
  float* sl = sm + p.S;
  float* sd = sl + p.S;
  float* slc = sd + p.S;
  stage<HD>(sq_, p.qkv, 3 * size_t(D), h * HD, n, p.N, e0, cnt);
  stage<HD>(sk, p.qkv, 3 * size_t(D), D + h * HD, n, p.N, e0, cnt);
  stage<HD>(sv, p.qkv, 3 * size_t(D), 2 * D + h * HD, n, p.N, e0, cnt);
  stage<HD>(sg, p.dmerged, size_t(D), h * HD, n, p.N, e0, cnt);
  for (int r = threadIdx.x; r < cnt; r += blockDim.x) {
    const size_t row = r == 0 ? size_t(n) : size_t(p.N) + e0 + r - 1;
    const float cf = r == 0 ? 1.0f : p.cut[e0 + r - 1];
    slc[r] = cf > 0.f ? __logf(cf) : kOff;
    sm[r] = p.ml[(row * p.H + h) * 2], sl[r] = p.ml[(row * p.H + h) * 2 + 1];
  }
  __syncthreads();
  // Queries: Dq = dO . O, dQ = sc sum_k dS K.
  for (int s = threadIdx.x; s < cnt; s += blockDim.x) {
    const size_t row = s == 0 ? size_t(n) : size_t(p.N) + e0 + s - 1;
    float q[HD], dout[HD], dq[HD];
    load_row<HD>(q, sq_ + s * HD);
    load_row<HD>(dout, sg + s * HD);
    const float Dq = dot_row<HD>(p.merged + row * D + h * HD, dout);
    sd[s] = Dq;
#pragma unroll
    for (int d = 0; d < HD; ++d) dq[d] = 0.f;
    const float m = sm[s], invl = sl[s];
    if (invl > 0.f)
      for (int k = 0; k < cnt; ++k) {
        const float lc = slc[k];
        if (is_off(lc)) continue;
        const float a = __expf(dot_row<HD>(sk + k * HD, q) * p.sc + lc - m) * invl;
        const float ds = a * (dot_row<HD>(sv + k * HD, dout) - Dq) * p.sc;
        axpby_row<HD>(dq, 1.0f, ds, sk + k * HD);
      }
    float* o = p.qkv_adj + row * 3 * D + h * HD;
#pragma unroll
    for (int d = 0; d < HD; d += 4) *reinterpret_cast<float4*>(o + d) = make_float4(dq[d], dq[d + 1], dq[d + 2], dq[d + 3]);
  }
  __syncthreads();
  // Keys: dK = sc sum_q dS Q, dV = sum_q A dO, and the key's dS summed over queries.
  for (int s = threadIdx.x; s < cnt; s += blockDim.x) {
    const size_t row = s == 0 ? size_t(n) : size_t(p.N) + e0 + s - 1;
    float k[HD], v[HD], dk[HD], dv[HD];
#pragma unroll
    for (int d = 0; d < HD; ++d) dk[d] = 0.f, dv[d] = 0.f;
    float cf_acc = 0.f;
    const float lcf = slc[s];
    if (!is_off(lcf)) {
      load_row<HD>(k, sk + s * HD);
      load_row<HD>(v, sv + s * HD);
      for (int q = 0; q < cnt; ++q) {
        const float invl = sl[q];
        if (invl <= 0.f) continue;
        const float a = __expf(dot_row<HD>(sq_ + q * HD, k) * p.sc + lcf - sm[q]) * invl;
        const float ds = a * (dot_row<HD>(sg + q * HD, v) - sd[q]);
        axpby_row<HD>(dk, 1.0f, ds * p.sc, sq_ + q * HD);
        axpby_row<HD>(dv, 1.0f, a, sg + q * HD);
        cf_acc += ds;
      }
    }
    float* ok = p.qkv_adj + row * 3 * D + D + h * HD;
    float* ov = p.qkv_adj + row * 3 * D + 2 * D + h * HD;
#pragma unroll
    for (int d = 0; d < HD; d += 4) {
      *reinterpret_cast<float4*>(ok + d) = make_float4(dk[d], dk[d + 1], dk[d + 2], dk[d + 3]);
      *reinterpret_cast<float4*>(ov + d) = make_float4(dv[d], dv[d + 1], dv[d + 2], dv[d + 3]);
    }
    p.cfh[row * p.H + h] = cf_acc;
  }
}

template <class K>
void launch(Stream& st, K kernel, const AttnArgs& p, size_t bytes, SmemOptIn& opted) {
  if (int(bytes) > 227 * 1024)
    throw Error(1, "attention: an atom with " + std::to_string(p.S - 1) + " neighbours needs " + std::to_string(bytes) +
                       " bytes of shared memory per block, above the device's 227 KiB");
  opt_in_shared_memory(kernel, bytes, opted);
  int threads = (p.S + 31) / 32 * 32;
  if (threads > 256) threads = 256;
  kernel<<<p.N * p.H, threads, bytes, st.s>>>(p);
  PETB_LAUNCH_CHECK(st);
}

template <int HD>
void fwd_hd(Stream& st, const AttnArgs& p) {
  static SmemOptIn opted;
  launch(st, k_attn_fwd<HD>, p, sizeof(float) * (2 * size_t(p.S) * HD + p.S), opted);
}
template <int HD>
void bwd_hd(Stream& st, const AttnArgs& p) {
  static SmemOptIn opted;
  launch(st, k_attn_bwd<HD>, p, sizeof(float) * (4 * size_t(p.S) * HD + 4 * size_t(p.S)), opted);
}

}  // namespace

void attention_forward(Stream& st, const AttnArgs& p) {
  if (p.N == 0) return;
  // The reference's own count (tools/roofline.py:188-202): 4 sum(cnt^2) D flops forward, 10 backward;
  // qkv read and the output written once.
  const double D = double(p.H) * p.hd;
  const ProfScope ps(st, PC_ATTN_FWD, 4.0 * p.pairs * D, 4.0 * p.T * (4.0 * D + 2.0 * p.H));
  if (p.mode != ATTN_NATIVE && attention_forward_mma(st, p)) return;
  if (attention_forward_tiled(st, p)) return;
  switch (p.hd) {
    case 16: return fwd_hd<16>(st, p);
    case 32: return fwd_hd<32>(st, p);
    case 48: return fwd_hd<48>(st, p);
    case 64: return fwd_hd<64>(st, p);
    case 80: return fwd_hd<80>(st, p);
    case 128: return fwd_hd<128>(st, p);
    default: throw Error(1, "attention: head_dim " + std::to_string(p.hd) + " is not one of 16, 32, 48, 64, 80, 128");
  }
}

void attention_backward(Stream& st, const AttnArgs& p) {
  if (p.N == 0) return;
  const double D = double(p.H) * p.hd;
  const ProfScope ps(st, PC_ATTN_BWD, 10.0 * p.pairs * D, 4.0 * p.T * (8.0 * D + 3.0 * p.H));
  if (p.mode != ATTN_NATIVE && attention_backward_mma(st, p)) return;
  if (attention_backward_tiled(st, p)) return;
  switch (p.hd) {
    case 16: return bwd_hd<16>(st, p);
    case 32: return bwd_hd<32>(st, p);
    case 48: return bwd_hd<48>(st, p);
    case 64: return bwd_hd<64>(st, p);
    case 80: return bwd_hd<80>(st, p);
    case 128: return bwd_hd<128>(st, p);
    default: throw Error(1, "attention: head_dim " + std::to_string(p.hd) + " is not one of 16, 32, 48, 64, 80, 128");
  }
}

}  // namespace petb
