// Attention on the tensor cores: warp-level mma.sync m16n8k8 with fp32 accumulation, in two forms. X3 (the
// reference's AttentionMode::TF32x3, src/attention.cpp:949-1011): every operand split into a leading tf32 part and
// its remainder, three products per tile, small terms first: fp32-class accuracy. Single pass (AttentionMode::TF32,
// src/attention.cpp:1031-1225 with X3 = false): operands rounded to tf32, one product per tile: the speed mode that
// goes with the tf32 and bf16 GEMM modes. Same mathematics as attention.cu; used when an atom's tokens fit shared
// memory.
//
// One CTA per (atom, head), one warp per block of 16 query rows (and, in the backward, one more per
// block of 16 keys). The head's Q, K, V (and dO) slices are staged once with a pitch
// of head_dim + 4 floats, which makes every fragment load below conflict-free:
//   X^T as B operand (scores Q K^T, dO V^T): b(k = t, n = g) = X[key 8kb + g][k0 + t]   -> banks 4g + t
//   X as B operand (P V, dS K, dS^T Q, P^T dO): the eight contraction indices of a step are taken in
//   the order 0,2,4,6,1,3,5,7, so b(k = t) = X[8kb + 2t][d0 + g], b(k = t + 4) = X[8kb + 2t + 1][d0 + g]
//   -> banks 8t + g; with that order the accumulator fragment of the scores (c0, c1 hold columns
//   2t, 2t + 1) IS the A fragment of the next product, so probabilities never leave registers.
// Forward: all scores of a query block stay in registers for the row max and sum. Backward, with the
// saved max and 1/sum: half of the warps take 16 queries each and form dQ = sc dS K key block by key
// block; the other half take 16 keys each and work transposed (S^T = K Q^T, dP^T = V dO^T), so that
// dS^T and P^T come out as A fragments for dK = sc dS^T Q and dV = P^T dO and each key's column sum of
// dS is a row sum. Nothing S x S is stored and the two halves never wait on each other.
// Every sum has one owner and a fixed order.
#include <cstdlib>

#include "attention.h"

namespace petb {

namespace {

constexpr float kOff = -1e30f;
__device__ __forceinline__ bool is_off(float lc) { return lc < -1e29f; }
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct Frag {
  uint32_t hi, lo;
};
// x = hi + lo with hi the leading 11 significant bits of x (truncated) and lo the remainder rounded to 11 bits
// (half of the last kept bit added, then masked). Integer and fp32-add instructions only: cvt.rna.tf32 runs on the
// quarter-rate conversion pipe, which two conversions per operand element had saturated.
// Single pass (X3 false): hi is x rounded to tf32 (nearest, half of the last kept bit added before the mask) and lo is
// never read, so the compiler drops it.
template <bool X3>
__device__ __forceinline__ Frag split(float x) {
  Frag f;
  if (X3) {
    f.hi = __float_as_uint(x) & 0xFFFFE000u;
    f.lo = (__float_as_uint(x - __uint_as_float(f.hi)) + 0x1000u) & 0xFFFFE000u;
  } else {
    f.hi = (__float_as_uint(x) + 0x1000u) & 0xFFFFE000u;
    f.lo = 0u;
  }
  return f;
}
__device__ __forceinline__ void mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// The same for G independent accumulators that share the A operand, one term at a time: consecutive
// instructions never depend on each other, so the tensor pipe's latency is covered inside one warp.
template <int G, bool X3>
__device__ __forceinline__ void mma3_shared_a(float (*c)[4], const Frag* a, const Frag (*b)[2]) {
  if (X3) {
#pragma unroll
    for (int j = 0; j < G; ++j) mma(c[j], a[0].lo, a[1].lo, a[2].lo, a[3].lo, b[j][0].hi, b[j][1].hi);
#pragma unroll
    for (int j = 0; j < G; ++j) mma(c[j], a[0].hi, a[1].hi, a[2].hi, a[3].hi, b[j][0].lo, b[j][1].lo);
  }
#pragma unroll
  for (int j = 0; j < G; ++j) mma(c[j], a[0].hi, a[1].hi, a[2].hi, a[3].hi, b[j][0].hi, b[j][1].hi);
}
// The same for two accumulators with their own A operands (two products that run side by side).
template <bool X3>
__device__ __forceinline__ void mma3_pair(float* c0, const Frag* a0, const Frag& p0, const Frag& p1, float* c1, const Frag* a1,
                                          const Frag& r0, const Frag& r1) {
  if (X3) {
    mma(c0, a0[0].lo, a0[1].lo, a0[2].lo, a0[3].lo, p0.hi, p1.hi);
    mma(c1, a1[0].lo, a1[1].lo, a1[2].lo, a1[3].lo, r0.hi, r1.hi);
    mma(c0, a0[0].hi, a0[1].hi, a0[2].hi, a0[3].hi, p0.lo, p1.lo);
    mma(c1, a1[0].hi, a1[1].hi, a1[2].hi, a1[3].hi, r0.lo, r1.lo);
  }
  mma(c0, a0[0].hi, a0[1].hi, a0[2].hi, a0[3].hi, p0.hi, p1.hi);
  mma(c1, a1[0].hi, a1[1].hi, a1[2].hi, a1[3].hi, r0.hi, r1.hi);
}

__host__ __device__ inline int round16(int s) { return (s + 15) / 16 * 16; }
// Pitch of the S x S tables: the smallest value >= S16 that is 4 modulo 32 (see the header).
__host__ __device__ inline int table_pitch(int S16) { return (S16 + 27) / 32 * 32 + 4; }

// Asynchronous 16-byte copies global -> shared: every tile's loads are in flight together, and no register waits on
// them; stage_wait() before the barrier that publishes the tiles.
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t) __cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void stage_wait() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

template <int HD>
__device__ __forceinline__ void stage(float* dst, const float* src, size_t ld, int col, int n, int N, int e0, int cnt, int rows) {
  constexpr int Q = HD / 4, P = HD + 4;
  for (int t = threadIdx.x; t < rows * Q; t += blockDim.x) {
    const int r = t / Q, c = (t % Q) * 4;
    if (r < cnt) {
      const size_t row = r == 0 ? size_t(n) : size_t(N) + e0 + r - 1;
      cp_async16(dst + r * P + c, src + row * ld + col + c);
    } else {
      *reinterpret_cast<float4*>(dst + r * P + c) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
}

// The A fragments (hi, lo) of rows r0.. r0+15 of X [.][P] for every 8-wide step of the head dimension.
template <int HD, bool X3>
__device__ __forceinline__ void load_a(Frag (*f)[4], const float* x, int r0, int g, int t) {
  constexpr int P = HD + 4;
#pragma unroll
  for (int ks = 0; ks < HD / 8; ++ks) {
    f[ks][0] = split<X3>(x[(r0 + g) * P + 8 * ks + t]);
    f[ks][1] = split<X3>(x[(r0 + g + 8) * P + 8 * ks + t]);
    f[ks][2] = split<X3>(x[(r0 + g) * P + 8 * ks + t + 4]);
    f[ks][3] = split<X3>(x[(r0 + g + 8) * P + 8 * ks + t + 4]);
  }
}

// One 8-wide step's A fragment, loaded where it is used: at head_dim 64 the fragments of all eight steps of two
// operands, split, would be 128 registers by themselves.
template <int HD, bool X3>
__device__ __forceinline__ void load_a_step(Frag* f, const float* x, int r0, int g, int t, int ks) {
  constexpr int P = HD + 4;
  f[0] = split<X3>(x[(r0 + g) * P + 8 * ks + t]);
  f[1] = split<X3>(x[(r0 + g + 8) * P + 8 * ks + t]);
  f[2] = split<X3>(x[(r0 + g) * P + 8 * ks + t + 4]);
  f[3] = split<X3>(x[(r0 + g + 8) * P + 8 * ks + t + 4]);
}

template <int HD, int MAXKB, bool X3>
__global__ void __launch_bounds__(32 * ((MAXKB + 1) / 2), MAXKB <= 10 ? 4 : 1) k_attn_fwd_mma(AttnArgs p) {
  constexpr int P = HD + 4, KS = HD / 8, R = 8 * MAXKB;  // R: staged token rows, the kernel's most (zero past the atom's)
  constexpr int G = MAXKB % 5 == 0 ? 5 : (MAXKB % 4 == 0 ? 4 : 2);  // key blocks whose score tiles advance together
  extern __shared__ __align__(16) float smem[];
  const int n = blockIdx.x / p.H, h = blockIdx.x % p.H, D = p.H * HD;
  const int e0 = p.off[n], cnt = p.off[n + 1] - e0 + 1;
  // key blocks of 8 that hold a token at all: a block past them is zero rows with their cutoff off, and adds nothing
  const int S16 = round16(cnt), nkb = (cnt + 7) / 8;
  float* sq = smem;
  float* sk = sq + R * P;
  float* sv = sk + R * P;
  float* slc = sv + R * P;
  stage<HD>(sq, p.qkv, 3 * size_t(D), h * HD, n, p.N, e0, cnt, S16);
  stage<HD>(sk, p.qkv, 3 * size_t(D), D + h * HD, n, p.N, e0, cnt, R);
  stage<HD>(sv, p.qkv, 3 * size_t(D), 2 * D + h * HD, n, p.N, e0, cnt, R);
  for (int r = threadIdx.x; r < R; r += blockDim.x) {
    const float cf = r == 0 ? 1.0f : (r < cnt ? p.cut[e0 + r - 1] : 0.f);
    slc[r] = cf > 0.f ? __logf(cf) : kOff;
  }
  stage_wait();
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int r0 = 16 * warp;
  if (r0 >= cnt) return;

  Frag qf[KS][4];
  load_a<HD, X3>(qf, sq, r0, g, t);
  float s[MAXKB][4];
#pragma unroll
  for (int kb = 0; kb < MAXKB; ++kb) s[kb][0] = s[kb][1] = s[kb][2] = s[kb][3] = 0.f;
#pragma unroll
  for (int kg = 0; kg < MAXKB; kg += G) {
    if (kg < nkb) {  // the same for the whole CTA; a group's blocks past the atom's keys read zero rows
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        Frag b[G][2];
#pragma unroll
        for (int j = 0; j < G; ++j) {
          b[j][0] = split<X3>(sk[(8 * (kg + j) + g) * P + 8 * ks + t]);
          b[j][1] = split<X3>(sk[(8 * (kg + j) + g) * P + 8 * ks + t + 4]);
        }
        mma3_shared_a<G, X3>(&s[kg], qf[ks], b);
      }
    }
  }
  // bias, row max, exponentials, row sum; this lane holds rows g and g + 8, keys 8kb + 2t and + 1
  float m0 = kOff, m1 = kOff;
#pragma unroll
  for (int kb = 0; kb < MAXKB; ++kb)
    if (kb < nkb) {
      const float lc0 = slc[8 * kb + 2 * t], lc1 = slc[8 * kb + 2 * t + 1];
      s[kb][0] = is_off(lc0) ? kOff : s[kb][0] * p.sc + lc0;
      s[kb][1] = is_off(lc1) ? kOff : s[kb][1] * p.sc + lc1;
      s[kb][2] = is_off(lc0) ? kOff : s[kb][2] * p.sc + lc0;
      s[kb][3] = is_off(lc1) ? kOff : s[kb][3] * p.sc + lc1;
      m0 = fmaxf(m0, fmaxf(s[kb][0], s[kb][1]));
      m1 = fmaxf(m1, fmaxf(s[kb][2], s[kb][3]));
    }
  m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 1)), m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 2));
  m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 1)), m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 2));
  float l0 = 0.f, l1 = 0.f;
#pragma unroll
  for (int kb = 0; kb < MAXKB; ++kb)
    if (kb < nkb) {
      s[kb][0] = is_off(s[kb][0]) ? 0.f : __expf(s[kb][0] - m0);
      s[kb][1] = is_off(s[kb][1]) ? 0.f : __expf(s[kb][1] - m0);
      s[kb][2] = is_off(s[kb][2]) ? 0.f : __expf(s[kb][2] - m1);
      s[kb][3] = is_off(s[kb][3]) ? 0.f : __expf(s[kb][3] - m1);
      l0 += s[kb][0] + s[kb][1];
      l1 += s[kb][2] + s[kb][3];
    }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1), l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1), l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const int q0 = r0 + g, q1 = r0 + g + 8;
  const bool dead0 = q0 > 0 && is_off(slc[q0]), dead1 = q1 > 0 && is_off(slc[q1]);  // a query on an edge at its cutoff
  const float il0 = (!dead0 && l0 > 0.f) ? 1.0f / l0 : 0.f, il1 = (!dead1 && l1 > 0.f) ? 1.0f / l1 : 0.f;

  // O = P V, the probabilities going straight from the accumulator layout into the A operand
  float o[KS][4];
#pragma unroll
  for (int db = 0; db < KS; ++db) o[db][0] = o[db][1] = o[db][2] = o[db][3] = 0.f;
#pragma unroll
  for (int kb = 0; kb < MAXKB; ++kb)
    if (kb < nkb) {
      const Frag a[4] = {split<X3>(s[kb][0] * il0), split<X3>(s[kb][2] * il1), split<X3>(s[kb][1] * il0), split<X3>(s[kb][3] * il1)};
      Frag b[KS][2];
#pragma unroll
      for (int db = 0; db < KS; ++db) {
        b[db][0] = split<X3>(sv[(8 * kb + 2 * t) * P + 8 * db + g]);
        b[db][1] = split<X3>(sv[(8 * kb + 2 * t + 1) * P + 8 * db + g]);
      }
      mma3_shared_a<KS, X3>(o, a, b);
    }
  const size_t g0 = q0 == 0 ? size_t(n) : size_t(p.N) + e0 + q0 - 1, g1 = size_t(p.N) + e0 + q1 - 1;
#pragma unroll
  for (int db = 0; db < KS; ++db) {
    if (q0 < cnt) *reinterpret_cast<float2*>(p.merged + g0 * D + h * HD + 8 * db + 2 * t) = make_float2(o[db][0], o[db][1]);
    if (q1 < cnt) *reinterpret_cast<float2*>(p.merged + g1 * D + h * HD + 8 * db + 2 * t) = make_float2(o[db][2], o[db][3]);
  }
  if (t == 0 && p.ml) {
    if (q0 < cnt) p.ml[(g0 * p.H + h) * 2] = dead0 ? kOff : m0, p.ml[(g0 * p.H + h) * 2 + 1] = il0;
    if (q1 < cnt) p.ml[(g1 * p.H + h) * 2] = dead1 ? kOff : m1, p.ml[(g1 * p.H + h) * 2 + 1] = il1;
  }
}

template <int HD, int MAXT, bool X3>
__global__ void __launch_bounds__(MAXT, MAXT <= 320 ? 2 : 1) k_attn_bwd_mma(AttnArgs p) {
  constexpr int P = HD + 4, KS = HD / 8;
  // The A fragments stay in registers over the whole key loop up to head_dim 32. At 64 they would be 128 registers
  // (two operands, eight steps, four values, two parts) and the compiler spilled a kilobyte per thread: there each
  // step's fragment is loaded and split where it is used (22.3 against 32.8 ms on a 1000-atom cell of the l shape).
  constexpr bool KEEP = HD <= 32;
  extern __shared__ __align__(16) float smem[];
  const int n = blockIdx.x / p.H, h = blockIdx.x % p.H, D = p.H * HD;
  const int e0 = p.off[n], cnt = p.off[n + 1] - e0 + 1;
  // nkb: blocks of 8 keys (or, on the key side, of 8 queries) that hold a token at all; the rows past them are zero
  // with zero weight, so leaving their block out changes no bit
  const int S16 = round16(cnt), nkb = (cnt + 7) / 8, SM = round16(p.S);
  float* sq = smem;
  float* sk = sq + SM * P;
  float* sv = sk + SM * P;
  float* sg = sv + SM * P;
  float* slc = sg + SM * P;
  float* sm = slc + SM;
  float* sl = sm + SM;
  float* sd = sl + SM;
  stage<HD>(sq, p.qkv, 3 * size_t(D), h * HD, n, p.N, e0, cnt, S16);
  stage<HD>(sk, p.qkv, 3 * size_t(D), D + h * HD, n, p.N, e0, cnt, S16);
  stage<HD>(sv, p.qkv, 3 * size_t(D), 2 * D + h * HD, n, p.N, e0, cnt, S16);
  stage<HD>(sg, p.dmerged, size_t(D), h * HD, n, p.N, e0, cnt, S16);
  for (int r = threadIdx.x; r < S16; r += blockDim.x) {
    float lc = kOff, m = 0.f, il = 0.f, dqv = 0.f;
    if (r < cnt) {
      const size_t row = r == 0 ? size_t(n) : size_t(p.N) + e0 + r - 1;
      const float cf = r == 0 ? 1.0f : p.cut[e0 + r - 1];
      lc = cf > 0.f ? __logf(cf) : kOff;
      m = p.ml[(row * p.H + h) * 2], il = p.ml[(row * p.H + h) * 2 + 1];
      // Dq = dO . O of this query's head slice, both rows straight from global memory: a thread per row, its loads
      // all in flight together
      const float4* o4 = reinterpret_cast<const float4*>(p.merged + row * D + h * HD);
      const float4* g4 = reinterpret_cast<const float4*>(p.dmerged + row * D + h * HD);
#pragma unroll
      for (int c = 0; c < HD / 4; ++c) {
        const float4 a = o4[c], b = g4[c];
        dqv += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
      }
    }
    slc[r] = lc, sm[r] = m, sl[r] = il, sd[r] = dqv;
  }
  stage_wait();
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5, g = lane >> 2, t = lane & 3;
  // The first half of the warps take 16 queries each (dQ), the second half 16 keys each (dK, dV and
  // the keys' cutoff shares), both recomputing the weights they need: no S x S table, no further barrier.
  // With more blocks than warps of a kind (long neighbour lists) a warp takes every half-th block in turn.
  const int half = nw >> 1;
  const bool keys = warp >= half;
  for (int r0 = 16 * (keys ? warp - half : warp); r0 < S16; r0 += 16 * half) {
  const int i0 = r0 + g, i1 = r0 + g + 8;  // this lane's two rows (queries or keys)
  const size_t g0 = i0 == 0 ? size_t(n) : size_t(p.N) + e0 + i0 - 1, g1 = size_t(p.N) + e0 + i1 - 1;
  if (!keys) {
    Frag qf[KEEP ? KS : 1][4], gf[KEEP ? KS : 1][4];
    if (KEEP) {
      load_a<HD, X3>(qf, sq, r0, g, t);
      load_a<HD, X3>(gf, sg, r0, g, t);
    }
    const float m0 = sm[i0], m1 = sm[i1], il0 = sl[i0], il1 = sl[i1], dq0 = sd[i0], dq1 = sd[i1];
    float dq[KS][4];
#pragma unroll
    for (int db = 0; db < KS; ++db) dq[db][0] = dq[db][1] = dq[db][2] = dq[db][3] = 0.f;
    for (int kb = 0; kb < nkb; ++kb) {
      if (!KEEP) asm volatile("" ::: "memory");  // or the fragment loads are hoisted out of the loop and live across it again
      float cs[4] = {0.f, 0.f, 0.f, 0.f}, cp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const Frag k0 = split<X3>(sk[(8 * kb + g) * P + 8 * ks + t]), k1 = split<X3>(sk[(8 * kb + g) * P + 8 * ks + t + 4]);
        const Frag v0 = split<X3>(sv[(8 * kb + g) * P + 8 * ks + t]), v1 = split<X3>(sv[(8 * kb + g) * P + 8 * ks + t + 4]);
        if (!KEEP) {
          load_a_step<HD, X3>(qf[0], sq, r0, g, t, ks);
          load_a_step<HD, X3>(gf[0], sg, r0, g, t, ks);
        }
        mma3_pair<X3>(cs, qf[KEEP ? ks : 0], k0, k1, cp, gf[KEEP ? ks : 0], v0, v1);
      }
      const int key = 8 * kb + 2 * t;
      const float lc0 = slc[key], lc1 = slc[key + 1];
      const float P0 = (il0 > 0.f && !is_off(lc0)) ? __expf(cs[0] * p.sc + lc0 - m0) * il0 : 0.f;
      const float P1 = (il0 > 0.f && !is_off(lc1)) ? __expf(cs[1] * p.sc + lc1 - m0) * il0 : 0.f;
      const float P2 = (il1 > 0.f && !is_off(lc0)) ? __expf(cs[2] * p.sc + lc0 - m1) * il1 : 0.f;
      const float P3 = (il1 > 0.f && !is_off(lc1)) ? __expf(cs[3] * p.sc + lc1 - m1) * il1 : 0.f;
      const Frag a[4] = {split<X3>(P0 * (cp[0] - dq0)), split<X3>(P2 * (cp[2] - dq1)), split<X3>(P1 * (cp[1] - dq0)), split<X3>(P3 * (cp[3] - dq1))};
      Frag b[KS][2];
#pragma unroll
      for (int db = 0; db < KS; ++db) {
        b[db][0] = split<X3>(sk[(8 * kb + 2 * t) * P + 8 * db + g]);
        b[db][1] = split<X3>(sk[(8 * kb + 2 * t + 1) * P + 8 * db + g]);
      }
      mma3_shared_a<KS, X3>(dq, a, b);
    }
#pragma unroll
    for (int db = 0; db < KS; ++db) {
      if (i0 < cnt)
        *reinterpret_cast<float2*>(p.qkv_adj + g0 * 3 * D + h * HD + 8 * db + 2 * t) = make_float2(dq[db][0] * p.sc, dq[db][1] * p.sc);
      if (i1 < cnt)
        *reinterpret_cast<float2*>(p.qkv_adj + g1 * 3 * D + h * HD + 8 * db + 2 * t) = make_float2(dq[db][2] * p.sc, dq[db][3] * p.sc);
    }
  } else {
    // transposed: rows are keys. S^T = K Q^T and dP^T = V dO^T per block of 8 queries; the accumulator
    // fragment of dS^T (and P^T) is the A operand of dK = dS^T Q (and dV = P^T dO).
    Frag kf[KEEP ? KS : 1][4], vf[KEEP ? KS : 1][4];
    if (KEEP) {
      load_a<HD, X3>(kf, sk, r0, g, t);
      load_a<HD, X3>(vf, sv, r0, g, t);
    }
    const float lc0 = slc[i0], lc1 = slc[i1];
    const bool on0 = !is_off(lc0), on1 = !is_off(lc1);
    float dk[KS][4], dv[KS][4], cf0 = 0.f, cf1 = 0.f;
#pragma unroll
    for (int db = 0; db < KS; ++db)
      dk[db][0] = dk[db][1] = dk[db][2] = dk[db][3] = dv[db][0] = dv[db][1] = dv[db][2] = dv[db][3] = 0.f;
    for (int qb = 0; qb < nkb; ++qb) {
      if (!KEEP) asm volatile("" ::: "memory");
      float cs[4] = {0.f, 0.f, 0.f, 0.f}, cp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const Frag q0 = split<X3>(sq[(8 * qb + g) * P + 8 * ks + t]), q1 = split<X3>(sq[(8 * qb + g) * P + 8 * ks + t + 4]);
        const Frag d0 = split<X3>(sg[(8 * qb + g) * P + 8 * ks + t]), d1 = split<X3>(sg[(8 * qb + g) * P + 8 * ks + t + 4]);
        if (!KEEP) {
          load_a_step<HD, X3>(kf[0], sk, r0, g, t, ks);
          load_a_step<HD, X3>(vf[0], sv, r0, g, t, ks);
        }
        mma3_pair<X3>(cs, kf[KEEP ? ks : 0], q0, q1, cp, vf[KEEP ? ks : 0], d0, d1);
      }
      const int qa = 8 * qb + 2 * t, qc = qa + 1;  // this lane's two queries of the block
      const float ma = sm[qa], mc = sm[qc], ila = sl[qa], ilc = sl[qc], da = sd[qa], dc = sd[qc];
      const float P0 = (on0 && ila > 0.f) ? __expf(cs[0] * p.sc + lc0 - ma) * ila : 0.f;  // key i0, query qa
      const float P1 = (on0 && ilc > 0.f) ? __expf(cs[1] * p.sc + lc0 - mc) * ilc : 0.f;  // key i0, query qc
      const float P2 = (on1 && ila > 0.f) ? __expf(cs[2] * p.sc + lc1 - ma) * ila : 0.f;  // key i1, query qa
      const float P3 = (on1 && ilc > 0.f) ? __expf(cs[3] * p.sc + lc1 - mc) * ilc : 0.f;
      const float S0 = P0 * (cp[0] - da), S1 = P1 * (cp[1] - dc), S2 = P2 * (cp[2] - da), S3 = P3 * (cp[3] - dc);
      cf0 += S0 + S1, cf1 += S2 + S3;
      const Frag as[4] = {split<X3>(S0), split<X3>(S2), split<X3>(S1), split<X3>(S3)};
      const Frag ap[4] = {split<X3>(P0), split<X3>(P2), split<X3>(P1), split<X3>(P3)};
      {
        Frag b[KS][2];
#pragma unroll
        for (int db = 0; db < KS; ++db) b[db][0] = split<X3>(sq[qa * P + 8 * db + g]), b[db][1] = split<X3>(sq[qc * P + 8 * db + g]);
        mma3_shared_a<KS, X3>(dk, as, b);
      }
      {
        Frag b[KS][2];
#pragma unroll
        for (int db = 0; db < KS; ++db) b[db][0] = split<X3>(sg[qa * P + 8 * db + g]), b[db][1] = split<X3>(sg[qc * P + 8 * db + g]);
        mma3_shared_a<KS, X3>(dv, ap, b);
      }
    }
    cf0 += __shfl_xor_sync(0xffffffffu, cf0, 1), cf0 += __shfl_xor_sync(0xffffffffu, cf0, 2);
    cf1 += __shfl_xor_sync(0xffffffffu, cf1, 1), cf1 += __shfl_xor_sync(0xffffffffu, cf1, 2);
#pragma unroll
    for (int db = 0; db < KS; ++db) {
      const int c = h * HD + 8 * db + 2 * t;
      if (i0 < cnt) {
        *reinterpret_cast<float2*>(p.qkv_adj + g0 * 3 * D + D + c) = make_float2(dk[db][0] * p.sc, dk[db][1] * p.sc);
        *reinterpret_cast<float2*>(p.qkv_adj + g0 * 3 * D + 2 * D + c) = make_float2(dv[db][0], dv[db][1]);
      }
      if (i1 < cnt) {
        *reinterpret_cast<float2*>(p.qkv_adj + g1 * 3 * D + D + c) = make_float2(dk[db][2] * p.sc, dk[db][3] * p.sc);
        *reinterpret_cast<float2*>(p.qkv_adj + g1 * 3 * D + 2 * D + c) = make_float2(dv[db][2], dv[db][3]);
      }
    }
    if (t == 0) {  // each key's dS summed over its queries: the cutoff factor's share from this head
      if (i0 < cnt) p.cfh[g0 * p.H + h] = cf0;
      if (i1 < cnt) p.cfh[g1 * p.H + h] = cf1;
    }
  }
  }
}

bool enabled() {
  static const bool on = [] {
    const char* e = std::getenv("PET_ATTN_MMA");
    return !(e && e[0] == '0');
  }();
  return on;
}

size_t fwd_bytes(int maxkb, int HD) {
  const int R = 8 * maxkb;
  return sizeof(float) * (3 * size_t(R) * (HD + 4) + R);
}
size_t bwd_bytes(int S, int HD) {
  const int SM = round16(S);
  return sizeof(float) * (4 * size_t(SM) * (HD + 4) + 4 * size_t(SM));
}

template <class K>
void launch(Stream& st, K kernel, const AttnArgs& p, size_t bytes, int threads, SmemOptIn& opted) {
  opt_in_shared_memory(kernel, bytes, opted);
  kernel<<<p.N * p.H, threads, bytes, st.s>>>(p);
  PETB_LAUNCH_CHECK(st);
}

template <int HD, bool X3>
bool fwd_hd(Stream& st, const AttnArgs& p) {
  const int S16 = round16(p.S), threads = 32 * (S16 / 16);
  if (S16 > 176 || fwd_bytes(22, HD) > 200 * 1024) return false;
  static SmemOptIn o10, o16, o22;
  if (S16 <= 80) launch(st, k_attn_fwd_mma<HD, 10, X3>, p, fwd_bytes(10, HD), threads, o10);
  else if (S16 <= 128) launch(st, k_attn_fwd_mma<HD, 16, X3>, p, fwd_bytes(16, HD), threads, o16);
  else launch(st, k_attn_fwd_mma<HD, 22, X3>, p, fwd_bytes(22, HD), threads, o22);
  return true;
}
template <int HD, bool X3>
bool bwd_hd(Stream& st, const AttnArgs& p) {
  const int S16 = round16(p.S);
  int threads = 2 * 32 * (S16 / 16);  // a warp per 16 queries and a warp per 16 keys, up to 512 threads: then blocks in turn
  if (threads > 512) threads = 512;
  const size_t bytes = bwd_bytes(p.S, HD);
  if (bytes > 200 * 1024) return false;
  static SmemOptIn o320, o512;
  if (threads <= 320) launch(st, k_attn_bwd_mma<HD, 320, X3>, p, bytes, threads, o320);
  else launch(st, k_attn_bwd_mma<HD, 512, X3>, p, bytes, threads, o512);
  return true;
}

template <bool X3>
bool fwd_any(Stream& st, const AttnArgs& p) {
  switch (p.hd) {
    case 16: return fwd_hd<16, X3>(st, p);
    case 32: return fwd_hd<32, X3>(st, p);
    case 64: return fwd_hd<64, X3>(st, p);
    default: return false;
  }
}
template <bool X3>
bool bwd_any(Stream& st, const AttnArgs& p) {
  switch (p.hd) {
    case 16: return bwd_hd<16, X3>(st, p);
    case 32: return bwd_hd<32, X3>(st, p);
    case 64: return bwd_hd<64, X3>(st, p);
    default: return false;
  }
}

}  // namespace

// True if the tensor-core kernel took the pass; false leaves it to the other kernels.
bool attention_forward_mma(Stream& st, const AttnArgs& p) {
  if (!enabled()) return false;
  return p.mode == ATTN_TF32 ? fwd_any<false>(st, p) : fwd_any<true>(st, p);
}

bool attention_backward_mma(Stream& st, const AttnArgs& p) {
  if (!enabled()) return false;
  return p.mode == ATTN_TF32 ? bwd_any<false>(st, p) : bwd_any<true>(st, p);
}

}  // namespace petb
