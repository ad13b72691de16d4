// The GEMM epilogues, on runs of four consecutive output columns of one row.
// Shared by the CUDA-core and the tensor-core kernels. Each epilogue is split into the global
// loads it needs (epilogue_load4) and the arithmetic and stores (epilogue_apply4), so that a
// kernel can issue the loads of several rows before it consumes any of them.
#pragma once

#include "gemm.h"

namespace petb {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x * sigmoid_f(x); }
// d silu / dx = s (1 + x (1 - s))
__device__ __forceinline__ float dsilu_f(float x) {
  const float s = sigmoid_f(x);
  return s * (1.0f + x * (1.0f - s));
}

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }

// What an epilogue reads from global memory for one run of four columns.
struct EpiLoad {
  float4 a, b;        // residual or saved pre-activation (two for the SwiGLU backward), species-table row
  float e0, e1, e2, e3;  // compress: the edge's (v, |v|) in float
};

template <int EPI>
__device__ __forceinline__ EpiLoad epilogue_load4(const GemmArgs& p, int row, int col) {
  const size_t r = size_t(row);
  EpiLoad l;
  l.a = l.b = make_float4(0.f, 0.f, 0.f, 0.f);
  l.e0 = l.e1 = l.e2 = l.e3 = 0.f;
  if (EPI == EPI_PLAIN) {
    if (p.res && row >= p.res_row0) l.a = ld4(p.res + r * p.ldr + col);
  } else if (EPI == EPI_SILU_BWD) {
    l.a = ld4(p.pre + r * p.ldp + col);
  } else if (EPI == EPI_SWIGLU_BWD) {
    l.a = ld4(p.pre + r * p.ldp + 2 * col);
    l.b = ld4(p.pre + r * p.ldp + 2 * col + 4);
  } else if (EPI == EPI_COMPRESS) {
    l.a = ld4(p.tab + size_t(p.sp[row]) * p.N + col);
    l.e0 = (float) p.vec[3 * r], l.e1 = (float) p.vec[3 * r + 1], l.e2 = (float) p.vec[3 * r + 2], l.e3 = (float) p.dist[r];
  }
  return l;
}

// acc[0..3] are the accumulators of C(row, col..col+3); col % 4 == 0 and col + 3 < N.
template <int EPI>
__device__ __forceinline__ void epilogue_apply4(const GemmArgs& p, int row, int col, const float* acc, const EpiLoad& l) {
  const size_t r = size_t(row);
  float z[4] = {acc[0], acc[1], acc[2], acc[3]};
  if (EPI == EPI_PLAIN || EPI == EPI_SILU || EPI == EPI_SWIGLU || EPI == EPI_COMPRESS) {
    if (p.bias) {
      const float4 b = ld4(p.bias + col);
      z[0] += b.x, z[1] += b.y, z[2] += b.z, z[3] += b.w;
    }
  }
  if (EPI == EPI_PLAIN) {
    if (p.res && row >= p.res_row0) z[0] += l.a.x, z[1] += l.a.y, z[2] += l.a.z, z[3] += l.a.w;
    st4(p.C + r * p.ldc + col, make_float4(z[0], z[1], z[2], z[3]));
  } else if (EPI == EPI_SILU) {
    if (p.pre) st4(p.pre + r * p.ldp + col, make_float4(z[0], z[1], z[2], z[3]));
    st4(p.C + r * p.ldc + col, make_float4(silu_f(z[0]), silu_f(z[1]), silu_f(z[2]), silu_f(z[3])));
  } else if (EPI == EPI_SWIGLU) {
    if (p.pre) st4(p.pre + r * p.ldp + col, make_float4(z[0], z[1], z[2], z[3]));
    if (p.C)
      *reinterpret_cast<float2*>(p.C + r * p.ldc + col / 2) = make_float2(z[0] * sigmoid_f(z[1]), z[2] * sigmoid_f(z[3]));
  } else if (EPI == EPI_SILU_BWD) {
    const float4 x = l.a;
    st4(p.C + r * p.ldc + col, make_float4(z[0] * dsilu_f(x.x), z[1] * dsilu_f(x.y), z[2] * dsilu_f(x.z), z[3] * dsilu_f(x.w)));
  } else if (EPI == EPI_SWIGLU_BWD) {
    const float4 xa = l.a, xb = l.b;
    const float v[4] = {xa.x, xa.z, xb.x, xb.z}, g[4] = {xa.y, xa.w, xb.y, xb.w};
    float o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float sg = sigmoid_f(g[j]);
      o[2 * j] = z[j] * sg;
      o[2 * j + 1] = z[j] * v[j] * sg * (1.0f - sg);
    }
    st4(p.C + r * p.ldc + 2 * col, make_float4(o[0], o[1], o[2], o[3]));
    st4(p.C + r * p.ldc + 2 * col + 4, make_float4(o[4], o[5], o[6], o[7]));
  } else if (EPI == EPI_COMPRESS) {
    const float tt[4] = {l.a.x, l.a.y, l.a.z, l.a.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 w = ld4(p.wx + size_t(col + j) * 4);
      z[j] = z[j] + tt[j] + w.x * l.e0 + w.y * l.e1 + w.z * l.e2 + w.w * l.e3;
    }
    if (p.pre) st4(p.pre + r * p.ldp + col, make_float4(z[0], z[1], z[2], z[3]));
    st4(p.C + r * p.ldc + col, make_float4(silu_f(z[0]), silu_f(z[1]), silu_f(z[2]), silu_f(z[3])));
  }
}

template <int EPI>
__device__ __forceinline__ void epilogue_run4(const GemmArgs& p, int row, int col, const float* acc) {
  const EpiLoad l = epilogue_load4<EPI>(p, row, col);
  epilogue_apply4<EPI>(p, row, col, acc, l);
}

}  // namespace petb
