// The GEMM epilogues, on runs of four consecutive output columns of one row.
// Shared by the CUDA-core and the tensor-core kernels.
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

// acc[0..3] are the accumulators of C(row, col..col+3); col % 4 == 0 and col + 3 < N.
template <int EPI>
__device__ __forceinline__ void epilogue_run4(const GemmArgs& p, int row, int col, const float* acc) {
  const size_t r = size_t(row);
  float z[4] = {acc[0], acc[1], acc[2], acc[3]};
  if (EPI == EPI_PLAIN || EPI == EPI_SILU || EPI == EPI_SWIGLU || EPI == EPI_COMPRESS) {
    if (p.bias) {
      const float4 b = ld4(p.bias + col);
      z[0] += b.x, z[1] += b.y, z[2] += b.z, z[3] += b.w;
    }
  }
  if (EPI == EPI_PLAIN) {
    if (p.res && row >= p.res_row0) {
      const float4 q = ld4(p.res + r * p.ldr + col);
      z[0] += q.x, z[1] += q.y, z[2] += q.z, z[3] += q.w;
    }
    st4(p.C + r * p.ldc + col, make_float4(z[0], z[1], z[2], z[3]));
  } else if (EPI == EPI_SILU) {
    if (p.pre) st4(p.pre + r * p.ldp + col, make_float4(z[0], z[1], z[2], z[3]));
    st4(p.C + r * p.ldc + col, make_float4(silu_f(z[0]), silu_f(z[1]), silu_f(z[2]), silu_f(z[3])));
  } else if (EPI == EPI_SWIGLU) {
    if (p.pre) st4(p.pre + r * p.ldp + col, make_float4(z[0], z[1], z[2], z[3]));
    if (p.C)
      *reinterpret_cast<float2*>(p.C + r * p.ldc + col / 2) = make_float2(z[0] * sigmoid_f(z[1]), z[2] * sigmoid_f(z[3]));
  } else if (EPI == EPI_SILU_BWD) {
    const float4 x = ld4(p.pre + r * p.ldp + col);
    st4(p.C + r * p.ldc + col, make_float4(z[0] * dsilu_f(x.x), z[1] * dsilu_f(x.y), z[2] * dsilu_f(x.z), z[3] * dsilu_f(x.w)));
  } else if (EPI == EPI_SWIGLU_BWD) {
    const float4 xa = ld4(p.pre + r * p.ldp + 2 * col), xb = ld4(p.pre + r * p.ldp + 2 * col + 4);
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
    const float e0 = (float) p.vec[3 * r], e1 = (float) p.vec[3 * r + 1], e2 = (float) p.vec[3 * r + 2], e3 = (float) p.dist[r];
    const float4 t = ld4(p.tab + size_t(p.sp[row]) * p.N + col);
    const float tt[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 w = ld4(p.wx + size_t(col + j) * 4);
      z[j] = z[j] + tt[j] + w.x * e0 + w.y * e1 + w.z * e2 + w.w * e3;
    }
    if (p.pre) st4(p.pre + r * p.ldp + col, make_float4(z[0], z[1], z[2], z[3]));
    st4(p.C + r * p.ldc + col, make_float4(silu_f(z[0]), silu_f(z[1]), silu_f(z[2]), silu_f(z[3])));
  }
}

}  // namespace petb
