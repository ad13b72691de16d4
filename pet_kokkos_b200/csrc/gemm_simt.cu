// The fp32 (native) GEMM on the CUDA cores and the GEMM dispatcher: see gemm.h.
//
// 128 x 128 x 16 tiles, 256 threads, 8 x 8 outputs per thread, operands staged in
// shared memory (transposed, so the inner loop reads float4s) with the next tile's
// global loads issued before the current tile's arithmetic. Each output is one
// chain of fused multiply-adds over k in increasing order, whatever the tile or
// the row count: a row's result depends on that row alone.
#include "epilogue.cuh"

namespace petb {

void gemm_tensor(Stream& st, Arena& arena, const GemmArgs& a, int mode);  // gemm_tc.cu
bool gemm_tensor_usable(const GemmArgs& a, int mode);

namespace {

constexpr int BM = 128, BN = 128, BK = 16, PAD = 4;

// Two fp32 values in one 64-bit register, and the packed fused multiply-add of sm_100: d.x = a.x * b.x + d.x and
// d.y = a.y * b.y + d.y, each rounded once (round to nearest even), as fmaf does.
__device__ __forceinline__ unsigned long long pack2(float x, float y) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(x), "f"(y));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& x, float& y) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(x), "=f"(y) : "l"(v));
}
__device__ __forceinline__ void fma2(unsigned long long& d, unsigned long long a, unsigned long long b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}

template <int EPI>
__global__ void __launch_bounds__(256, 2) k_gemm_native(GemmArgs p) {
  __shared__ __align__(16) float As[2][BK][BM + PAD];
  __shared__ __align__(16) float Bs[2][BK][BN + PAD];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int m0 = (blockIdx.x / tiles_n) * BM, n0 = (blockIdx.x % tiles_n) * BN;

  // Loader: a thread brings rows lr and lr + 64 of each tile, four k values at lk.
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  float4 ra[2], rb[2];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int am = m0 + lr + 64 * h, bn = n0 + lr + 64 * h, k = k0 + lk;
      ra[h] = (am < p.M && k < p.K) ? ld4(p.A + size_t(am) * p.lda + k) : make_float4(0, 0, 0, 0);
      rb[h] = (bn < p.N && k < p.K) ? ld4(p.B + size_t(bn) * p.ldb + k) : make_float4(0, 0, 0, 0);
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = lr + 64 * h;
      As[buf][lk + 0][r] = ra[h].x, As[buf][lk + 1][r] = ra[h].y, As[buf][lk + 2][r] = ra[h].z, As[buf][lk + 3][r] = ra[h].w;
      Bs[buf][lk + 0][r] = rb[h].x, Bs[buf][lk + 1][r] = rb[h].y, Bs[buf][lk + 2][r] = rb[h].z, Bs[buf][lk + 3][r] = rb[h].w;
    }
  };

  // The accumulators as pairs of neighbouring columns: one fma.rn.f32x2 advances two of them with the IEEE fp32
  // fused multiply-add of the scalar instruction (same bits), for half the issue slots.
  unsigned long long acc2[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc2[i][j] = 0ull;

  fetch(0);
  stash(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < p.K; k0 += BK) {
    const bool more = k0 + BK < p.K;
    if (more) fetch(k0 + BK);
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a0 = ld4(&As[buf][k][ty * 4]), a1 = ld4(&As[buf][k][64 + ty * 4]);
      const float4 b0 = ld4(&Bs[buf][k][tx * 4]), b1 = ld4(&Bs[buf][k][64 + tx * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const unsigned long long b2[4] = {pack2(b0.x, b0.y), pack2(b0.z, b0.w), pack2(b1.x, b1.y), pack2(b1.z, b1.w)};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const unsigned long long aa = pack2(a[i], a[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) fma2(acc2[i][j], aa, b2[j]);
      }
    }
    if (more) {
      stash(buf ^ 1);
      __syncthreads();
      buf ^= 1;
    }
  }

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) unpack2(acc2[i][j], acc[i][2 * j], acc[i][2 * j + 1]);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (row >= p.M) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int col = n0 + 64 * h + tx * 4;
      if (col < p.N) epilogue_run4<EPI>(p, row, col, &acc[i][4 * h]);
    }
  }
}

__global__ void k_gemv_rows(const float* __restrict__ A, int lda, const float* __restrict__ w, const float* __restrict__ bias,
                            float* __restrict__ out, int M, int K) {
  const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (r >= M) return;
  float s = 0.0f;
  for (int k = lane; k < K; k += 32) s = fmaf(A[size_t(r) * lda + k], w[k], s);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) out[r] = s + (bias ? bias[0] : 0.0f);
}

template <int EPI>
void launch_native(Stream& st, const GemmArgs& a) {
  const long long tiles = (long long) cdiv(a.M, BM) * cdiv(a.N, BN);
  k_gemm_native<EPI><<<(unsigned) tiles, 256, 0, st.s>>>(a);
  PETB_LAUNCH_CHECK(st);
}

}  // namespace

void gemm(Stream& st, Arena& arena, const GemmArgs& a, int mode) {
  if (a.M <= 0 || a.N <= 0) return;
  if (a.N % 4 || a.K % 4 || a.lda % 4 || a.ldb % 4 || a.ldc % 2)
    throw Error(2, "gemm: widths must be multiples of 4 (N=" + std::to_string(a.N) + ", K=" + std::to_string(a.K) + ")");
  // Algorithmic work: 2MNK flops; A, B, C once each, plus what the epilogue reads and writes.
  double bytes = 4.0 * (double(a.M) * a.K + double(a.N) * a.K + double(a.M) * a.N);
  if (a.res) bytes += 4.0 * a.M * a.N;
  if (a.pre) bytes += 4.0 * a.M * a.N * (a.epi == EPI_SWIGLU_BWD ? 2.0 : 1.0);
  if (a.epi == EPI_SWIGLU) bytes -= 2.0 * a.M * a.N;      // h is half as wide as the product
  if (a.epi == EPI_SWIGLU_BWD) bytes += 4.0 * a.M * a.N;  // pre_adj is twice as wide
  const ProfScope ps(st, PC_GEMM, 2.0 * a.M * a.N * a.K, bytes);
  if (mode != GEMM_NATIVE && gemm_tensor_usable(a, mode)) return gemm_tensor(st, arena, a, mode);
  switch (a.epi) {
    case EPI_PLAIN: return launch_native<EPI_PLAIN>(st, a);
    case EPI_SILU: return launch_native<EPI_SILU>(st, a);
    case EPI_SWIGLU: return launch_native<EPI_SWIGLU>(st, a);
    case EPI_SILU_BWD: return launch_native<EPI_SILU_BWD>(st, a);
    case EPI_SWIGLU_BWD: return launch_native<EPI_SWIGLU_BWD>(st, a);
    case EPI_COMPRESS: return launch_native<EPI_COMPRESS>(st, a);
    default: throw Error(3, "gemm: unknown epilogue");
  }
}

void gemv_rows(Stream& st, const float* A, int lda, const float* w, const float* bias, float* out, int M, int K) {
  if (M <= 0) return;
  const ProfScope ps(st, PC_GEMM, 2.0 * M * K, 4.0 * (double(M) * K + K + M));
  k_gemv_rows<<<cdiv((long long) M * 32, 256), 256, 0, st.s>>>(A, lda, w, bias, out, M, K);
  PETB_LAUNCH_CHECK(st);
}

}  // namespace petb
