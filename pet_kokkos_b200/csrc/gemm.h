// Weight GEMMs with fused epilogues: C[M,N] = A[M,K] . B[N,K]^T (+ bias, residual, activation).
//
// Every dense contraction of the network has a weight as its second operand
// (the reference's weight_gemm, src/ops.cpp:18-24). Weights are held in both
// orientations so that B is always K-major: forward GEMMs read W [N_out, K_in],
// backward (input-adjoint) GEMMs read W^T [K_in, N_out]; no weight gradients are
// formed. The epilogues are the reference's fused ones (src/fused_gemm.cpp:441-563)
// plus the residual add and compress.0's folded geometry/species terms
// (src/ops.cpp:326-365).
//
// Two kernel families share the epilogue code:
//   * native: fp32 FMA on the CUDA cores, one accumulation chain per output in k
//     order, so a row's bits do not depend on how many rows the GEMM has;
//   * tensor: tcgen05.mma (kind::tf32 or kind::f16 with bf16 operands) with TMA-fed
//     shared-memory tiles and the accumulator in tensor memory.
#pragma once

#include "common.h"

namespace petb {

enum Epilogue {
  EPI_PLAIN = 0,       // C = acc + bias (+ res for rows >= res_row0)
  EPI_SILU = 1,        // z = acc + bias; pre (optional) = z; C = silu(z)
  EPI_SWIGLU = 2,      // z = acc + bias, columns interleaved (v_j, g_j); pre = z; C[M,N/2] = v * sigmoid(g)
  EPI_SILU_BWD = 3,    // C = acc * silu'(pre)
  EPI_SWIGLU_BWD = 4,  // acc = h_adj [M,N]; C[M,2N]: (acc*sg, acc*v*sg*(1-sg)) from pre [M,2N]
  EPI_COMPRESS = 5     // z = acc + b + tab[sp[row]] + wx . (v, |v|); pre = z; C = silu(z)
};

enum GemmMode { GEMM_NATIVE = 0, GEMM_TF32 = 1, GEMM_BF16 = 2, GEMM_TF32X3 = 3 };

struct GemmArgs {
  const float* A = nullptr;  // [M,K]
  int lda = 0;
  const float* B = nullptr;  // [N,K]
  int ldb = 0;
  // Non-zero: B + b_lo_offset holds the low parts of B's 3xTF32 split, computed once when the weights were loaded
  // (same shape and pitch); the tensor-core kernel then loads them instead of splitting every B tile it stages.
  size_t b_lo_offset = 0;
  // B again as bf16 [N,K] with the same pitch in elements (round to nearest even, made when the weights were loaded):
  // what the bf16 mode's tensor-core kernel reads. Null: the bf16 mode runs this GEMM as tf32.
  const uint16_t* B16 = nullptr;
  float* C = nullptr;        // [M, N] (EPI_SWIGLU: [M,N/2]; EPI_SWIGLU_BWD: [M,2N])
  int ldc = 0;
  int M = 0, N = 0, K = 0;
  const float* bias = nullptr;  // [N]
  const float* res = nullptr;   // [M,N] residual, read before C is written (may alias C)
  int ldr = 0;
  int res_row0 = 0;
  float* pre = nullptr;  // saved or read pre-activation
  int ldp = 0;
  // EPI_COMPRESS
  const float* tab = nullptr;    // [n_species, N]
  const int* sp = nullptr;       // [M]
  const float* wx = nullptr;     // [N,4]
  const double* vec = nullptr;   // [M,3]
  const double* dist = nullptr;  // [M]
  int epi = EPI_PLAIN;
};

// Runs the GEMM in `mode`. The tensor modes need K % 8 == 0 (tf32) or K % 16 == 0
// (bf16), N % 8 == 0 and 16-byte aligned rows; anything else takes the native kernel.
void gemm(Stream& st, Arena& arena, const GemmArgs& a, int mode);

// out[M] = A[M,K] . w[K] + b (a one-column linear layer), one warp per row.
void gemv_rows(Stream& st, const float* A, int lda, const float* w, const float* bias, float* out, int M, int K);

// Non-zero if a tensor-core kernel launched on this stream gave up on a bounded wait since the
// last call (synchronizes the stream; clears the flag).
int gemm_tensor_error(Stream& st);

// True once the tensor-core path has been initialised on this device (driver entry point found).
bool tensor_gemm_available();

}  // namespace petb
