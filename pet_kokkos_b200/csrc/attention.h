// Per-atom multi-head attention over neighbour tokens: see attention.cu.
#pragma once

#include "common.h"

namespace petb {

enum AttnMode { ATTN_NATIVE = 0, ATTN_TF32X3 = 1, ATTN_TF32 = 2 };

struct AttnArgs {
  int N = 0, H = 0, hd = 0, S = 0;  // atoms, heads, head_dim, most tokens of any atom (max neighbours + 1)
  float sc = 1.f;                   // 1 / (sqrt(head_dim) * temperature)
  // How the products run (the reference's AttentionMode, include/pet/gemm.hpp): ATTN_NATIVE, fp32 on the CUDA
  // cores; ATTN_TF32X3, the split products on the tensor cores, as accurate but for the tensor core's truncating
  // accumulate; ATTN_TF32, one tf32 product per tile (a speed mode, about three decimal digits).
  int mode = 0;
  double pairs = 0.0;               // sum over atoms of tokens^2 (work accounting only)
  double T = 0.0;                   // token rows (work accounting only)
  const int* off = nullptr;         // [N+1] each atom's range of edge rows
  const float* cut = nullptr;       // [E] cutoff factor of each edge token
  const float* qkv = nullptr;       // [T,3D] columns Q | K | V
  float* merged = nullptr;          // [T,D] attention output before the output projection
  float* ml = nullptr;              // [T,H,2] each query's running max and 1/sum (null: not saved)
  // backward
  const float* dmerged = nullptr;   // [T,D]
  float* qkv_adj = nullptr;         // [T,3D]
  float* cfh = nullptr;             // [T,H] each key's score adjoint summed over its queries
};

void attention_forward(Stream& st, const AttnArgs& a);
void attention_backward(Stream& st, const AttnArgs& a);

}  // namespace petb
