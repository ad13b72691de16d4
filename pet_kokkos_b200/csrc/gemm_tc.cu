// The tensor-core GEMM: tcgen05.mma with TMA-fed shared-memory tiles and the accumulators in
// tensor memory (sm_100a). See gemm.h for the interface and the epilogues.
//
// A persistent kernel, one CTA per SM, each walking 128 x BN tiles of C = A . B^T (A [M,K],
// B [N,K], both K-major fp32) in an N-fastest order so that CTAs running side by side share
// their A rows in L2. Roles, by warp:
//   warp 0      producer: one thread issues cp.async.bulk.tensor (TMA) loads of a 128 x BK slab
//               of A and a BN x BK slab of B per stage, landing on an mbarrier. BK = 32 columns of K
//               (128-byte swizzle), or 16 (64-byte swizzle) with twice the stages where that hides
//               more of a TMA round trip (the 3xTF32 mode's 256-wide tiles);
//   warp 1      issuer: one thread issues tcgen05.mma kind::tf32 (M = 128, N = BN, K = 8) for every
//               8 columns of a stage into one of TWO accumulators in tensor memory, releases the
//               stage with tcgen05.commit and hands the finished accumulator to the epilogue;
//   warps 4-11  epilogue: tcgen05.ld the accumulator (a thread owns a row, a warp pair splits the
//               columns), turn each 32 x 32 chunk through a per-warp shared-memory pad so that
//               lanes run along columns, issue the epilogue's global loads for four row groups
//               before consuming them, and write 16 bytes per lane. The accumulator is handed
//               back as soon as it has been read, so the next tile's products overlap this
//               tile's stores;
//   warps 12-15 (3xTF32 mode) splitter: for every landed stage write A's lo = x - hi(x) beside the
//               tile, hi(x) being x with its 13 low mantissa bits cleared, which is what the
//               tensor core reads of an fp32 operand (lo is rounded to tf32 by adding half of its
//               last kept bit, since the tensor core would truncate it too). The weights' lo parts
//               are computed once when the model is loaded and arrive by a third TMA map. The
//               issuer accumulates hi.lo + lo.hi + hi.hi in fp32, small terms first: fp32-class
//               accuracy without reading the activations from L2 a second time.
//               (bf16 mode) converter: the activations stay fp32 in memory; for every landed stage these warps
//               round A's 128 x 32 fp32 slab to bf16 into a second, half-sized tile in the 64-byte-swizzled
//               K-major layout the tensor core reads, while the weights arrive as bf16 (converted once when
//               the model was loaded) by their own TMA map. The issuer then runs tcgen05.mma kind::f16 (K = 16
//               per instruction) on the two bf16 tiles: twice the tf32 rate on half the operand bytes.
// No TMA load here uses cluster multicast. Every wait is bounded: a wait that runs out sets an
// error word the host checks, every role then leaves its loop, and the CTA still reaches its
// tensor-memory release.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "epilogue.cuh"

namespace petb {

namespace {

constexpr int TBM = 128;  // rows per tile
constexpr int kEpiWarp0 = 4, kEpiWarps = 8, kSplitWarp0 = 12;
constexpr int kPad = 32;            // floats per row of an epilogue warp's 32 x 32 pad (16-byte slots XOR-swizzled by row)
constexpr unsigned long long kSpinLimit = 1ull << 31;  // clock64 ticks (~1 s) before a wait gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false once kSpinLimit clock ticks have passed or another role has given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if ((unsigned long long) (clock64() - t0) > kSpinLimit) {
      *abort_flag = 1;
      return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: start address >> 4 in bits 0-13,
// leading byte offset (unused for swizzled K-major: 1) in 16-29, stride byte offset (1024 B between
// 8-row groups) >> 4 in 32-45, descriptor version 1 in 46-47, layout type 2 (SWIZZLE_128B) in 61-63.
// With 16 fp32 per row (64-byte rows, 64-byte swizzle) the 8-row groups are 512 B apart and the layout type is 4.
template <int BK>
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  constexpr uint64_t sbo = BK == 32 ? 1024 : 512, layout = BK == 32 ? 2 : 4;
  return uint64_t((addr & 0x3FFFF) >> 4) | (uint64_t(1) << 16) | (uint64_t(sbo >> 4) << 32) | (uint64_t(1) << 46) | (layout << 61);
}
// Instruction descriptor, kind::tf32: D fp32 (bits 4-5 = 1), A and B tf32 (bits 7-9, 10-12 = 2), both
// K-major (bits 15, 16 = 0), N >> 3 in bits 17-22, M >> 4 in bits 24-28.
__host__ __device__ constexpr uint32_t idesc_tf32(int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(TBM >> 4) << 24);
}

// kind::f16 with bf16 operands: D fp32 (bits 4-5 = 1), A and B bf16 (bits 7-9, 10-12 = 1), K-major, N >> 3, M >> 4.
__host__ __device__ constexpr uint32_t idesc_bf16(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(TBM >> 4) << 24);
}
__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
        "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
        "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

enum TcMode { TC_TF32 = 0, TC_X3 = 1, TC_BF16 = 2 };

template <int BN, int STAGES, int MODE>
struct Smem {
  static constexpr bool X3 = MODE == TC_X3, B16 = MODE == TC_BF16;
  // fp32 elements of K per stage: a 128-byte swizzled row, or half of one where four stages of the widest 3x tile
  // have to fit (finer stages hide the load latency that two coarse ones cannot)
  static constexpr int BK = (X3 && BN == 256 && STAGES == 4) ? 16 : 32;
  static constexpr int kA = TBM * BK * 4;                     // A as it lands, fp32
  static constexpr int kA16 = B16 ? TBM * BK * 2 : 0;         // A again as bf16 (64-byte rows)
  static constexpr int kB = BN * BK * (B16 ? 2 : 4);          // B: fp32, or bf16 straight from memory
  static constexpr int kHi = kA + kA16 + kB;
  static constexpr int kStage = kHi * (X3 ? 2 : 1);           // with the lo tiles in the 3x mode
  static constexpr int kTiles = STAGES * kStage;
  static constexpr int kPads = kEpiWarps * 32 * kPad * 4;
  static constexpr int kTotal = kTiles + kPads + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static constexpr int kThreads = (X3 || B16) ? 512 : 384;
};

// The low part of the 3xTF32 split. The tensor core reads the top 19 bits of an fp32 operand (sign, exponent, 10
// mantissa bits) and ignores the rest, so hi(x) is x truncated; x - hi(x) is exact and has up to 13 significant
// bits, of which the tensor core would again keep the top 11 by truncation -- a bias toward zero that adds up along
// K. Adding half of the last kept bit here makes that truncation a rounding to nearest (ties away from zero, one
// case in 8192), which leaves an unbiased error of 2^-25 of x instead; the add carries into the exponent when the
// mantissa overflows, as rounding should, and a zero remainder stays below the kept bits.
__device__ __forceinline__ float tf32_lo(float x) {
  return __uint_as_float(__float_as_uint(x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u)) + 0x1000u);
}

// ---- the epilogue of one tile, shared by the kernels below -------------------------------------
//
// What an epilogue reads from global memory (a residual, a saved pre-activation) does not depend on the accumulator,
// and a DRAM round trip per batch of rows was what made an epilogue last longer than the next tile's MMAs: with two
// accumulators in tensor memory the tile period is then (epilogue + MMAs) / 2 instead of the MMAs' time. So (1) while
// an epilogue warp waits for its tile's accumulator it asks the L2 for the lines it is going to read, and (2) inside
// a 32-column chunk the loads of all eight row groups are issued before the accumulator is fetched from tensor memory.
template <int EPI>
__device__ __forceinline__ void epilogue_prefetch(const GemmArgs& p, int row, int col0, int ncols) {
  if (row >= p.M) return;
  const float* base = nullptr;
  size_t ld = 0;
  int wide = 1;
  if (EPI == EPI_PLAIN) {
    if (!p.res || row < p.res_row0) return;
    base = p.res, ld = size_t(p.ldr);
  } else if (EPI == EPI_SILU_BWD) {
    base = p.pre, ld = size_t(p.ldp);
  } else if (EPI == EPI_SWIGLU_BWD) {
    base = p.pre, ld = size_t(p.ldp), wide = 2;
  } else {
    return;
  }
  if (col0 + ncols > p.N) ncols = p.N - col0;
  const float* r = base + size_t(row) * ld + size_t(wide) * col0;
  for (int c = 0; c < wide * ncols; c += 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(r + c));
}

// Rows m0 + 32 q .. + 31, columns n0 + half BN/2 .. of the accumulator at `acc` (this warp's quarter of the lanes
// already in the address), through this warp's pad; `release` runs once the accumulator has been read.
template <int EPI, int BN, class Release>
__device__ __forceinline__ void epilogue_tile(const GemmArgs& p, uint32_t acc, float* pad, int m0, int n0, int q, int half, int lane,
                                              Release release) {
  constexpr int kBatch = (EPI == EPI_SWIGLU_BWD || EPI == EPI_COMPRESS) ? 4 : 8;  // row groups whose loads are in flight together
  const int sub = lane >> 3, c4 = (lane & 7) * 4;  // row-within-group and column of this lane's 16 bytes
#pragma unroll 1
  for (int c0 = half * (BN / 2); c0 < (half + 1) * (BN / 2); c0 += 32) {
    const int col = n0 + c0 + c4;
    EpiLoad ld[8];
    if (kBatch == 8 && col < p.N) {
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int row = m0 + q * 32 + u * 4 + sub;
        if (row < p.M) ld[u] = epilogue_load4<EPI>(p, row, col);
      }
    }
    float v[32];
    tmem_ld32(acc + c0, v);
    if (c0 + 32 == (half + 1) * (BN / 2)) {  // the accumulator has been read: the issuer may reuse it
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) release();
    }
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 32; j += 4)
      *reinterpret_cast<float4*>(pad + lane * kPad + (((j >> 2) ^ (lane & 7)) << 2)) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    __syncwarp();
    if (col < p.N) {
#pragma unroll
      for (int h = 0; h < 8 / kBatch; ++h) {
        if (kBatch == 4) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int row = m0 + q * 32 + (h * 4 + u) * 4 + sub;
            if (row < p.M) ld[u] = epilogue_load4<EPI>(p, row, col);
          }
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const int rr = (h * kBatch + u) * 4 + sub, row = m0 + q * 32 + rr;
          if (row < p.M) {
            const float4 a = *reinterpret_cast<const float4*>(pad + rr * kPad + (((lane & 7) ^ (rr & 7)) << 2));
            const float accv[4] = {a.x, a.y, a.z, a.w};
            epilogue_apply4<EPI>(p, row, col, accv, ld[u]);
          }
        }
      }
    }
  }
}

template <int EPI, int BN, int STAGES, int MODE>
__global__ void __launch_bounds__(Smem<BN, STAGES, MODE>::kThreads, 1)
    k_gemm_tc(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
              const __grid_constant__ CUtensorMap map_blo, GemmArgs p, int* err) {
  using L = Smem<BN, STAGES, MODE>;
  constexpr bool X3 = L::X3, B16 = L::B16;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* pads = reinterpret_cast<float*>(tiles + L::kTiles);
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + L::kTiles + L::kPads);  // [STAGES] TMA landed
  uint64_t* empty = full + STAGES;   // [STAGES] the stage's MMAs are done
  uint64_t* split = empty + STAGES;  // [STAGES] lo tiles written (3x mode)
  uint64_t* tfull = split + STAGES;  // [2] accumulator complete
  uint64_t* tempty = tfull + 2;      // [2] accumulator read back
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (p.N + BN - 1) / BN, tiles_m = (p.M + TBM - 1) / TBM;
  const int n_tiles = tiles_m * tiles_n;
  constexpr int TBK = L::BK;
  const int nkb = (p.K + TBK - 1) / TBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
      mbar_init(split + s, X3 ? 192 : 128);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull + b, 1);
      mbar_init(tempty + b, kEpiWarps);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // tensor memory: two accumulators of BN fp32 columns x 128 lanes
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int g = 0;  // k-blocks issued so far, across tiles
      for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        const int m0 = (t / tiles_n) * TBM, n0 = (t % tiles_n) * BN;
        bool ok = true;
        for (int kb = 0; kb < nkb; ++kb, ++g) {
          const int s = g % STAGES;
          if (!(ok = mbar_wait(empty + s, ((g / STAGES) & 1) ^ 1, abort_flag))) break;
          uint8_t* sa = tiles + size_t(s) * L::kStage;
          const bool b_lo = X3 && p.b_lo_offset != 0;  // B's low parts come from memory, not from the splitter
          mbar_expect_tx(full + s, L::kA + L::kB + (b_lo ? L::kB : 0));  // what TMA brings: not the converter's bf16 A tile
          tma_load_2d(sa, &map_a, full + s, kb * TBK, m0);
          tma_load_2d(sa + L::kA + L::kA16, &map_b, full + s, kb * TBK, n0);
          if (b_lo) tma_load_2d(sa + L::kHi + L::kA, &map_blo, full + s, kb * TBK, n0);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_tf32(BN);
      int g = 0, i = 0;
      for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++i) {
        const int b = i & 1;
        bool ok = mbar_wait(tempty + b, ((i >> 1) & 1) ^ 1, abort_flag);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem + uint32_t(b * BN);
        for (int kb = 0; ok && kb < nkb; ++kb, ++g) {
          const int s = g % STAGES;
          if (!(ok = mbar_wait((X3 || B16) ? split + s : full + s, (g / STAGES) & 1, abort_flag))) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a0 = smem_u32(tiles + size_t(s) * L::kStage), b0 = a0 + L::kA + L::kA16;
          if (B16) {  // 16 bf16 = 32 bytes along K per instruction, on the converted A tile and the bf16 B tile
            constexpr uint32_t idesc16 = idesc_bf16(BN);
#pragma unroll
            for (int k = 0; k < TBK / 16; ++k)
              mma_bf16(acc, smem_desc<16>(a0 + L::kA + 32 * k), smem_desc<16>(b0 + 32 * k), idesc16, (kb | k) != 0);
            mma_commit(empty + s);
            continue;
          }
#pragma unroll
          for (int k = 0; k < TBK / 8; ++k) {  // 8 tf32 = 32 bytes along K per instruction
            const uint64_t da = smem_desc<TBK>(a0 + 32 * k), db = smem_desc<TBK>(b0 + 32 * k);
            if (X3) {  // the two small cross terms first, then hi.hi on top of them
              const uint64_t dal = smem_desc<TBK>(a0 + L::kHi + 32 * k), dbl = smem_desc<TBK>(b0 + L::kHi + 32 * k);
              mma_tf32(acc, da, dbl, idesc, (kb | k) != 0);
              mma_tf32(acc, dal, db, idesc, 1);
              mma_tf32(acc, da, db, idesc, 1);
            } else {
              mma_tf32(acc, da, db, idesc, (kb | k) != 0);
            }
          }
          mma_commit(empty + s);
        }
        if (!ok) break;
        mma_commit(tfull + b);
      }
    }
  } else if (warp >= kEpiWarp0 && warp < kEpiWarp0 + kEpiWarps) {
    const int ew = warp - kEpiWarp0;
    const int q = warp & 3;          // the quarter of the 128 lanes this warp may read
    const int half = ew >> 2;        // which half of the BN columns
    float* pad = pads + size_t(ew) * 32 * kPad;
    int i = 0;
    for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++i) {
      const int b = i & 1;
      const int m0 = (t / tiles_n) * TBM, n0 = (t % tiles_n) * BN;
      epilogue_prefetch<EPI>(p, m0 + q * 32 + lane, n0 + half * (BN / 2), BN / 2);
      if (!mbar_wait(tfull + b, (i >> 1) & 1, abort_flag)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t acc = tmem + uint32_t(b * BN) + (uint32_t(q * 32) << 16);
      epilogue_tile<EPI, BN>(p, acc, pad, m0, n0, q, half, lane, [&] { mbar_arrive(tempty + b); });
    }
  } else if (B16 && warp >= kSplitWarp0) {
    // A's fp32 slab (128-byte rows, 16-byte chunk c of row r at chunk c ^ (r & 7)) rounded to bf16 into the tile beside
    // it (64-byte rows, chunk c of row r at chunk c ^ ((r >> 1) & 3): the 64-byte swizzle). A thread owns a row: the
    // eight lanes of a quarter warp then touch eight different 16-byte columns on the reads and on the writes.
    const int r = threadIdx.x - kSplitWarp0 * 32;
    int g = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x) {
      for (int kb = 0; kb < nkb; ++kb, ++g) {
        const int s = g % STAGES;
        if (!(ok = mbar_wait(full + s, (g / STAGES) & 1, abort_flag))) break;
        const uint8_t* src = tiles + size_t(s) * L::kStage + size_t(r) * 128;
        uint8_t* dst = tiles + size_t(s) * L::kStage + L::kA + size_t(r) * 64;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float4 x = *reinterpret_cast<const float4*>(src + (((2 * c) ^ (r & 7)) << 4));
          const float4 y = *reinterpret_cast<const float4*>(src + (((2 * c + 1) ^ (r & 7)) << 4));
          const __nv_bfloat162 q0 = __floats2bfloat162_rn(x.x, x.y), q1 = __floats2bfloat162_rn(x.z, x.w);
          const __nv_bfloat162 q2 = __floats2bfloat162_rn(y.x, y.y), q3 = __floats2bfloat162_rn(y.z, y.w);
          uint4 o;
          o.x = *reinterpret_cast<const uint32_t*>(&q0), o.y = *reinterpret_cast<const uint32_t*>(&q1);
          o.z = *reinterpret_cast<const uint32_t*>(&q2), o.w = *reinterpret_cast<const uint32_t*>(&q3);
          *reinterpret_cast<uint4*>(dst + ((c ^ ((r >> 1) & 3)) << 4)) = o;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes visible to the tensor core
        mbar_arrive(split + s);
      }
    }
  } else if (X3 && (warp >= kSplitWarp0 || warp == 2 || warp == 3)) {
    // lo = x - hi(x), written beside the stage's tiles at the same swizzled positions, so the same
    // descriptors, offset by the size of the hi tiles, address them. Six warps: the four splitter warps and the two
    // that have no other role (2 % on the 1728-atom benchmark over four).
    const int tid = warp >= kSplitWarp0 ? threadIdx.x - kSplitWarp0 * 32 : 128 + threadIdx.x - 64;
    const int n16 = (p.b_lo_offset != 0 ? L::kA : L::kHi) / 16;  // 16-byte pieces to split: A's, and B's unless they came split
    int g = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x) {
      for (int kb = 0; kb < nkb; ++kb, ++g) {
        const int s = g % STAGES;
        if (!(ok = mbar_wait(full + s, (g / STAGES) & 1, abort_flag))) break;
        const float4* hi = reinterpret_cast<const float4*>(tiles + size_t(s) * L::kStage);
        float4* lo = reinterpret_cast<float4*>(tiles + size_t(s) * L::kStage + L::kHi);
#pragma unroll 8
        for (int e = tid; e < n16; e += 192) {
          const float4 x = hi[e];
          float4 y;
          y.x = tf32_lo(x.x), y.y = tf32_lo(x.y), y.z = tf32_lo(x.z), y.w = tf32_lo(x.w);
          lo[e] = y;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes visible to the tensor core
        mbar_arrive(split + s);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * BN) : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(err, 1);
}


// ---- the 3xTF32 product with A on its own, deeper ring ---------------------------------------
//
// In k_gemm_tc's 3xTF32 form a stage holds 16 columns of A, A's low part and both parts of the 256-row B tile: 48 KB,
// of which A itself is 8 KB, so four stages keep at most 24 KB of A in flight per SM. A comes from HBM (B, the weights,
// sits in L2), and an SM's share of the HBM bandwidth times a DRAM round trip under load is about 50 KB: the A stream
// runs short of bytes in flight, a tile takes 19.6 k clocks against 12.3 k of MMA, and the tf32 form, whose four
// stages hold 64 KB of A, does not have the problem. Here A gets its own ring of eight 8 KB slots (seven in flight),
// while B (hi and lo) and A's low part, which need no look-ahead beyond hiding an L2 round trip and the splitter,
// share a ring of three. One producer thread feeds each ring. Same MMAs in the same order: same bits.
template <int NA_, int NB_>
struct SmemRing {
  static constexpr int BN = 256, BK = 16, kASlots = NA_, kBSlots = NB_;
  static constexpr int kA = TBM * BK * 4, kB = BN * BK * 4;     // 8 KB, 16 KB
  static constexpr int kRingA = kASlots * kA;                   // A as it lands
  static constexpr int kSlotB = 2 * kB + kA;                    // B hi, B lo, A lo
  static constexpr int kTiles = kRingA + kBSlots * kSlotB;
  static constexpr int kPads = kEpiWarps * 32 * kPad * 4;
  static constexpr int kTotal = kTiles + kPads + 1024 + 256;
  static constexpr int kThreads = 512;
};

template <int EPI, int NA_, int NB_>
__global__ void __launch_bounds__(512, 1)
    k_gemm_tc_ring(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ CUtensorMap map_blo, GemmArgs p, int* err) {
  using L = SmemRing<NA_, NB_>;
  constexpr int BN = L::BN, TBK = L::BK, NA = L::kASlots, NB = L::kBSlots;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring_b = tiles + L::kRingA;
  float* pads = reinterpret_cast<float*>(tiles + L::kTiles);
  uint64_t* full_a = reinterpret_cast<uint64_t*>(tiles + L::kTiles + L::kPads);  // [NA] A slot landed
  uint64_t* empty_a = full_a + NA;    // [NA] the slot's MMAs are done
  uint64_t* full_b = empty_a + NA;    // [NB] B hi and lo landed
  uint64_t* empty_b = full_b + NB;    // [NB] the slot's MMAs are done (B and A's low part with them)
  uint64_t* split = empty_b + NB;     // [NB] A's low part written
  uint64_t* tfull = split + NB;       // [2]
  uint64_t* tempty = tfull + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (p.N + BN - 1) / BN, tiles_m = (p.M + TBM - 1) / TBM;
  const int n_tiles = tiles_m * tiles_n;
  const int nkb = (p.K + TBK - 1) / TBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NA; ++s) mbar_init(full_a + s, 1), mbar_init(empty_a + s, 1);
    for (int s = 0; s < NB; ++s) mbar_init(full_b + s, 1), mbar_init(empty_b + s, 1), mbar_init(split + s, 128);
    for (int b = 0; b < 2; ++b) mbar_init(tfull + b, 1), mbar_init(tempty + b, kEpiWarps);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {  // A: up to seven slots ahead of the MMAs
      int g = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x) {
        const int m0 = (t / tiles_n) * TBM;
        for (int kb = 0; kb < nkb; ++kb, ++g) {
          const int s = g % NA;
          if (!(ok = mbar_wait(empty_a + s, ((g / NA) & 1) ^ 1, abort_flag))) break;
          mbar_expect_tx(full_a + s, L::kA);
          tma_load_2d(tiles + size_t(s) * L::kA, &map_a, full_a + s, kb * TBK, m0);
        }
      }
    }
  } else if (warp == 2) {
    if (lane == 0) {  // B, both parts
      int g = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x) {
        const int n0 = (t % tiles_n) * BN;
        for (int kb = 0; kb < nkb; ++kb, ++g) {
          const int s = g % NB;
          if (!(ok = mbar_wait(empty_b + s, ((g / NB) & 1) ^ 1, abort_flag))) break;
          uint8_t* sb = ring_b + size_t(s) * L::kSlotB;
          mbar_expect_tx(full_b + s, 2 * L::kB);
          tma_load_2d(sb, &map_b, full_b + s, kb * TBK, n0);
          tma_load_2d(sb + L::kB, &map_blo, full_b + s, kb * TBK, n0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_tf32(BN);
      int g = 0, i = 0;
      for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++i) {
        const int b = i & 1;
        bool ok = mbar_wait(tempty + b, ((i >> 1) & 1) ^ 1, abort_flag);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem + uint32_t(b * BN);
        for (int kb = 0; ok && kb < nkb; ++kb, ++g) {
          const int sa = g % NA, sb = g % NB;
          if (!(ok = mbar_wait(split + sb, (g / NB) & 1, abort_flag))) break;   // A landed and its low part is written
          if (!(ok = mbar_wait(full_b + sb, (g / NB) & 1, abort_flag))) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a0 = smem_u32(tiles + size_t(sa) * L::kA);
          const uint32_t b0 = smem_u32(ring_b + size_t(sb) * L::kSlotB), bl0 = b0 + L::kB, al0 = b0 + 2 * L::kB;
#pragma unroll
          for (int k = 0; k < TBK / 8; ++k) {
            const uint64_t da = smem_desc<TBK>(a0 + 32 * k), db = smem_desc<TBK>(b0 + 32 * k);
            const uint64_t dal = smem_desc<TBK>(al0 + 32 * k), dbl = smem_desc<TBK>(bl0 + 32 * k);
            mma_tf32(acc, da, dbl, idesc, (kb | k) != 0);
            mma_tf32(acc, dal, db, idesc, 1);
            mma_tf32(acc, da, db, idesc, 1);
          }
          mma_commit(empty_a + sa);
          mma_commit(empty_b + sb);
        }
        if (!ok) break;
        mma_commit(tfull + b);
      }
    }
  } else if (warp >= kEpiWarp0 && warp < kEpiWarp0 + kEpiWarps) {
    const int ew = warp - kEpiWarp0;
    const int q = warp & 3;
    const int half = ew >> 2;
    float* pad = pads + size_t(ew) * 32 * kPad;
    int i = 0;
    for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++i) {
      const int b = i & 1;
      const int m0 = (t / tiles_n) * TBM, n0 = (t % tiles_n) * BN;
      epilogue_prefetch<EPI>(p, m0 + q * 32 + lane, n0 + half * (BN / 2), BN / 2);
      if (!mbar_wait(tfull + b, (i >> 1) & 1, abort_flag)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t acc = tmem + uint32_t(b * BN) + (uint32_t(q * 32) << 16);
      epilogue_tile<EPI, BN>(p, acc, pad, m0, n0, q, half, lane, [&] { mbar_arrive(tempty + b); });
    }
  } else if (warp >= kSplitWarp0) {
    // A's low part, from its ring slot into the B slot that travels with it: needs the A slot landed and the B slot free
    const int tid = threadIdx.x - kSplitWarp0 * 32;
    constexpr int n16 = L::kA / 16;
    int g = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x) {
      for (int kb = 0; kb < nkb; ++kb, ++g) {
        const int sa = g % NA, sb = g % NB;
        if (!(ok = mbar_wait(empty_b + sb, ((g / NB) & 1) ^ 1, abort_flag))) break;
        if (!(ok = mbar_wait(full_a + sa, (g / NA) & 1, abort_flag))) break;
        const float4* hi = reinterpret_cast<const float4*>(tiles + size_t(sa) * L::kA);
        float4* lo = reinterpret_cast<float4*>(ring_b + size_t(sb) * L::kSlotB + 2 * L::kB);
#pragma unroll 4
        for (int e = tid; e < n16; e += 128) {
          const float4 x = hi[e];
          float4 y;
          y.x = tf32_lo(x.x), y.y = tf32_lo(x.y), y.z = tf32_lo(x.z), y.w = tf32_lo(x.w);
          lo[e] = y;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(split + sb);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * BN) : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(err, 1);
}

// ---- the same product on a pair of CTAs ------------------------------------------------------
//
// k_gemm_tc above is short of shared-memory bandwidth in the 3xTF32 mode: per 8 columns of K a CTA moves 64 KB through
// shared memory (TMA writes, the splitter, three MMAs' operand reads) against 384 clocks of MMA, and two thirds of it
// is the B tile. Here two CTAs of a cluster share one 256 x 256 tile: each stages its own 128 rows of A and HALF of
// the B tile (128 of its 256 rows, hi and lo), and one thread of the even CTA issues tcgen05.mma.cta_group::2
// (M = 256, N = 256, K = 8): the tensor cores of both SMs read both halves of B, each half once. Per CTA and 8
// columns of K that is 44 KB of shared-memory traffic against the same 384 clocks.
//
// Who signals whom (every barrier exists in both CTAs at the same offset; "leader" is the even CTA):
//   full[s]    own CTA's TMA loads landed (each CTA loads with the plain, CTA-local form; no multicast anywhere)
//   split[s]   LEADER's: 12 arrivals, one per splitter warp of both CTAs (the odd CTA's arrive remotely) once the warp
//              has written its share of the lo tile: both CTAs' operands are then complete
//   empty[s]   own CTA's: the leader's issuer commits the stage's MMAs to its own and to the odd CTA's barrier
//   tfull[b]   own CTA's: the leader commits the finished accumulator to both
//   tempty[b]  LEADER's: 16 arrivals, the epilogue warps of both CTAs once they have read the accumulator
// Tensor memory is allocated by warp 1 of both CTAs together (cta_group::2); each CTA's half of the accumulator is in
// its own tensor memory and its own epilogue warps write its 128 rows. Every wait is bounded as above; the CTAs meet
// at a cluster barrier after set-up and before release, so neither signals a peer that is not there.

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address of the same shared-memory location in another CTA of the cluster.
__device__ __forceinline__ uint32_t peer_smem(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// A bounded wait that also acquires what the other CTA of the cluster wrote before it arrived.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const long long t0 = clock64();
  for (;;) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
    if (*abort_flag) return false;
    if ((unsigned long long) (clock64() - t0) > kSpinLimit) {
      *abort_flag = 1;
      return false;
    }
  }
}
__device__ __forceinline__ void mma_tf32_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on a barrier (of this CTA or, by its cluster address, of the peer) once the pair's MMAs issued so far are done.
__device__ __forceinline__ void mma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}
__host__ __device__ constexpr uint32_t idesc_tf32_pair(int n) {  // M = 256 over the two CTAs
  return (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(256 >> 4) << 24);
}

template <int STAGES, int BK_ = 32>
struct SmemPair {
  static constexpr int BN = 256, BK = BK_;
  static constexpr int kA = TBM * BK * 4, kBh = (BN / 2) * BK * 4;  // A's rows, and this CTA's half of B's
  static constexpr int kHi = kA + kBh;
  static constexpr int kStage = 2 * kHi;  // with the lo tiles
  static constexpr int kTiles = STAGES * kStage;
  static constexpr int kPads = kEpiWarps * 32 * kPad * 4;
  static constexpr int kTotal = kTiles + kPads + 1024 + 256;
  static constexpr int kThreads = 512;
};

template <int EPI, int STAGES, int BK_>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(512, 1)
    k_gemm_tc_pair(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ CUtensorMap map_blo, GemmArgs p, int* err) {
  using L = SmemPair<STAGES, BK_>;
  constexpr int BN = L::BN, TBK = L::BK;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* pads = reinterpret_cast<float*>(tiles + L::kTiles);
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + L::kTiles + L::kPads);
  uint64_t* empty = full + STAGES;
  uint64_t* split = empty + STAGES;
  uint64_t* tfull = split + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int tiles_n = (p.N + BN - 1) / BN, tiles_m = (p.M + 2 * TBM - 1) / (2 * TBM);
  const int n_tiles = tiles_m * tiles_n, pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int nkb = (p.K + TBK - 1) / TBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
      mbar_init(split + s, 12);  // six splitter warps in each CTA
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull + b, 1);
      mbar_init(tempty + b, 2 * kEpiWarps);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // both CTAs' warp 1, together: two accumulators of 256 columns in each CTA's tensor memory
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {  // each CTA loads its own rows of A and its half of B
      int g = 0;
      for (int t = pair; t < n_tiles; t += n_pairs) {
        const int m0 = (t / tiles_n) * 2 * TBM + int(rank) * TBM, n0 = (t % tiles_n) * BN + int(rank) * (BN / 2);
        bool ok = true;
        for (int kb = 0; kb < nkb; ++kb, ++g) {
          const int s = g % STAGES;
          if (!(ok = mbar_wait(empty + s, ((g / STAGES) & 1) ^ 1, abort_flag))) break;
          uint8_t* sa = tiles + size_t(s) * L::kStage;
          mbar_expect_tx(full + s, L::kA + 2 * L::kBh);
          tma_load_2d(sa, &map_a, full + s, kb * TBK, m0);
          tma_load_2d(sa + L::kA, &map_b, full + s, kb * TBK, n0);
          tma_load_2d(sa + L::kHi + L::kA, &map_blo, full + s, kb * TBK, n0);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = idesc_tf32_pair(BN);
      int g = 0, i = 0;
      for (int t = pair; t < n_tiles; t += n_pairs, ++i) {
        const int b = i & 1;
        bool ok = mbar_wait_cluster(tempty + b, ((i >> 1) & 1) ^ 1, abort_flag);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem + uint32_t(b * BN);
        for (int kb = 0; ok && kb < nkb; ++kb, ++g) {
          const int s = g % STAGES;
          if (!(ok = mbar_wait_cluster(split + s, (g / STAGES) & 1, abort_flag))) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a0 = smem_u32(tiles + size_t(s) * L::kStage), b0 = a0 + L::kA;
#pragma unroll
          for (int k = 0; k < TBK / 8; ++k) {
            const uint64_t da = smem_desc<TBK>(a0 + 32 * k), db = smem_desc<TBK>(b0 + 32 * k);
            const uint64_t dal = smem_desc<TBK>(a0 + L::kHi + 32 * k), dbl = smem_desc<TBK>(b0 + L::kHi + 32 * k);
            mma_tf32_pair(acc, da, dbl, idesc, (kb | k) != 0);
            mma_tf32_pair(acc, dal, db, idesc, 1);
            mma_tf32_pair(acc, da, db, idesc, 1);
          }
          mma_commit_pair(smem_u32(empty + s));
          mma_commit_pair(peer_smem(empty + s, 1));
        }
        if (!ok) break;
        mma_commit_pair(smem_u32(tfull + b));
        mma_commit_pair(peer_smem(tfull + b, 1));

      }
    }
  } else if (warp >= kEpiWarp0 && warp < kEpiWarp0 + kEpiWarps) {
    const int ew = warp - kEpiWarp0;
    const int q = warp & 3;
    const int half = ew >> 2;
    float* pad = pads + size_t(ew) * 32 * kPad;
    int i = 0;
    for (int t = pair; t < n_tiles; t += n_pairs, ++i) {
      const int b = i & 1;
      const int m0 = (t / tiles_n) * 2 * TBM + int(rank) * TBM, n0 = (t % tiles_n) * BN;
      epilogue_prefetch<EPI>(p, m0 + q * 32 + lane, n0 + half * (BN / 2), BN / 2);
      if (!mbar_wait(tfull + b, (i >> 1) & 1, abort_flag)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t acc = tmem + uint32_t(b * BN) + (uint32_t(q * 32) << 16);
      epilogue_tile<EPI, BN>(p, acc, pad, m0, n0, q, half, lane, [&] { mbar_arrive_cluster(peer_smem(tempty + b, 0)); });
    }
  } else if (warp >= kSplitWarp0 || warp == 2 || warp == 3) {  // six warps, as in k_gemm_tc
    const int tid = warp >= kSplitWarp0 ? threadIdx.x - kSplitWarp0 * 32 : 128 + threadIdx.x - 64;
    constexpr int n16 = L::kA / 16;  // A's 16-byte pieces; B's lo half arrives split
    const uint32_t split0 = peer_smem(split, 0);  // the leader's barriers
    int g = 0;
    bool ok = true;
    for (int t = pair; ok && t < n_tiles; t += n_pairs) {
      for (int kb = 0; kb < nkb; ++kb, ++g) {
        const int s = g % STAGES;
        // a warp goes on or gives up as one, and arrives once: no barrier among the splitter warps that a warp
        // which gave up could leave the others waiting at
        if (!(ok = __all_sync(0xffffffffu, mbar_wait(full + s, (g / STAGES) & 1, abort_flag)))) break;
        const float4* hi = reinterpret_cast<const float4*>(tiles + size_t(s) * L::kStage);
        float4* lo = reinterpret_cast<float4*>(tiles + size_t(s) * L::kStage + L::kHi);
#pragma unroll 8
        for (int e = tid; e < n16; e += 192) {
          const float4 x = hi[e];
          float4 y;
          y.x = tf32_lo(x.x), y.y = tf32_lo(x.y), y.z = tf32_lo(x.z), y.w = tf32_lo(x.w);
          lo[e] = y;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(split0 + 8u * uint32_t(s));
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();  // nobody leaves while the other CTA may still signal it or read its tiles
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * BN) : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(err, 1);
}

// ---- host side ---------------------------------------------------------------------------

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// What the tensor-core path needs of one device: its SM count and an error word in its memory (with a pinned
// mirror), plus the driver's tensor-map encoder (the same function for every device). One per device ordinal,
// built on first use with that device current.
struct TensorState {
  EncodeFn encode = nullptr;
  int* err = nullptr;       // device error word
  int* err_host = nullptr;  // pinned mirror
  int sms = 0;
  bool ok = false;
};

TensorState& state() {
  static PerDevice<TensorState> table;
  int dev = 0;
  cudaGetDevice(&dev);
  return table.get(dev, [dev](TensorState& s) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return;
    int major = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&s.sms, cudaDevAttrMultiProcessorCount, dev);
    if (major != 10 || s.sms <= 0) return;
    if (cudaMalloc(&s.err, sizeof(int)) != cudaSuccess) return;
    cudaMemset(s.err, 0, sizeof(int));
    cudaStreamSynchronize(cudaStreamLegacy);  // the callers' streams do not wait for the legacy one
    if (cudaMallocHost(&s.err_host, sizeof(int)) != cudaSuccess) return;
    *s.err_host = 0;
    s.encode = reinterpret_cast<EncodeFn>(fn);
    s.ok = true;
  });
}

// A [rows, K] fp32 row-major matrix as a 2-D tensor map with a 32 x box_rows box, 128-byte swizzle,
// zero fill outside the matrix.
CUtensorMap make_map(const float* base, int rows, int K, int ld, int box_rows, int bk) {
  CUtensorMap m;
  const cuuint64_t dims[2] = {cuuint64_t(K), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(ld) * 4};
  const cuuint32_t box[2] = {cuuint32_t(bk), cuuint32_t(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = state().encode(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw Error(5, "gemm: cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
  return m;
}

// B [rows, K] bf16 row-major as a 2-D tensor map with a 32 x box_rows box (64-byte rows), 64-byte swizzle.
CUtensorMap make_map_bf16(const uint16_t* base, int rows, int K, int ld, int box_rows) {
  CUtensorMap m;
  const cuuint64_t dims[2] = {cuuint64_t(K), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(ld) * 2};
  const cuuint32_t box[2] = {32, cuuint32_t(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = state().encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t*>(base), dims, strides, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw Error(5, "gemm: cuTensorMapEncodeTiled (bf16) failed with code " + std::to_string(int(r)));
  return m;
}

template <int EPI, int BN, int STAGES, int MODE>
void launch_tc(Stream& st, const GemmArgs& a) {
  using L = Smem<BN, STAGES, MODE>;
  static_assert(L::kTotal <= 227 * 1024, "the tile pipeline does not fit shared memory");
  static SmemOptIn opted;
  auto kernel = k_gemm_tc<EPI, BN, STAGES, MODE>;
  opt_in_shared_memory(kernel, L::kTotal, opted);
  const CUtensorMap ma = make_map(a.A, a.M, a.K, a.lda, TBM, L::BK);
  const CUtensorMap mb = L::B16 ? make_map_bf16(a.B16, a.N, a.K, a.ldb, BN) : make_map(a.B, a.N, a.K, a.ldb, BN, L::BK);
  const CUtensorMap mblo = (L::X3 && a.b_lo_offset) ? make_map(a.B + a.b_lo_offset, a.N, a.K, a.ldb, BN, L::BK) : mb;
  const long long tiles = (long long) cdiv(a.M, TBM) * cdiv(a.N, BN);
  const int grid = int(tiles < state().sms ? tiles : state().sms);
  kernel<<<grid, L::kThreads, L::kTotal, st.s>>>(ma, mb, mblo, a, state().err);
  PETB_LAUNCH_CHECK(st);
}

// The ring kernel serves the 3xTF32 mode's widest tiles with pre-split weights when PET_GEMM_RING=1 (eight A slots,
// three B slots) or 2 (four and four). It measures the same as the staged kernel, which stays the default.
bool ring_enabled() {
  const char* e = std::getenv("PET_GEMM_RING");
  return e && (e[0] == '1' || e[0] == '2');
}

template <int EPI, int NA_, int NB_>
void launch_tc_ring(Stream& st, const GemmArgs& a) {
  using L = SmemRing<NA_, NB_>;
  static_assert(L::kTotal <= 227 * 1024, "the rings do not fit shared memory");
  static SmemOptIn opted;
  auto kernel = k_gemm_tc_ring<EPI, NA_, NB_>;
  opt_in_shared_memory(kernel, L::kTotal, opted);
  const CUtensorMap ma = make_map(a.A, a.M, a.K, a.lda, TBM, L::BK), mb = make_map(a.B, a.N, a.K, a.ldb, L::BN, L::BK);
  const CUtensorMap mblo = make_map(a.B + a.b_lo_offset, a.N, a.K, a.ldb, L::BN, L::BK);
  const long long tiles = (long long) cdiv(a.M, TBM) * cdiv(a.N, L::BN);
  const int grid = int(tiles < state().sms ? tiles : state().sms);
  kernel<<<grid, L::kThreads, L::kTotal, st.s>>>(ma, mb, mblo, a, state().err);
  PETB_LAUNCH_CHECK(st);
}

// The pair kernel serves the 3xTF32 mode's widest tiles (N a multiple of 256, weights pre-split) when PET_GEMM_PAIR=1.
bool pair_enabled() {  // read at every call, so that one process can compare the two kernels
  const char* e = std::getenv("PET_GEMM_PAIR");
  return e && e[0] == '1';
}

template <int EPI, int STAGES = 3, int BK_ = 32>
void launch_tc_pair(Stream& st, const GemmArgs& a) {
  using L = SmemPair<STAGES, BK_>;
  static_assert(L::kTotal <= 227 * 1024, "the pair's tile pipeline does not fit shared memory");
  static SmemOptIn opted;
  auto kernel = k_gemm_tc_pair<EPI, STAGES, BK_>;
  opt_in_shared_memory(kernel, L::kTotal, opted);
  const CUtensorMap ma = make_map(a.A, a.M, a.K, a.lda, TBM, L::BK);
  const CUtensorMap mb = make_map(a.B, a.N, a.K, a.ldb, L::BN / 2, L::BK);
  const CUtensorMap mblo = make_map(a.B + a.b_lo_offset, a.N, a.K, a.ldb, L::BN / 2, L::BK);
  const long long tiles = (long long) cdiv(a.M, 2 * TBM) * cdiv(a.N, L::BN);
  // as many pairs as the device can hold at once (a pair needs two SMs of one GPC: fewer than half the SMs may fit),
  // or the kernel's last pairs would start when the first ones end
  static PerDevice<int> resident;
  int dev = 0;
  cudaGetDevice(&dev);
  const int fit = resident.get(dev, [&](int& out) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(state().sms / 2 * 2)), cfg.blockDim = dim3(L::kThreads), cfg.dynamicSmemBytes = L::kTotal;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2, attr.val.clusterDim.y = 1, attr.val.clusterDim.z = 1;
    cfg.attrs = &attr, cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) n = state().sms / 2;
    if (std::getenv("PET_GEMM_PAIR_VERBOSE")) std::fprintf(stderr, "pair kernel: %d clusters fit on %d SMs\n", n, state().sms);
    out = n;
  });
  const long long pairs = std::min<long long>(tiles, std::min(fit, state().sms / 2));
  kernel<<<unsigned(2 * pairs), L::kThreads, L::kTotal, st.s>>>(ma, mb, mblo, a, state().err);
  PETB_LAUNCH_CHECK(st);
}

// The widest 3x tile runs four 16-column stages (64-byte swizzle) rather than two 32-column ones: the same bytes in
// flight, handed over in finer pieces (2 % faster on the 1728-atom benchmark). PET_GEMM_FINE=0 picks the coarse form.
bool fine_stages() {
  static const bool on = [] {
    const char* e = std::getenv("PET_GEMM_FINE");
    return !(e && e[0] == '0');
  }();
  return on;
}

template <int EPI>
void dispatch_tc(Stream& st, const GemmArgs& a, int mode) {
  const bool x3 = mode == GEMM_TF32X3, b16 = mode == GEMM_BF16;
  // The tile width that finishes first. A tile's time per step of K goes with the shared-memory wavefronts it needs
  // (operand reads, fills, the splitter, its share of the epilogue), which a narrower tile needs fewer of per tile
  // and more of per output column; the launch takes as many rounds as its fullest CTA has tiles. The token GEMMs
  // (thousands of row tiles) come out at 256; a GEMM over the atoms' rows (14 row tiles at 1728 atoms) at whatever
  // gives one round: 64 for 256 columns, 128 for 1024, 256 for 2048.
  const long long mt = cdiv(a.M, TBM);
  const int sms = state().sms;
  const int widths[3] = {256, 128, 64};
  const int wavefronts[3] = {x3 ? 550 : 300, x3 ? 350 : 185, x3 ? 270 : 125};
  int bn = 0;
  long long best = 0;
  for (int i = 0; i < 3; ++i) {
    if (a.N % widths[i] != 0) continue;
    const long long tiles = mt * (a.N / widths[i]), rounds = (tiles + sms - 1) / sms;
    if (bn == 0 || rounds * wavefronts[i] < best) bn = widths[i], best = rounds * wavefronts[i];
  }
  if (bn == 0) bn = 128;  // ragged widths: a wide tile with a zero-filled edge
  if (bn == 256) {
    if (x3 && a.b_lo_offset && pair_enabled() && cdiv(a.M, 2 * TBM) * (a.N / 256) >= sms / 2) {
      const char* e = std::getenv("PET_GEMM_PAIR");
      if (e[1] == '6') return launch_tc_pair<EPI, 6, 16>(st, a);  // "16": six stages of 16 columns
      return launch_tc_pair<EPI, 3, 32>(st, a);
    }
    if (x3 && a.b_lo_offset && ring_enabled()) {
      const char* e = std::getenv("PET_GEMM_RING");
      if (e && e[0] == '2') return launch_tc_ring<EPI, 4, 4>(st, a);
      return launch_tc_ring<EPI, 8, 3>(st, a);
    }
    if (b16) return launch_tc<EPI, 256, 4, TC_BF16>(st, a);
    if (x3) return fine_stages() ? launch_tc<EPI, 256, 4, TC_X3>(st, a) : launch_tc<EPI, 256, 2, TC_X3>(st, a);
    return launch_tc<EPI, 256, 4, TC_TF32>(st, a);
  }
  if (bn == 128) {
    if (b16) return launch_tc<EPI, 128, 6, TC_BF16>(st, a);
    if (x3) return launch_tc<EPI, 128, 3, TC_X3>(st, a);
    return launch_tc<EPI, 128, 4, TC_TF32>(st, a);
  }
  if (b16) return launch_tc<EPI, 64, 6, TC_BF16>(st, a);
  if (x3) return launch_tc<EPI, 64, 4, TC_X3>(st, a);
  return launch_tc<EPI, 64, 6, TC_TF32>(st, a);
}

}  // namespace

bool tensor_gemm_available() { return state().ok; }

bool gemm_tensor_usable(const GemmArgs& a, int mode) {
  if (mode != GEMM_TF32 && mode != GEMM_TF32X3 && mode != GEMM_BF16) return false;
  if (!state().ok) return false;
  // TMA: 16-byte aligned bases and row strides; the epilogue walks runs of four columns (N % 4 == 0, checked by gemm()).
  if ((reinterpret_cast<uintptr_t>(a.A) | reinterpret_cast<uintptr_t>(a.B)) & 15) return false;
  if (a.lda % 4 || a.ldb % 4 || a.K % 8) return false;
  if (a.M < 64 || a.N < 32) return false;  // too small to be worth a 128-row tensor tile
  return true;
}

void gemm_tensor(Stream& st, Arena&, const GemmArgs& a, int mode) {
  // a GEMM without a bf16 copy of its second operand (a caller's own matrix) or with rows that a bf16 TMA map cannot
  // stride runs as tf32, which is more exact
  if (mode == GEMM_BF16 && (!a.B16 || a.ldb % 8 || (reinterpret_cast<uintptr_t>(a.B16) & 15))) mode = GEMM_TF32;
  switch (a.epi) {
    case EPI_PLAIN: return dispatch_tc<EPI_PLAIN>(st, a, mode);
    case EPI_SILU: return dispatch_tc<EPI_SILU>(st, a, mode);
    case EPI_SWIGLU: return dispatch_tc<EPI_SWIGLU>(st, a, mode);
    case EPI_SILU_BWD: return dispatch_tc<EPI_SILU_BWD>(st, a, mode);
    case EPI_SWIGLU_BWD: return dispatch_tc<EPI_SWIGLU_BWD>(st, a, mode);
    case EPI_COMPRESS: return dispatch_tc<EPI_COMPRESS>(st, a, mode);
    default: throw Error(3, "gemm: unknown epilogue");
  }
}

// Non-zero once a tensor-core kernel gave up on a wait; cleared by the read.
int gemm_tensor_error(Stream& st) {
  TensorState& s = state();
  if (!s.ok) return 0;
  cudaMemcpyAsync(s.err_host, s.err, sizeof(int), cudaMemcpyDeviceToHost, st.s);
  cudaStreamSynchronize(st.s);
  const int e = *s.err_host;
  if (e) cudaMemsetAsync(s.err, 0, sizeof(int), st.s);
  return e;
}

}  // namespace petb
