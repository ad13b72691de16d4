// Shared plumbing of the evaluator: error type, device scratch pool, launch accounting.
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "per_device.h"

namespace petb {

// An error that crosses the C ABI as a status code plus a message.
struct Error : std::runtime_error {
  int code;
  Error(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};

#define PETB_CUDA(expr)                                                                         \
  do {                                                                                          \
    cudaError_t err__ = (expr);                                                                 \
    if (err__ != cudaSuccess)                                                                   \
      throw ::petb::Error(err__ == cudaErrorMemoryAllocation ? 4 : 5,                           \
                          std::string(#expr) + ": " + cudaGetErrorString(err__));               \
  } while (0)

inline int cdiv(long long a, long long b) { return int((a + b - 1) / b); }

// Failure injection for tests, on the host: when >= 0, the pools' cudaMalloc number g_fail_alloc_in from now reports
// out of memory instead of allocating (once). No GPU fault is involved.
inline long g_fail_alloc_in = -1;

// PET_WS_POISON=1 (the reference's switch of the same name, include/pet/kokkos.hpp) or PET_B200_WS_POISON=1 (this
// library alone, for a process that also runs the reference): every pool block is filled with
// 0xFF bytes (NaNs as floats and doubles, -1 as ints) when it is allocated and again whenever the pool is reset, so
// that a kernel reading something nobody wrote this evaluation shows up as NaNs in the results instead of passing
// by the luck of what the memory held. A debugging aid: the fills synchronize the device.
inline bool poison_pools() {
  static const bool on = [] {
    for (const char* name : {"PET_WS_POISON", "PET_B200_WS_POISON"})
      if (const char* e = std::getenv(name))
        if (e[0] == '1') return true;
    return false;
  }();
  return on;
}

// The fill runs on the legacy stream, which the evaluators' non-blocking streams do not wait for: fence it on both
// sides, or it lands on top of what the next kernels write.
inline void poison_fill(void* p, size_t bytes) {
  PETB_CUDA(cudaDeviceSynchronize());
  PETB_CUDA(cudaMemset(p, 0xFF, bytes));
  PETB_CUDA(cudaDeviceSynchronize());
}

// Device scratch for one evaluation: a bump allocator over a few large blocks.
// The first evaluations grow it (cudaMalloc); later ones of the same shapes
// allocate nothing, so the pointers repeat and a captured graph stays valid.
// reset() rewinds; when more than one block was needed the blocks are merged
// into one of the total size at the next reset, so the layout becomes stable.
// The reference's counterpart is the Workspace pool (include/pet/kokkos.hpp:84-198).
class Arena {
 public:
  explicit Arena(size_t first_block = size_t(64) << 20) : next_block_(first_block) {}
  ~Arena() { release(); }
  Arena(const Arena&) = delete;
  Arena& operator=(const Arena&) = delete;

  void* alloc_bytes(size_t bytes) {
    bytes = (bytes + 255) & ~size_t(255);
    if (bytes == 0) bytes = 256;
    while (cur_ < blocks_.size()) {
      Block& b = blocks_[cur_];
      if (b.used + bytes <= b.size) {
        void* p = b.ptr + b.used;
        b.used += bytes;
        used_total_ += bytes;
        return p;
      }
      ++cur_;
    }
    // a block of the pool's step, or exactly this allocation when that is larger: nothing is rounded up to a power
    // of two, so a pool of a hundred gigabytes wastes none of it; the step grows with the pool so that a large pool
    // is not made of thousands of small blocks
    const size_t size = std::max(next_block_, bytes);
    next_block_ = std::max(next_block_, std::min(capacity() / 4, size_t(2) << 30));
    Block b;
    if (g_fail_alloc_in >= 0 && g_fail_alloc_in-- == 0)
      throw Error(4, "cudaMalloc: out of memory (injected for a test)");
    PETB_CUDA(cudaMalloc(&b.ptr, size));
    if (poison_pools()) poison_fill(b.ptr, size);
    b.size = size;
    b.used = bytes;
    blocks_.push_back(b);
    cur_ = blocks_.size() - 1;
    used_total_ += bytes;
    ++generation_;
    return b.ptr;
  }
  template <class T>
  T* alloc(size_t n) { return static_cast<T*>(alloc_bytes(n * sizeof(T))); }

  // Rewind; merges several blocks into one so the next pass of the same shapes
  // gets one stable layout. Must not be called while kernels still read the pool.
  void reset() {
    if (blocks_.size() > 1) {
      size_t total = 0;
      for (auto& b : blocks_) total += b.size;
      PETB_CUDA(cudaDeviceSynchronize());
      for (auto& b : blocks_) cudaFree(b.ptr);
      blocks_.clear();
      Block b;
      PETB_CUDA(cudaMalloc(&b.ptr, total));
      b.size = total;
      blocks_.push_back(b);
      ++generation_;
    }
    if (poison_pools())
      for (auto& b : blocks_) poison_fill(b.ptr, b.size);
    for (auto& b : blocks_) b.used = 0;
    cur_ = 0;
    used_total_ = 0;
  }
  // Before a pass whose need is known: one block of at least `bytes`, so that the pass allocates nothing on the way
  // and the layout is the steady one from the first evaluation on. Only while nothing of the pool is in use.
  void reserve(size_t bytes) {
    if (used_total_ != 0 || capacity() >= bytes) return;
    release();
    Block b;
    if (g_fail_alloc_in >= 0 && g_fail_alloc_in-- == 0) throw Error(4, "cudaMalloc: out of memory (injected for a test)");
    PETB_CUDA(cudaMalloc(&b.ptr, bytes));
    if (poison_pools()) poison_fill(b.ptr, bytes);
    b.size = bytes;
    blocks_.push_back(b);
    ++generation_;
  }
  // A stack discipline for temporaries: everything allocated after mark() is handed
  // back by rewind(). Kernels run in stream order, so a later pass may reuse it.
  struct Mark {
    size_t cur, used, total;
  };
  Mark mark() const { return {cur_, cur_ < blocks_.size() ? blocks_[cur_].used : 0, used_total_}; }
  void rewind(const Mark& m) {
    for (size_t b = m.cur + 1; b < blocks_.size(); ++b) blocks_[b].used = 0;
    if (m.cur < blocks_.size()) blocks_[m.cur].used = m.used;
    cur_ = m.cur;
    used_total_ = m.total;
  }
  void release() {
    for (auto& b : blocks_) cudaFree(b.ptr);
    blocks_.clear();
    cur_ = 0;
    used_total_ = 0;
    ++generation_;
  }
  // Trades everything with another pool (the pools are not copyable: they own device memory).
  void swap(Arena& o) {
    blocks_.swap(o.blocks_);
    std::swap(cur_, o.cur_), std::swap(next_block_, o.next_block_), std::swap(used_total_, o.used_total_);
    std::swap(generation_, o.generation_);
    ++generation_, ++o.generation_;
  }
  size_t capacity() const {
    size_t t = 0;
    for (auto& b : blocks_) t += b.size;
    return t;
  }
  size_t used() const { return used_total_; }
  // Changes whenever device memory was (re)allocated: part of a graph's key.
  uint64_t generation() const { return generation_; }

 private:
  struct Block {
    char* ptr = nullptr;
    size_t size = 0, used = 0;
  };
  std::vector<Block> blocks_;
  size_t cur_ = 0, next_block_, used_total_ = 0;
  uint64_t generation_ = 0;
};

// Kernel classes for the per-class timing a profiling pass collects; the names are
// the classes the reference's own roofline model reports (tools/roofline.md:16-24).
enum ProfClass { PC_GEMM = 0, PC_ATTN_FWD, PC_ATTN_BWD, PC_NORM, PC_ELEMENTWISE, PC_GATHER, PC_GEOMETRY, PC_FORCES, PC_COUNT };
inline const char* prof_class_name(int c) {
  static const char* names[] = {"gemm", "attention_fwd", "attention_bwd", "norm", "elementwise", "gather", "geometry", "forces"};
  return c >= 0 && c < PC_COUNT ? names[c] : "?";
}

// CUDA-event brackets around launches, on the launching stream, summed per class after a
// synchronize. Off by default: an evaluation records nothing unless a profiling pass asked.
struct Profiler {
  struct Rec {
    cudaEvent_t a, b;
    int cls;
    double flops, bytes;
  };
  bool on = false;
  std::vector<Rec> recs;
  std::vector<cudaEvent_t> pool;
  cudaEvent_t get() {
    if (!pool.empty()) {
      cudaEvent_t e = pool.back();
      pool.pop_back();
      return e;
    }
    cudaEvent_t e;
    cudaEventCreate(&e);
    return e;
  }
  ~Profiler() {
    for (auto& r : recs) cudaEventDestroy(r.a), cudaEventDestroy(r.b);
    for (auto e : pool) cudaEventDestroy(e);
  }
};

// The stream every kernel of a calculator runs on, with a count of launches.
struct Stream {
  cudaStream_t s = nullptr;
  long long launches = 0;
  Profiler* prof = nullptr;
  cudaEvent_t legacy_fence = nullptr;  // made at first use by order_after_legacy_stream, destroyed with the stream's owner
};

// After a caller's callback returns: what it put on the legacy default stream (a blocking cudaMemcpy from pageable
// memory returns once the bytes are staged, before they have landed) is ordered before this stream's next work.
// The evaluators' streams are non-blocking and would not wait for it otherwise.
inline void order_after_legacy_stream(Stream& st) {
  if (!st.legacy_fence) PETB_CUDA(cudaEventCreateWithFlags(&st.legacy_fence, cudaEventDisableTiming));
  PETB_CUDA(cudaEventRecord(st.legacy_fence, cudaStreamLegacy));
  PETB_CUDA(cudaStreamWaitEvent(st.s, st.legacy_fence, 0));
}

// Brackets the launches made in its lifetime; `flops` and `bytes` are the algorithmic work
// of those launches (2MNK for a GEMM, the tensors an op must read and write once).
struct ProfScope {
  Stream& st;
  int idx = -1;
  ProfScope(Stream& s, int cls, double flops, double bytes) : st(s) {
    if (!s.prof || !s.prof->on) return;
    Profiler::Rec r{s.prof->get(), s.prof->get(), cls, flops, bytes};
    cudaEventRecord(r.a, s.s);
    s.prof->recs.push_back(r);
    idx = int(s.prof->recs.size()) - 1;
  }
  ~ProfScope() {
    if (idx >= 0) cudaEventRecord(st.prof->recs[idx].b, st.s);
  }
};

#define PETB_LAUNCH_CHECK(st)                                     \
  do {                                                            \
    ++(st).launches;                                              \
    cudaError_t err__ = cudaGetLastError();                       \
    if (err__ != cudaSuccess)                                     \
      throw ::petb::Error(5, std::string("kernel launch failed at ") + __FILE__ + ":" + \
                                 std::to_string(__LINE__) + ": " + cudaGetErrorString(err__)); \
  } while (0)

// Raises a kernel's dynamic shared-memory limit on the CURRENT device when `bytes` is more than this device has been
// granted for it so far (the attribute is per device; `memo` is the kernel's own table).
template <class K>
void opt_in_shared_memory(K kernel, size_t bytes, SmemOptIn& memo) {
  int dev = 0;
  PETB_CUDA(cudaGetDevice(&dev));
  cudaError_t e = cudaSuccess;
  memo.ensure(dev, int(bytes), [&](int b) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, b);
    return e == cudaSuccess ? 0 : 1;
  });
  PETB_CUDA(e);
}

}  // namespace petb
