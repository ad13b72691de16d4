// pet_gemm_host_static: the fp32 weight GEMM for callers that must not allocate device memory.
//
// Who cannot allocate: a host program that has already handed the whole device to its own
// memory pool (an MD engine's device allocator, a framework's caching allocator) so that a
// cudaMalloc from a plug-in fails or fragments it; code that runs while another thread of the
// process is capturing a stream, where cudaMalloc is an error; and latency-critical loops that
// may not take the driver's allocation lock. pet_gemm_host stages its operands in the
// calculator's growable pool, which calls cudaMalloc when it grows. This variant stages them in
// a fixed array that is part of the library image instead, so it allocates nothing, ever.
//
// The price: the array (kStaticFloats floats, 12 MiB) is resident on every GPU that loads the
// library, from load to process exit, whether or not this entry point is called; problems that
// do not fit are refused; and all calls share the one array, so two calls that overlap on a GPU
// (different host threads) race on it. The copies and the kernel run on the calling thread's
// own stream (cudaStreamPerThread: it exists without being created, does not wait on the
// process-wide default stream and is not implicitly joined to other streams), and each call
// waits for that stream before it returns.
#include <atomic>
#include <cstdio>

#include "../../include/pet_b200.h"
#include "gemm.h"

namespace {

constexpr size_t kStaticFloats = size_t(3) << 20;  // 3 Mi floats = 12 MiB per GPU
using petb::kMaxDevices;

// The staging array. In host code this name is only a handle: its device address is obtained
// with cudaGetSymbolAddress below and that pointer is what kernels receive.
static __device__ __align__(256) float g_static_scratch[kStaticFloats];

// Device address of g_static_scratch, per device ordinal. Two threads that race on a device's first call both
// resolve the same address, so a relaxed atomic store is all the cache needs.
std::atomic<float*> g_scratch_ptr[kMaxDevices];

size_t round64(size_t n) { return (n + 63) & ~size_t(63); }

// While some thread of the process has a stream capture open in the global mode, CUDA refuses calls it counts as
// potentially unsafe from every thread, and a refused call also spoils that capture. Copies from and to pageable
// host memory are among them, and this entry point's operands are ordinary host arrays. For the length of a call
// the calling thread therefore declares its own calls unrelated to any capture (the relaxed mode), and puts back
// the mode it found when the call ends.
struct RelaxedCaptureMode {
  cudaStreamCaptureMode mode = cudaStreamCaptureModeRelaxed;
  RelaxedCaptureMode() { cudaThreadExchangeStreamCaptureMode(&mode); }
  ~RelaxedCaptureMode() { cudaThreadExchangeStreamCaptureMode(&mode); }
};

int fail(char* buf, size_t len, int code, const char* msg) {
  if (buf && len) snprintf(buf, len, "%s", msg);
  return code;
}

}  // namespace

extern "C" int pet_gemm_host_static(int m, int n, int k, const float* A, const float* W, float* C, char* errbuf,
                                    size_t errbuf_len) {
  if (m <= 0 || n <= 0 || k <= 0 || !A || !W || !C) return fail(errbuf, errbuf_len, PET_ERR_INVALID, "pet_gemm_host_static: bad arguments");
  if (n % 4 || k % 4) return fail(errbuf, errbuf_len, PET_ERR_INVALID, "pet_gemm_host_static: n and k must be multiples of 4");
  const size_t na = round64(size_t(m) * k), nw = round64(size_t(n) * k), nc = round64(size_t(m) * n);
  if (na + nw + nc > kStaticFloats) {
    char msg[256];
    snprintf(msg, sizeof(msg),
             "pet_gemm_host_static: m*k + n*k + m*n = %zu floats exceeds the fixed staging array of %zu floats; "
             "use pet_gemm_host (which may allocate) for this size",
             na + nw + nc, kStaticFloats);
    return fail(errbuf, errbuf_len, PET_ERR_INVALID, msg);
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return fail(errbuf, errbuf_len, PET_ERR_CUDA, "pet_gemm_host_static: no CUDA device");
  if (dev < 0 || dev >= kMaxDevices) return fail(errbuf, errbuf_len, PET_ERR_INVALID, "pet_gemm_host_static: device ordinal out of range");
  // Set-up, once per device, with that device current: the first call on a device resolves the
  // array's address there. Make that first call before any stream capture begins.
  float* dA = g_scratch_ptr[dev].load(std::memory_order_relaxed);
  if (!dA) {
    float* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress((void**) &ptr, g_static_scratch);
    if (e != cudaSuccess || !ptr) {
      char msg[256];
      snprintf(msg, sizeof(msg), "pet_gemm_host_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return fail(errbuf, errbuf_len, PET_ERR_CUDA, msg);
    }
    g_scratch_ptr[dev].store(ptr, std::memory_order_relaxed);
    dA = ptr;
  }
  float* dW = dA + na;
  float* dC = dW + nw;
  const RelaxedCaptureMode not_part_of_any_capture;
  try {
    petb::Stream st;  // this thread's own stream; nothing here allocates
    st.s = cudaStreamPerThread;
    petb::Arena unused;
    PETB_CUDA(cudaMemcpyAsync(dA, A, sizeof(float) * size_t(m) * k, cudaMemcpyHostToDevice, st.s));
    PETB_CUDA(cudaMemcpyAsync(dW, W, sizeof(float) * size_t(n) * k, cudaMemcpyHostToDevice, st.s));
    // The array keeps the previous call's contents. Every element of C is written by the kernel
    // (no accumulation onto old values), so nothing needs clearing first.
    petb::GemmArgs a;
    a.A = dA, a.lda = k, a.B = dW, a.ldb = k, a.C = dC, a.ldc = n, a.M = m, a.N = n, a.K = k;
    petb::gemm(st, unused, a, petb::GEMM_NATIVE);
    PETB_CUDA(cudaMemcpyAsync(C, dC, sizeof(float) * size_t(m) * n, cudaMemcpyDeviceToHost, st.s));
    PETB_CUDA(cudaStreamSynchronize(st.s));
  } catch (const petb::Error& err) {
    return fail(errbuf, errbuf_len, err.code, err.what());
  }
  return PET_OK;
}
