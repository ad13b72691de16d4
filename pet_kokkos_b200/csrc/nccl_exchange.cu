// The engine's side of exchange mode over NCCL, inside the library: rows of edges to ghosts cross between the
// ranks' GPUs with ncclSend / ncclRecv on the calculator's own stream, packed and unpacked by kernels here, and the
// ghost forces are folded onto their owners on the device and reduced with one ncclAllReduce.
//
// It stands for what the reference's LAMMPS pair style does around pet::Exchange
// (lammps/ML-PET/pair_pet.cpp:268-360 routing, :396-472 exchange_rows: pack, GPU-aware send/recv, unpack,
// :479-555 set_live and edges). The routing itself (which edge of which rank is the partner of each edge to a
// ghost) is host logic the caller supplies once per list as `dest[n_remote][2]` = (rank, index among that rank's
// edges to ghosts); partnership is symmetric, which makes the whole schedule static:
//   * to rank q this rank sends the rows of its edges whose partner lives on q, ordered by the partner's index;
//   * from rank q it receives q's rows ordered by ITS OWN edges' indices (the same set, seen from the other side).
// So counts, offsets and slots are known from `dest` alone: no handshake per evaluation and no host synchronisation
// inside a pass. Every edge to a ghost has a slot whether or not it is inside the cutoff in this evaluation; rows of
// edges that are not live are never read by the receiver (an edge and its partner have the same length, so they
// are live together).
//
// NCCL is taken from the process at run time (dlopen of libnccl.so.2: the copy PyTorch or the MD engine already
// loaded), so the library links without it and a build without NCCL still serves one GPU.
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <numeric>
#include <vector>

#include "../../include/pet_b200.h"
#include "common.h"

namespace {

struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

const NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    // PET_NCCL_LIB names the library file; otherwise the soname, which resolves to a copy the process has already
    // loaded (PyTorch's bundled one, an MD engine's) before it looks on the search path. A process that will load
    // PyTorch later should load it first: two different NCCL versions under one soname do not mix.
    void* h = nullptr;
    if (const char* path = std::getenv("PET_NCCL_LIB")) h = dlopen(path, RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return;
    auto sym = [&](const char* n) { return dlsym(h, n); };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.Send = reinterpret_cast<decltype(api.Send)>(sym("ncclSend"));
    api.Recv = reinterpret_cast<decltype(api.Recv)>(sym("ncclRecv"));
    api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
    api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.Send && api.Recv && api.GroupStart && api.GroupEnd &&
             api.AllReduce && api.GetErrorString;
  });
  return api;
}

thread_local std::string g_error;

#define PETX_NCCL(expr)                                                                                              \
  do {                                                                                                               \
    ncclResult_t r__ = (expr);                                                                                       \
    if (r__ != ncclSuccess) throw petb::Error(5, std::string(#expr) + ": " + nccl().GetErrorString(r__));            \
  } while (0)

// send(slot of live row l) = out(l), 16 bytes per thread
__global__ void k_pack_rows(float4* __restrict__ send, const float4* __restrict__ out, const int* __restrict__ live,
                            const int* __restrict__ slot_of, int n_live, int w4) {
  const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= size_t(n_live) * w4) return;
  const int l = int(i / w4), c = int(i % w4);
  send[size_t(slot_of[live[l]]) * w4 + c] = out[i];
}
// in(l) = recv(slot of live row l)
__global__ void k_unpack_rows(float4* __restrict__ in, const float4* __restrict__ recv, const int* __restrict__ live,
                              const int* __restrict__ slot_of, int n_live, int w4) {
  const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= size_t(n_live) * w4) return;
  const int l = int(i / w4), c = int(i % w4);
  in[i] = recv[size_t(slot_of[live[l]]) * w4 + c];
}
// One thread per atom of the whole cell: buf = [energy, virial(6), forces(3 n_total)]; the forces this rank has for
// the atom (its own, and those on its ghost images of it) summed in list order.
__global__ void k_fold_to_owners(double* __restrict__ buf, const double* __restrict__ forces, const double* __restrict__ energy,
                                 const double* __restrict__ vir6, const int* __restrict__ off, const int* __restrict__ listed,
                                 int n_total) {
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a == 0) {
    buf[0] = energy[0];
    for (int k = 0; k < 6; ++k) buf[1 + k] = vir6 ? vir6[k] : 0.0;
  }
  if (a >= n_total) return;
  double f[3] = {0.0, 0.0, 0.0};
  for (int k = off[a]; k < off[a + 1]; ++k)
    for (int c = 0; c < 3; ++c) f[c] += forces[3 * size_t(listed[k]) + c];
  for (int c = 0; c < 3; ++c) buf[7 + 3 * size_t(a) + c] = f[c];
}

}  // namespace

struct pet_nccl_exchange {
  int rank = 0, world = 1, device = 0, n_remote = 0;
  ncclComm_t comm = nullptr;
  std::vector<int> count, offset;  // rows to (= from) each rank, and where that rank's block starts
  int* send_slot = nullptr;        // [n_remote] device: slot of each edge to a ghost in the send buffer
  int* recv_slot = nullptr;        // [n_remote] device: slot of its partner's row in the receive buffer
  float* send = nullptr;
  float* recv = nullptr;
  size_t buf_floats = 0;
  const int* live = nullptr;  // device, this evaluation's (set_live)
  int n_live = 0;
  pet_exchange callbacks{};
  // the fold of forces onto owners
  int n_total = 0, n_listed = 0;
  int* fold_off = nullptr;
  int* fold_listed = nullptr;
  double* reduce_buf = nullptr;   // device [7 + 3 n_total]
  double* reduce_host = nullptr;  // pinned
  // CUDA events around the rows in flight (edges() calls), summed when asked
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> timed, spare;
  bool timing = false;
};

namespace {

void ensure_buffers(pet_nccl_exchange* x, int width) {
  const size_t need = size_t(x->n_remote > 0 ? x->n_remote : 1) * width;
  if (need <= x->buf_floats) return;
  if (x->send) cudaFree(x->send);
  if (x->recv) cudaFree(x->recv);
  x->send = x->recv = nullptr;
  PETB_CUDA(cudaMalloc(&x->send, need * sizeof(float)));
  PETB_CUDA(cudaMalloc(&x->recv, need * sizeof(float)));
  x->buf_floats = need;
}

int cb_set_live(void* user, const int* live, int n_live, void*) {
  auto* x = static_cast<pet_nccl_exchange*>(user);
  x->live = live, x->n_live = n_live;
  return 0;
}

int cb_edges(void* user, const float* out, float* in, int n_live, int width, void* stream) {
  auto* x = static_cast<pet_nccl_exchange*>(user);
  try {
    if (width % 4) throw petb::Error(2, "exchange: row width must be a multiple of 4");
    if (n_live != x->n_live) throw petb::Error(3, "exchange: edges() does not follow this evaluation's set_live()");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    ensure_buffers(x, width);
    std::pair<cudaEvent_t, cudaEvent_t> ev{};
    if (x->timing) {
      if (!x->spare.empty()) ev = x->spare.back(), x->spare.pop_back();
      else cudaEventCreate(&ev.first), cudaEventCreate(&ev.second);
      cudaEventRecord(ev.first, s);
    }
    const int w4 = width / 4;
    const size_t work = size_t(n_live) * w4;
    if (work) {
      k_pack_rows<<<unsigned((work + 255) / 256), 256, 0, s>>>(reinterpret_cast<float4*>(x->send), reinterpret_cast<const float4*>(out),
                                                              x->live, x->send_slot, n_live, w4);
      PETB_CUDA(cudaGetLastError());
    }
    // every rank makes the same calls whether or not it has live edges of its own: the schedule is the list's
    const NcclApi& api = nccl();
    bool grouped = false;
    for (int q = 0; q < x->world; ++q) {
      const size_t n = size_t(x->count[q]) * width, at = size_t(x->offset[q]) * width;
      if (!n) continue;
      if (q == x->rank) {  // images of this rank's own atoms: the partner rows are here already
        PETB_CUDA(cudaMemcpyAsync(x->recv + at, x->send + at, n * sizeof(float), cudaMemcpyDeviceToDevice, s));
        continue;
      }
      if (!grouped) {
        PETX_NCCL(api.GroupStart());
        grouped = true;
      }
      PETX_NCCL(api.Send(x->send + at, n, ncclFloat32, q, x->comm, s));
      PETX_NCCL(api.Recv(x->recv + at, n, ncclFloat32, q, x->comm, s));
    }
    if (grouped) PETX_NCCL(api.GroupEnd());
    if (work) {
      k_unpack_rows<<<unsigned((work + 255) / 256), 256, 0, s>>>(reinterpret_cast<float4*>(in), reinterpret_cast<const float4*>(x->recv),
                                                                x->live, x->recv_slot, n_live, w4);
      PETB_CUDA(cudaGetLastError());
    }
    if (x->timing) {
      cudaEventRecord(ev.second, s);
      x->timed.push_back(ev);
    }
    return 0;
  } catch (const std::exception& e) {
    g_error = e.what();
    return 1;
  }
}

// The static schedule of one rank from its routing: rows per peer, each edge's slot in the send buffer (blocks by
// destination rank, within a block by the partner's index there) and the slot its partner's row arrives in (blocks
// by source rank, within a block by this rank's own index). Host arithmetic only.
void make_schedule(const int* dest, int n_remote, int world, std::vector<int>& count, std::vector<int>& offset,
                   std::vector<int>& send_slot, std::vector<int>& recv_slot) {
  count.assign(world, 0), offset.assign(world, 0);
  for (int r = 0; r < n_remote; ++r) {
    const int q = dest[2 * r];
    if (q < 0 || q >= world) throw petb::Error(2, "exchange: a partner on a rank that does not exist");
    ++count[q];
  }
  for (int q = 1; q < world; ++q) offset[q] = offset[q - 1] + count[q - 1];
  send_slot.assign(n_remote, 0), recv_slot.assign(n_remote, 0);
  std::vector<int> order(n_remote), at(offset);
  for (int r = 0; r < n_remote; ++r) recv_slot[r] = at[dest[2 * r]]++;
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) {
    return dest[2 * a] != dest[2 * b] ? dest[2 * a] < dest[2 * b] : dest[2 * a + 1] < dest[2 * b + 1];
  });
  for (int k = 0; k < n_remote; ++k) send_slot[order[k]] = k;
}

template <class F>
int guarded(F&& f) {
  try {
    f();
    return PET_OK;
  } catch (const petb::Error& e) {
    g_error = e.what();
    return e.code;
  } catch (const std::exception& e) {
    g_error = e.what();
    return PET_ERR_RUNTIME;
  }
}

}  // namespace

extern "C" {

const char* pet_nccl_last_error(void) { return g_error.c_str(); }

int pet_exchange_schedule(const int* dest, int n_remote, int world, int* count, int* send_slot, int* recv_slot) {
  return guarded([&] {
    if (n_remote < 0 || world < 1 || (n_remote > 0 && !dest)) throw petb::Error(2, "exchange: bad arguments");
    std::vector<int> c, o, ss, rs;
    make_schedule(dest, n_remote, world, c, o, ss, rs);
    if (count) std::copy(c.begin(), c.end(), count);
    if (send_slot) std::copy(ss.begin(), ss.end(), send_slot);
    if (recv_slot) std::copy(rs.begin(), rs.end(), recv_slot);
  });
}

int pet_nccl_unique_id(char* id128) {
  return guarded([&] {
    if (!id128) throw petb::Error(2, "exchange: no buffer for the id");
    if (!nccl().ok) throw petb::Error(1, "exchange: libnccl.so.2 is not available in this process");
    ncclUniqueId id;
    PETX_NCCL(nccl().GetUniqueId(&id));
    static_assert(sizeof(ncclUniqueId) == 128, "the id is passed around as 128 bytes");
    std::memcpy(id128, &id, 128);
  });
}

int pet_nccl_exchange_create(const char* id128, int rank, int world, int device, const int* dest, int n_remote,
                             const int* owner, int n_listed, int n_total, pet_nccl_exchange** out) {
  return guarded([&] {
    if (!id128 || !out || world < 1 || rank < 0 || rank >= world || n_remote < 0 || (n_remote > 0 && !dest))
      throw petb::Error(2, "exchange: bad arguments");
    if (!nccl().ok) throw petb::Error(1, "exchange: libnccl.so.2 is not available in this process");
    PETB_CUDA(cudaSetDevice(device));
    auto x = new pet_nccl_exchange();
    *out = x;
    x->rank = rank, x->world = world, x->device = device, x->n_remote = n_remote;
    ncclUniqueId id;
    std::memcpy(&id, id128, 128);
    PETX_NCCL(nccl().CommInitRank(&x->comm, world, id, rank));
    std::vector<int> send_slot, recv_slot;
    make_schedule(dest, n_remote, world, x->count, x->offset, send_slot, recv_slot);
    const size_t nr = size_t(n_remote > 0 ? n_remote : 1);
    PETB_CUDA(cudaMalloc(&x->send_slot, nr * sizeof(int)));
    PETB_CUDA(cudaMalloc(&x->recv_slot, nr * sizeof(int)));
    PETB_CUDA(cudaMemcpy(x->send_slot, send_slot.data(), size_t(n_remote) * sizeof(int), cudaMemcpyHostToDevice));
    PETB_CUDA(cudaMemcpy(x->recv_slot, recv_slot.data(), size_t(n_remote) * sizeof(int), cudaMemcpyHostToDevice));
    x->callbacks.user = x, x->callbacks.set_live = cb_set_live, x->callbacks.edges = cb_edges;
    // the fold: for every atom of the whole cell, this rank's listed atoms (owned or ghost images) that are it
    if (owner && n_total > 0) {
      x->n_total = n_total, x->n_listed = n_listed;
      std::vector<int> off(size_t(n_total) + 1, 0), listed(n_listed > 0 ? n_listed : 1);
      for (int i = 0; i < n_listed; ++i) {
        if (owner[i] < 0 || owner[i] >= n_total) throw petb::Error(2, "exchange: an owner outside the cell's atoms");
        ++off[owner[i] + 1];
      }
      for (int a = 0; a < n_total; ++a) off[a + 1] += off[a];
      std::vector<int> cur(off.begin(), off.end() - 1);
      for (int i = 0; i < n_listed; ++i) listed[cur[owner[i]]++] = i;
      PETB_CUDA(cudaMalloc(&x->fold_off, off.size() * sizeof(int)));
      PETB_CUDA(cudaMalloc(&x->fold_listed, listed.size() * sizeof(int)));
      PETB_CUDA(cudaMemcpy(x->fold_off, off.data(), off.size() * sizeof(int), cudaMemcpyHostToDevice));
      PETB_CUDA(cudaMemcpy(x->fold_listed, listed.data(), listed.size() * sizeof(int), cudaMemcpyHostToDevice));
      PETB_CUDA(cudaMalloc(&x->reduce_buf, (7 + 3 * size_t(n_total)) * sizeof(double)));
      PETB_CUDA(cudaMallocHost(&x->reduce_host, (7 + 3 * size_t(n_total)) * sizeof(double)));
    }
    PETB_CUDA(cudaDeviceSynchronize());  // the tables above were copied on the legacy stream; they are read on the caller's
  });
}

void pet_nccl_exchange_destroy(pet_nccl_exchange* x) {
  if (!x) return;
  cudaSetDevice(x->device);
  cudaDeviceSynchronize();
  if (x->comm && nccl().ok) nccl().CommDestroy(x->comm);
  cudaFree(x->send_slot), cudaFree(x->recv_slot), cudaFree(x->send), cudaFree(x->recv);
  cudaFree(x->fold_off), cudaFree(x->fold_listed), cudaFree(x->reduce_buf);
  if (x->reduce_host) cudaFreeHost(x->reduce_host);
  for (auto& e : x->timed) cudaEventDestroy(e.first), cudaEventDestroy(e.second);
  for (auto& e : x->spare) cudaEventDestroy(e.first), cudaEventDestroy(e.second);
  delete x;
}

const pet_exchange* pet_nccl_exchange_callbacks(pet_nccl_exchange* x) { return x ? &x->callbacks : nullptr; }

int pet_nccl_exchange_reduce(pet_nccl_exchange* x, const double* forces, const double* energy, const double* virial6,
                             void* stream, double* out_host) {
  return guarded([&] {
    if (!x || !x->reduce_buf || !forces || !energy || !out_host) throw petb::Error(2, "exchange: nothing to reduce");
    PETB_CUDA(cudaSetDevice(x->device));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t n = 7 + 3 * size_t(x->n_total);
    k_fold_to_owners<<<(x->n_total + 255) / 256, 256, 0, s>>>(x->reduce_buf, forces, energy, virial6, x->fold_off, x->fold_listed,
                                                              x->n_total);
    PETB_CUDA(cudaGetLastError());
    if (x->world > 1) PETX_NCCL(nccl().AllReduce(x->reduce_buf, x->reduce_buf, n, ncclFloat64, ncclSum, x->comm, s));
    PETB_CUDA(cudaMemcpyAsync(x->reduce_host, x->reduce_buf, n * sizeof(double), cudaMemcpyDeviceToHost, s));
    PETB_CUDA(cudaStreamSynchronize(s));
    std::memcpy(out_host, x->reduce_host, n * sizeof(double));
  });
}

int pet_nccl_exchange_timing(pet_nccl_exchange* x, int enable, double* ms, int* calls) {
  return guarded([&] {
    if (!x) throw petb::Error(2, "exchange: no exchange");
    PETB_CUDA(cudaSetDevice(x->device));
    double total = 0.0;
    int n = 0;
    for (auto& e : x->timed) {
      cudaEventSynchronize(e.second);
      float t = 0.f;
      if (cudaEventElapsedTime(&t, e.first, e.second) == cudaSuccess) total += t, ++n;
      x->spare.push_back(e);
    }
    x->timed.clear();
    if (ms) *ms = total;
    if (calls) *calls = n;
    x->timing = enable != 0;
  });
}

}  // extern "C"
