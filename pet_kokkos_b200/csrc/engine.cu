// The calculator behind the C ABI: see engine.h.
#include "engine.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "gemm.h"

namespace petb {

namespace {

int env_int(const char* name, int dflt) {
  const char* e = std::getenv(name);
  return e && *e ? std::atoi(e) : dflt;
}

int env_gemm_mode() {
  const char* e = std::getenv("PET_GEMM");
  if (!e) return GEMM_NATIVE;
  const std::string v(e);
  if (v == "tf32") return GEMM_TF32;
  if (v == "bf16") return GEMM_BF16;
  if (v == "3xtf32" || v == "tf32x3") return GEMM_TF32X3;
  return GEMM_NATIVE;
}

// eg(e) = scale * g(packed row of raw edge e), 0 for a dropped edge (the reference's raw_edge_grad).
__global__ void k_raw_edge_grad(double* __restrict__ eg, const double* __restrict__ grad, const int* __restrict__ packed_of_raw,
                                int R, double scale) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= R) return;
  const int p = packed_of_raw[e];
  for (int c = 0; c < 3; ++c) eg[3 * size_t(e) + c] = p >= 0 ? scale * grad[3 * size_t(p) + c] : 0.0;
}

// Which of the edges to ghosts kept a row this time, and where (the reference's remote_map, src/model.cpp:459-497).
__global__ void k_live_flag(int* __restrict__ flag, const int* __restrict__ remote_raw, const int* __restrict__ packed_of_raw,
                            int R) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < R) flag[r] = packed_of_raw[remote_raw[r]] >= 0;
}
__global__ void k_live_fill(int* __restrict__ live, int* __restrict__ live_packed, int* __restrict__ remote_of,
                            const int* __restrict__ at, const int* __restrict__ remote_raw,
                            const int* __restrict__ packed_of_raw, int R) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  const int k = packed_of_raw[remote_raw[r]];
  if (k < 0) return;
  const int l = at[r];
  live[l] = r, live_packed[l] = k, remote_of[k] = l;
}

// eg(e) += gmag(e) v(e)
// A flat pair list's columns into a dense [P,5] block, whatever its strides.
__global__ void k_dense_pairs(int* __restrict__ out, const int* __restrict__ pairs, long sp, long sc, int P) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= 5 * P) return;
  out[t] = pairs[(t / 5) * sp + (t % 5) * sc];
}

// An engine's 2-D neighbour array into a dense list: centre ii's neighbours at out[off[ii] ...], index bits only.
__global__ void k_dense_neighbors(int* __restrict__ out, const int* __restrict__ ilist, const int* __restrict__ off,
                                  const int* __restrict__ nbr, long si, long sk, int mask, int NC) {
  const int ii = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (ii >= NC) return;
  const int i = ilist[ii], e0 = off[ii], n = off[ii + 1] - e0;
  for (int k = lane; k < n; k += 32) out[e0 + k] = nbr[i * si + k * sk] & mask;
}

// The engine's positions into the list's numbering.
__global__ void k_renumber_positions(double* __restrict__ out, const double* __restrict__ x, const int* __restrict__ ren, int N) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N) return;
  const int to = ren[i];
  for (int c = 0; c < 3; ++c) out[3 * to + c] = x[3 * i + c];
}

__global__ void k_add_radial(double* __restrict__ eg, const double* __restrict__ gmag, const double* __restrict__ vec, int E) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  for (int c = 0; c < 3; ++c) eg[3 * size_t(e) + c] += gmag[e] * vec[3 * size_t(e) + c];
}

// An edge with no partner gives its target's share of the force itself (orphan_forces, src/forces.cpp:400-410).
__global__ void k_orphan_forces(double* __restrict__ forces, const double* __restrict__ eg, const int* __restrict__ ooff,
                                const int* __restrict__ oedge, int N) {
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= N) return;
  for (int k = ooff[a]; k < ooff[a + 1]; ++k)
    for (int c = 0; c < 3; ++c) forces[3 * size_t(a) + c] -= eg[3 * size_t(oedge[k]) + c];
}

// out(k) = in(idx(k)): the edge offsets at structure boundaries, for the host.
__global__ void k_pick(int* __restrict__ out, const int* __restrict__ in, const int* __restrict__ idx, int n) {
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k < n) out[k] = in[idx[k]];
}
// out(i, :) = in(map(i), :), `w` doubles per row.
__global__ void k_gather_rows_f64(double* __restrict__ out, const double* __restrict__ in, const int* __restrict__ map, int n, int w) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < n * w) out[t] = in[size_t(map[t / w]) * w + t % w];
}
// The cached pairs of the structures that stay, renumbered for where each structure now sits (the reference's
// cache_reassemble, src/device_geometry.cpp:203-246). Slot k of the smaller batch holds the structure whose atoms
// were at atom_old(k).. and whose pairs were at edge_old(k)..; they move to atom_new(k).. and edge_new(k)...
// Pairs never cross structures, so a block's partners stay inside it.
__global__ void k_reassemble_pairs(RawEdges out, RawEdges in, const int* __restrict__ edge_new, const int* __restrict__ edge_old,
                                   const int* __restrict__ atom_new, const int* __restrict__ atom_old, int slots, int E) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  int lo = 0, hi = slots - 1;  // the slot whose range of new pairs holds e
  while (lo < hi) {
    const int mid = (lo + hi + 1) / 2;
    if (edge_new[mid] <= e) lo = mid;
    else hi = mid - 1;
  }
  const int from = edge_old[lo] + e - edge_new[lo], moved = atom_new[lo] - atom_old[lo];
  out.i[e] = in.i[from] + moved, out.j[e] = in.j[from] + moved;
  out.reverse[e] = in.reverse[from] < 0 ? -1 : in.reverse[from] - edge_old[lo] + edge_new[lo];
  for (int d = 0; d < 3; ++d) out.shift[3 * size_t(e) + d] = in.shift[3 * size_t(from) + d];
}
__global__ void k_reassemble_offsets(int* __restrict__ off_new, const int* __restrict__ off_old, const int* __restrict__ atom_map,
                                     const int* __restrict__ slot_of_atom, const int* __restrict__ edge_new,
                                     const int* __restrict__ edge_old, int N, int E) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i > N) return;
  if (i == N) {
    off_new[N] = E;
    return;
  }
  const int k = slot_of_atom[i];
  off_new[i] = off_old[atom_map[i]] - edge_old[k] + edge_new[k];
}

// `skip`, unless null, is the fixed-shape overflow flag: a step that did not fit adds nothing (it is redone).
__global__ void k_add_arrays(double* __restrict__ f, const double* __restrict__ forces, double* __restrict__ e,
                             const double* __restrict__ per_atom, int N, const int* __restrict__ skip) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N || (skip && *skip)) return;
  if (f)
    for (int c = 0; c < 3; ++c) f[3 * size_t(i) + c] += forces[3 * size_t(i) + c];
  if (e) e[i] += per_atom[i];
}

// Each directed edge's sym(v (x) g), half to each end, gathered per atom (md_atom_virial, src/calculator.cpp:846-868).
__global__ void k_atom_virial(double* __restrict__ w, const double* __restrict__ eg, const double* __restrict__ vec,
                              const int* __restrict__ roff, const int* __restrict__ rrev, const int* __restrict__ ooff,
                              const int* __restrict__ oedge, int N, double scale, const int* __restrict__ skip) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N || (skip && *skip)) return;
  double s[6] = {0, 0, 0, 0, 0, 0};
  auto add = [&](int e) {
    const double* v = vec + 3 * size_t(e);
    const double* g = eg + 3 * size_t(e);
    s[0] += v[0] * g[0], s[1] += v[1] * g[1], s[2] += v[2] * g[2];
    s[3] += 0.5 * (v[0] * g[1] + v[1] * g[0]);
    s[4] += 0.5 * (v[0] * g[2] + v[2] * g[0]);
    s[5] += 0.5 * (v[1] * g[2] + v[2] * g[1]);
  };
  for (int e = roff[i]; e < roff[i + 1]; ++e) {
    add(e);
    if (rrev[e] >= 0) add(rrev[e]);
  }
  if (ooff)
    for (int k = ooff[i]; k < ooff[i + 1]; ++k) add(oedge[k]);
  for (int k = 0; k < 6; ++k) w[6 * size_t(i) + k] += scale * s[k];
}

}  // namespace

Engine::Engine(const std::string& json, const std::string& weights, const pet_options* opts)
    : ckpt(json, weights), geom_arena(size_t(1) << 20), nbr_arena(size_t(16) << 20), save_arena(size_t(64) << 20),
      tmp_arena(size_t(64) << 20), session_arena(size_t(4) << 20), cache_arena(size_t(4) << 20), cache_spare(size_t(4) << 20) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0)
    throw Error(5, "no CUDA device: this evaluator has no CPU path");
  device = opts && opts->device >= 0 ? opts->device : -1;
  if (device >= 0) PETB_CUDA(cudaSetDevice(device));
  else PETB_CUDA(cudaGetDevice(&device));
  gemm_mode = opts && opts->gemm_mode >= 0 ? opts->gemm_mode : env_gemm_mode();
  graphs = (opts && opts->graphs >= 0 ? opts->graphs : env_int("PET_GRAPHS", 1)) != 0;
  md_fixed = (opts && opts->md_fixed_shapes >= 0 ? opts->md_fixed_shapes : env_int("PET_MD_FIXED", 0)) != 0;
  cache_neighbors = (opts && opts->cache_neighbors > 0) || env_int("PET_CACHE_NEIGHBORS", 0) != 0;
  memory_budget = opts ? opts->memory_budget_bytes : 0;
  max_batch_atoms = opts && opts->max_batch_atoms > 0 ? opts->max_batch_atoms : 0;
  recompute = opts && opts->recompute > 0 ? opts->recompute : RECOMPUTE_AUTO;
  if (recompute == RECOMPUTE_AUTO)
    if (const char* e = std::getenv("PET_RECOMPUTE")) {  // auto | never | wide | layers (Options::recompute)
      const std::string v(e);
      recompute = v == "never" ? RECOMPUTE_NEVER : v == "wide" ? RECOMPUTE_WIDE : v == "layers" ? RECOMPUTE_LAYERS : RECOMPUTE_AUTO;
    }
  if (recompute > RECOMPUTE_LAYERS) throw Error(2, "pet: unknown recompute tier " + std::to_string(recompute));
  PETB_CUDA(cudaStreamCreateWithFlags(&st.s, cudaStreamNonBlocking));
  PETB_CUDA(cudaEventCreate(&ev0));
  PETB_CUDA(cudaEventCreate(&ev1));
  PETB_CUDA(cudaMallocHost(&pinned, 64 * sizeof(int)));
  model.reset(new Model(ckpt));
}

Engine::~Engine() {
  cudaSetDevice(device);
  cudaDeviceSynchronize();
  drop_graphs();
  model.reset();
  if (pinned) cudaFreeHost(pinned);
  if (host_stage) cudaFreeHost(host_stage);
  if (ev0) cudaEventDestroy(ev0);
  if (ev1) cudaEventDestroy(ev1);
  if (st.legacy_fence) cudaEventDestroy(st.legacy_fence);
  if (st.s) cudaStreamDestroy(st.s);
}

void* Engine::staging(size_t bytes) {
  if (bytes > host_stage_bytes) {
    if (host_stage) cudaFreeHost(host_stage);
    host_stage = nullptr;
    size_t cap = host_stage_bytes ? host_stage_bytes : size_t(1) << 20;
    while (cap < bytes) cap *= 2;
    PETB_CUDA(cudaMallocHost(&host_stage, cap));
    host_stage_bytes = cap;
  }
  return host_stage;
}

int Engine::species_index(int Z) const {
  const int s = (Z >= 0 && Z < (int) ckpt.species_to_index.size()) ? ckpt.species_to_index[Z] : -1;
  if (s < 0) throw Error(1, "pet: unsupported atomic number " + std::to_string(Z));
  return s;
}

// ---- staging (stage_systems, src/device_geometry.cpp:368-401) -------------------

void Engine::stage(const pet_system* systems, int B, bool keep_cache) {
  PETB_CUDA(cudaSetDevice(device));
  if (B < 0 || (B > 0 && !systems)) throw Error(2, "pet: no systems given");
  long long Nll = 0;
  for (int b = 0; b < B; ++b) {
    if (systems[b].n_atoms < 0) throw Error(2, "pet: negative atom count");
    Nll += systems[b].n_atoms;
  }
  if (Nll >= (1LL << 24)) throw Error(1, "pet: too many atoms for the edge key");
  const int N = int(Nll);
  // One host block, one copy: doubles first, then ints.
  const size_t nd = size_t(N) * 3 + size_t(B) * 18, ni = size_t(N) * 2 + size_t(B) * 9 + 2;
  char* hb = static_cast<char*>(staging(nd * 8 + ni * 4));
  double* h_pos = reinterpret_cast<double*>(hb);
  double* h_cell = h_pos + size_t(N) * 3;
  double* h_cinv = h_cell + size_t(B) * 9;
  int* h_sid = reinterpret_cast<int*>(h_cinv + size_t(B) * 9);
  int* h_spec = h_sid + N;
  int* h_soff = h_spec + N;
  int* h_sper = h_soff + B + 1;
  int* h_gnc = h_sper + B;
  int* h_gnr = h_gnc + 3 * B;
  int* h_goff = h_gnr + 3 * B;
  const std::vector<int> was_natoms = h_natoms, was_per = h_per, was_species = h_species;
  h_cells.assign(size_t(B) * 9, 0.0);
  h_natoms.assign(B, 0);
  h_per.assign(B, 0);
  int gi = 0, bins = 0;
  for (int b = 0; b < B; ++b) {
    const pet_system& s = systems[b];
    h_soff[b] = gi;
    h_natoms[b] = s.n_atoms;
    h_per[b] = h_sper[b] = (s.pbc[0] ? 1 : 0) | (s.pbc[1] ? 2 : 0) | (s.pbc[2] ? 4 : 0);
    for (int e = 0; e < 9; ++e) h_cells[size_t(b) * 9 + e] = h_cell[size_t(b) * 9 + e] = s.cell[e];
    invert_cell(s.cell, h_cinv + size_t(b) * 9);
    grid_for_cell(s.cell, h_sper[b], s.n_atoms, ckpt.hypers.cutoff, h_gnc + 3 * b, h_gnr + 3 * b);
    h_goff[b] = bins;
    bins += h_gnc[3 * b] * h_gnc[3 * b + 1] * h_gnc[3 * b + 2];
    for (int i = 0; i < s.n_atoms; ++i, ++gi) {
      for (int d = 0; d < 3; ++d) h_pos[size_t(gi) * 3 + d] = s.positions[size_t(i) * 3 + d];
      h_sid[gi] = b;
      h_spec[gi] = species_index(s.atomic_numbers[i]);
    }
  }
  h_soff[B] = gi;
  h_goff[B] = bins;
  PETB_CUDA(cudaStreamSynchronize(st.s));  // the previous evaluation may still read the staged block
  geom_arena.reset();
  char* db = static_cast<char*>(geom_arena.alloc_bytes(nd * 8 + ni * 4));
  PETB_CUDA(cudaMemcpyAsync(db, hb, nd * 8 + ni * 4, cudaMemcpyHostToDevice, st.s));
  Geom g;
  g.Ntot = N, g.B = B, g.nbins = bins;
  g.pos = reinterpret_cast<double*>(db);
  g.scell = g.pos + size_t(N) * 3;
  g.cinv = g.scell + size_t(B) * 9;
  g.sid = reinterpret_cast<int*>(g.cinv + size_t(B) * 9);
  g.spec = g.sid + N;
  g.soff = g.spec + N;
  g.sper = g.soff + B + 1;
  g.gnc = g.sper + B;
  g.gnr = g.gnc + 3 * B;
  g.goff = g.gnr + 3 * B;
  geom = g;
  h_species.assign(h_spec, h_spec + N);
  // Calculator::stage resets the neighbour cache (include/pet/calculator.hpp:210-212); an evaluation that stages
  // the same atoms again keeps it
  verlet.valid = verlet.valid && keep_cache && was_natoms == h_natoms && was_per == h_per && was_species == h_species;
  // the copy must finish before the staging block is reused by another stage()
  PETB_CUDA(cudaStreamSynchronize(st.s));
}

// A batch being stepped shrinks as its structures finish (a batched relaxation): the structures `keep` (indices into
// the staged batch, in the order they shall have from now on) stay, with the positions they have on the device now,
// and the Verlet cache follows them without a new search: each kept structure's block of cached pairs is copied and
// renumbered. The reference does the same when compute_device is given a smaller DeviceGeom whose `staged` says
// where each structure went (include/pet/calculator.hpp:214-218, src/device_geometry.cpp:203-246,262-310).
void Engine::keep_staged(const int* keep, int n_keep) {
  PETB_CUDA(cudaSetDevice(device));
  const int B = geom.B, N = geom.Ntot;
  if (n_keep < 0 || (n_keep > 0 && !keep)) throw Error(2, "pet: no structures given to keep");
  if (B == 0 && N == 0) throw Error(3, "pet: nothing is staged");
  std::vector<char> seen(B, 0);
  for (int k = 0; k < n_keep; ++k) {
    if (keep[k] < 0 || keep[k] >= B || seen[keep[k]]) throw Error(2, "pet: keep names a structure twice or one that is not staged");
    seen[keep[k]] = 1;
  }
  PETB_CUDA(cudaStreamSynchronize(st.s));
  std::vector<int> soff_old(B + 1, 0);
  for (int b = 0; b < B; ++b) soff_old[b + 1] = soff_old[b] + h_natoms[b];
  // the kept structures, slot by slot: their atoms' old indices, and host copies of what staging needs
  std::vector<int> atom_map, slot_of_atom, atom_new(n_keep + 1, 0), atom_old(n_keep > 0 ? n_keep : 1, 0);
  for (int k = 0; k < n_keep; ++k) {
    const int b = keep[k];
    atom_old[k] = soff_old[b], atom_new[k + 1] = atom_new[k] + h_natoms[b];
    for (int a = 0; a < h_natoms[b]; ++a) atom_map.push_back(soff_old[b] + a), slot_of_atom.push_back(k);
  }
  const int Nn = atom_new[n_keep];
  tmp_arena.reset();
  int* d_map = tmp_arena.alloc<int>(size_t(Nn > 0 ? Nn : 1));
  double* d_pos = tmp_arena.alloc<double>(3 * size_t(Nn > 0 ? Nn : 1));
  std::vector<double> pos(3 * size_t(Nn));
  if (Nn) {
    PETB_CUDA(cudaMemcpyAsync(d_map, atom_map.data(), 4 * size_t(Nn), cudaMemcpyHostToDevice, st.s));
    k_gather_rows_f64<<<cdiv(3 * size_t(Nn), 256), 256, 0, st.s>>>(d_pos, geom.pos, d_map, Nn, 3);
    PETB_LAUNCH_CHECK(st);
    PETB_CUDA(cudaMemcpyAsync(pos.data(), d_pos, 24 * size_t(Nn), cudaMemcpyDeviceToHost, st.s));
  }
  // the cache's pairs for the smaller batch, in the pool that is not holding the current ones
  VerletCache next;
  const bool follow = cache_neighbors && verlet.valid && Nn > 0;
  if (follow) {
    const VerletCache& c = verlet;
    std::vector<int> bounds(n_keep + 1), edge_at(size_t(n_keep) * 2);
    int* d_idx = tmp_arena.alloc<int>(size_t(n_keep) * 2);
    int* d_val = tmp_arena.alloc<int>(size_t(n_keep) * 2);
    std::vector<int> idx(size_t(n_keep) * 2);
    for (int k = 0; k < n_keep; ++k) idx[2 * k] = soff_old[keep[k]], idx[2 * k + 1] = soff_old[keep[k] + 1];
    PETB_CUDA(cudaMemcpyAsync(d_idx, idx.data(), 4 * idx.size(), cudaMemcpyHostToDevice, st.s));
    k_pick<<<cdiv(idx.size(), 256), 256, 0, st.s>>>(d_val, c.ref.off, d_idx, int(idx.size()));
    PETB_LAUNCH_CHECK(st);
    PETB_CUDA(cudaMemcpyAsync(edge_at.data(), d_val, 4 * edge_at.size(), cudaMemcpyDeviceToHost, st.s));
    PETB_CUDA(cudaStreamSynchronize(st.s));
    std::vector<int> edge_old(n_keep), edge_new(n_keep + 1, 0);
    for (int k = 0; k < n_keep; ++k) edge_old[k] = edge_at[2 * k], edge_new[k + 1] = edge_new[k] + edge_at[2 * k + 1] - edge_at[2 * k];
    const int En = edge_new[n_keep];
    Arena& pool = cache_spare;
    pool.reset();
    const size_t Ea = En > 0 ? En : 1;
    RawEdges r;
    r.E = En;
    r.i = pool.alloc<int>(Ea), r.j = pool.alloc<int>(Ea), r.shift = pool.alloc<int>(3 * Ea);
    r.vec = pool.alloc<double>(3 * Ea), r.dist = pool.alloc<double>(Ea);
    r.off = pool.alloc<int>(size_t(Nn) + 1), r.reverse = pool.alloc<int>(Ea);
    next.pos0 = pool.alloc<double>(3 * size_t(Nn)), next.cinv0 = pool.alloc<double>(9 * size_t(n_keep));
    next.worst = pool.alloc<double>(1);
    int* d_tab = tmp_arena.alloc<int>(4 * size_t(n_keep) + 2 + size_t(Nn));
    int *d_enew = d_tab, *d_eold = d_enew + n_keep + 1, *d_anew = d_eold + n_keep, *d_aold = d_anew + n_keep + 1;
    int* d_slot = d_aold + n_keep;
    int* d_keep = tmp_arena.alloc<int>(n_keep);
    PETB_CUDA(cudaMemcpyAsync(d_enew, edge_new.data(), 4 * size_t(n_keep + 1), cudaMemcpyHostToDevice, st.s));
    PETB_CUDA(cudaMemcpyAsync(d_eold, edge_old.data(), 4 * size_t(n_keep), cudaMemcpyHostToDevice, st.s));
    PETB_CUDA(cudaMemcpyAsync(d_anew, atom_new.data(), 4 * size_t(n_keep + 1), cudaMemcpyHostToDevice, st.s));
    PETB_CUDA(cudaMemcpyAsync(d_aold, atom_old.data(), 4 * size_t(n_keep), cudaMemcpyHostToDevice, st.s));
    PETB_CUDA(cudaMemcpyAsync(d_slot, slot_of_atom.data(), 4 * size_t(Nn), cudaMemcpyHostToDevice, st.s));
    PETB_CUDA(cudaMemcpyAsync(d_keep, keep, 4 * size_t(n_keep), cudaMemcpyHostToDevice, st.s));
    if (En) {
      k_reassemble_pairs<<<cdiv(En, 256), 256, 0, st.s>>>(r, c.ref, d_enew, d_eold, d_anew, d_aold, n_keep, En);
      PETB_LAUNCH_CHECK(st);
    }
    k_reassemble_offsets<<<cdiv(Nn + 1, 256), 256, 0, st.s>>>(r.off, c.ref.off, d_map, d_slot, d_enew, d_eold, Nn, En);
    PETB_LAUNCH_CHECK(st);
    k_gather_rows_f64<<<cdiv(3 * size_t(Nn), 256), 256, 0, st.s>>>(next.pos0, c.pos0, d_map, Nn, 3);
    PETB_LAUNCH_CHECK(st);
    k_gather_rows_f64<<<cdiv(9 * size_t(n_keep), 256), 256, 0, st.s>>>(next.cinv0, c.cinv0, d_keep, n_keep, 9);
    PETB_LAUNCH_CHECK(st);
    next.ref = r, next.valid = true, next.searches = c.searches, next.reuses = c.reuses;
  }
  PETB_CUDA(cudaStreamSynchronize(st.s));
  // stage the kept structures again from what the host knows of them and the positions just read
  std::vector<int> z_of_species(ckpt.n_species > 0 ? ckpt.n_species : 1, 0);
  for (int Z = int(ckpt.species_to_index.size()) - 1; Z >= 0; --Z)
    if (ckpt.species_to_index[Z] >= 0 && ckpt.species_to_index[Z] < int(z_of_species.size())) z_of_species[ckpt.species_to_index[Z]] = Z;
  std::vector<int> numbers(Nn > 0 ? Nn : 1);
  for (int i = 0; i < Nn; ++i) numbers[i] = z_of_species[h_species[atom_map[i]]];
  std::vector<pet_system> sys(n_keep);
  for (int k = 0; k < n_keep; ++k) {
    const int b = keep[k];
    pet_system& s = sys[k];
    s = pet_system{};
    s.n_atoms = h_natoms[b], s.atomic_numbers = numbers.data() + atom_new[k], s.positions = pos.data() + 3 * size_t(atom_new[k]);
    for (int e = 0; e < 9; ++e) s.cell[e] = h_cells[size_t(b) * 9 + e];
    for (int d = 0; d < 3; ++d) s.pbc[d] = (h_per[b] >> d) & 1;
    s.spin_multiplicity = 1;
  }
  const long long searches = verlet.searches, reuses = verlet.reuses;
  stage(sys.data(), n_keep, false);
  if (follow) {
    cache_arena.swap(cache_spare);  // the new pairs' pool becomes the cache's; the old one is spare from now on
    verlet = next;
  }
  verlet.searches = searches, verlet.reuses = reuses;
}

void Engine::update_staged(const double* positions, const double* cells) {
  PETB_CUDA(cudaSetDevice(device));
  if (geom.Ntot == 0 && geom.B == 0) throw Error(3, "pet: nothing is staged");
  if (positions)
    PETB_CUDA(cudaMemcpyAsync(geom.pos, positions, sizeof(double) * 3 * size_t(geom.Ntot), cudaMemcpyHostToDevice, st.s));
  if (cells) {
    const int B = geom.B;
    std::vector<double> hc(size_t(B) * 18);
    std::vector<int> gi(size_t(B) * 7 + 1);
    int bins = 0;
    for (int b = 0; b < B; ++b) {
      for (int e = 0; e < 9; ++e) h_cells[size_t(b) * 9 + e] = hc[size_t(b) * 9 + e] = cells[size_t(b) * 9 + e];
      invert_cell(cells + size_t(b) * 9, hc.data() + size_t(B) * 9 + size_t(b) * 9);
      grid_for_cell(cells + size_t(b) * 9, h_per[b], h_natoms[b], ckpt.hypers.cutoff, gi.data() + 3 * b, gi.data() + 3 * B + 3 * b);
      gi[6 * B + b] = bins;
      bins += gi[3 * b] * gi[3 * b + 1] * gi[3 * b + 2];
    }
    gi[7 * B] = bins;
    geom.nbins = bins;
    PETB_CUDA(cudaMemcpyAsync(geom.scell, hc.data(), sizeof(double) * 18 * size_t(B), cudaMemcpyHostToDevice, st.s));
    PETB_CUDA(cudaMemcpyAsync(geom.gnc, gi.data(), sizeof(int) * (7 * size_t(B) + 1), cudaMemcpyHostToDevice, st.s));
  }
  PETB_CUDA(cudaStreamSynchronize(st.s));
}

// ---- one evaluation -----------------------------------------------------------------

void Engine::drop_graphs() {
  for (auto& g : graph_cache)
    if (g.exec) cudaGraphExecDestroy(g.exec);
  graph_cache.clear();
  graph_seen.clear();
}

// One pass of the network over packed edges: eagerly, or as a recorded CUDA graph once the same shapes and
// buffers have been seen before (eager first, capture second, replay after). The key holds everything the
// recorded launches depend on besides the weights: shapes, the input pointers, and the pools' generations.
// What a pass may keep: the tier asked for, or under Auto the first one whose estimate fits the budget (the given
// one, else nine tenths of what the device has free plus what the pools already hold).
RunOptions Engine::run_options() const {
  RunOptions o;
  o.recompute = recompute, o.tier_floor = tier_floor;
  o.budget = memory_budget;
  if (o.budget == 0 && recompute == RECOMPUTE_AUTO) {
    size_t free_b = 0, total_b = 0;
    if (device_memory(&free_b, &total_b)) {
      const double pool = double(save_arena.capacity() + tmp_arena.capacity());
      o.budget = size_t(std::min(double(free_b) + pool, double(total_b)) * 0.9);
    }
  }
  return o;
}

// What the device has free, asked of the driver only when this engine's pools have changed size since the last
// answer. cudaMemGetInfo goes into the kernel-mode driver, where it queues behind whoever else is talking to it
// (a monitoring agent's NVML polls, nvidia-smi): asked at every evaluation it held one 20 ms step in ten or so up for
// 50-100 ms on a shared box, the GPU idle meanwhile. Between two evaluations of the same shapes nothing this engine
// does changes the answer.
bool Engine::device_memory(size_t* free_b, size_t* total_b) const {
  const size_t pools = save_arena.capacity() + tmp_arena.capacity() + nbr_arena.capacity() + cache_arena.capacity() +
                       cache_spare.capacity() + session_arena.capacity() + geom_arena.capacity();
  if (!mem_known || pools != mem_pools) {
    ++mem_queries;
    if (cudaMemGetInfo(&mem_free, &mem_total) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    mem_known = true, mem_pools = pools;
  }
  *free_b = mem_free, *total_b = mem_total;
  return true;
}

void Engine::run_model(const PackedEdges& pk, bool forces) {
  taps.clear();
  const RunOptions ro = run_options();
  const int tier = model->hypers().feedforward && forces ? model->choose_tier(ro, pk.N, pk.E) : int(RECOMPUTE_NEVER);
  RunOptions fixed = ro;  // the tier is part of a recorded pass's key: run exactly the one chosen here
  fixed.recompute = tier;
  if (model->hypers().feedforward && forces) {  // size both pools for the pass before it starts
    const MemoryNeed need = model->memory_need(tier, pk.N, pk.E, pk.n_live);
    save_arena.reserve(need.save), tmp_arena.reserve(need.tmp);
  }
  // An exchanged list calls back into the engine in the middle of the pass: it is never recorded.
  const bool eager_only = !graphs || want_taps || prof.on || pk.exchange != nullptr;
  if (eager_only) {
    last_out = model->run(st, save_arena, tmp_arena, pk, forces, gemm_mode, want_taps ? &taps : nullptr, fixed);
    last_pk = pk, have_out = true;
    return;
  }
  auto ptr = [](const void* q) { return uint64_t(reinterpret_cast<uintptr_t>(q)); };
  const std::vector<uint64_t> key = {uint64_t(pk.N),      uint64_t(pk.E),     uint64_t(pk.M),       uint64_t(pk.B),
                                     uint64_t(pk.n_atoms), uint64_t(pk.n_local), uint64_t(forces),   uint64_t(gemm_mode) | (uint64_t(tier) << 8),
                                     ptr(pk.off),          ptr(pk.center),     ptr(pk.species),      ptr(pk.reverse),
                                     ptr(pk.vec),          ptr(pk.dist),       ptr(pk.cut),          ptr(pk.atom_species),
                                     ptr(pk.soff),         save_arena.generation(), tmp_arena.generation(),
                                     ptr(save_arena.alloc_bytes(0)),
                                     // the rest of what the recorded kernels read: the neighbour atoms, the maps between
                                     // packed and raw edges, and an adaptive cutoff's per-atom data and raw list
                                     ptr(pk.nbr),          ptr(pk.rc),         ptr(pk.raw_of),       ptr(pk.packed_of_raw),
                                     ptr(pk.sid),          ptr(pk.adaptive.acut), ptr(pk.adaptive.root), ptr(pk.adaptive.slope),
                                     ptr(pk.adaptive.eff), ptr(pk.adaptive.probes), uint64_t(pk.adaptive.P),
                                     uint64_t(pk.adaptive.n_atoms), uint64_t(pk.adaptive.raw.E), ptr(pk.adaptive.raw.i),
                                     ptr(pk.adaptive.raw.j), ptr(pk.adaptive.raw.vec), ptr(pk.adaptive.raw.dist),
                                     ptr(pk.adaptive.raw.off), ptr(pk.adaptive.raw.reverse)};
  for (auto& g : graph_cache)
    if (g.key == key) {
      PETB_CUDA(cudaGraphLaunch(g.exec, st.s));
      st.launches += g.launches;
      ++graph_replays;
      g.stamp = ++graph_clock;
      save_arena.rewind(g.save_after), tmp_arena.rewind(g.tmp_after);
      last_out = g.out, last_pk = pk, have_out = true;
      return;
    }
  bool seen = false;
  for (auto& k : graph_seen) seen = seen || k == key;
  if (!seen) {  // first time: eagerly (the pools may still grow, which a capture cannot contain)
    if (graph_seen.size() >= 32) graph_seen.erase(graph_seen.begin());
    graph_seen.push_back(key);
    last_out = model->run(st, save_arena, tmp_arena, pk, forces, gemm_mode, nullptr, fixed);
    last_pk = pk, have_out = true;
    return;
  }
  GraphEntry g;
  g.key = key;
  const long long before = st.launches;
  const uint64_t gen_s = save_arena.generation(), gen_t = tmp_arena.generation();
  cudaGraph_t graph = nullptr;
  PETB_CUDA(cudaStreamBeginCapture(st.s, cudaStreamCaptureModeRelaxed));
  try {
    g.out = model->run(st, save_arena, tmp_arena, pk, forces, gemm_mode, nullptr, fixed);
  } catch (...) {
    cudaStreamEndCapture(st.s, &graph);
    if (graph) cudaGraphDestroy(graph);
    throw;
  }
  PETB_CUDA(cudaStreamEndCapture(st.s, &graph));
  g.launches = st.launches - before;
  g.save_after = save_arena.mark(), g.tmp_after = tmp_arena.mark();
  if (gen_s != save_arena.generation() || gen_t != tmp_arena.generation()) {
    // A pool grew during the capture (it should not, after the eager pass): do not keep the recording.
    cudaGraphDestroy(graph);
    throw Error(3, "pet: the scratch pool grew while a pass was being recorded");
  }
  const cudaError_t ie = cudaGraphInstantiate(&g.exec, graph, 0);
  cudaGraphDestroy(graph);
  if (ie != cudaSuccess) throw Error(5, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(ie));
  PETB_CUDA(cudaGraphLaunch(g.exec, st.s));
  g.stamp = ++graph_clock;
  if (graph_cache.size() >= 8) {  // least recently used out
    size_t lru = 0;
    for (size_t i = 1; i < graph_cache.size(); ++i)
      if (graph_cache[i].stamp < graph_cache[lru].stamp) lru = i;
    cudaGraphExecDestroy(graph_cache[lru].exec);
    graph_cache.erase(graph_cache.begin() + lru);
  }
  last_out = g.out, last_pk = pk, have_out = true;
  graph_cache.push_back(g);
}

void Engine::compute_staged(bool forces) {
  PETB_CUDA(cudaSetDevice(device));
  have_out = false;
  PETB_CUDA(cudaStreamSynchronize(st.s));
  nbr_arena.reset();
  save_arena.reset();
  tmp_arena.reset();
  PETB_CUDA(cudaEventRecord(ev0, st.s));
  const Geom& g = geom;
  RawEdges re;
  if (cache_neighbors) {
    re = cached_edges();
  } else {
    posw = nbr_arena.alloc<double>(3 * size_t(g.Ntot > 0 ? g.Ntot : 1));
    wrap_positions(st, g, posw);
    re = cell_list_search(st, nbr_arena, g, posw, ckpt.hypers.cutoff);
    find_reverse(st, re, g.Ntot);
  }
  const CutoffSpec cs = model->cutoff_spec();
  const AdaptiveCut ad = adaptive_cutoffs(st, nbr_arena, re, g.Ntot, cs);
  PackedEdges pk = pack_edges(st, nbr_arena, re, g.Ntot, g.spec, cs, pinned, ad);
  pk.n_atoms = g.Ntot, pk.n_local = g.Ntot, pk.B = g.B, pk.sid = g.sid, pk.soff = g.soff;
  last_B = g.B, last_N = g.Ntot;
  peak_slots = std::max(peak_slots, double(g.Ntot) * double(pk.M + 1));
  if (g.Ntot > 0 && g.B > 0) run_model(pk, forces);
  else last_pk = pk;
  PETB_CUDA(cudaEventRecord(ev1, st.s));
}

// The staged batch's pairs from the Verlet cache (cached_edges, src/device_geometry.cpp:262-352): one readback
// decides between the cached pairs and a new search to cutoff + skin; either way the pairs' vectors come from the
// positions and cells as they are now, and the packing drops those past the cutoff as it does for an engine's list.
RawEdges Engine::cached_edges() {
  const Geom& g = geom;
  VerletCache& c = verlet;
  const int N = g.Ntot, B = g.B;
  const double reach = ckpt.hypers.cutoff + VerletCache::kSkin;
  bool again = !c.valid;
  if (!again && N > 0) {
    verlet_check(st, g, c.pos0, c.cinv0, reach, c.worst);
    double* h = reinterpret_cast<double*>(pinned + 16);
    PETB_CUDA(cudaMemcpyAsync(h, c.worst, sizeof(double), cudaMemcpyDeviceToHost, st.s));
    PETB_CUDA(cudaStreamSynchronize(st.s));
    again = !(*h < VerletCache::kSkin);
  }
  if (again) {
    // the bins for the longer reach, chosen on the host from the staged cells as staging chooses the model's
    std::vector<int> gi(7 * size_t(B) + 1);
    int bins = 0;
    for (int b = 0; b < B; ++b) {
      grid_for_cell(h_cells.data() + 9 * size_t(b), h_per[b], h_natoms[b], reach, gi.data() + 3 * b, gi.data() + 3 * B + 3 * b);
      gi[6 * size_t(B) + b] = bins;
      bins += gi[3 * b] * gi[3 * b + 1] * gi[3 * b + 2];
    }
    gi[7 * size_t(B)] = bins;
    Geom gr = g;
    gr.gnc = nbr_arena.alloc<int>(7 * size_t(B) + 1);
    gr.gnr = gr.gnc + 3 * B, gr.goff = gr.gnr + 3 * B, gr.nbins = bins;
    PETB_CUDA(cudaMemcpyAsync(gr.gnc, gi.data(), sizeof(int) * gi.size(), cudaMemcpyHostToDevice, st.s));
    PETB_CUDA(cudaStreamSynchronize(st.s));  // gi leaves scope
    posw = nbr_arena.alloc<double>(3 * size_t(N > 0 ? N : 1));
    wrap_positions(st, gr, posw);
    const RawEdges found = cell_list_search(st, nbr_arena, gr, posw, reach);
    find_reverse(st, found, N);
    cache_arena.reset();
    const size_t E = found.E, Ea = E > 0 ? E : 1, Na = N > 0 ? N : 1;
    RawEdges r;
    r.E = found.E;
    r.i = cache_arena.alloc<int>(Ea), r.j = cache_arena.alloc<int>(Ea), r.shift = cache_arena.alloc<int>(3 * Ea);
    r.vec = cache_arena.alloc<double>(3 * Ea), r.dist = cache_arena.alloc<double>(Ea);
    r.off = cache_arena.alloc<int>(size_t(N) + 1), r.reverse = cache_arena.alloc<int>(Ea);
    c.pos0 = cache_arena.alloc<double>(3 * Na), c.cinv0 = cache_arena.alloc<double>(9 * size_t(B > 0 ? B : 1));
    c.worst = cache_arena.alloc<double>(1);
    PETB_CUDA(cudaMemcpyAsync(r.off, found.off, 4 * (size_t(N) + 1), cudaMemcpyDeviceToDevice, st.s));
    if (E) {
      PETB_CUDA(cudaMemcpyAsync(r.i, found.i, 4 * E, cudaMemcpyDeviceToDevice, st.s));
      PETB_CUDA(cudaMemcpyAsync(r.j, found.j, 4 * E, cudaMemcpyDeviceToDevice, st.s));
      PETB_CUDA(cudaMemcpyAsync(r.reverse, found.reverse, 4 * E, cudaMemcpyDeviceToDevice, st.s));
      unwrap_shifts(st, found, g, r.shift);
    }
    if (N) PETB_CUDA(cudaMemcpyAsync(c.pos0, g.pos, 24 * size_t(N), cudaMemcpyDeviceToDevice, st.s));
    if (B) PETB_CUDA(cudaMemcpyAsync(c.cinv0, g.cinv, 72 * size_t(B), cudaMemcpyDeviceToDevice, st.s));
    c.ref = r, c.valid = true, ++c.searches;
  } else {
    ++c.reuses;
  }
  edge_vectors_batch(st, c.ref, g);
  return c.ref;
}

void Engine::fetch(pet_results* out) {
  PETB_CUDA(cudaSetDevice(device));
  if (!out) throw Error(2, "pet: no results struct given");
  const int B = last_B, N = last_N;
  if (have_out) {
    const PassOut& o = last_out;
    if (out->energy) PETB_CUDA(cudaMemcpyAsync(out->energy, o.f.energy, sizeof(double) * B, cudaMemcpyDeviceToHost, st.s));
    if (out->per_atom_energy)
      PETB_CUDA(cudaMemcpyAsync(out->per_atom_energy, o.per_atom, sizeof(double) * N, cudaMemcpyDeviceToHost, st.s));
    if (o.has_forces) {
      if (out->forces) PETB_CUDA(cudaMemcpyAsync(out->forces, o.f.forces, sizeof(double) * 3 * N, cudaMemcpyDeviceToHost, st.s));
      if (out->virial) PETB_CUDA(cudaMemcpyAsync(out->virial, o.f.vir6, sizeof(double) * 6 * B, cudaMemcpyDeviceToHost, st.s));
    }
    if (out->struct_id && last_pk.sid)
      PETB_CUDA(cudaMemcpyAsync(out->struct_id, last_pk.sid, sizeof(int) * N, cudaMemcpyDeviceToHost, st.s));
  }
  PETB_CUDA(cudaStreamSynchronize(st.s));
  float ms = 0.f;
  if (cudaEventElapsedTime(&ms, ev0, ev1) == cudaSuccess) last_ms = ms;
  if (gemm_mode != GEMM_NATIVE && gemm_tensor_error(st))
    throw Error(5, "pet: a tensor-core GEMM gave up waiting on its pipeline; the results of this evaluation are invalid");
}

// How many neighbours an atom of this structure has, roughly: the density times the cutoff sphere for a periodic
// structure, every other atom for a small one (the reference's neighbors_estimate).
static double neighbors_estimate(const pet_system& s, double cutoff) {
  const double all = s.n_atoms > 1 ? double(s.n_atoms - 1) : 1.0;
  if (!(s.pbc[0] || s.pbc[1] || s.pbc[2])) return all;
  const double* c = s.cell;
  const double vol = std::fabs(c[0] * (c[4] * c[8] - c[5] * c[7]) - c[1] * (c[3] * c[8] - c[5] * c[6]) +
                               c[2] * (c[3] * c[7] - c[4] * c[6]));
  if (!(vol > 1e-9)) return all;
  const double est = 4.18879020478639 * cutoff * cutoff * cutoff * double(s.n_atoms) / vol;
  return est > 1.0 ? est : 1.0;
}

std::vector<std::pair<int, int>> Engine::memory_runs(const pet_system* systems, int B) const {
  const Hypers& h = ckpt.hypers;
  const double pool = double(save_arena.capacity() + tmp_arena.capacity() + nbr_arena.capacity());
  // bytes per edge slot: measured once an evaluation of some size has run, else from the widths of what a pass saves
  // (about 64 floats of d_pet per token row of a 2 x 2 model), a quarter more for what else the pools hold
  const double blocks = double(h.num_gnn_layers) * double(h.num_attention_layers);
  const double estimate = 1.25 * 4.0 * double(h.d_pet) * (12.0 * blocks + 8.0 * h.num_gnn_layers);
  const double per_slot = (pool > 0.0 && peak_slots >= 4096.0) ? pool / peak_slots : estimate;
  double budget = double(memory_budget);
  if (memory_budget == 0) {
    size_t free_b = 0, total_b = 0;
    if (!device_memory(&free_b, &total_b)) free_b = total_b = size_t(64) << 30;
    budget = std::min(double(free_b) + pool, double(total_b)) * 0.9;
  }
  const double cap = budget / per_slot;
  const long max_atoms = max_batch_atoms > 0 ? max_batch_atoms : (1L << 40);
  std::vector<std::pair<int, int>> runs;
  int b0 = 0;
  long atoms = 0;
  double m = 0.0;
  for (int i = 0; i < B; ++i) {
    const long a = systems[i].n_atoms;
    const double mi = std::max(m, neighbors_estimate(systems[i], h.cutoff));
    if (i > b0 && (double(atoms + a) * (mi + 1.0) > cap || atoms + a > max_atoms)) {
      runs.emplace_back(b0, i);
      b0 = i, atoms = 0, m = 0.0;
    }
    atoms += a;
    m = std::max(m, neighbors_estimate(systems[i], h.cutoff));
  }
  runs.emplace_back(b0, B);
  return runs;
}

void Engine::compute_runs(const pet_system* systems, int B, const std::vector<std::pair<int, int>>& runs, bool forces,
                          pet_results* out) {
  if (runs.size() == 1) {
    stage(systems, B, true);
    compute_staged(forces);
    fetch(out);
    return;
  }
  // A batch too large for the device: consecutive pieces, the results in order, struct_id counted over the whole
  // batch (Calculator::compute, src/calculator.cpp:589-624).
  if (!out) throw Error(2, "pet: no results struct given");
  ++batch_splits;
  size_t a0 = 0;
  for (const auto& run : runs) {
    const int b0 = run.first, nb = run.second - run.first;
    size_t na = 0;
    for (int b = b0; b < run.second; ++b) na += size_t(systems[b].n_atoms);
    stage(systems + b0, nb, false);
    compute_staged(forces);
    pet_results piece{};
    piece.energy = out->energy ? out->energy + b0 : nullptr;
    piece.per_atom_energy = out->per_atom_energy ? out->per_atom_energy + a0 : nullptr;
    piece.forces = out->forces ? out->forces + 3 * a0 : nullptr;
    piece.virial = out->virial ? out->virial + 6 * size_t(b0) : nullptr;
    piece.struct_id = out->struct_id ? out->struct_id + a0 : nullptr;
    fetch(&piece);
    if (piece.struct_id && have_out)
      for (size_t i = 0; i < na; ++i) piece.struct_id[i] += b0;
    a0 += na;
  }
  last_B = B, last_N = int(a0);
}

// Out of device memory is recovered from where that can help (the reference drops a recompute tier, releases its
// pool and retries, src/model.cpp:952-971): the pools are released, so that the next pass allocates one block of
// the size it needs instead of growing in steps, and a batch is cut into pieces half the size; three rounds of
// that, then the error goes to the caller with what the pools held.
void Engine::compute(const pet_system* systems, int B, bool forces, pet_results* out) {
  if (B < 0 || (B > 0 && !systems)) throw Error(2, "pet: no systems given");
  for (int b = 0; b < B; ++b)
    if (systems[b].n_atoms < 0) throw Error(2, "pet: negative atom count");
  auto runs = B > 1 ? memory_runs(systems, B) : std::vector<std::pair<int, int>>{{0, B}};
  for (int round = 0;; ++round) {
    try {
      compute_runs(systems, B, runs, forces, out);
      return;
    } catch (const Error& e) {
      if (e.code != 4 || round == 3) {
        if (e.code != 4) throw;
        throw Error(4, std::string(e.what()) + " (pet: out of device memory after " + std::to_string(round) +
                           " retries; the pools held " + std::to_string((save_arena.capacity() + tmp_arena.capacity() +
                           nbr_arena.capacity()) >> 20) + " MiB, the batch was cut into " + std::to_string(runs.size()) +
                           " pieces)");
      }
      cudaGetLastError();  // the failed allocation leaves its error behind
      PETB_CUDA(cudaDeviceSynchronize());
      drop_graphs();       // they replay into pool addresses
      graph_seen.clear();
      have_out = false, verlet.valid = false;
      save_arena.release(), tmp_arena.release(), nbr_arena.release(), cache_arena.release(), cache_spare.release();
      ++oom_recoveries;
      // one structure cannot be cut: keep less of its forward instead (the reference's tier drop, src/model.cpp:952-971)
      bool cuttable = false;
      for (const auto& r : runs) cuttable = cuttable || r.second - r.first > 1;
      if (!cuttable && recompute == RECOMPUTE_AUTO && model->hypers().feedforward && tier_floor < RECOMPUTE_LAYERS) {
        tier_floor = std::max(tier_floor, model->last_tier()) + 1;
        continue;
      }
      std::vector<std::pair<int, int>> halved;
      for (const auto& r : runs) {
        const int n = r.second - r.first;
        if (n <= 1) {
          halved.push_back(r);
        } else {
          halved.emplace_back(r.first, r.first + n / 2);
          halved.emplace_back(r.first + n / 2, r.second);
        }
      }
      runs = halved;
    }
  }
}

void Engine::neighbor_list(const pet_system* systems, int B, pet_raw_edges* out) {
  if (!out) throw Error(2, "pet: no edge struct given");
  stage(systems, B);
  PETB_CUDA(cudaStreamSynchronize(st.s));
  nbr_arena.reset();
  const Geom& g = geom;
  posw = nbr_arena.alloc<double>(3 * size_t(g.Ntot > 0 ? g.Ntot : 1));
  wrap_positions(st, g, posw);
  RawEdges re = cell_list_search(st, nbr_arena, g, posw, ckpt.hypers.cutoff);
  find_reverse(st, re, g.Ntot);
  out->n_edges = re.E;
  if (re.E > out->capacity) throw Error(2, "pet: " + std::to_string(re.E) + " edges, above the given capacity");
  const size_t E = re.E;
  if (E) {
    if (out->i) PETB_CUDA(cudaMemcpyAsync(out->i, re.i, 4 * E, cudaMemcpyDeviceToHost, st.s));
    if (out->j) PETB_CUDA(cudaMemcpyAsync(out->j, re.j, 4 * E, cudaMemcpyDeviceToHost, st.s));
    if (out->shift) PETB_CUDA(cudaMemcpyAsync(out->shift, re.shift, 12 * E, cudaMemcpyDeviceToHost, st.s));
    if (out->vec) PETB_CUDA(cudaMemcpyAsync(out->vec, re.vec, 24 * E, cudaMemcpyDeviceToHost, st.s));
    if (out->dist) PETB_CUDA(cudaMemcpyAsync(out->dist, re.dist, 8 * E, cudaMemcpyDeviceToHost, st.s));
    if (out->reverse) PETB_CUDA(cudaMemcpyAsync(out->reverse, re.reverse, 4 * E, cudaMemcpyDeviceToHost, st.s));
    if (out->cutoff) {
      CutoffSpec cs = model->cutoff_spec();
      cs.adaptive = 0;  // the raw list's own factors: the model's fixed cutoff
      PackedEdges pk = pack_edges(st, nbr_arena, re, g.Ntot, g.spec, cs, pinned);
      if (pk.E != re.E) throw Error(3, "pet: a raw edge lies past the cutoff");
      PETB_CUDA(cudaMemcpyAsync(out->cutoff, pk.cut, 4 * E, cudaMemcpyDeviceToHost, st.s));
    }
  }
  PETB_CUDA(cudaStreamSynchronize(st.s));
}

// ---- an engine's own list (EdgeSession, src/device_geometry.cpp:410-454,673-778) --------

void Engine::set_neighbors(const pet_edge_list* v) {
  PETB_CUDA(cudaSetDevice(device));
  if (!v || v->n_atoms < 0 || (v->n_atoms > 0 && (!v->offsets || !v->atomic_numbers)))
    throw Error(2, "pet: an edge list needs offsets and atomic numbers");
  const int N = v->n_atoms, L = N > 0 ? v->offsets[N] : 0;
  if (N >= (1 << 24)) throw Error(1, "pet: too many atoms for the edge key");
  const int n_own = v->n_local < 0 ? N : v->n_local;
  if (v->exchange) {  // ghosts one cutoff deep: they are neighbours only (src/device_geometry.cpp:679)
    if (v->half) throw Error(2, "pet: an exchanged list must be a full list");
    if (!v->exchange->set_live || !v->exchange->edges) throw Error(2, "pet: an exchange needs set_live and edges callbacks");
    if (n_own < N && v->offsets[N] != v->offsets[n_own]) throw Error(2, "pet: with an exchange, ghosts have no pairs of their own");
  }
  std::vector<int> sp(N);
  for (int i = 0; i < N; ++i) sp[i] = species_index(v->atomic_numbers[i]);
  // Directed edges grouped by centre: each atom's listed pairs, then the mirrors of the pairs that list it.
  std::vector<int> off(N + 1, 0);
  for (int i = 0; i < N; ++i) {
    off[i + 1] += v->offsets[i + 1] - v->offsets[i];
    if (v->half)
      for (int e = v->offsets[i]; e < v->offsets[i + 1]; ++e) ++off[v->neighbors[e] + 1];
  }
  for (int i = 0; i < N; ++i) off[i + 1] += off[i];
  const int E = off[N];
  std::vector<int> ri(E), rj(E), sh(3 * size_t(E), 0), cur(off.begin(), off.end() - 1);
  Session& s = md;
  s.src.assign(E, 0), s.dir.assign(E, 1);
  auto put = [&](int c, int n, int e, int sign) {
    const int k = cur[c]++;
    ri[k] = c, rj[k] = n, s.src[k] = e, s.dir[k] = sign;
    if (!v->shifts) return;
    for (int d = 0; d < 3; ++d) {
      sh[3 * size_t(k) + d] = sign * v->shifts[3 * size_t(e) + d];
      if (std::abs(sh[3 * size_t(k) + d]) > 15) throw Error(1, "pet: cell shift too large for the edge key");
    }
  };
  for (int i = 0; i < N; ++i)
    for (int e = v->offsets[i]; e < v->offsets[i + 1]; ++e) {
      if (v->neighbors[e] < 0 || v->neighbors[e] >= N) throw Error(2, "pet: a neighbour index is out of range");
      put(i, v->neighbors[e], e, 1);
    }
  if (v->half)
    for (int i = 0; i < N; ++i)
      for (int e = v->offsets[i]; e < v->offsets[i + 1]; ++e) put(v->neighbors[e], i, e, -1);

  PETB_CUDA(cudaStreamSynchronize(st.s));
  session_arena.reset();
  Arena& A = session_arena;
  const size_t Ea = E > 0 ? E : 1, Na = N > 0 ? N : 1;
  s.valid = false;
  s.n_atoms = N, s.n_local = v->n_local < 0 ? N : v->n_local, s.n_pairs = L, s.E = E;
  s.shifted = v->shifts != nullptr, s.half = v->half != 0;
  s.species = A.alloc<int>(Na);
  s.sid = A.alloc<int>(Na);
  s.soff = A.alloc<int>(2);
  s.pos = A.alloc<double>(3 * Na);
  s.cell = A.alloc<double>(9);
  s.re = RawEdges();
  s.re.E = E;
  s.re.i = A.alloc<int>(Ea), s.re.j = A.alloc<int>(Ea), s.re.shift = A.alloc<int>(3 * Ea);
  s.re.vec = A.alloc<double>(3 * Ea), s.re.dist = A.alloc<double>(Ea);
  s.re.off = A.alloc<int>(N + 1), s.re.reverse = A.alloc<int>(Ea);
  const int soff[2] = {0, N};
  PETB_CUDA(cudaMemcpyAsync(s.species, sp.data(), 4 * size_t(N), cudaMemcpyHostToDevice, st.s));
  PETB_CUDA(cudaMemsetAsync(s.sid, 0, 4 * Na, st.s));
  PETB_CUDA(cudaMemcpyAsync(s.soff, soff, 8, cudaMemcpyHostToDevice, st.s));
  PETB_CUDA(cudaMemsetAsync(s.cell, 0, 72, st.s));
  PETB_CUDA(cudaMemcpyAsync(s.re.off, off.data(), 4 * size_t(N + 1), cudaMemcpyHostToDevice, st.s));
  std::vector<int> rrev(E, -1);
  if (E) {
    PETB_CUDA(cudaMemcpyAsync(s.re.i, ri.data(), 4 * size_t(E), cudaMemcpyHostToDevice, st.s));
    PETB_CUDA(cudaMemcpyAsync(s.re.j, rj.data(), 4 * size_t(E), cudaMemcpyHostToDevice, st.s));
    PETB_CUDA(cudaMemcpyAsync(s.re.shift, sh.data(), 12 * size_t(E), cudaMemcpyHostToDevice, st.s));
    find_reverse(st, s.re, N);
    PETB_CUDA(cudaMemcpyAsync(rrev.data(), s.re.reverse, 4 * size_t(E), cudaMemcpyDeviceToHost, st.s));
  }
  PETB_CUDA(cudaStreamSynchronize(st.s));
  // Partnerless edges by target atom, each atom's in edge order.
  std::vector<int> ooff(N + 1, 0), oedge;
  for (int e = 0; e < E; ++e)
    if (rrev[e] < 0) ++ooff[rj[e] + 1];
  for (int i = 0; i < N; ++i) ooff[i + 1] += ooff[i];
  s.n_orphan = ooff[N];
  s.ooff = s.oedge = nullptr;
  if (s.n_orphan > 0) {
    oedge.resize(s.n_orphan);
    std::vector<int> at(ooff.begin(), ooff.end() - 1);
    for (int e = 0; e < E; ++e)
      if (rrev[e] < 0) oedge[at[rj[e]]++] = e;
    s.ooff = A.alloc<int>(N + 1), s.oedge = A.alloc<int>(s.n_orphan);
    PETB_CUDA(cudaMemcpyAsync(s.ooff, ooff.data(), 4 * size_t(N + 1), cudaMemcpyHostToDevice, st.s));
    PETB_CUDA(cudaMemcpyAsync(s.oedge, oedge.data(), 4 * size_t(s.n_orphan), cudaMemcpyHostToDevice, st.s));
    PETB_CUDA(cudaStreamSynchronize(st.s));
  }
  s.caps_valid = false, s.e_cap = s.m_cap = 0;
  s.overflow = A.alloc<int>(1);
  PETB_CUDA(cudaMemsetAsync(s.overflow, 0, sizeof(int), st.s));
  s.has_exchange = v->exchange != nullptr;
  s.n_remote = 0, s.remote_raw = nullptr, s.renumber = nullptr;
  if (s.has_exchange) {
    s.exchange = *v->exchange;
    std::vector<int> remote;
    for (int e = 0; e < E; ++e)
      if (rj[e] >= s.n_local) remote.push_back(e);
    s.n_remote = int(remote.size());
    s.remote_raw = A.alloc<int>(s.n_remote > 0 ? s.n_remote : 1);
    if (s.n_remote > 0) {
      PETB_CUDA(cudaMemcpyAsync(s.remote_raw, remote.data(), 4 * size_t(s.n_remote), cudaMemcpyHostToDevice, st.s));
      PETB_CUDA(cudaStreamSynchronize(st.s));
    }
  }
  s.valid = true;
}

namespace {

struct StepOut {
  double* eg_raw = nullptr;  // [E_raw,3] scaled edge gradients in the session's edge order
};

}  // namespace

static StepOut session_step(Engine& I, const double* positions, bool on_device, const double* cell, bool forces) {
  Session& s = I.md;
  Stream& st = I.st;
  if (!s.valid) throw Error(1, "pet: no neighbour list set");
  if (s.shifted && !cell) throw Error(1, "pet: an edge list with shifts needs the cell");
  PETB_CUDA(cudaStreamSynchronize(st.s));
  I.have_out = false;
  I.nbr_arena.reset();
  I.save_arena.reset();
  I.tmp_arena.reset();
  PETB_CUDA(cudaEventRecord(I.ev0, st.s));
  const int N = s.n_atoms;
  if (s.renumber && !on_device) throw Error(1, "pet: a renumbered list takes device positions");
  if (N && s.renumber) {
    k_renumber_positions<<<cdiv(N, 256), 256, 0, st.s>>>(s.pos, positions, s.renumber, N);
    PETB_LAUNCH_CHECK(st);
  } else if (N) {
    PETB_CUDA(cudaMemcpyAsync(s.pos, positions, 24 * size_t(N), on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, st.s));
  }
  if (cell) PETB_CUDA(cudaMemcpyAsync(s.cell, cell, 72, cudaMemcpyHostToDevice, st.s));
  edge_vectors(st, s.re, s.pos, s.cell);
  // With an exchange only the owned atoms are centres (token rows); ghosts are neighbours.
  const int NC = s.has_exchange ? s.n_local : N;
  const bool fixed = I.md_fixed && s.caps_valid && !s.has_exchange && N > 0;
  const CutoffSpec cs = I.model->cutoff_spec();
  if (cs.adaptive && s.has_exchange)
    throw Error(1, "pet: an adaptive cutoff over an exchange needs the per-atom moves (atoms_forward/atoms_reverse), which are not built");
  // every listed atom's adaptive cutoff from the pairs it lists (ghosts without pairs keep the model's reach)
  const AdaptiveCut ad = adaptive_cutoffs(st, I.nbr_arena, s.re, N, cs);
  PackedEdges pk;
  if (fixed) {  // nothing is read back: the shapes are the capacities, the overflow flag travels with the results
    pk = pack_edges_fixed(st, I.nbr_arena, s.re, NC, s.species, cs, s.e_cap, s.m_cap, s.pairs, s.overflow, ad);
  } else {
    pk = pack_edges(st, I.nbr_arena, s.re, NC, s.species, cs, I.pinned, ad);
    if (I.md_fixed && !s.has_exchange) {  // size the capacities with room to move (src/device_geometry.cpp:749-777)
      s.e_cap = pk.E + pk.E / 20 + 64, s.m_cap = pk.M + 2, s.pairs = pk.pairs, s.caps_valid = true;
      PETB_CUDA(cudaMemsetAsync(s.overflow, 0, sizeof(int), st.s));
    }
  }
  pk.n_atoms = N, pk.n_local = s.n_local, pk.B = 1, pk.sid = s.sid, pk.soff = s.soff;
  if (s.has_exchange) {
    Arena& A = I.nbr_arena;
    const int R = s.n_remote, Ra = R > 0 ? R : 1;
    int* flag = A.alloc<int>(Ra + 1);
    int* at = A.alloc<int>(Ra + 1);
    int* live = A.alloc<int>(Ra);
    int* live_packed = A.alloc<int>(Ra);
    int* remote_of = A.alloc<int>(pk.E > 0 ? pk.E : 1);
    PETB_CUDA(cudaMemsetAsync(remote_of, 0xFF, 4 * size_t(pk.E > 0 ? pk.E : 1), st.s));
    int n_live = 0;
    if (R > 0) {
      k_live_flag<<<cdiv(R, 256), 256, 0, st.s>>>(flag, s.remote_raw, pk.packed_of_raw, R);
      PETB_LAUNCH_CHECK(st);
      exclusive_scan(st, A, flag, at, R);
      k_live_fill<<<cdiv(R, 256), 256, 0, st.s>>>(live, live_packed, remote_of, at, s.remote_raw, pk.packed_of_raw, R);
      PETB_LAUNCH_CHECK(st);
      PETB_CUDA(cudaMemcpyAsync(I.pinned, at + R, sizeof(int), cudaMemcpyDeviceToHost, st.s));
      PETB_CUDA(cudaStreamSynchronize(st.s));
      n_live = I.pinned[0];
    }
    pk.n_live = n_live, pk.live_packed = live_packed, pk.remote_of = remote_of, pk.exchange = &s.exchange;
    if (s.exchange.set_live(s.exchange.user, live, n_live, static_cast<void*>(st.s)) != 0)
      throw Error(1, "pet: the exchange's set_live() failed");
    order_after_legacy_stream(st);
  }
  I.last_B = 1, I.last_N = N;
  StepOut so;
  if (N == 0) return so;
  I.run_model(pk, forces);
  if (forces && s.E > 0) {
    so.eg_raw = I.save_arena.alloc<double>(3 * size_t(s.E));
    k_raw_edge_grad<<<cdiv(s.E, 256), 256, 0, st.s>>>(so.eg_raw, I.last_out.f.edge_grad, pk.packed_of_raw, s.E,
                                                      I.model->energy_scale());
    PETB_LAUNCH_CHECK(st);
    if (I.last_out.f.adaptive_gmag) {  // the adaptive cutoff's radial share, on every listed pair (src/forces.cpp:198-203)
      k_add_radial<<<cdiv(s.E, 256), 256, 0, st.s>>>(so.eg_raw, I.last_out.f.adaptive_gmag, s.re.vec, s.E);
      PETB_LAUNCH_CHECK(st);
    }
    if (s.n_orphan > 0) {
      k_orphan_forces<<<cdiv(N, 256), 256, 0, st.s>>>(I.last_out.f.forces, so.eg_raw, s.ooff, s.oedge, N);
      PETB_LAUNCH_CHECK(st);
    }
  }
  PETB_CUDA(cudaEventRecord(I.ev1, st.s));
  return so;
}

// True when the latest fixed-shape step outgrew its capacities: they are dropped, and the caller redoes the step,
// which then runs with the shapes read back and sizes new ones.
static bool fixed_step_overflowed(Engine& I) {
  Session& s = I.md;
  if (!I.md_fixed || !s.caps_valid || s.has_exchange || !s.overflow) return false;
  PETB_CUDA(cudaMemcpyAsync(I.pinned + 8, s.overflow, sizeof(int), cudaMemcpyDeviceToHost, I.st.s));
  PETB_CUDA(cudaStreamSynchronize(I.st.s));
  if (I.pinned[8] == 0) return false;
  s.caps_valid = false;
  return true;
}

void Engine::compute_step(const double* positions, const double* cell, bool forces, bool edge_gradients, pet_results* out) {
  PETB_CUDA(cudaSetDevice(device));
  if (!positions && md.n_atoms > 0) throw Error(2, "pet: no positions given");
  StepOut so = session_step(*this, positions, false, cell, forces);
  if (fixed_step_overflowed(*this)) so = session_step(*this, positions, false, cell, forces);
  std::vector<double> g;
  if (forces && edge_gradients && out && out->edge_gradient && so.eg_raw) {
    g.resize(3 * size_t(md.E));
    PETB_CUDA(cudaMemcpyAsync(g.data(), so.eg_raw, 24 * size_t(md.E), cudaMemcpyDeviceToHost, st.s));
  }
  if (!out) return;  // the results stay on the device (pet_device_results_of): a caller that reduces them there
  fetch(out);
  if (forces && edge_gradients && out && out->edge_gradient) {
    // A half list's pair gets both directions: g(i -> j) - g(j -> i)  (src/calculator.cpp:689-699).
    std::fill(out->edge_gradient, out->edge_gradient + 3 * size_t(md.n_pairs), 0.0);
    for (size_t e = 0; e < g.size() / 3; ++e)
      for (int c = 0; c < 3; ++c) out->edge_gradient[size_t(md.src[e]) * 3 + c] += md.dir[e] * g[e * 3 + c];
  }
}

void Engine::compute_step_device(const pet_device_arrays* a, const double* cell, pet_totals* totals) {
  PETB_CUDA(cudaSetDevice(device));
  if (!a || !a->positions) throw Error(2, "pet: no device positions given");
  const bool forces = a->forces != nullptr;
  const int N = md.n_atoms;
  pet_totals t{};
  for (int attempt = 0; attempt < 2; ++attempt) {
    const StepOut so = session_step(*this, a->positions, true, cell, forces);
    if (!(have_out && N > 0)) break;
    // the adds are skipped on the device when a fixed-shape step did not fit: that step is redone below
    const int* skip = (md_fixed && md.caps_valid && !md.has_exchange) ? md.overflow : nullptr;
    k_add_arrays<<<cdiv(N, 256), 256, 0, st.s>>>(a->forces, last_out.f.forces, a->per_atom_energy, last_out.per_atom, N, skip);
    PETB_LAUNCH_CHECK(st);
    if (a->per_atom_virial && forces && so.eg_raw) {
      k_atom_virial<<<cdiv(N, 256), 256, 0, st.s>>>(a->per_atom_virial, so.eg_raw, md.re.vec, md.re.off, md.re.reverse,
                                                    md.n_orphan > 0 ? md.ooff : nullptr, md.oedge, N, 0.5 * a->virial_scale, skip);
      PETB_LAUNCH_CHECK(st);
    }
    double* h = reinterpret_cast<double*>(pinned + 16);
    PETB_CUDA(cudaMemcpyAsync(h, last_out.f.energy, 8, cudaMemcpyDeviceToHost, st.s));
    if (forces) PETB_CUDA(cudaMemcpyAsync(h + 1, last_out.f.vir6, 48, cudaMemcpyDeviceToHost, st.s));
    if (skip) PETB_CUDA(cudaMemcpyAsync(pinned + 8, md.overflow, sizeof(int), cudaMemcpyDeviceToHost, st.s));
    PETB_CUDA(cudaStreamSynchronize(st.s));
    // a tensor-core GEMM that gave up on a wait left garbage behind, and the adds above have put it into the caller's arrays
    if (gemm_mode != GEMM_NATIVE && gemm_tensor_error(st))
      throw Error(5, "pet: a tensor-core GEMM gave up waiting on its pipeline; the arrays this step added into are invalid");
    if (skip && pinned[8] != 0) {  // outgrown: drop the capacities and run the step again, read back and resized
      md.caps_valid = false;
      continue;
    }
    t.energy = h[0];
    if (forces)
      for (int k = 0; k < 6; ++k) t.virial[k] = h[1 + k];
    break;
  }
  if (totals) *totals = t;
}

// An engine's full list in device memory (EdgeSession::set(DeviceEdgeListView), src/device_geometry.cpp:456-545).
// As for the flat pair list, the list comes to the host once per set (the counts first, then the neighbours
// gathered dense by a kernel) and goes through the host list's path; every step stays on the device.
void Engine::set_neighbors_device(const pet_device_edge_list* v) {
  PETB_CUDA(cudaSetDevice(device));
  if (!v || v->n_atoms < 0 || v->n_centres < 0) throw Error(2, "pet: no edge list given");
  const int N = v->n_atoms, NC = v->n_centres;
  if (N > 0 && !v->atomic_numbers) throw Error(2, "pet: an edge list needs atomic numbers");
  if (NC > 0 && (!v->ilist || !v->numneigh || !v->neighbors)) throw Error(2, "pet: an edge list needs ilist, numneigh and neighbors");
  if (N >= (1 << 24)) throw Error(1, "pet: too many atoms for the edge key");
  if (v->image_of && (!v->cell || !v->positions)) throw Error(1, "pet: images need the positions and the cell");
  const long si = v->stride_i, sk = v->stride_k ? v->stride_k : 1;
  const int mask = v->mask ? v->mask : ~0;
  PETB_CUDA(cudaStreamSynchronize(st.s));
  tmp_arena.reset();
  std::vector<int> ilist(NC), numneigh(N), z(N), image(v->image_of ? N : 0);
  std::vector<double> x(v->image_of ? 3 * size_t(N) : 0);
  if (NC) PETB_CUDA(cudaMemcpyAsync(ilist.data(), v->ilist, 4 * size_t(NC), cudaMemcpyDeviceToHost, st.s));
  if (N) {
    PETB_CUDA(cudaMemcpyAsync(numneigh.data(), v->numneigh, 4 * size_t(N), cudaMemcpyDeviceToHost, st.s));
    PETB_CUDA(cudaMemcpyAsync(z.data(), v->atomic_numbers, 4 * size_t(N), cudaMemcpyDeviceToHost, st.s));
    if (v->image_of) {
      PETB_CUDA(cudaMemcpyAsync(image.data(), v->image_of, 4 * size_t(N), cudaMemcpyDeviceToHost, st.s));
      PETB_CUDA(cudaMemcpyAsync(x.data(), v->positions, 24 * size_t(N), cudaMemcpyDeviceToHost, st.s));
    }
  }
  PETB_CUDA(cudaStreamSynchronize(st.s));
  // the centres' counts, in ilist order for the gather and in atom order for the list
  std::vector<int> coff(size_t(NC) + 1, 0), off(size_t(N) + 1, 0);
  for (int ii = 0; ii < NC; ++ii) {
    const int i = ilist[ii];
    if (i < 0 || i >= N || numneigh[i] < 0) throw Error(2, "pet: a centre of the list is not one of its atoms");
    coff[ii + 1] = coff[ii] + numneigh[i];
    off[i + 1] = numneigh[i];
  }
  for (int i = 0; i < N; ++i) off[i + 1] += off[i];
  const int E = off[N];
  if (E != coff[NC]) throw Error(2, "pet: a centre is listed twice");
  std::vector<int> dense(E), nb(E), sh;
  if (E) {
    int* d_off = tmp_arena.alloc<int>(size_t(NC) + 1);
    int* d_dense = tmp_arena.alloc<int>(E);
    PETB_CUDA(cudaMemcpyAsync(d_off, coff.data(), 4 * (size_t(NC) + 1), cudaMemcpyHostToDevice, st.s));
    k_dense_neighbors<<<cdiv(size_t(NC) * 32, 256), 256, 0, st.s>>>(d_dense, v->ilist, d_off, v->neighbors, si, sk, mask, NC);
    PETB_LAUNCH_CHECK(st);
    PETB_CUDA(cudaMemcpyAsync(dense.data(), d_dense, 4 * size_t(E), cudaMemcpyDeviceToHost, st.s));
    PETB_CUDA(cudaStreamSynchronize(st.s));
  }
  for (int ii = 0; ii < NC; ++ii)  // ilist order -> atom order
    std::copy(dense.begin() + coff[ii], dense.begin() + coff[ii + 1], nb.begin() + off[ilist[ii]]);
  for (int e = 0; e < E; ++e)
    if (nb[e] < 0 || nb[e] >= N) throw Error(2, "pet: a neighbour index is out of range");
  if (v->image_of) {  // each neighbour becomes the owned atom it is an image of, with the shift between them
    double inv[9];
    invert_cell(v->cell, inv);
    const double* c = v->cell;
    const double det = c[0] * (c[4] * c[8] - c[5] * c[7]) - c[1] * (c[3] * c[8] - c[5] * c[6]) + c[2] * (c[3] * c[7] - c[4] * c[6]);
    if (std::fabs(det) < 1e-12) throw Error(1, "pet: images need a cell with volume");
    sh.assign(3 * size_t(E), 0);
    for (int e = 0; e < E; ++e) {
      const int j = nb[e], o = image[j];
      if (o < 0 || o >= N) throw Error(1, "pet: a neighbour is not an image of an owned atom");
      const double d0 = x[3 * size_t(j)] - x[3 * size_t(o)], d1 = x[3 * size_t(j) + 1] - x[3 * size_t(o) + 1],
                   d2 = x[3 * size_t(j) + 2] - x[3 * size_t(o) + 2];
      for (int d = 0; d < 3; ++d) sh[3 * size_t(e) + d] = int(std::lround(d0 * inv[d] + d1 * inv[3 + d] + d2 * inv[6 + d]));
      nb[e] = o;
    }
  }
  pet_edge_list list{};
  list.n_atoms = N, list.n_local = v->n_local;
  list.atomic_numbers = z.data(), list.offsets = off.data(), list.neighbors = nb.data();
  list.shifts = v->image_of ? sh.data() : nullptr;
  list.cell = v->cell, list.half = 0, list.exchange = v->exchange;
  set_neighbors(&list);
}

// An engine's pairs as a flat device list (EdgeSession::set(DevicePairListView), src/device_geometry.cpp:547-669;
// Calculator::compute_pairs). The list comes to the host once per set, where each centre's pairs are gathered in
// list order (the reference's run and scattered cases give the same order); every step stays on the device.
void Engine::compute_pairs(const pet_pair_list* v, const double* positions, const double* cell, bool forces,
                           pet_device_results* out) {
  PETB_CUDA(cudaSetDevice(device));
  if (!v || v->n_atoms < 0 || v->n_pairs < 0) throw Error(2, "pet: no pair list given");
  const int N = v->n_atoms, P = v->n_pairs;
  if ((P > 0 && !v->pairs) || (N > 0 && !v->atomic_numbers)) throw Error(2, "pet: a pair list needs pairs and atomic numbers");
  if (N > 0 && !positions) throw Error(2, "pet: no device positions given");
  if (N >= (1 << 24)) throw Error(1, "pet: too many atoms for the edge key");
  const long sp = v->stride_pair ? v->stride_pair : 5, sc = v->stride_col ? v->stride_col : 1;
  PETB_CUDA(cudaStreamSynchronize(st.s));
  tmp_arena.reset();
  std::vector<int> hp(5 * size_t(P)), z(N), ren(v->renumber ? N : 0);
  if (P) {
    int* dense = tmp_arena.alloc<int>(5 * size_t(P));
    k_dense_pairs<<<cdiv(5 * size_t(P), 256), 256, 0, st.s>>>(dense, v->pairs, sp, sc, P);
    PETB_LAUNCH_CHECK(st);
    PETB_CUDA(cudaMemcpyAsync(hp.data(), dense, 20 * size_t(P), cudaMemcpyDeviceToHost, st.s));
  }
  if (N) PETB_CUDA(cudaMemcpyAsync(z.data(), v->atomic_numbers, 4 * size_t(N), cudaMemcpyDeviceToHost, st.s));
  if (N && v->renumber) PETB_CUDA(cudaMemcpyAsync(ren.data(), v->renumber, 4 * size_t(N), cudaMemcpyDeviceToHost, st.s));
  PETB_CUDA(cudaStreamSynchronize(st.s));

  const bool has_ren = v->renumber != nullptr;
  if (has_ren) {  // it must be a permutation
    std::vector<char> seen(N, 0);
    for (int a = 0; a < N; ++a) {
      if (ren[a] < 0 || ren[a] >= N || seen[ren[a]]) throw Error(1, "pet: the renumbering is not a permutation of the atoms");
      seen[ren[a]] = 1;
    }
  }
  auto ours = [&](int a) { return has_ren ? ren[a] : a; };
  std::vector<int> zz(N);
  int uncovered = 0;
  for (int a = 0; a < N; ++a) {
    zz[ours(a)] = z[a];
    uncovered += ckpt.species_to_index.empty() || z[a] < 0 || z[a] >= int(ckpt.species_to_index.size()) ||
                 ckpt.species_to_index[z[a]] < 0;
  }
  if (uncovered) throw Error(1, "pet: " + std::to_string(uncovered) + " atoms have elements the model does not cover");
  std::vector<int> off(size_t(N) + 1, 0);
  int bad = 0;
  for (int k = 0; k < P; ++k) {
    const int i = hp[5 * size_t(k)], j = hp[5 * size_t(k) + 1];
    if (i < 0 || i >= N || j < 0 || j >= N) ++bad;
    else ++off[ours(i) + 1];
  }
  if (bad) throw Error(1, "pet: " + std::to_string(bad) + " pairs name atoms that do not exist");
  for (int a = 0; a < N; ++a) off[a + 1] += off[a];
  std::vector<int> cur(off.begin(), off.end() - 1), nb(P), sh(3 * size_t(P));
  bool shifted = false;
  for (int k = 0; k < P; ++k) {
    const int e = cur[ours(hp[5 * size_t(k)])]++;
    nb[e] = ours(hp[5 * size_t(k) + 1]);
    for (int d = 0; d < 3; ++d) {
      sh[3 * size_t(e) + d] = hp[5 * size_t(k) + 2 + d];
      shifted = shifted || sh[3 * size_t(e) + d] != 0;
    }
  }
  pet_edge_list list{};
  list.n_atoms = N, list.n_local = v->n_local;
  list.atomic_numbers = zz.data(), list.offsets = off.data(), list.neighbors = nb.data();
  list.shifts = shifted ? sh.data() : nullptr;
  list.cell = cell, list.half = 0, list.exchange = nullptr;
  set_neighbors(&list);
  if (has_ren && N) {
    md.renumber = session_arena.alloc<int>(N);
    PETB_CUDA(cudaMemcpyAsync(md.renumber, ren.data(), 4 * size_t(N), cudaMemcpyHostToDevice, st.s));
    PETB_CUDA(cudaStreamSynchronize(st.s));
  }
  session_step(*this, positions, true, cell, forces);
  if (fixed_step_overflowed(*this)) session_step(*this, positions, true, cell, forces);
  if (gemm_mode != GEMM_NATIVE && gemm_tensor_error(st))  // synchronizes the stream
    throw Error(5, "pet: a tensor-core GEMM gave up waiting on its pipeline; the results of this evaluation are invalid");
  if (out) {
    *out = pet_device_results{};
    out->n_atoms = N;
    if (have_out) {
      out->energy = last_out.f.energy, out->per_atom_energy = last_out.per_atom;
      if (last_out.has_forces) out->forces = last_out.f.forces, out->virial = last_out.f.vir6;
    }
  }
}

// ---- testing aids ---------------------------------------------------------------------

void Engine::debug_fetch(const char* name, float* out, size_t capacity, size_t* n) {
  PETB_CUDA(cudaSetDevice(device));
  const auto it = taps.find(name ? name : "");
  if (it == taps.end()) throw Error(2, std::string("pet: no intermediate named '") + (name ? name : "") + "'");
  if (n) *n = it->second.second;
  if (!out) return;
  if (capacity < it->second.second) throw Error(2, "pet: the buffer is too small for this intermediate");
  PETB_CUDA(cudaStreamSynchronize(st.s));
  PETB_CUDA(cudaMemcpy(out, it->second.first, 4 * it->second.second, cudaMemcpyDeviceToHost));
}

void Engine::gemm_host(int mode, bool w_transposed, int m, int n, int k, const float* A, const float* W, float* C) {
  PETB_CUDA(cudaSetDevice(device));
  if (m <= 0 || n <= 0 || k <= 0 || !A || !W || !C) throw Error(2, "pet: bad GEMM arguments");
  PETB_CUDA(cudaStreamSynchronize(st.s));
  tmp_arena.reset();
  float* dA = tmp_arena.alloc<float>(size_t(m) * k);
  float* dW = tmp_arena.alloc<float>(2 * size_t(n) * k);  // and, for the 3xTF32 mode, the low parts of its split behind it
  float* dC = tmp_arena.alloc<float>(size_t(m) * n);
  PETB_CUDA(cudaMemcpyAsync(dA, A, 4 * size_t(m) * k, cudaMemcpyHostToDevice, st.s));
  // The kernels take the weight K-major, [n, k]; the other orientation is transposed here, as a
  // loaded weight is kept in both.
  std::vector<float> wt;
  const float* hw = W;
  if (!w_transposed) {
    wt.resize(size_t(n) * k);
    for (int p = 0; p < k; ++p)
      for (int j = 0; j < n; ++j) wt[size_t(j) * k + p] = W[size_t(p) * n + j];
    hw = wt.data();
  }
  PETB_CUDA(cudaMemcpyAsync(dW, hw, 4 * size_t(n) * k, cudaMemcpyHostToDevice, st.s));
  GemmArgs a;
  a.A = dA, a.lda = k, a.B = dW, a.ldb = k, a.C = dC, a.ldc = n, a.M = m, a.N = n, a.K = k;
  std::vector<float> wlo;
  if (mode == GEMM_TF32X3) {  // the weight's low parts, made once as for a loaded weight (x minus its leading 11 bits, rounded)
    wlo.resize(size_t(n) * k);
    for (size_t i = 0; i < wlo.size(); ++i) {
      uint32_t bits, lo;
      std::memcpy(&bits, &hw[i], 4);
      bits &= 0xFFFFE000u;
      float hi;
      std::memcpy(&hi, &bits, 4);
      const float r = hw[i] - hi;
      std::memcpy(&lo, &r, 4);
      lo += 0x1000u;
      std::memcpy(&wlo[i], &lo, 4);
    }
    PETB_CUDA(cudaMemcpyAsync(dW + size_t(n) * k, wlo.data(), 4 * wlo.size(), cudaMemcpyHostToDevice, st.s));
    a.b_lo_offset = size_t(n) * k;
  }
  std::vector<uint16_t> w16;
  if (mode == GEMM_BF16) {  // the weight again as bf16, round to nearest even, as a loaded weight is kept
    w16.resize(size_t(n) * k);
    for (size_t i = 0; i < w16.size(); ++i) {
      uint32_t u;
      std::memcpy(&u, &hw[i], 4);
      w16[i] = uint16_t((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
    }
    uint16_t* d16 = tmp_arena.alloc<uint16_t>(w16.size());
    PETB_CUDA(cudaMemcpyAsync(d16, w16.data(), 2 * w16.size(), cudaMemcpyHostToDevice, st.s));
    a.B16 = d16;
  }
  gemm(st, tmp_arena, a, mode);
  PETB_CUDA(cudaMemcpyAsync(C, dC, 4 * size_t(m) * n, cudaMemcpyDeviceToHost, st.s));
  PETB_CUDA(cudaStreamSynchronize(st.s));
  if (mode != GEMM_NATIVE && gemm_tensor_error(st)) throw Error(5, "pet: a tensor-core GEMM gave up waiting on its pipeline");
}

}  // namespace petb
