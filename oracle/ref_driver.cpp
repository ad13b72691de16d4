// A C entry layer over the reference's own pet::Calculator, compiled here from the
// reference's unmodified sources (see build_ref.sh) against the host stand-in for
// Kokkos in kokkos_host/. TEST INFRASTRUCTURE ONLY: the parity tests and the CPU
// baseline call it through ctypes as the checker; the product never links it.
//
// The reference's DFT-D3 correction (src/d3.cpp, out of the evaluated path) is not
// compiled; the members of pet::D3 that calculator.cpp refers to are defined below
// and throw, which no caller reaches with Options::d3 unset.
#include <Kokkos_Core.hpp>

#include <cstdio>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "pet/calculator.hpp"
#include "pet/checkpoint.hpp"
#include "pet/d3.hpp"
#include "pet/device_geometry.hpp"
#include "pet/gemm.hpp"
#include "pet/neighbors.hpp"

namespace pet {
struct D3::Impl {};
static void no_d3() { throw std::runtime_error("D3 dispersion is not part of this build of the reference"); }
D3::D3(D3Settings) { no_d3(); }
D3::~D3() = default;
Results D3::compute(const System&, bool) const { no_d3(); return {}; }
Results D3::compute(const std::vector<System>&, bool) const { no_d3(); return {}; }
D3::Out D3::evaluate(const Atoms&, bool, bool) const { no_d3(); return {}; }
double D3::ghost_cutoff(bool) const { return 0.0; }
bool D3::overflowed() const { return false; }
IView1D D3::overflow_flag() const { return {}; }
void D3::reset_grid() const {}
}  // namespace pet

namespace {

void put_error(char* buf, size_t len, const char* what) {
  if (buf && len) std::snprintf(buf, len, "%s", what);
}

std::vector<pet::System> make_systems(int B, const int* n_atoms, const int* Z, const double* pos, const double* cells,
                                      const int* pbc) {
  std::vector<pet::System> out(B);
  size_t a0 = 0;
  for (int b = 0; b < B; ++b) {
    pet::System& s = out[b];
    s.n_atoms = n_atoms[b];
    s.atomic_numbers.assign(Z + a0, Z + a0 + s.n_atoms);
    s.positions.assign(pos + 3 * a0, pos + 3 * (a0 + s.n_atoms));
    for (int k = 0; k < 9; ++k) s.cell[k] = cells[9 * b + k];
    for (int k = 0; k < 3; ++k) s.pbc[k] = pbc[3 * b + k] != 0;
    a0 += s.n_atoms;
  }
  return out;
}

template <class T>
void copy_out(T* dst, const std::vector<T>& src) {
  if (dst && !src.empty()) std::memcpy(dst, src.data(), src.size() * sizeof(T));
}

void results_out(const pet::Results& r, double* energy, double* per_atom, double* forces, double* virial,
                 double* edge_gradient) {
  copy_out(energy, r.energy);
  copy_out(per_atom, r.per_atom_energy);
  copy_out(forces, r.forces);
  copy_out(virial, r.virial);
  copy_out(edge_gradient, r.edge_gradient);
}

struct Handle {
  std::unique_ptr<pet::Calculator> calc;
  std::string json, weights;
};

}  // namespace

#if defined(PET_HAVE_CBLAS)
// The build of the reference whose GEMMs go through a CBLAS (its PET_USE_BLAS option): the two
// calls are bound at run time to whichever BLAS library petref_bind_blas is pointed at.
#include <dlfcn.h>
namespace {
using SgemmFn = void (*)(CBLAS_LAYOUT, CBLAS_TRANSPOSE, CBLAS_TRANSPOSE, int, int, int, float, const float*, int,
                         const float*, int, float, float*, int);
using DgemmFn = void (*)(CBLAS_LAYOUT, CBLAS_TRANSPOSE, CBLAS_TRANSPOSE, int, int, int, double, const double*, int,
                         const double*, int, double, double*, int);
SgemmFn g_sgemm = nullptr;
DgemmFn g_dgemm = nullptr;
}  // namespace
extern "C" void cblas_sgemm(CBLAS_LAYOUT l, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k, float alpha,
                            const float* A, int lda, const float* B, int ldb, float beta, float* C, int ldc) {
  if (!g_sgemm) throw std::runtime_error("no BLAS bound: call petref_bind_blas first");
  g_sgemm(l, ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc);
}
extern "C" void cblas_dgemm(CBLAS_LAYOUT l, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k, double alpha,
                            const double* A, int lda, const double* B, int ldb, double beta, double* C, int ldc) {
  if (!g_dgemm) throw std::runtime_error("no BLAS bound: call petref_bind_blas first");
  g_dgemm(l, ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc);
}
// path: a shared library exporting cblas_sgemm/cblas_dgemm, plain or with the given prefix ("scipy_").
extern "C" int petref_bind_blas(const char* path, const char* prefix) {
  void* h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (!h) return 1;
  const std::string p = prefix ? prefix : "";
  g_sgemm = reinterpret_cast<SgemmFn>(dlsym(h, (p + "cblas_sgemm").c_str()));
  g_dgemm = reinterpret_cast<DgemmFn>(dlsym(h, (p + "cblas_dgemm").c_str()));
  return g_sgemm && g_dgemm ? 0 : 2;
}
#else
extern "C" int petref_bind_blas(const char*, const char*) { return 3; }  // this build runs the reference's own GEMM loop
#endif

extern "C" {

// Calculator(model_json, model_weights, Options): the options at their defaults (Native GEMMs) but for the two
// neighbour-search switches; graphs are off (there is no device).
void* petref_create(const char* json, const char* weights, int device_neighbors, int builtin_search, char* err,
                    size_t errlen) {
  try {
    if (!Kokkos::is_initialized()) Kokkos::initialize();
    pet::Options o;
    o.device_neighbors = device_neighbors != 0;
    o.neighbors = builtin_search ? pet::Options::Neighbors::Builtin : pet::Options::Neighbors::Vesin;
    o.graphs = false;
    auto h = std::make_unique<Handle>();
    h->json = json, h->weights = weights;
    h->calc = std::make_unique<pet::Calculator>(h->json, h->weights, o);
    return h.release();
  } catch (const std::exception& e) {
    put_error(err, errlen, e.what());
    return nullptr;
  }
}

void petref_destroy(void* p) { delete static_cast<Handle*>(p); }

double petref_cutoff(void* p) { return static_cast<Handle*>(p)->calc->cutoff(); }
double petref_ghost_cutoff(void* p) { return static_cast<Handle*>(p)->calc->ghost_cutoff(); }
double petref_energy_scale(void* p) { return static_cast<Handle*>(p)->calc->energy_scale(); }

// Calculator::compute over B structures given as concatenated arrays.
int petref_compute(void* p, int B, const int* n_atoms, const int* Z, const double* pos, const double* cells,
                   const int* pbc, int compute_forces, double* energy, double* per_atom, double* forces, double* virial,
                   char* err, size_t errlen) {
  try {
    const auto systems = make_systems(B, n_atoms, Z, pos, cells, pbc);
    const pet::Results r = B == 1 ? static_cast<Handle*>(p)->calc->compute(systems[0], compute_forces != 0)
                                  : static_cast<Handle*>(p)->calc->compute(systems, compute_forces != 0);
    results_out(r, energy, per_atom, forces, virial, nullptr);
    return 0;
  } catch (const std::exception& e) {
    put_error(err, errlen, e.what());
    return 1;
  }
}

static pet::EdgeListView list_view(int n_atoms, int n_local, const double* pos, const int* Z, const int* offsets,
                                   const int* neighbors, const int* shifts, const double* cell, int half) {
  pet::EdgeListView v;
  v.n_atoms = n_atoms, v.n_local = n_local;
  v.positions = pos, v.atomic_numbers = Z, v.offsets = offsets, v.neighbors = neighbors;
  v.shifts = shifts, v.cell = cell, v.half = half != 0;
  return v;
}

// Calculator::compute_edges.
int petref_compute_edges(void* p, int n_atoms, int n_local, const double* pos, const int* Z, const int* offsets,
                         const int* neighbors, const int* shifts, const double* cell, int half, int compute_forces,
                         int edge_gradients, double* energy, double* per_atom, double* forces, double* virial,
                         double* edge_gradient, char* err, size_t errlen) {
  try {
    const pet::EdgeListView v = list_view(n_atoms, n_local, pos, Z, offsets, neighbors, shifts, cell, half);
    const pet::Results r = static_cast<Handle*>(p)->calc->compute_edges(v, compute_forces != 0, edge_gradients != 0);
    results_out(r, energy, per_atom, forces, virial, edge_gradient);
    return 0;
  } catch (const std::exception& e) {
    put_error(err, errlen, e.what());
    return 1;
  }
}

// Calculator::set_neighbors then n_steps of compute_step, positions [n_steps][n_atoms*3]; the outputs hold every step's.
int petref_steps(void* p, int n_atoms, int n_local, const double* pos0, const int* Z, const int* offsets,
                 const int* neighbors, const int* shifts, const double* cell, int half, int n_steps,
                 const double* positions, double* energy, double* forces, double* virial, char* err, size_t errlen) {
  try {
    auto& calc = *static_cast<Handle*>(p)->calc;
    calc.set_neighbors(list_view(n_atoms, n_local, pos0, Z, offsets, neighbors, shifts, cell, half));
    for (int s = 0; s < n_steps; ++s) {
      const pet::Results r = calc.compute_step(positions + size_t(s) * n_atoms * 3, cell, true, false);
      copy_out(energy + s, r.energy);
      copy_out(forces + size_t(s) * n_atoms * 3, r.forces);
      copy_out(virial + size_t(s) * 6, r.virial);
    }
    return 0;
  } catch (const std::exception& e) {
    put_error(err, errlen, e.what());
    return 1;
  }
}

// The packed neighbour list the reference's device search builds for a batch
// (build_device_batch): M, then per slot n*M+m the neighbour vector, distance,
// mask, cutoff factor and reverse slot. Call with null outputs first for N and M.
int petref_device_edges(void* p, int B, const int* n_atoms, const int* Z, const double* pos, const double* cells,
                        const int* pbc, int* N_out, int* M_out, double* edge_vec, double* dist, double* mask,
                        float* cutoff_factor, int* reverse_index, int* neigh_species, char* err, size_t errlen) {
  try {
    const auto systems = make_systems(B, n_atoms, Z, pos, cells, pbc);
    Handle* h = static_cast<Handle*>(p);
    const pet::Checkpoint ck(h->json, h->weights);
    pet::Workspace ws;
    pet::EdgeMap map(16);
    int m_high = 0;
    const pet::DeviceEdgeData d =
        pet::build_device_batch(systems, ck.hypers, ck.species_to_index, pet::RView1D(), 0, ws, map, m_high);
    const int N = d.n_atoms, M = d.max_neighbors;
    if (N_out) *N_out = N;
    if (M_out) *M_out = M;
    const size_t S = size_t(N) * M;
    for (size_t s = 0; s < S; ++s) {
      if (edge_vec)
        for (int c = 0; c < 3; ++c) edge_vec[3 * s + c] = d.edge_vec(s, c);
      if (dist) dist[s] = d.dist(s);
      if (mask) mask[s] = d.mask(s);
      if (cutoff_factor) cutoff_factor[s] = float(d.cutoff_factor(s));
      if (reverse_index) reverse_index[s] = d.reverse_index(s);
      if (neigh_species) neigh_species[s] = d.neigh_species(s);
    }
    return 0;
  } catch (const std::exception& e) {
    put_error(err, errlen, e.what());
    return 1;
  }
}

// The host search's raw list for one structure (detail::build_raw_edges): count, then i, j, shift, vec, dist.
int petref_host_raw_edges(int n_atoms, const int* Z, const double* pos, const double* cell, const int* pbc,
                          double cutoff, int capacity, int* count, int* i, int* j, int* shift, double* vec,
                          double* dist, char* err, size_t errlen) {
  try {
    const int one[1] = {n_atoms};
    const auto systems = make_systems(1, one, Z, pos, cell, pbc);
    const auto e = pet::detail::build_raw_edges(systems[0], cutoff);
    *count = int(e.size());
    if (int(e.size()) > capacity) return 0;
    for (size_t k = 0; k < e.size(); ++k) {
      i[k] = e[k].i, j[k] = e[k].j;
      shift[3 * k] = e[k].sa, shift[3 * k + 1] = e[k].sb, shift[3 * k + 2] = e[k].sc;
      vec[3 * k] = e[k].vx, vec[3 * k + 1] = e[k].vy, vec[3 * k + 2] = e[k].vz;
      dist[k] = e[k].dist;
    }
    return 0;
  } catch (const std::exception& e) {
    put_error(err, errlen, e.what());
    return 1;
  }
}

}  // extern "C"
