// A header-only C++ facade over the C ABI (pet_b200.h) with the names of the reference's
// include/pet/calculator.hpp:32-319, so that a caller of pet::Calculator recompiles against it.
// Status codes are rethrown as the exception types the reference throws.
#pragma once

#include <array>
#include <cstdlib>
#include <filesystem>
#include <new>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../pet_b200.h"

namespace pet {

// How much of the forward the backward keeps (the reference's include/pet/config.hpp:19-24).
enum class Recompute { Auto = 0, Never = 1, Wide = 2, Layers = 3 };
inline const char* recompute_name(Recompute r) {
  const char* names[] = {"auto", "never", "wide", "layers"};
  return names[int(r)];
}

enum class GemmMode { Native = PET_GEMM_NATIVE, TF32 = PET_GEMM_TF32, BF16 = PET_GEMM_BF16, TF32x3 = PET_GEMM_TF32X3 };

// pet::System (the reference's include/pet/neighbors.hpp:15-25).
struct System {
  int n_atoms = 0;
  std::vector<int> atomic_numbers;
  std::vector<double> positions;
  std::array<double, 9> cell{};
  std::array<bool, 3> pbc{false, false, false};
  int charge = 0;
  int spin_multiplicity = 1;
};

// pet::Options (calculator.hpp:32-117): the fields this path uses.
struct Options {
  std::optional<GemmMode> gemm;
  bool graphs = true;
  bool md_fixed_shapes = false;
  bool cache_neighbors = false;  // a Verlet cache for a staged batch being stepped (stage / compute_device)
  std::size_t memory_budget_bytes = 0;
  Recompute recompute = Recompute::Auto;
  int max_batch_atoms = 0;
  int device = -1;
};

// The latest evaluation's memory decision (the reference's MemoryPlan, include/pet/model.hpp:23-28).
struct MemoryPlan {
  int atoms = 0, max_neighbors = 0;
  long edges = 0;
  Recompute tier = Recompute::Never;
  std::size_t estimate = 0, budget = 0;
};

// Where a named model is looked for, in order (calculator.hpp:152-156 of the reference): $PET_MODEL_DIR
// (':'-separated), ./models and ., $XDG_DATA_HOME/pet/models (else ~/.local/share/pet/models). A directory counts only
// if it holds both <name>.json and <name>.safetensors.
inline std::vector<std::string> model_search_dirs() {
  std::vector<std::string> dirs;
  const char* e = std::getenv("PET_MODEL_DIR");
  const std::string env = e ? e : "";
  std::size_t p = 0;
  while (p <= env.size()) {
    const std::size_t q = std::min(env.find(':', p), env.size());
    if (q > p) dirs.push_back(env.substr(p, q - p));
    p = q + 1;
  }
  dirs.push_back("models");
  dirs.push_back(".");
  const char* x = std::getenv("XDG_DATA_HOME");
  const char* home = std::getenv("HOME");
  if (x && x[0]) dirs.push_back(std::string(x) + "/pet/models");
  else if (home && home[0]) dirs.push_back(std::string(home) + "/.local/share/pet/models");
  return dirs;
}

// A model name ("pet-mad-s") or a path prefix to <spec>.json and <spec>.safetensors, to the two paths
// (calculator.hpp:164-167). Throws, listing where it looked, if a named model is not found. There is no default model
// in this library: an empty spec is refused.
inline void resolve_model(const std::string& spec, std::string& json_out, std::string& weights_out) {
  namespace fs = std::filesystem;
  std::error_code ec;
  if (spec.empty()) throw std::invalid_argument("pet: no model given (this library ships no default model)");
  if (spec.find('/') != std::string::npos || fs::exists(spec + ".json", ec)) {
    json_out = spec + ".json", weights_out = spec + ".safetensors";
    return;
  }
  std::string looked;
  for (const std::string& d : model_search_dirs()) {
    const std::string base = d + "/" + spec;
    if (fs::exists(base + ".json", ec) && fs::exists(base + ".safetensors", ec)) {
      json_out = base + ".json", weights_out = base + ".safetensors";
      return;
    }
    looked += (looked.empty() ? "" : ", ") + d;
  }
  throw std::runtime_error("pet: model '" + spec + "' not found in " + looked);
}

// pet::Results (calculator.hpp:120-142).
struct Results {
  std::vector<double> energy, per_atom_energy, forces, virial;
  std::vector<int> struct_id, n_atoms;
  std::vector<double> edge_gradient;
};

// pet::EdgeListView (the reference's include/pet/device_geometry.hpp:93-110).
// What an engine supplies when it runs PET over several ranks with ghosts one cutoff deep: the reference's
// pet::Exchange (include/pet/exchange.hpp:19-41) with device pointers and the calculator's CUDA stream in place of
// Kokkos views. Work enqueued on `stream` is ordered with the evaluation; anything else must be complete on return.
class Exchange {
 public:
  virtual ~Exchange() = default;
  // Once per evaluation: the kept edges to ghosts, ascending indices into the list's owned-atom -> ghost pairs.
  virtual void set_live(const int* live, int n_live, void* stream) = 0;
  // out[n_live, width]: one row per live edge to send to the ghost's owner; in[n_live, width]: the partners' rows.
  virtual void edges(const float* out, float* in, int n_live, int width, void* stream) = 0;
};

struct EdgeListView {
  int n_atoms = 0, n_local = -1;
  const double* positions = nullptr;
  const int* atomic_numbers = nullptr;
  const int* offsets = nullptr;
  const int* neighbors = nullptr;
  const int* shifts = nullptr;
  const double* cell = nullptr;
  bool half = false;
  Exchange* exchange = nullptr;  // must outlive the list
};

// pet::DeviceEdgeListView (include/pet/device_geometry.hpp:113-135): device memory throughout, except cell.
struct DeviceEdgeListView {
  int n_atoms = 0, n_local = -1, n_centres = 0;
  const int* ilist = nullptr;
  const int* numneigh = nullptr;
  const int* neighbors = nullptr;
  long stride_i = 0, stride_k = 1;
  int mask = ~0;
  const int* atomic_numbers = nullptr;
  const int* image_of = nullptr;
  const double* positions = nullptr;
  const double* cell = nullptr;
};

// pet::DevicePairListView (include/pet/device_geometry.hpp:137-154): device memory throughout.
struct DevicePairListView {
  int n_atoms = 0, n_local = -1, n_pairs = 0;
  const int* pairs = nullptr;
  long stride_pair = 5, stride_col = 1;
  const int* atomic_numbers = nullptr;
  const int* renumber = nullptr;
};

// pet::DeviceGeom (Calculator::stage, calculator.hpp:210-213): the staged batch on the device. `positions` may be
// written in place (on `stream`, or after synchronizing with it) between evaluations; cells move through
// Calculator::update_staged, which also refreshes what is derived from them.
struct DeviceGeom {
  int B = 0, Ntot = 0;
  double* pos = nullptr;          // [Ntot * 3] device
  const double* scell = nullptr;  // [B * 9] device
  const int* struct_id = nullptr; // [Ntot] device
  void* stream = nullptr;         // the calculator's cudaStream_t
};

// pet::BatchResult (calculator.hpp:144-165): a batch's results left on the device, valid until the next evaluation.
struct BatchResult {
  int B = 0, Ntot = 0;
  const double* energy = nullptr;           // [B]
  const double* per_atom_energy = nullptr;  // [Ntot]
  const double* forces = nullptr;           // [Ntot * 3], null without forces
  const double* virial = nullptr;           // [B * 6]
  void* stream = nullptr;
};

// pet::BatchResult for one structure: device pointers, valid until the calculator's next evaluation.
struct DeviceResults {
  int n_atoms = 0;
  const double* energy = nullptr;
  const double* per_atom_energy = nullptr;
  const double* forces = nullptr;
  const double* virial = nullptr;
};

class Calculator {
 public:
  struct DeviceArrays {
    const double* positions = nullptr;
    double* forces = nullptr;
    double* per_atom_energy = nullptr;
    double* per_atom_virial = nullptr;
    double virial_scale = 1.0;
  };
  struct Totals {
    double energy = 0.0;
    double virial[6] = {0, 0, 0, 0, 0, 0};
  };

  // A model name or path prefix (resolve_model above).
  explicit Calculator(const std::string& spec, Options opts = {}) : opts_(opts) {
    std::string json, weights;
    resolve_model(spec, json, weights);
    open(json, weights);
  }
  Calculator(const std::string& model_json, const std::string& model_weights, Options opts = {}) : opts_(opts) {
    open(model_json, model_weights);
  }
  ~Calculator() { pet_calc_destroy(h_); }
  Calculator(Calculator&& o) noexcept : h_(o.h_), opts_(o.opts_), pairs_(o.pairs_), atoms_(o.atoms_) { o.h_ = nullptr; }
  Calculator& operator=(Calculator&& o) noexcept {
    if (this != &o) {
      pet_calc_destroy(h_);
      h_ = o.h_, opts_ = o.opts_, pairs_ = o.pairs_, atoms_ = o.atoms_;
      o.h_ = nullptr;
    }
    return *this;
  }
  Calculator(const Calculator&) = delete;
  Calculator& operator=(const Calculator&) = delete;

  Results compute(const System& system, bool compute_forces = true) const {
    return compute(std::vector<System>{system}, compute_forces);
  }
  Results compute(const std::vector<System>& systems, bool compute_forces = true) const {
    Results r;
    if (systems.empty()) return r;
    std::vector<pet_system> ps = packed(systems);
    std::size_t N = 0;
    for (const System& s : systems) {
      r.n_atoms.push_back(s.n_atoms);
      N += std::size_t(s.n_atoms);
    }
    pet_results out = sized(r, systems.size(), N, compute_forces, 0);
    check(pet_compute(h_, ps.data(), int(ps.size()), compute_forces, &out));
    return r;
  }
  // Structures staged on the device for a caller that steps them there (calculator.hpp:210-218).
  DeviceGeom stage(const std::vector<System>& systems) const {
    std::vector<pet_system> ps = packed(systems);
    check(pet_stage(h_, ps.data(), int(ps.size())));
    return staged();
  }
  DeviceGeom staged() const {
    pet_device_geom g{};
    check(pet_staged_geometry(h_, &g));
    return DeviceGeom{g.n_structures, g.n_atoms, g.positions, g.cells, g.struct_id, g.stream};
  }
  // The staged batch shrinks to the structures `still_running` (indices into it, in their new order), e.g. as the
  // structures of a batched relaxation converge; a Verlet cache follows them without searching again.
  DeviceGeom keep(const std::vector<int>& still_running) const {
    check(pet_keep_staged(h_, still_running.data(), int(still_running.size())));
    return staged();
  }
  // New positions [Ntot * 3] and / or cells [B * 9] for the staged batch, from host arrays.
  void update_staged(const double* positions, const double* cells = nullptr) const { check(pet_update_staged(h_, positions, cells)); }
  // From the staged geometry, results left on the device.
  BatchResult compute_device(const DeviceGeom& geom, bool compute_forces = true) const {
    check(pet_compute_staged(h_, compute_forces ? 1 : 0));
    pet_device_results d{};
    void* stream = nullptr;
    check(pet_device_results_of(h_, &d, &stream));
    return BatchResult{geom.B, geom.Ntot, d.energy, d.per_atom_energy, d.forces, d.virial, stream};
  }
  // The staged batch's results to the host (what Results-returning compute gives).
  Results fetch(const DeviceGeom& geom, bool with_forces = true) const {
    Results r;
    pet_results out = sized(r, std::size_t(geom.B), std::size_t(geom.Ntot), with_forces, 0);
    check(pet_fetch_results(h_, &out));
    return r;
  }

  Results compute_edges(const EdgeListView& v, bool compute_forces = true, bool edge_gradients = true) const {
    pet_exchange ex{};
    const pet_edge_list l = list(v, ex);
    atoms_ = v.n_atoms, pairs_ = v.n_atoms > 0 ? v.offsets[v.n_atoms] : 0;
    Results r;
    r.n_atoms = {v.n_atoms};
    pet_results out = sized(r, 1, std::size_t(v.n_atoms), compute_forces, edge_gradients ? pairs_ : 0);
    check(pet_compute_edges(h_, &l, compute_forces, edge_gradients, &out));
    return r;
  }
  void set_neighbors(const EdgeListView& v) {
    pet_exchange ex{};
    const pet_edge_list l = list(v, ex);
    check(pet_set_neighbors(h_, &l));
    atoms_ = v.n_atoms, pairs_ = v.n_atoms > 0 ? v.offsets[v.n_atoms] : 0;
  }
  Results compute_step(const double* positions, const double* cell = nullptr, bool compute_forces = true,
                       bool edge_gradients = false) const {
    Results r;
    r.n_atoms = {atoms_};
    pet_results out = sized(r, 1, std::size_t(atoms_), compute_forces, edge_gradients ? pairs_ : 0);
    check(pet_compute_step(h_, positions, cell, compute_forces, edge_gradients, &out));
    return r;
  }
  Totals compute_step(const DeviceArrays& a, const double* cell = nullptr) const {
    const pet_device_arrays d{a.positions, a.forces, a.per_atom_energy, a.per_atom_virial, a.virial_scale};
    pet_totals t{};
    check(pet_compute_step_device(h_, &d, cell, &t));
    Totals out;
    out.energy = t.energy;
    for (int k = 0; k < 6; ++k) out.virial[k] = t.virial[k];
    return out;
  }

  void set_neighbors(const DeviceEdgeListView& v) {
    const pet_device_edge_list l{v.n_atoms, v.n_local,  v.n_centres, v.ilist,     v.numneigh, v.neighbors, v.stride_i,
                                 v.stride_k, v.mask,    v.atomic_numbers, v.image_of, v.positions, v.cell, nullptr};
    check(pet_set_neighbors_device(h_, &l));
    atoms_ = v.n_atoms, pairs_ = 0;
  }
  // An engine's flat pair list on the device, set and evaluated in one call (calculator.hpp:260-268).
  DeviceResults compute_pairs(const DevicePairListView& v, const double* positions, const double* cell = nullptr,
                              bool compute_forces = true) {
    const pet_pair_list l{v.n_atoms, v.n_local, v.n_pairs, v.pairs, v.stride_pair, v.stride_col, v.atomic_numbers, v.renumber};
    pet_device_results d{};
    check(pet_compute_pairs(h_, &l, positions, cell, compute_forces ? 1 : 0, &d));
    atoms_ = v.n_atoms, pairs_ = v.n_pairs;
    return DeviceResults{d.n_atoms, d.energy, d.per_atom_energy, d.forces, d.virial};
  }

  double cutoff() const { return pet_cutoff(h_); }
  double ghost_cutoff() const { return pet_ghost_cutoff(h_); }
  double exchange_ghost_cutoff() const { return pet_exchange_ghost_cutoff(h_); }
  double energy_scale() const { return pet_energy_scale(h_); }
  bool supports(int atomic_number) const { return pet_supports(h_, atomic_number) != 0; }
  std::size_t workspace_bytes() const { return pet_workspace_bytes(h_); }
  int recommended_batch_atoms() const { return pet_recommended_batch_atoms(h_); }
  MemoryPlan memory_plan() const {
    pet_memory_plan_info p{};
    check(pet_memory_plan(h_, &p));
    return MemoryPlan{p.atoms, p.max_neighbors, p.edges, Recompute(p.tier), p.estimate_bytes, p.budget_bytes};
  }
  std::string memory_report() const {
    char buf[1024] = {0};
    check(pet_memory_report(h_, buf, sizeof(buf)));
    return buf;
  }
  Options& options() { return opts_; }
  const Options& options() const { return opts_; }

 private:
  void open(const std::string& model_json, const std::string& model_weights) {
    pet_options o{};
    o.device = opts_.device;
    o.gemm_mode = opts_.gemm ? int(*opts_.gemm) : -1;
    o.graphs = opts_.graphs ? 1 : 0;
    o.md_fixed_shapes = opts_.md_fixed_shapes ? 1 : 0;
    o.cache_neighbors = opts_.cache_neighbors ? 1 : 0;
    o.memory_budget_bytes = opts_.memory_budget_bytes;
    o.max_batch_atoms = opts_.max_batch_atoms;
    o.recompute = int(opts_.recompute);
    const int rc = pet_calc_create(model_json.c_str(), model_weights.c_str(), &o, &h_);
    if (rc) raise(rc, pet_last_error(nullptr));
  }
  static std::vector<pet_system> packed(const std::vector<System>& systems) {
    std::vector<pet_system> ps(systems.size());
    for (std::size_t b = 0; b < systems.size(); ++b) {
      const System& s = systems[b];
      ps[b].n_atoms = s.n_atoms;
      ps[b].atomic_numbers = s.atomic_numbers.data();
      ps[b].positions = s.positions.data();
      for (int k = 0; k < 9; ++k) ps[b].cell[k] = s.cell[k];
      for (int k = 0; k < 3; ++k) ps[b].pbc[k] = s.pbc[k];
      ps[b].charge = s.charge, ps[b].spin_multiplicity = s.spin_multiplicity;
    }
    return ps;
  }
  // The library copies the callbacks out of `ex` during the call; the Exchange object itself is the caller's.
  static pet_edge_list list(const EdgeListView& v, pet_exchange& ex) {
    const pet_exchange* pex = nullptr;
    if (v.exchange) {
      ex.user = v.exchange;
      ex.set_live = [](void* u, const int* live, int n, void* stream) -> int {
        try {
          static_cast<Exchange*>(u)->set_live(live, n, stream);
          return 0;
        } catch (...) {
          return 1;
        }
      };
      ex.edges = [](void* u, const float* out, float* in, int n, int width, void* stream) -> int {
        try {
          static_cast<Exchange*>(u)->edges(out, in, n, width, stream);
          return 0;
        } catch (...) {
          return 1;
        }
      };
      pex = &ex;
    }
    return pet_edge_list{v.n_atoms, v.n_local, v.positions, v.atomic_numbers, v.offsets, v.neighbors,
                         v.shifts,  v.cell,    v.half ? 1 : 0, pex};
  }
  static pet_results sized(Results& r, std::size_t B, std::size_t N, bool forces, int pairs) {
    pet_results out{};
    r.energy.assign(B, 0.0), r.per_atom_energy.assign(N, 0.0);
    out.energy = r.energy.data(), out.per_atom_energy = r.per_atom_energy.data();
    if (forces) {
      r.forces.assign(3 * N, 0.0), r.virial.assign(6 * B, 0.0), r.struct_id.assign(N, 0);
      out.forces = r.forces.data(), out.virial = r.virial.data(), out.struct_id = r.struct_id.data();
      if (pairs > 0) {
        r.edge_gradient.assign(3 * std::size_t(pairs), 0.0);
        out.edge_gradient = r.edge_gradient.data();
      }
    }
    return out;
  }
  [[noreturn]] static void raise(int rc, const char* msg) {
    const std::string m = msg ? msg : "pet: unknown error";
    switch (rc) {
      case PET_ERR_INVALID: throw std::invalid_argument(m);
      case PET_ERR_LOGIC: throw std::logic_error(m);
      case PET_ERR_ALLOC: throw std::bad_alloc();
      default: throw std::runtime_error(m);
    }
  }
  void check(int rc) const {
    if (rc) raise(rc, pet_last_error(h_));
  }

  pet_calc* h_ = nullptr;
  Options opts_;
  mutable int pairs_ = 0, atoms_ = 0;
};

}  // namespace pet
