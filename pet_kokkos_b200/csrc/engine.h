// The calculator behind the C ABI: owns the device, the stream, the scratch pools,
// the model and the staged geometry, and runs one evaluation end to end.
//
// Stands for the reference's Calculator::Impl (src/calculator.cpp) on its device
// neighbour path: stage_systems -> build_nef_device -> PetModel::compute -> results.
#pragma once

#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../../include/pet_b200.h"
#include "checkpoint.h"
#include "common.h"
#include "model.h"
#include "neighbors.h"

namespace petb {

// An engine's neighbour list held on the device between its rebuilds
// (the reference's EdgeSession, src/device_geometry.cpp:410-778).
struct Session {
  bool valid = false, shifted = false, half = false;
  int n_atoms = 0, n_local = 0, n_pairs = 0, E = 0;
  RawEdges re;            // directed edges grouped by centre; vec/dist refreshed each step
  int* species = nullptr;  // [n_atoms]
  int* sid = nullptr;      // [n_atoms] zeros
  int* soff = nullptr;     // [2] = {0, n_atoms}
  double* pos = nullptr;   // [n_atoms,3]
  double* cell = nullptr;  // [9]
  int* ooff = nullptr;     // [n_atoms+1] partnerless edges by target atom
  int* oedge = nullptr;    // [n_orphan]
  int n_orphan = 0;
  std::vector<int> src, dir;  // each directed edge's pair in the engine's list, and its sign
  // Over several ranks with ghosts one cutoff deep (EdgeListView::exchange): the engine's callbacks, and the
  // owned-atom -> ghost edges in list order as raw edge indices (the reference's remote_raw).
  // Fixed shapes (Options::md_fixed_shapes): row and neighbour capacities kept from step to step, sized by an
  // eager step with room to move, and grown (the step redone) when a step outgrows them.
  bool caps_valid = false;
  int e_cap = 0, m_cap = 0;
  double pairs = 0.0;
  int* overflow = nullptr;  // device flag: the latest fixed-shape step did not fit
  bool has_exchange = false;
  pet_exchange exchange{};
  int n_remote = 0;
  int* remote_raw = nullptr;  // [n_remote]
  int* renumber = nullptr;    // [n_atoms] a flat pair list's renumbering (device); null: none
};

// The pairs of a staged batch within cutoff + skin, kept between evaluations while no atom has moved (and no cell
// strained) far enough for a pair outside to have come inside the cutoff: the reference's NefCache
// (include/pet/device_geometry.hpp:198-228, src/device_geometry.cpp:165-352). The shifts are in terms of the
// unwrapped positions, so a pair survives an atom crossing a cell face. Staging drops it; a batch that shrinks
// (Engine::keep_staged) keeps the pairs of the structures that stay, renumbered.
struct VerletCache {
  static constexpr double kSkin = 1.0;  // Angstrom, as the reference's
  bool valid = false;
  RawEdges ref;              // i, j, unwrapped shift, off, reverse; vec and dist refreshed each evaluation
  double* pos0 = nullptr;    // [N,3] the positions at the search
  double* cinv0 = nullptr;   // [B,9] the inverse cells then
  double* worst = nullptr;   // [1] the test's result
  long long searches = 0, reuses = 0;
};

struct Engine {
  explicit Engine(const std::string& json, const std::string& weights, const pet_options* opts);
  ~Engine();

  // Calculator::compute(vector<System>) on the device path.
  void compute(const pet_system* systems, int B, bool forces, pet_results* out);
  // keep_cache: the Verlet cache survives when the batch is the same atoms as the last one staged (compute() with
  // Options::cache_neighbors steps a structure this way, src/calculator.cpp:638-644); Calculator::stage drops it.
  void stage(const pet_system* systems, int B, bool keep_cache = false);
  void update_staged(const double* positions, const double* cells);
  void keep_staged(const int* keep, int n_keep);
  void compute_staged(bool forces);
  void fetch(pet_results* out);
  void neighbor_list(const pet_system* systems, int B, pet_raw_edges* out);
  void set_neighbors(const pet_edge_list* list);
  void compute_step(const double* positions, const double* cell, bool forces, bool edge_gradients, pet_results* out);
  void compute_step_device(const pet_device_arrays* arrays, const double* cell, pet_totals* totals);
  void set_neighbors_device(const pet_device_edge_list* list);
  void compute_pairs(const pet_pair_list* pairs, const double* positions, const double* cell, bool forces,
                     pet_device_results* out);
  void debug_fetch(const char* name, float* out, size_t capacity, size_t* n);
  void gemm_host(int mode, bool w_transposed, int m, int n, int k, const float* A, const float* W, float* C);

  int species_index(int Z) const;

  int device = 0;
  int gemm_mode = 0;
  bool graphs = true;
  bool md_fixed = false;  // Options::md_fixed_shapes / PET_MD_FIXED
  bool cache_neighbors = false;  // Options::cache_neighbors / PET_CACHE_NEIGHBORS
  size_t memory_budget = 0;      // Options::memory_budget_bytes; 0: what the device has
  int max_batch_atoms = 0;       // Options::max_batch_atoms; 0: no limit
  int recompute = RECOMPUTE_AUTO;  // Options::recompute / PET_RECOMPUTE: how much of the forward the backward keeps
  int tier_floor = RECOMPUTE_NEVER;  // raised when an evaluation of one structure ran out of memory under Auto
  RunOptions run_options() const;
  bool device_memory(size_t* free_b, size_t* total_b) const;  // cached while the pools keep their size
  mutable bool mem_known = false;
  mutable size_t mem_free = 0, mem_total = 0, mem_pools = 0;
  mutable long long mem_queries = 0;
  double peak_slots = 0.0;       // the most atoms x (neighbours + 1) one evaluation has held: samples bytes per slot
  long long batch_splits = 0;    // batches evaluated as more than one piece
  long long oom_recoveries = 0;  // evaluations retried after the device ran out of memory
  void compute_runs(const pet_system* systems, int B, const std::vector<std::pair<int, int>>& runs, bool forces,
                    pet_results* out);
  // Consecutive runs of a batch, each at least one structure, whose estimated edge slots fit the memory budget and
  // whose atoms fit max_batch_atoms (memory_runs, src/calculator.cpp:326-345).
  std::vector<std::pair<int, int>> memory_runs(const pet_system* systems, int B) const;
  Stream st;
  Profiler prof;
  Checkpoint ckpt;
  std::unique_ptr<Model> model;
  Arena geom_arena, nbr_arena, save_arena, tmp_arena, session_arena, cache_arena, cache_spare;
  VerletCache verlet;
  Geom geom;                  // staged batch
  std::vector<double> h_cells;  // staged cells on the host (the grid is chosen there)
  std::vector<int> h_natoms, h_per, h_species;
  double* posw = nullptr;
  PackedEdges last_pk;
  PassOut last_out;
  bool have_out = false;
  int last_B = 0, last_N = 0;
  int* pinned = nullptr;  // small pinned scratch for readbacks
  void* host_stage = nullptr;
  size_t host_stage_bytes = 0;
  std::map<std::string, std::pair<const float*, size_t>> taps;
  bool want_taps = false;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  double last_ms = 0.0;
  Session md;
  std::string error;

  // Recorded passes (the reference's GraphCache, include/pet/graph.hpp:68-146): a pass of given shapes and
  // buffers runs eagerly the first time, is captured the second time and replayed afterwards.
  struct GraphEntry {
    std::vector<uint64_t> key;
    cudaGraphExec_t exec = nullptr;
    PassOut out;
    Arena::Mark save_after{}, tmp_after{};
    long long launches = 0;
    uint64_t stamp = 0;
  };
  std::vector<GraphEntry> graph_cache;
  std::vector<std::vector<uint64_t>> graph_seen;
  uint64_t graph_clock = 0;
  long long graph_replays = 0;
  void run_model(const PackedEdges& pk, bool forces);
  RawEdges cached_edges();
  void drop_graphs();

 private:
  void* staging(size_t bytes);
};

}  // namespace petb
