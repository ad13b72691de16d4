// extern "C" entry points: include/pet_b200.h. Exceptions become status codes.
#include <new>
#include <string>

#include "engine.h"

using petb::Engine;

struct pet_calc {
  Engine* e = nullptr;
  std::string error;
};

namespace {

thread_local std::string g_create_error;

template <class F>
int guarded(pet_calc* c, F&& f) {
  try {
    if (!c || !c->e) throw petb::Error(PET_ERR_INVALID, "pet: null calculator");
    f(*c->e);
    return PET_OK;
  } catch (const petb::Error& err) {
    if (c) c->error = err.what();
    return err.code;
  } catch (const std::bad_alloc&) {
    if (c) c->error = "out of host memory";
    return PET_ERR_ALLOC;
  } catch (const std::exception& err) {
    if (c) c->error = err.what();
    return PET_ERR_RUNTIME;
  }
}

}  // namespace

extern "C" {

int pet_calc_create(const char* model_json, const char* model_weights, const pet_options* opts, pet_calc** out) {
  if (!out) return PET_ERR_INVALID;
  *out = nullptr;
  try {
    if (!model_json || !model_weights) throw petb::Error(PET_ERR_INVALID, "pet: model paths are required");
    pet_calc* c = new pet_calc;
    try {
      c->e = new Engine(model_json, model_weights, opts);
    } catch (...) {
      delete c;
      throw;
    }
    *out = c;
    return PET_OK;
  } catch (const petb::Error& err) {
    g_create_error = err.what();
    return err.code;
  } catch (const std::bad_alloc&) {
    g_create_error = "out of host memory";
    return PET_ERR_ALLOC;
  } catch (const std::exception& err) {
    g_create_error = err.what();
    return PET_ERR_RUNTIME;
  }
}

void pet_calc_destroy(pet_calc* c) {
  if (!c) return;
  delete c->e;
  delete c;
}

const char* pet_last_error(const pet_calc* c) { return c ? c->error.c_str() : g_create_error.c_str(); }

int pet_compute(pet_calc* c, const pet_system* systems, int n, int forces, pet_results* out) {
  return guarded(c, [&](Engine& e) { e.compute(systems, n, forces != 0, out); });
}
int pet_stage(pet_calc* c, const pet_system* systems, int n) {
  return guarded(c, [&](Engine& e) { e.stage(systems, n); });
}
int pet_compute_staged(pet_calc* c, int forces) {
  return guarded(c, [&](Engine& e) { e.compute_staged(forces != 0); });
}
int pet_fetch_results(pet_calc* c, pet_results* out) {
  return guarded(c, [&](Engine& e) { e.fetch(out); });
}
int pet_update_staged(pet_calc* c, const double* positions, const double* cells) {
  return guarded(c, [&](Engine& e) { e.update_staged(positions, cells); });
}
int pet_compute_edges(pet_calc* c, const pet_edge_list* list, int forces, int edge_gradients, pet_results* out) {
  return guarded(c, [&](Engine& e) {
    e.set_neighbors(list);
    e.compute_step(list->positions, list->cell, forces != 0, edge_gradients != 0, out);
  });
}
int pet_set_neighbors(pet_calc* c, const pet_edge_list* list) {
  return guarded(c, [&](Engine& e) { e.set_neighbors(list); });
}
int pet_compute_step(pet_calc* c, const double* positions, const double* cell, int forces, int edge_gradients,
                     pet_results* out) {
  return guarded(c, [&](Engine& e) { e.compute_step(positions, cell, forces != 0, edge_gradients != 0, out); });
}
int pet_compute_step_device(pet_calc* c, const pet_device_arrays* arrays, const double* cell, pet_totals* totals) {
  return guarded(c, [&](Engine& e) { e.compute_step_device(arrays, cell, totals); });
}
int pet_set_neighbors_device(pet_calc* c, const pet_device_edge_list* list) {
  return guarded(c, [&](Engine& e) { e.set_neighbors_device(list); });
}
int pet_compute_pairs(pet_calc* c, const pet_pair_list* pairs, const double* positions, const double* cell, int forces,
                      pet_device_results* out) {
  return guarded(c, [&](Engine& e) { e.compute_pairs(pairs, positions, cell, forces != 0, out); });
}
int pet_neighbor_list(pet_calc* c, const pet_system* systems, int n, pet_raw_edges* out) {
  return guarded(c, [&](Engine& e) { e.neighbor_list(systems, n, out); });
}

double pet_cutoff(const pet_calc* c) { return c && c->e ? c->e->ckpt.hypers.cutoff : 0.0; }
double pet_ghost_cutoff(const pet_calc* c) {
  // One cutoff per message-passing layer, and one more for an adaptive cutoff, which needs each of those atoms'
  // complete neighbourhoods (Calculator::ghost_cutoff, src/calculator.cpp:890-894).
  if (!c || !c->e) return 0.0;
  const petb::Hypers& h = c->e->ckpt.hypers;
  return (h.num_gnn_layers + (h.adaptive() ? 1 : 0)) * h.cutoff;
}
double pet_exchange_ghost_cutoff(const pet_calc* c) { return pet_cutoff(c); }
double pet_energy_scale(const pet_calc* c) { return c && c->e ? c->e->ckpt.energy_scale : 0.0; }
int pet_supports(const pet_calc* c, int Z) {
  if (!c || !c->e) return 0;
  const auto& m = c->e->ckpt.species_to_index;
  return Z >= 0 && Z < (int) m.size() && m[Z] >= 0;
}
size_t pet_workspace_bytes(const pet_calc* c) {
  if (!c || !c->e) return 0;
  const Engine& e = *c->e;
  return e.geom_arena.capacity() + e.nbr_arena.capacity() + e.save_arena.capacity() + e.tmp_arena.capacity() +
         e.session_arena.capacity();
}
int pet_last_shapes(const pet_calc* c, int* n_atoms, int* n_edges, int* max_neighbors) {
  if (!c || !c->e) return PET_ERR_INVALID;
  if (n_atoms) *n_atoms = c->e->last_pk.n_atoms;
  if (n_edges) *n_edges = c->e->last_pk.E;
  if (max_neighbors) *max_neighbors = c->e->last_pk.M;
  return PET_OK;
}
int pet_keep_staged(pet_calc* c, const int* keep, int n_keep) {
  return guarded(c, [&](Engine& e) { e.keep_staged(keep, n_keep); });
}
int pet_staged_geometry(pet_calc* c, pet_device_geom* out) {
  if (!c || !c->e || !out) return PET_ERR_INVALID;
  const Engine& e = *c->e;
  *out = pet_device_geom{};
  out->n_structures = e.geom.B, out->n_atoms = e.geom.Ntot;
  out->positions = e.geom.pos, out->cells = e.geom.scell, out->struct_id = e.geom.sid;
  out->stream = static_cast<void*>(e.st.s);
  return PET_OK;
}
int pet_device_results_of(pet_calc* c, pet_device_results* out, void** stream) {
  if (!c || !c->e || !out) return PET_ERR_INVALID;
  const Engine& e = *c->e;
  *out = pet_device_results{};
  out->n_atoms = e.last_N;
  if (e.have_out) {
    out->energy = e.last_out.f.energy, out->per_atom_energy = e.last_out.per_atom;
    if (e.last_out.has_forces) out->forces = e.last_out.f.forces, out->virial = e.last_out.f.vir6;
  }
  if (stream) *stream = static_cast<void*>(e.st.s);
  return PET_OK;
}
int pet_memory_plan(const pet_calc* c, pet_memory_plan_info* out) {
  if (!c || !c->e || !out) return PET_ERR_INVALID;
  const Engine& e = *c->e;
  *out = pet_memory_plan_info{};
  out->atoms = e.last_pk.n_atoms, out->max_neighbors = e.last_pk.M, out->edges = e.last_pk.E;
  out->tier = e.model->last_tier(), out->estimate_bytes = e.model->last_estimate();
  out->budget_bytes = e.memory_budget;
  out->pool_bytes = e.save_arena.capacity() + e.tmp_arena.capacity() + e.nbr_arena.capacity();
  return PET_OK;
}
int pet_memory_report(const pet_calc* c, char* buf, size_t len) {
  pet_memory_plan_info p;
  if (!buf || !len || pet_memory_plan(c, &p) != PET_OK) return PET_ERR_INVALID;
  size_t free_b = 0, total_b = 0;
  cudaSetDevice(c->e->device);
  cudaMemGetInfo(&free_b, &total_b);
  const double GiB = 1024.0 * 1024.0 * 1024.0;
  snprintf(buf, len,
           "  %d atoms, %d neighbours at most, %ld edges; recompute %s\n"
           "  estimated %.2f GiB for this tier, budget %.2f GiB (0: what the device has)\n"
           "  pools hold %.2f GiB; device %.2f GiB free of %.2f GiB\n",
           p.atoms, p.max_neighbors, p.edges, petb::recompute_name(p.tier), p.estimate_bytes / GiB, p.budget_bytes / GiB,
           p.pool_bytes / GiB, free_b / GiB, total_b / GiB);
  return PET_OK;
}
int pet_recommended_batch_atoms(const pet_calc* c) {
  if (!c || !c->e) return 0;
  const Engine& e = *c->e;
  if (e.max_batch_atoms > 0) return e.max_batch_atoms;
  // before anything has been evaluated the neighbour count is unknown: sizes that fit a small card
  const double pool = double(e.save_arena.capacity() + e.tmp_arena.capacity() + e.nbr_arena.capacity());
  if (pool <= 0.0 || e.peak_slots < 4096.0 || e.last_pk.M <= 0) return e.ckpt.hypers.feedforward ? 4096 : 2048;
  size_t free_b = 0, total_b = 0;
  cudaSetDevice(e.device);
  if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) return 4096;
  const double per_slot = pool / e.peak_slots;
  const double budget = e.memory_budget ? double(e.memory_budget) : 0.8 * double(total_b);
  const double by_memory = budget / per_slot / double(e.last_pk.M + 1);
  const double by_throughput = double(1 << 22) / double(e.last_pk.M + 1);  // past ~4 M edge slots a batch gains nothing
  const double atoms = std::min(by_memory, by_throughput);
  return int(std::min(std::max(atoms, 256.0), 65536.0));
}
long long pet_kernel_launches(const pet_calc* c) { return c && c->e ? c->e->st.launches : 0; }
long long pet_graph_replays(const pet_calc* c) { return c && c->e ? c->e->graph_replays : 0; }
long long pet_oom_recoveries(const pet_calc* c) { return c && c->e ? c->e->oom_recoveries : 0; }
long long pet_driver_memory_queries(const pet_calc* c) { return c && c->e ? c->e->mem_queries : 0; }
void pet_debug_fail_alloc(long k) { petb::g_fail_alloc_in = k; }
long long pet_batch_splits(const pet_calc* c) { return c && c->e ? c->e->batch_splits : 0; }
long long pet_neighbor_searches(const pet_calc* c) { return c && c->e ? c->e->verlet.searches : 0; }
long long pet_neighbor_reuses(const pet_calc* c) { return c && c->e ? c->e->verlet.reuses : 0; }
double pet_last_device_ms(const pet_calc* c) { return c && c->e ? c->e->last_ms : 0.0; }

int pet_profile(pet_calc* c, int enable) {
  return guarded(c, [&](Engine& e) {
    e.st.prof = &e.prof;
    e.prof.on = enable != 0;
  });
}
int pet_profile_read(pet_calc* c, pet_profile_entry* out, int capacity, int* n) {
  return guarded(c, [&](Engine& e) {
    PETB_CUDA(cudaSetDevice(e.device));
    PETB_CUDA(cudaStreamSynchronize(e.st.s));
    pet_profile_entry acc[petb::PC_COUNT] = {};
    for (auto& r : e.prof.recs) {
      float ms = 0.f;
      cudaEventElapsedTime(&ms, r.a, r.b);
      pet_profile_entry& a = acc[r.cls];
      a.launches += 1, a.ms += ms, a.flops += r.flops, a.bytes += r.bytes;
      e.prof.pool.push_back(r.a), e.prof.pool.push_back(r.b);
    }
    e.prof.recs.clear();
    int k = 0;
    for (int cls = 0; cls < petb::PC_COUNT; ++cls) {
      if (!acc[cls].launches) continue;
      if (out && k < capacity) {
        out[k] = acc[cls];
        snprintf(out[k].name, sizeof(out[k].name), "%s", petb::prof_class_name(cls));
      }
      ++k;
    }
    if (n) *n = k;
  });
}

int pet_debug_fetch(pet_calc* c, const char* name, float* out, size_t capacity, size_t* n) {
  return guarded(c, [&](Engine& e) {
    if (!e.want_taps) {
      e.want_taps = true;
      throw petb::Error(PET_ERR_LOGIC, "pet: intermediates are recorded from the next evaluation on");
    }
    e.debug_fetch(name, out, capacity, n);
  });
}
int pet_gemm_host(pet_calc* c, int mode, int w_transposed, int m, int n, int k, const float* A, const float* W, float* C) {
  return guarded(c, [&](Engine& e) { e.gemm_host(mode, w_transposed != 0, m, n, k, A, W, C); });
}

}  // extern "C"
