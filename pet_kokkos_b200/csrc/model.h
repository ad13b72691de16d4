// The PET network on the device: weights, the forward pass, the analytic backward.
//
// Stands for the reference's PetModel (include/pet/model.hpp, src/model.cpp:180-344
// load_all, :656-778 readout and readout_bwd), ff_layer / ff_layer_bwd / ff_pass
// (src/feedforward.cpp:34-426) and residual_layer / residual_pass (src/residual.cpp).
#pragma once

#include <map>
#include <string>
#include <utility>
#include <vector>

#include "checkpoint.h"
#include "common.h"
#include "neighbors.h"
#include "ops.h"

namespace petb {

// A weight on the device in both orientations: w [rows, cols] as stored, wt [cols, rows].
struct Mat {
  const float* w = nullptr;
  const float* wt = nullptr;
  int rows = 0, cols = 0;
  size_t lo_off = 0;  // w + lo_off and wt + lo_off: the low parts of the 3xTF32 split of w and wt
  const uint16_t* w16 = nullptr;   // w and wt again as bf16 (round to nearest even), for the bf16 GEMM mode
  const uint16_t* wt16 = nullptr;
};

struct PassOut {
  double* per_atom = nullptr;  // [n_atoms]
  ForceOut f;                  // forces, virial, per-structure energy (device)
  bool has_forces = false;
};

// How much of the forward the backward keeps (the reference's Recompute, include/pet/config.hpp:19-24).
enum RecomputeTier { RECOMPUTE_AUTO = 0, RECOMPUTE_NEVER = 1, RECOMPUTE_WIDE = 2, RECOMPUTE_LAYERS = 3 };
inline const char* recompute_name(int t) {
  static const char* names[] = {"auto", "never", "wide", "layers"};
  return t >= 0 && t < 4 ? names[t] : "?";
}

// Bytes of the two scratch pools at their fullest during one evaluation.
struct MemoryNeed {
  size_t save = 0, tmp = 0;
};

struct RunOptions {
  int recompute = RECOMPUTE_AUTO;    // a tier, or Auto: the first that fits `budget`
  int tier_floor = RECOMPUTE_NEVER;  // Auto starts here (raised after an evaluation ran out of memory)
  size_t budget = 0;                 // bytes the pools may hold; 0: no limit known, keep everything
};

class Model {
 public:
  explicit Model(const Checkpoint& ckpt);
  ~Model();
  Model(const Model&) = delete;
  Model& operator=(const Model&) = delete;

  const Hypers& hypers() const { return h_; }
  double energy_scale() const { return scale_; }
  CutoffSpec cutoff_spec() const {
    CutoffSpec cs{h_.cutoff, h_.cutoff_width, h_.cutoff_function};
    if (h_.adaptive()) {
      cs.adaptive = h_.adaptive_solver ? 2 : 1;
      cs.target = h_.num_neighbors_adaptive, cs.width_adaptive = h_.cutoff_width_adaptive;
      cs.probes = probes_, cs.n_probes = n_probes_;
    }
    return cs;
  }

  // One evaluation over packed edges. Saved activations come from `save`, temporaries
  // from `tmp`; both are rewound by the caller. With `taps`, named intermediates are
  // recorded as (pointer, element count) for inspection after the pass.
  PassOut run(Stream& st, Arena& save, Arena& tmp, const PackedEdges& pk, bool grad, int gemm_mode,
              std::map<std::string, std::pair<const float*, size_t>>* taps, const RunOptions& opt = RunOptions());

  // The tier the latest pass ran under and the bytes estimated for it (Calculator::memory_plan / memory_report).
  int last_tier() const { return last_tier_; }
  size_t last_estimate() const { return last_estimate_; }
  // Bytes the pools hold for one evaluation with forces of N atoms and E kept edges under a tier.
  size_t memory_estimate(int tier, int N, int E) const;
  MemoryNeed memory_need(int tier, int N, int E, int n_live) const;
  int choose_tier(const RunOptions& opt, int N, int E) const;
  // Rows of a chunk of the edge MLP under Wide and Layers: an eighth of the edges, at least 64 Ki; PET_EDGE_CHUNK=rows
  // overrides it so that small structures exercise the chunking (edge_chunk_rows, src/model.cpp:813-817).
  static int edge_chunk_rows(int E);

 private:
  PassOut run_feedforward(Stream& st, Arena& save, Arena& tmp, const PackedEdges& pk, bool grad, int mode,
                          std::map<std::string, std::pair<const float*, size_t>>* taps, const RunOptions& opt);
  PassOut run_residual(Stream& st, Arena& save, Arena& tmp, const PackedEdges& pk, bool grad, int mode,
                       std::map<std::string, std::pair<const float*, size_t>>* taps);
  PassOut finish(Stream& st, Arena& save, const PackedEdges& pk, bool grad, float* x4_adj, const float* cutoff_adj,
                 float* cf_adj, double* per_atom);

  const Mat& mat(const std::string& name) const;
  const float* vec(const std::string& name) const;
  // `src` are doubles in DEVICE memory; the layouts the kernels read are made from them by kernels.
  void put_mat(const std::string& name, const double* src, int ld, int rows, int cols, bool paired);
  void put_vec(const std::string& name, const double* src, int len, bool paired);
  void fold_compress(const Checkpoint& ck, const std::string& c0, int layer);

  Hypers h_;
  double scale_ = 1.0;
  int last_tier_ = RECOMPUTE_NEVER;
  size_t last_estimate_ = 0;
  double* comp_ = nullptr;  // [n_species] composition energies
  double* probes_ = nullptr;  // [n_probes_] the grid adaptive cutoff's radii (adaptive_probes, src/neighbors.cpp:23-27)
  int n_probes_ = 0;
  std::map<std::string, Mat> mat_;
  std::map<std::string, const float*> vec_;
  std::vector<void*> owned_;
};

}  // namespace petb
