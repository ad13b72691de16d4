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
              std::map<std::string, std::pair<const float*, size_t>>* taps);

 private:
  PassOut run_feedforward(Stream& st, Arena& save, Arena& tmp, const PackedEdges& pk, bool grad, int mode,
                          std::map<std::string, std::pair<const float*, size_t>>* taps);
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
  double* comp_ = nullptr;  // [n_species] composition energies
  double* probes_ = nullptr;  // [n_probes_] the grid adaptive cutoff's radii (adaptive_probes, src/neighbors.cpp:23-27)
  int n_probes_ = 0;
  std::map<std::string, Mat> mat_;
  std::map<std::string, const float*> vec_;
  std::vector<void*> owned_;
};

}  // namespace petb
