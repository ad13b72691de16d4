// Model files: <name>.json (hyperparameters, species map, composition energies,
// energy scale) and <name>.safetensors (F32/F64 tensors). The on-disk format is
// the reference's (src/checkpoint.cpp:12-139, tools/convert_pet.py:342-420).
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace petb {

// A minimal JSON value: enough for the checkpoint header and the safetensors index.
struct Json {
  enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
  bool b = false;
  double num = 0.0;
  std::string str;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;

  static Json parse(const std::string& text);
  const Json* find(const std::string& key) const;
  const Json& at(const std::string& key) const;  // throws if missing
  bool is_null() const { return kind == Null; }
  double number() const;
  int integer() const { return int(number()); }
  bool boolean() const;
  const std::string& string() const;
  double number_or(const std::string& key, double dflt) const;
  bool bool_or(const std::string& key, bool dflt) const;
  std::string string_or(const std::string& key, const std::string& dflt) const;
};

// The hyperparameters evaluation needs (the reference's include/pet/config.hpp:30-68).
struct Hypers {
  int d_pet = 128, d_head = 128, d_node = 512, d_feedforward = 256;
  int num_heads = 8, head_dim = 16;
  int num_attention_layers = 1, num_gnn_layers = 2, num_readout_layers = 1;
  bool layernorm = false;   // normalization: RMSNorm | LayerNorm
  bool swiglu = true;       // activation: SwiGLU | SiLU
  bool preln = true;        // transformer_type: PreLN | PostLN
  bool feedforward = true;  // featurizer_type: feedforward | residual
  int cutoff_function = 0;  // 0 Bump, 1 Cosine
  double attention_temperature = 1.0, cutoff = 7.5, cutoff_width = 0.5;
  double num_neighbors_adaptive = -1.0;
  bool adaptive_solver = false;        // adaptive_cutoff_method: grid | solver
  double cutoff_width_adaptive = 0.5;
  bool adaptive() const { return num_neighbors_adaptive > 0.0; }
  bool expanded_node() const { return d_node != d_pet; }
};

struct Tensor {
  std::vector<int64_t> shape;
  std::vector<double> data;  // widened to double, as the reference's loader holds them
  int64_t numel() const {
    int64_t n = 1;
    for (auto s : shape) n *= s;
    return n;
  }
  int64_t dim(int i) const { return shape.at(i); }
};

struct Checkpoint {
  Hypers hypers;
  double energy_scale = 1.0;
  int n_species = 0;
  std::vector<int> species_to_index;
  std::vector<double> composition_energies;
  std::map<std::string, Tensor> tensors;

  Checkpoint(const std::string& json_path, const std::string& safetensors_path);
  const Tensor& at(const std::string& name) const;
};

}  // namespace petb
