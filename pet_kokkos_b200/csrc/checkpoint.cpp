// Checkpoint reader: see checkpoint.h.
#include "checkpoint.h"

#include <cctype>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>

#include "common.h"

namespace petb {

namespace {

struct Parser {
  const std::string& s;
  size_t p = 0;
  explicit Parser(const std::string& t) : s(t) {}
  [[noreturn]] void fail(const char* what) const {
    throw Error(1, std::string("json: ") + what + " at byte " + std::to_string(p));
  }
  void ws() {
    while (p < s.size() && std::isspace((unsigned char) s[p])) ++p;
  }
  bool eat(char c) {
    ws();
    if (p < s.size() && s[p] == c) return ++p, true;
    return false;
  }
  std::string string_body() {
    std::string out;
    if (!eat('"')) fail("expected a string");
    while (p < s.size() && s[p] != '"') {
      char c = s[p++];
      if (c == '\\' && p < s.size()) {
        char e = s[p++];
        switch (e) {
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'r': out += '\r'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'u': {  // only the BMP, encoded as UTF-8
            if (p + 4 > s.size()) fail("short \\u escape");
            unsigned cp = std::strtoul(s.substr(p, 4).c_str(), nullptr, 16);
            p += 4;
            if (cp < 0x80) out += char(cp);
            else if (cp < 0x800) out += char(0xC0 | (cp >> 6)), out += char(0x80 | (cp & 0x3F));
            else out += char(0xE0 | (cp >> 12)), out += char(0x80 | ((cp >> 6) & 0x3F)), out += char(0x80 | (cp & 0x3F));
            break;
          }
          default: out += e;
        }
      } else {
        out += c;
      }
    }
    if (p >= s.size()) fail("unterminated string");
    ++p;
    return out;
  }
  Json value() {
    ws();
    if (p >= s.size()) fail("unexpected end");
    Json j;
    const char c = s[p];
    if (c == '{') {
      ++p;
      j.kind = Json::Object;
      if (eat('}')) return j;
      do {
        std::string k = string_body();
        if (!eat(':')) fail("expected ':'");
        j.obj.emplace_back(std::move(k), value());
      } while (eat(','));
      if (!eat('}')) fail("expected '}'");
    } else if (c == '[') {
      ++p;
      j.kind = Json::Array;
      if (eat(']')) return j;
      do j.arr.push_back(value());
      while (eat(','));
      if (!eat(']')) fail("expected ']'");
    } else if (c == '"') {
      j.kind = Json::String;
      j.str = string_body();
    } else if (!s.compare(p, 4, "true")) {
      j.kind = Json::Bool, j.b = true, p += 4;
    } else if (!s.compare(p, 5, "false")) {
      j.kind = Json::Bool, j.b = false, p += 5;
    } else if (!s.compare(p, 4, "null")) {
      p += 4;
    } else if (!s.compare(p, 3, "NaN")) {
      j.kind = Json::Number, j.num = std::strtod("nan", nullptr), p += 3;
    } else {
      char* end = nullptr;
      j.num = std::strtod(s.c_str() + p, &end);
      if (end == s.c_str() + p) fail("unexpected character");
      j.kind = Json::Number;
      p = size_t(end - s.c_str());
    }
    return j;
  }
};

}  // namespace

Json Json::parse(const std::string& text) {
  Parser ps(text);
  Json j = ps.value();
  ps.ws();
  if (ps.p != text.size()) ps.fail("trailing characters");
  return j;
}
const Json* Json::find(const std::string& key) const {
  for (const auto& kv : obj)
    if (kv.first == key) return &kv.second;
  return nullptr;
}
const Json& Json::at(const std::string& key) const {
  const Json* j = find(key);
  if (!j) throw Error(1, "json: missing key '" + key + "'");
  return *j;
}
double Json::number() const {
  if (kind == Bool) return b ? 1.0 : 0.0;
  if (kind != Number) throw Error(1, "json: expected a number");
  return num;
}
bool Json::boolean() const {
  if (kind == Number) return num != 0.0;
  if (kind != Bool) throw Error(1, "json: expected a boolean");
  return b;
}
const std::string& Json::string() const {
  if (kind != String) throw Error(1, "json: expected a string");
  return str;
}
double Json::number_or(const std::string& key, double dflt) const {
  const Json* j = find(key);
  return j && !j->is_null() ? j->number() : dflt;
}
bool Json::bool_or(const std::string& key, bool dflt) const {
  const Json* j = find(key);
  return j && !j->is_null() ? j->boolean() : dflt;
}
std::string Json::string_or(const std::string& key, const std::string& dflt) const {
  const Json* j = find(key);
  return j && !j->is_null() ? j->string() : dflt;
}

static bool choose(const std::string& key, const std::string& v, const char* a, const char* b) {
  if (v == a) return true;
  if (v == b) return false;
  throw Error(1, "checkpoint: unknown " + key + " '" + v + "'");
}

Checkpoint::Checkpoint(const std::string& json_path, const std::string& safetensors_path) {
  // ---- <name>.json ----
  {
    std::ifstream f(json_path);
    if (!f) throw Error(1, "checkpoint: cannot open '" + json_path + "'");
    std::stringstream ss;
    ss << f.rdbuf();
    const Json j = Json::parse(ss.str());
    const Json& h = j.at("hypers");
    Hypers& p = hypers;
    p.d_pet = h.at("d_pet").integer();
    p.d_head = h.at("d_head").integer();
    p.d_node = h.at("d_node").integer();
    p.d_feedforward = h.at("d_feedforward").integer();
    p.num_heads = h.at("num_heads").integer();
    p.head_dim = h.at("head_dim").integer();
    p.num_attention_layers = h.at("num_attention_layers").integer();
    p.num_gnn_layers = h.at("num_gnn_layers").integer();
    p.attention_temperature = h.at("attention_temperature").number();
    p.cutoff = h.at("cutoff").number();
    p.cutoff_width = h.at("cutoff_width").number();
    p.num_neighbors_adaptive = h.number_or("num_neighbors_adaptive", -1.0);
    p.layernorm = !choose("normalization", h.at("normalization").string(), "RMSNorm", "LayerNorm");
    p.swiglu = choose("activation", h.at("activation").string(), "SwiGLU", "SiLU");
    p.preln = choose("transformer_type", h.at("transformer_type").string(), "PreLN", "PostLN");
    p.feedforward = choose("featurizer_type", h.at("featurizer_type").string(), "feedforward", "residual");
    p.cutoff_function = choose("cutoff_function", h.at("cutoff_function").string(), "Bump", "Cosine") ? 0 : 1;
    p.num_readout_layers = int(h.number_or("num_readout_layers", p.feedforward ? 1 : p.num_gnn_layers));
    if (h.bool_or("long_range_enabled", false)) throw Error(1, "checkpoint: long-range models are not supported");
    if (h.bool_or("zbl", false)) throw Error(1, "checkpoint: the ZBL term is not supported");
    if (h.bool_or("system_conditioning", false))
      throw Error(1, "checkpoint: system_conditioning models are outside this evaluator's scope");
    if (p.adaptive()) {
      // older adaptive checkpoints carry neither key: the grid scheme and the plain taper width (src/checkpoint.cpp:91-95)
      p.adaptive_solver = !choose("adaptive_cutoff_method", h.string_or("adaptive_cutoff_method", "grid"), "grid", "solver");
      p.cutoff_width_adaptive = h.number_or("cutoff_width_adaptive", p.cutoff_width);
      // as the reference (src/model.cpp): the adaptive cutoff is implemented for the feedforward featurizer
      if (!p.feedforward) throw Error(1, "checkpoint: the residual featurizer with an adaptive cutoff is not implemented");
    }
    energy_scale = j.at("energy_scale").number();
    n_species = j.at("n_species").integer();
    for (const auto& v : j.at("species_to_index").arr) species_to_index.push_back(v.integer());
    for (const auto& v : j.at("composition_energies").arr) composition_energies.push_back(v.number());
  }
  // ---- <name>.safetensors ----
  std::ifstream f(safetensors_path, std::ios::binary);
  if (!f) throw Error(1, "safetensors: cannot open '" + safetensors_path + "'");
  uint64_t header_len = 0;
  f.read(reinterpret_cast<char*>(&header_len), 8);
  if (!f || header_len > (uint64_t(1) << 30)) throw Error(1, "safetensors: bad header length");
  std::string header(size_t(header_len), '\0');
  f.read(header.data(), std::streamsize(header_len));
  if (!f) throw Error(1, "safetensors: truncated header");
  const std::streampos data_start = f.tellg();
  const Json j = Json::parse(header);
  for (const auto& kv : j.obj) {
    if (kv.first == "__metadata__") continue;
    const Json& e = kv.second;
    const std::string dtype = e.at("dtype").string();
    const int64_t begin = int64_t(e.at("data_offsets").arr.at(0).number());
    const int64_t end = int64_t(e.at("data_offsets").arr.at(1).number());
    Tensor t;
    for (const auto& s : e.at("shape").arr) t.shape.push_back(int64_t(s.number()));
    const int64_t n = t.numel();
    const int64_t item = dtype == "F32" ? 4 : dtype == "F64" ? 8 : 0;
    if (!item) throw Error(1, "safetensors: unsupported dtype '" + dtype + "' for '" + kv.first + "'");
    if (begin < 0 || end - begin != n * item)
      throw Error(1, "safetensors: '" + kv.first + "' byte range does not match its shape");
    f.seekg(data_start + std::streamoff(begin));
    t.data.resize(size_t(n));
    if (item == 8) {
      f.read(reinterpret_cast<char*>(t.data.data()), end - begin);
    } else {
      std::vector<float> raw((size_t) n);
      f.read(reinterpret_cast<char*>(raw.data()), end - begin);
      for (int64_t i = 0; i < n; ++i) t.data[size_t(i)] = raw[size_t(i)];
    }
    if (!f) throw Error(1, "safetensors: truncated data for '" + kv.first + "'");
    tensors.emplace(kv.first, std::move(t));
  }
}

const Tensor& Checkpoint::at(const std::string& name) const {
  auto it = tensors.find(name);
  if (it == tensors.end()) throw Error(1, "safetensors: missing tensor '" + name + "'");
  return it->second;
}

}  // namespace petb
