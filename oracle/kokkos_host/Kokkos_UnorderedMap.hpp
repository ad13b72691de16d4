// Host stand-in for Kokkos::UnorderedMap (see Kokkos_Core.hpp in this folder): a
// fixed-capacity hash map whose copies share one table, insert() callable on a
// const copy from inside a parallel loop, find() returning a slot index.
// Open addressing with linear probing; an insert of a key already present keeps
// the first value. Test infrastructure only.
#pragma once
#include <Kokkos_Core.hpp>

#include <mutex>

namespace Kokkos {

struct UnorderedMapInsertResult {
  enum : int { kSuccess, kExisting, kFailed };
  int state = kFailed;
  uint32_t slot = ~uint32_t(0);
  bool success() const { return state == kSuccess; }
  bool existing() const { return state == kExisting; }
  bool failed() const { return state == kFailed; }
  uint32_t index() const { return slot; }
};

template <class Key, class Value, class Device = Serial>
class UnorderedMap {
 public:
  using size_type = uint32_t;
  using key_type = Key;
  using value_type = Value;
  static constexpr size_type invalid_index = ~size_type(0);

  UnorderedMap() : UnorderedMap(0) {}
  explicit UnorderedMap(size_type capacity_hint) : t_(std::make_shared<Table>()) { t_->reset(capacity_hint); }

  size_type capacity() const { return size_type(t_->keys.size()); }
  size_type size() const { return t_->count.load(); }
  bool failed_insert() const { return t_->failed.load(); }
  bool rehash(size_type n) {
    // Like the real map, a rehash keeps what is stored.
    std::vector<std::pair<Key, Value>> old;
    for (size_type i = 0; i < capacity(); ++i)
      if (t_->used[i]) old.emplace_back(t_->keys[i], t_->values[i]);
    t_->reset(std::max<size_type>(n, size_type(old.size())));
    for (const auto& kv : old) insert(kv.first, kv.second);
    return true;
  }
  void clear() { t_->reset(capacity()); }

  UnorderedMapInsertResult insert(const Key& k, const Value& v = Value()) const {
    UnorderedMapInsertResult r;
    const size_type cap = capacity();
    if (cap == 0) {
      t_->failed = true;
      return r;
    }
    std::lock_guard<std::mutex> lock(t_->mutex);
    size_type s = hash(k) % cap;
    for (size_type probe = 0; probe < cap; ++probe, s = (s + 1 == cap ? 0 : s + 1)) {
      if (!t_->used[s]) {
        t_->used[s] = 1, t_->keys[s] = k, t_->values[s] = v;
        ++t_->count;
        r.state = UnorderedMapInsertResult::kSuccess, r.slot = s;
        return r;
      }
      if (t_->keys[s] == k) {
        r.state = UnorderedMapInsertResult::kExisting, r.slot = s;
        return r;
      }
    }
    t_->failed = true;
    return r;
  }
  size_type find(const Key& k) const {
    const size_type cap = capacity();
    if (cap == 0) return invalid_index;
    size_type s = hash(k) % cap;
    for (size_type probe = 0; probe < cap; ++probe, s = (s + 1 == cap ? 0 : s + 1)) {
      if (!t_->used[s]) return invalid_index;
      if (t_->keys[s] == k) return s;
    }
    return invalid_index;
  }
  bool exists(const Key& k) const { return find(k) != invalid_index; }
  bool valid_at(size_type i) const { return i < capacity() && t_->used[i]; }
  Value& value_at(size_type i) const { return t_->values[i]; }
  const Key& key_at(size_type i) const { return t_->keys[i]; }

 private:
  struct Table {
    std::vector<Key> keys;
    std::vector<Value> values;
    std::vector<char> used;
    std::atomic<size_type> count{0};
    std::atomic<bool> failed{false};
    std::mutex mutex;
    void reset(size_type n) {
      keys.assign(n, Key()), values.assign(n, Value()), used.assign(n, 0);
      count = 0, failed = false;
    }
  };
  static size_type hash(const Key& k) {
    uint64_t x = uint64_t(k);
    x ^= x >> 33, x *= 0xff51afd7ed558ccdULL, x ^= x >> 33, x *= 0xc4ceb9fe1a85ec53ULL, x ^= x >> 33;
    return size_type(x);
  }
  std::shared_ptr<Table> t_;
};

}  // namespace Kokkos
