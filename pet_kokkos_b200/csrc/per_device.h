// State that CUDA keeps per device, cached per device.
//
// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) applies to the device that is current when it
// is called, an error word lives in one device's memory, and the SM count is a property of one
// device. A process may hold calculators on several GPUs (pet_options.device) and drive them
// from several host threads, so every cache of such a fact is a table indexed by device ordinal
// behind a mutex. This header is free of CUDA types so that the tables can be unit-tested on a
// host without a GPU: the CUDA call is passed in as a callable.
#pragma once

#include <mutex>

namespace petb {

constexpr int kMaxDevices = 64;

// The largest opt-in made so far for one kernel, per device. ensure(dev, bytes, set) calls
// set(bytes) when `bytes` exceeds what this device has been given and remembers it only when
// set succeeds (returns 0); a smaller request never lowers the value.
class SmemOptIn {
 public:
  explicit SmemOptIn(int initial = 48 * 1024) {
    for (int& b : bytes_) b = initial;
  }
  template <class Set>
  int ensure(int dev, int bytes, Set&& set) {
    if (dev < 0 || dev >= kMaxDevices) return set(bytes);  // beyond the table: no memo, always ask
    std::lock_guard<std::mutex> lock(mu_);
    if (bytes <= bytes_[dev]) return 0;
    const int rc = set(bytes);
    if (rc == 0) bytes_[dev] = bytes;
    return rc;
  }
  int granted(int dev) const { return dev >= 0 && dev < kMaxDevices ? bytes_[dev] : 0; }

 private:
  std::mutex mu_;
  int bytes_[kMaxDevices];
};

// One lazily built T per device. get(dev, make) runs make(T&) the first time a device asks.
template <class T>
class PerDevice {
 public:
  template <class Make>
  T& get(int dev, Make&& make) {
    if (dev < 0 || dev >= kMaxDevices) dev = kMaxDevices - 1;
    std::lock_guard<std::mutex> lock(mu_);
    if (!made_[dev]) {
      make(slot_[dev]);
      made_[dev] = true;
    }
    return slot_[dev];
  }

 private:
  std::mutex mu_;
  T slot_[kMaxDevices];
  bool made_[kMaxDevices] = {};
};

}  // namespace petb
