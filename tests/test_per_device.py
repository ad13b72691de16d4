"""The per-device tables behind the kernels' shared-memory opt-ins and the tensor-core state.

cudaFuncSetAttribute(MaxDynamicSharedMemorySize) applies to the device that is current when it is called, so a
process that holds calculators on several GPUs (pet_options.device) must opt in once per device, not once per
process. pet_kokkos_b200/csrc/per_device.h keeps those facts per device ordinal; it is free of CUDA types, so this
test compiles it with g++ and drives it with a counting stand-in for the CUDA call, threads included.
"""
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

SRC = r'''
#include "per_device.h"
#include <atomic>
#include <cstdio>
#include <thread>
#include <vector>
using namespace petb;
int main() {
  SmemOptIn memo;  // starts at the 48 KiB every kernel has without asking
  std::vector<int> calls(4, 0);
  auto set_on = [&](int dev) { return [&calls, dev](int) { ++calls[dev]; return 0; }; };
  // device 0 opts in; device 1 must still be asked although device 0 already was
  if (memo.ensure(0, 100 << 10, set_on(0)) != 0 || calls[0] != 1) return 1;
  if (memo.ensure(1, 100 << 10, set_on(1)) != 0 || calls[1] != 1) return 2;
  // no new call for the same or a smaller size, one more for a larger one, and the grant never shrinks
  memo.ensure(0, 100 << 10, set_on(0)), memo.ensure(0, 60 << 10, set_on(0));
  if (calls[0] != 1 || memo.granted(0) != (100 << 10)) return 3;
  memo.ensure(0, 200 << 10, set_on(0));
  if (calls[0] != 2 || memo.granted(0) != (200 << 10) || memo.granted(1) != (100 << 10)) return 4;
  // below the default nothing is asked; a failing set is not remembered
  if (memo.ensure(2, 16 << 10, set_on(2)) != 0 || calls[2] != 0) return 5;
  if (memo.ensure(3, 100 << 10, [](int) { return 7; }) != 7 || memo.granted(3) != (48 << 10)) return 6;
  // threads racing on one device: the largest request wins and stays
  SmemOptIn raced;
  std::atomic<int> n{0};
  std::vector<std::thread> ts;
  for (int t = 0; t < 8; ++t)
    ts.emplace_back([&, t] {
      for (int k = 0; k < 1000; ++k) raced.ensure(5, (64 + 8 * ((t * 1000 + k) % 16)) << 10, [&](int) { ++n; return 0; });
    });
  for (auto& t : ts) t.join();
  if (raced.granted(5) != ((64 + 8 * 15) << 10) || n.load() > 16) return 7;
  // one lazily made state per device
  PerDevice<int> state;
  int made = 0;
  int& a = state.get(0, [&](int& v) { v = 10; ++made; });
  int& b = state.get(1, [&](int& v) { v = 11; ++made; });
  int& c = state.get(0, [&](int& v) { v = 99; ++made; });
  if (&a != &c || a != 10 || b != 11 || made != 2) return 8;
  std::puts("PER_DEVICE_OK");
  return 0;
}
'''


def test_opt_ins_and_state_are_kept_per_device(tmp_path):
    src = tmp_path / "per_device_test.cpp"
    src.write_text(SRC)
    exe = tmp_path / "per_device_test"
    subprocess.run(["g++", "-std=c++17", "-O1", "-pthread", f"-I{ROOT / 'pet_kokkos_b200' / 'csrc'}", str(src), "-o", str(exe)],
                   check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and "PER_DEVICE_OK" in r.stdout, (r.returncode, r.stdout, r.stderr)
