"""A C++ caller of the header-only facade (include/pet/calculator.hpp) evaluates on the GPU, and every number it gets
equals what the ctypes mirror gets from the same library to the bit.

The driver below is what a user of the reference's pet::Calculator would write: `compute` on a System, `stage` +
`compute_device`, `set_neighbors` + `compute_step` on an engine's list with shifts, and `compute_edges` over a
pet::Exchange subclass (one rank whose ghosts are images of its own atoms, rows crossing through host memory, the
reference's ImageExchange test, tests/test_edges.cpp:385-439). It exercises the facade's marshalling (`sized`, `list`,
the exchange trampolines), which nothing else does.
"""
import subprocess
from pathlib import Path

import numpy as np
import pytest

from pet_kokkos_b200 import EdgeListView, exchange, structures as st

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

DRIVER = r'''
#include <cuda_runtime_api.h>
#include <cstdio>
#include <fstream>
#include <vector>
#include "pet/calculator.hpp"

template <class T> std::vector<T> rd(std::ifstream& f, size_t n) {
  std::vector<T> v(n);
  f.read(reinterpret_cast<char*>(v.data()), n * sizeof(T));
  return v;
}
void wr(std::ofstream& f, const std::vector<double>& v) { f.write(reinterpret_cast<const char*>(v.data()), v.size() * sizeof(double)); }
void wr(std::ofstream& f, const pet::Results& r) { wr(f, r.energy), wr(f, r.per_atom_energy), wr(f, r.forces), wr(f, r.virial); }

// One rank, every ghost an image of an own atom: the partner of edge r is edge partner[r] of the same rank.
struct ImageExchange : pet::Exchange {
  std::vector<int> partner, live;
  int calls = 0;
  void set_live(const int* d_live, int n, void* stream) override {
    cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    live.resize(n);
    cudaMemcpy(live.data(), d_live, n * sizeof(int), cudaMemcpyDeviceToHost);
  }
  void edges(const float* out, float* in, int n, int width, void* stream) override {
    cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    std::vector<float> rows(size_t(n) * width), got(size_t(n) * width, 0.f);
    cudaMemcpy(rows.data(), out, rows.size() * sizeof(float), cudaMemcpyDeviceToHost);
    std::vector<int> where(partner.size(), -1);
    for (int l = 0; l < n; ++l) where[live[l]] = l;
    for (int l = 0; l < n; ++l) {
      const int src = where[partner[live[l]]];
      if (src < 0) throw std::runtime_error("a live edge's partner is not live");
      for (int c = 0; c < width; ++c) got[size_t(l) * width + c] = rows[size_t(src) * width + c];
    }
    // on the calculator's stream: a blocking copy from pageable memory returns once staged, before the rows have
    // landed, and the calculator's non-blocking stream would not wait for it
    cudaMemcpyAsync(in, got.data(), got.size() * sizeof(float), cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream));
    cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    ++calls;
  }
};

int main(int argc, char** argv) {
  if (argc < 4) return 2;
  try {
    std::ifstream f(argv[2], std::ios::binary);
    std::ofstream o(argv[3], std::ios::binary);
    pet::Options opts;
    opts.recompute = pet::Recompute::Never;
    pet::Calculator calc(argv[1], opts);  // a path prefix: resolve_model appends .json / .safetensors
    // 1. a periodic System through compute, then staged and evaluated in place
    const int n = rd<int>(f, 1)[0];
    pet::System s;
    s.n_atoms = n, s.atomic_numbers = rd<int>(f, n), s.positions = rd<double>(f, 3 * size_t(n));
    const auto cell = rd<double>(f, 9);
    for (int k = 0; k < 9; ++k) s.cell[k] = cell[k];
    s.pbc = {true, true, true};
    wr(o, calc.compute(s, true));
    const pet::DeviceGeom geom = calc.stage({s});
    if (geom.B != 1 || geom.Ntot != n || !geom.pos) return 3;
    const pet::BatchResult br = calc.compute_device(geom, true);
    if (!br.energy || !br.forces) return 4;
    wr(o, calc.fetch(geom, true));
    const pet::MemoryPlan plan = calc.memory_plan();
    if (plan.atoms != n || plan.tier != pet::Recompute::Never || calc.memory_report().empty()) return 5;
    // 2. an engine's list with shifts: set_neighbors + compute_step on moved positions, with edge gradients
    const int pairs = rd<int>(f, 1)[0];
    const auto off = rd<int>(f, size_t(n) + 1), nbr = rd<int>(f, pairs), sh = rd<int>(f, 3 * size_t(pairs));
    const auto moved = rd<double>(f, 3 * size_t(n));
    pet::EdgeListView v;
    v.n_atoms = n, v.positions = s.positions.data(), v.atomic_numbers = s.atomic_numbers.data();
    v.offsets = off.data(), v.neighbors = nbr.data(), v.shifts = sh.data(), v.cell = cell.data();
    calc.set_neighbors(v);
    const pet::Results step = calc.compute_step(moved.data(), cell.data(), true, true);
    wr(o, step), wr(o, step.edge_gradient);
    // 3. a one-rank exchanged list
    const auto hdr = rd<int>(f, 4);  // listed atoms, owned atoms, pairs, edges to ghosts
    const auto z2 = rd<int>(f, hdr[0]), off2 = rd<int>(f, size_t(hdr[0]) + 1), nbr2 = rd<int>(f, hdr[2]);
    ImageExchange ex;
    ex.partner = rd<int>(f, hdr[3]);
    const auto x2 = rd<double>(f, 3 * size_t(hdr[0]));
    pet::EdgeListView w;
    w.n_atoms = hdr[0], w.n_local = hdr[1], w.positions = x2.data(), w.atomic_numbers = z2.data();
    w.offsets = off2.data(), w.neighbors = nbr2.data(), w.exchange = &ex;
    wr(o, calc.compute_edges(w, true, false));
    if (ex.calls == 0) return 6;
    std::printf("FACADE_OK %d\n", ex.calls);
  } catch (const std::exception& e) {
    std::printf("caught: %s\n", e.what());
    return 1;
  }
  return 0;
}
'''


def engine_list(s, cutoff, skin):
    from oracle import neighbors_oracle as nbo
    idx, _, _ = nbo.brute_force_edges(s, cutoff + skin)
    idx = idx[np.lexsort((idx[:, 4], idx[:, 3], idx[:, 2], idx[:, 1], idx[:, 0]))]
    off = np.concatenate([[0], np.cumsum(np.bincount(idx[:, 0], minlength=s["n_atoms"]))]).astype(np.int32)
    return off, idx[:, 1].astype(np.int32), idx[:, 2:5].astype(np.int32)


def test_a_cpp_caller_gets_the_bits_the_ctypes_mirror_gets(lib_path, models, tmp_path):
    from pet_kokkos_b200 import Calculator
    jp, sp = models("tiny", "feedforward", "scaled", 41)
    prefix = str(jp)[:-len(".json")]
    s = st.diamond(2, jitter=0.05, seed=9)
    n = s["n_atoms"]
    off, nbr, sh = engine_list(s, 4.5, 0.5)
    moved = s["positions"] + np.random.default_rng(2).normal(0, 0.03, s["positions"].shape)
    fields, owner, _, remote = exchange.exchange_domain(s, 0, 1, 4.5)
    partner = exchange.route([(fields, owner, None, remote)])[0][:, 1].astype(np.int32)
    with open(tmp_path / "in.bin", "wb") as f:
        for a in (np.int32([n]), s["atomic_numbers"].astype(np.int32), s["positions"].astype(np.float64),
                  s["cell"].astype(np.float64).reshape(9), np.int32([len(nbr)]), off, nbr, sh, moved.astype(np.float64),
                  np.int32([len(fields["positions"]), fields["n_local"], len(fields["neighbors"]), len(remote)]),
                  fields["atomic_numbers"].astype(np.int32), fields["offsets"].astype(np.int32),
                  fields["neighbors"].astype(np.int32), partner, fields["positions"].astype(np.float64)):
            f.write(np.ascontiguousarray(a).tobytes())
    src, exe = tmp_path / "driver.cpp", tmp_path / "driver"
    src.write_text(DRIVER)
    subprocess.run(["g++", "-std=c++17", "-O1", f"-I{ROOT / 'include'}", "-I/usr/local/cuda/include", str(src), "-o", str(exe),
                    f"-L{lib_path.parent}", "-lpet_b200", "-L/usr/local/cuda/lib64", "-lcudart",
                    f"-Wl,-rpath,{lib_path.parent}", "-Wl,-rpath,/usr/local/cuda/lib64"], check=True)
    r = subprocess.run([str(exe), prefix, str(tmp_path / "in.bin"), str(tmp_path / "out.bin")], capture_output=True, text=True)
    assert r.returncode == 0 and "FACADE_OK" in r.stdout, (r.returncode, r.stdout, r.stderr)
    got = np.fromfile(tmp_path / "out.bin", dtype=np.float64)

    c = Calculator(jp, sp, recompute="never")
    want = []
    r1 = c.compute(s)
    c.stage([s])
    c.compute_staged(True)
    r2 = c.fetch()
    view = EdgeListView(s["positions"], s["atomic_numbers"], off, nbr, sh, s["cell"])
    c.set_neighbors(view)
    r3 = c.compute_step(moved, s["cell"], True, True)
    calcs = [Calculator(jp, sp, recompute="never")]
    hub = exchange.ThreadHub(exchange.route([(fields, owner, None, remote)]))
    r4 = calcs[0].compute_edges(exchange.view_of(fields, exchange.ThreadExchange(hub, 0)), True, False)
    for r in (r1, r2, r3):
        want += [r.energy, r.per_atom_energy, r.forces.ravel(), r.virial.ravel()]
        if r is r3:
            want.append(r.edge_gradient.ravel())
    want += [r4.energy, r4.per_atom_energy, r4.forces.ravel(), r4.virial.ravel()]
    sizes = [len(np.ravel(w)) for w in want]
    want = np.concatenate(want)
    assert got.shape == want.shape
    at = 0
    for k, n in enumerate(sizes):  # which block differs, for the failure message
        if not np.array_equal(got[at:at + n], want[at:at + n]):
            print(f"block {k} (of {len(sizes)}, {n} numbers) differs by {np.abs(got[at:at + n] - want[at:at + n]).max():.3e}; "
                  f"first values {got[at:at + 3]} vs {want[at:at + 3]}")
        at += n
    assert np.array_equal(got, want), np.abs(got - want).max()
    assert np.array_equal(r1.forces, r2.forces), "staged evaluation equals compute"
    c.close()
    calcs[0].close()
