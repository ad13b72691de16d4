// The device neighbour pipeline: see neighbors.h. Compiled with -fmad=false so that
// every fp64 product and sum below is rounded on its own, in the written order.
#include "neighbors.h"

#include <cmath>

namespace petb {

namespace {

constexpr int kCellListMinAtoms = 256;    // the reference's device_cell_list.hpp:46
constexpr int kCellListMinChecks = 2048;  // :47

__host__ __device__ inline int floor_div(int a, int n) {
  const int q = a / n;
  return (a % n != 0 && ((a < 0) != (n < 0))) ? q - 1 : q;
}
__host__ __device__ inline int floor_mod(int a, int n) { return a - floor_div(a, n) * n; }

// Images to search along each lattice vector: ceil(cutoff / interplanar spacing) on
// periodic axes (the reference's image_ranges_rows, device_geometry.hpp:28-44).
void image_ranges(const double c[9], double cutoff, int periodic, int n[3]) {
  n[0] = n[1] = n[2] = 0;
  const double *a = c, *b = c + 3, *cc = c + 6;
  const double bc[3] = {b[1] * cc[2] - b[2] * cc[1], b[2] * cc[0] - b[0] * cc[2], b[0] * cc[1] - b[1] * cc[0]};
  const double ca[3] = {cc[1] * a[2] - cc[2] * a[1], cc[2] * a[0] - cc[0] * a[2], cc[0] * a[1] - cc[1] * a[0]};
  const double ab[3] = {a[1] * b[2] - a[2] * b[1], a[2] * b[0] - a[0] * b[2], a[0] * b[1] - a[1] * b[0]};
  const double vol = std::fabs(a[0] * bc[0] + a[1] * bc[1] + a[2] * bc[2]);
  if (vol < 1e-12) return;
  const double nbc = std::sqrt(bc[0] * bc[0] + bc[1] * bc[1] + bc[2] * bc[2]);
  const double nca = std::sqrt(ca[0] * ca[0] + ca[1] * ca[1] + ca[2] * ca[2]);
  const double nab = std::sqrt(ab[0] * ab[0] + ab[1] * ab[1] + ab[2] * ab[2]);
  if (periodic & 1) n[0] = (int) std::ceil(cutoff / (vol / nbc));
  if (periodic & 2) n[1] = (int) std::ceil(cutoff / (vol / nca));
  if (periodic & 4) n[2] = (int) std::ceil(cutoff / (vol / nab));
}

}  // namespace

void invert_cell(const double c[9], double inv[9]) {
  const double a0 = c[0], a1 = c[1], a2 = c[2], b0 = c[3], b1 = c[4], b2 = c[5], c0 = c[6], c1 = c[7], c2 = c[8];
  const double det = a0 * (b1 * c2 - b2 * c1) - a1 * (b0 * c2 - b2 * c0) + a2 * (b0 * c1 - b1 * c0);
  const double id = (det != 0.0) ? 1.0 / det : 0.0;
  inv[0] = (b1 * c2 - b2 * c1) * id, inv[1] = (a2 * c1 - a1 * c2) * id, inv[2] = (a1 * b2 - a2 * b1) * id;
  inv[3] = (b2 * c0 - b0 * c2) * id, inv[4] = (a0 * c2 - a2 * c0) * id, inv[5] = (a2 * b0 - a0 * b2) * id;
  inv[6] = (b0 * c1 - b1 * c0) * id, inv[7] = (a1 * c0 - a0 * c1) * id, inv[8] = (a0 * b1 - a1 * b0) * id;
}

void grid_for_cell(const double c[9], int periodic, int n_atoms, double cutoff, int nc[3], int nr[3]) {
  int rng[3];
  image_ranges(c, cutoff, periodic, rng);
  // A structure the brute-force search could take gets one bin and that search's
  // image ranges, so its edges come out in that search's order (images, then atoms).
  if (n_atoms < kCellListMinAtoms &&
      n_atoms * (2 * rng[0] + 1) * (2 * rng[1] + 1) * (2 * rng[2] + 1) < kCellListMinChecks) {
    for (int d = 0; d < 3; ++d) nc[d] = 1, nr[d] = rng[d];
    return;
  }
  const double *a = c, *b = c + 3, *cc = c + 6;
  const double bc[3] = {b[1] * cc[2] - b[2] * cc[1], b[2] * cc[0] - b[0] * cc[2], b[0] * cc[1] - b[1] * cc[0]};
  const double ca[3] = {cc[1] * a[2] - cc[2] * a[1], cc[2] * a[0] - cc[0] * a[2], cc[0] * a[1] - cc[1] * a[0]};
  const double ab[3] = {a[1] * b[2] - a[2] * b[1], a[2] * b[0] - a[0] * b[2], a[0] * b[1] - a[1] * b[0]};
  const double vol = std::fabs(a[0] * bc[0] + a[1] * bc[1] + a[2] * bc[2]);
  const double area[3] = {std::sqrt(bc[0] * bc[0] + bc[1] * bc[1] + bc[2] * bc[2]),
                          std::sqrt(ca[0] * ca[0] + ca[1] * ca[1] + ca[2] * ca[2]),
                          std::sqrt(ab[0] * ab[0] + ab[1] * ab[1] + ab[2] * ab[2])};
  for (int d = 0; d < 3; ++d) {
    int k = 1, r = 0;
    if (periodic && vol > 1e-12 && area[d] > 0.0) {
      const double perp = vol / area[d];
      k = (int) std::floor(perp / cutoff);
      if (k < 1) k = 1;
      const double w = perp / (double) k;
      r = (int) std::ceil(cutoff / w);
      if (r < 1) r = 1;
    }
    nc[d] = k, nr[d] = r;
  }
}

// ---- scan ---------------------------------------------------------------------

namespace {

constexpr int kScanThreads = 256, kScanItems = 8, kScanChunk = kScanThreads * kScanItems;

__device__ inline int warp_inclusive(int v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  return v;
}

// Exclusive scan of a block's chunk into out, its total into sums[block].
__global__ void __launch_bounds__(kScanThreads) k_scan_chunks(const int* __restrict__ in, int* __restrict__ out,
                                                              int* __restrict__ sums, int n) {
  __shared__ int warp_tot[kScanThreads / 32];
  const int base = blockIdx.x * kScanChunk + threadIdx.x * kScanItems;
  int v[kScanItems], t = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    v[k] = base + k < n ? in[base + k] : 0;
    t += v[k];
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int inc = warp_inclusive(t, lane);
  if (lane == 31) warp_tot[w] = inc;
  __syncthreads();
  if (w == 0) {
    int x = lane < kScanThreads / 32 ? warp_tot[lane] : 0;
    x = warp_inclusive(x, lane);
    if (lane < kScanThreads / 32) warp_tot[lane] = x;
  }
  __syncthreads();
  int run = inc - t + (w > 0 ? warp_tot[w - 1] : 0);
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    if (base + k < n) out[base + k] = run;
    run += v[k];
  }
  if (threadIdx.x == kScanThreads - 1) sums[blockIdx.x] = run;
}

// One block: exclusive scan of the chunk totals in place, the grand total into *total.
__global__ void __launch_bounds__(1024) k_scan_sums(int* __restrict__ sums, int nb, int* __restrict__ total) {
  __shared__ int warp_tot[32];
  __shared__ int carry_s;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  for (int b0 = 0; b0 < nb; b0 += 1024) {
    const int i = b0 + threadIdx.x;
    const int x = i < nb ? sums[i] : 0;
    const int inc = warp_inclusive(x, lane);
    if (lane == 31) warp_tot[w] = inc;
    __syncthreads();
    if (w == 0) warp_tot[lane] = warp_inclusive(warp_tot[lane], lane);
    __syncthreads();
    const int carry = carry_s;
    const int excl = carry + inc - x + (w > 0 ? warp_tot[w - 1] : 0);
    if (i < nb) sums[i] = excl;
    __syncthreads();
    if (threadIdx.x == 1023) carry_s = carry + warp_tot[31];
    __syncthreads();
  }
  if (threadIdx.x == 0) *total = carry_s;
}

__global__ void __launch_bounds__(kScanThreads) k_scan_add(int* __restrict__ out, const int* __restrict__ sums, int n) {
  const int add = sums[blockIdx.x];
  const int base = blockIdx.x * kScanChunk + threadIdx.x * kScanItems;
#pragma unroll
  for (int k = 0; k < kScanItems; ++k)
    if (base + k < n) out[base + k] += add;
}

}  // namespace

void exclusive_scan(Stream& st, Arena& arena, const int* in, int* out, int n) {
  if (n <= 0) {
    PETB_CUDA(cudaMemsetAsync(out, 0, sizeof(int), st.s));
    return;
  }
  const int nb = cdiv(n, kScanChunk);
  int* sums = arena.alloc<int>(nb);
  k_scan_chunks<<<nb, kScanThreads, 0, st.s>>>(in, out, sums, n);
  PETB_LAUNCH_CHECK(st);
  k_scan_sums<<<1, 1024, 0, st.s>>>(sums, nb, out + n);
  PETB_LAUNCH_CHECK(st);
  if (nb > 1) {
    k_scan_add<<<nb, kScanThreads, 0, st.s>>>(out, sums, n);
    PETB_LAUNCH_CHECK(st);
  }
}

// ---- wrap, bins ------------------------------------------------------------------

namespace {

__global__ void k_wrap(Geom g, double* __restrict__ posw) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= g.Ntot) return;
  const int b = g.sid[i], per = g.sper[b];
  const double x = g.pos[3 * i], y = g.pos[3 * i + 1], z = g.pos[3 * i + 2];
  if (!per) {
    posw[3 * i] = x, posw[3 * i + 1] = y, posw[3 * i + 2] = z;
    return;
  }
  const double* ci = g.cinv + 9 * b;
  const double* c = g.scell + 9 * b;
  double f[3];
  for (int d = 0; d < 3; ++d) {
    f[d] = x * ci[d] + y * ci[3 + d] + z * ci[6 + d];
    const double w = (per >> d & 1) ? floor(f[d]) : 0.0;
    f[d] -= w;
  }
  for (int d = 0; d < 3; ++d) posw[3 * i + d] = f[0] * c[d] + f[1] * c[3 + d] + f[2] * c[6 + d];
}

__global__ void k_assign_bins(Geom g, const double* __restrict__ posw, int* __restrict__ abin, int* __restrict__ bcnt) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= g.Ntot) return;
  const int b = g.sid[i];
  int ijk[3] = {0, 0, 0};
  const int* nc = g.gnc + 3 * b;
  if (g.sper[b]) {
    const double x = posw[3 * i], y = posw[3 * i + 1], z = posw[3 * i + 2];
    const double* ci = g.cinv + 9 * b;
    for (int d = 0; d < 3; ++d) {
      const double f = x * ci[d] + y * ci[3 + d] + z * ci[6 + d];
      int c = (int) floor(f * (double) nc[d]);
      if (c < 0) c = 0;
      if (c >= nc[d]) c = nc[d] - 1;
      ijk[d] = c;
    }
  }
  const int bin = g.goff[b] + (ijk[0] * nc[1] + ijk[1]) * nc[2] + ijk[2];
  abin[i] = bin;
  atomicAdd(&bcnt[bin], 1);
}

// Atoms into their bins in arrival order; k_sort_bins then orders each bin by atom index.
__global__ void k_fill_bins(int N, const int* __restrict__ abin, const int* __restrict__ bstart, int* __restrict__ fill,
                            int* __restrict__ unsorted) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N) return;
  const int c = abin[i];
  unsorted[bstart[c] + atomicAdd(&fill[c], 1)] = i;
}

// One warp per bin: each member goes to its rank among the bin's members.
__global__ void k_sort_bins(int nbins, const int* __restrict__ bstart, const int* __restrict__ unsorted,
                            int* __restrict__ sorted) {
  const int bin = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (bin >= nbins) return;
  const int lo = bstart[bin], n = bstart[bin + 1] - lo;
  for (int q = lane; q < n; q += 32) {
    const int a = unsorted[lo + q];
    int rank = 0;
    for (int p = 0; p < n; ++p) rank += unsorted[lo + p] < a;
    sorted[lo + rank] = a;
  }
}

// The search for one atom, shared by the count and fill passes: candidate bins in
// (da, db, dc) order, a bin's members by atom index, lanes across the members.
struct Walk {
  Geom g;
  const double* posw;
  const int *abin, *bstart, *batom;
  double cutoff2;

  // v = x_j + (shift . cell - x_i), the image offset first and then the atom.
  __device__ inline bool edge(int gi, int j, const int* sh, const double* c, double* v) const {
#pragma unroll
    for (int d = 0; d < 3; ++d)
      v[d] = posw[3 * j + d] + (sh[0] * c[d] + sh[1] * c[3 + d] + sh[2] * c[6 + d] - posw[3 * gi + d]);
    v[3] = v[0] * v[0] + v[1] * v[1] + v[2] * v[2];
    return v[3] >= 1e-24 && v[3] <= cutoff2;
  }
};

template <bool FILL>
__global__ void __launch_bounds__(128) k_walk(Walk w, int* __restrict__ ecnt, const int* __restrict__ eoff, RawEdges re) {
  const int gi = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (gi >= w.g.Ntot) return;
  const int b = w.g.sid[gi];
  const int nca = w.g.gnc[3 * b], ncb = w.g.gnc[3 * b + 1], ncc = w.g.gnc[3 * b + 2];
  const int nra = w.g.gnr[3 * b], nrb = w.g.gnr[3 * b + 1], nrc = w.g.gnr[3 * b + 2];
  const int g0 = w.g.goff[b];
  const int loc = w.abin[gi] - g0;
  const int ca = loc / (ncb * ncc), cb = (loc / ncc) % ncb, cc = loc % ncc;
  const double* cell = w.g.scell + 9 * b;
  int e = FILL ? eoff[gi] : 0;
  for (int da = -nra; da <= nra; ++da)
    for (int db = -nrb; db <= nrb; ++db)
      for (int dc = -nrc; dc <= nrc; ++dc) {
        const int ta = ca + da, tb = cb + db, tc = cc + dc;
        const int sh[3] = {floor_div(ta, nca), floor_div(tb, ncb), floor_div(tc, ncc)};
        const int bin = g0 + (floor_mod(ta, nca) * ncb + floor_mod(tb, ncb)) * ncc + floor_mod(tc, ncc);
        const int k0 = w.bstart[bin], nk = w.bstart[bin + 1] - k0;
        for (int q0 = 0; q0 < nk; q0 += 32) {
          const int q = q0 + lane;
          double v[4];
          int j = -1;
          bool hit = false;
          if (q < nk) {
            j = w.batom[k0 + q];
            hit = w.edge(gi, j, sh, cell, v);
          }
          const unsigned m = __ballot_sync(0xffffffffu, hit);
          if (FILL && hit) {
            const int pos = e + __popc(m & ((1u << lane) - 1u));
            re.i[pos] = gi;
            re.j[pos] = j;
            re.shift[3 * pos] = sh[0], re.shift[3 * pos + 1] = sh[1], re.shift[3 * pos + 2] = sh[2];
            re.vec[3 * pos] = v[0], re.vec[3 * pos + 1] = v[1], re.vec[3 * pos + 2] = v[2];
            re.dist[pos] = sqrt(v[3]);
          }
          e += __popc(m);
        }
      }
  if (!FILL && lane == 0) ecnt[gi] = e;
}

// Each edge's partner: the (j, i, -shift) entry in j's own range.
__global__ void k_reverse(RawEdges re) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= re.E) return;
  const int i = re.i[e], j = re.j[e];
  const int sa = -re.shift[3 * e], sb = -re.shift[3 * e + 1], sc = -re.shift[3 * e + 2];
  int r = -1;
  for (int f = re.off[j]; f < re.off[j + 1]; ++f)
    if (re.j[f] == i && re.shift[3 * f] == sa && re.shift[3 * f + 1] == sb && re.shift[3 * f + 2] == sc) {
      r = f;
      break;
    }
  re.reverse[e] = r;
}

__global__ void k_edge_vectors(RawEdges re, const double* __restrict__ pos, const double* __restrict__ hc) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= re.E) return;
  const int i = re.i[e], j = re.j[e], a = re.shift[3 * e], b = re.shift[3 * e + 1], c = re.shift[3 * e + 2];
  const double x = pos[3 * j] + (a * hc[0] + b * hc[3] + c * hc[6]) - pos[3 * i];
  const double y = pos[3 * j + 1] + (a * hc[1] + b * hc[4] + c * hc[7]) - pos[3 * i + 1];
  const double z = pos[3 * j + 2] + (a * hc[2] + b * hc[5] + c * hc[8]) - pos[3 * i + 2];
  const double d2 = x * x + y * y + z * z;
  re.vec[3 * e] = x, re.vec[3 * e + 1] = y, re.vec[3 * e + 2] = z;
  re.dist[e] = d2 > 1e-24 ? sqrt(d2) : 1e30;  // a coincident pair weighs nothing
}

// The same for a batch whose structures each have their own cell (the Verlet cache's pairs).
__global__ void k_edge_vectors_batch(RawEdges re, Geom g) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= re.E) return;
  const int i = re.i[e], j = re.j[e], a = re.shift[3 * e], b = re.shift[3 * e + 1], c = re.shift[3 * e + 2];
  const double* hc = g.scell + 9 * g.sid[i];
  const double* pos = g.pos;
  const double x = pos[3 * j] + (a * hc[0] + b * hc[3] + c * hc[6]) - pos[3 * i];
  const double y = pos[3 * j + 1] + (a * hc[1] + b * hc[4] + c * hc[7]) - pos[3 * i + 1];
  const double z = pos[3 * j + 2] + (a * hc[2] + b * hc[5] + c * hc[8]) - pos[3 * i + 2];
  const double d2 = x * x + y * y + z * z;
  re.vec[3 * e] = x, re.vec[3 * e + 1] = y, re.vec[3 * e + 2] = z;
  re.dist[e] = d2 > 1e-24 ? sqrt(d2) : 1e30;
}

// How many cells k_wrap moved atom i by along each periodic axis: the same expression, so the same floor.
__device__ inline void wrap_count(const Geom& g, int i, int n[3]) {
  const int b = g.sid[i], per = g.sper[b];
  n[0] = n[1] = n[2] = 0;
  if (!per) return;
  const double* ci = g.cinv + 9 * b;
  const double x = g.pos[3 * i], y = g.pos[3 * i + 1], z = g.pos[3 * i + 2];
  for (int d = 0; d < 3; ++d) {
    const double f = x * ci[d] + y * ci[3 + d] + z * ci[6 + d];
    n[d] = (per >> d & 1) ? (int) floor(f) : 0;
  }
}

// A searched pair's image in terms of the unwrapped positions: posw = pos - n.cell, so
// posw_j + s.cell - posw_i = pos_j + (s - n_j + n_i).cell - pos_i (src/device_geometry.cpp:176-181).
__global__ void k_unwrap_shifts(RawEdges re, Geom g, int* __restrict__ out) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= re.E) return;
  int ni[3], nj[3];
  wrap_count(g, re.i[e], ni);
  wrap_count(g, re.j[e], nj);
  for (int d = 0; d < 3; ++d) out[3 * e + d] = re.shift[3 * e + d] - nj[d] + ni[d];
}

// The Verlet test (src/device_geometry.cpp:283-307): a pair outside the cached list was more than `reach` apart at
// the search; it cannot be inside the cutoff now while 2 d + reach |D - I|_F < skin, d the largest move in the
// strained frame and D = H0^-1 H the strain since. worst = the largest such sum over the atoms.
__global__ void k_verlet_check(Geom g, const double* __restrict__ pos0, const double* __restrict__ cinv0, double reach,
                               unsigned long long* __restrict__ worst) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= g.Ntot) return;
  const int b = g.sid[i];
  const double* c0 = cinv0 + 9 * b;
  const double* h = g.scell + 9 * b;
  double e2 = 0.0;
  for (int a = 0; a < 3; ++a)
    for (int d = 0; d < 3; ++d) {
      double x = a == d ? -1.0 : 0.0;
      for (int k = 0; k < 3; ++k) x += c0[3 * a + k] * h[3 * k + d];
      e2 += x * x;
    }
  double ds[3], d2 = 0.0;
  for (int d = 0; d < 3; ++d) {
    ds[d] = 0.0;
    for (int k = 0; k < 3; ++k) ds[d] += (g.pos[3 * i + k] - pos0[3 * i + k]) * c0[3 * k + d];
  }
  for (int d = 0; d < 3; ++d) {
    const double x = ds[0] * h[d] + ds[1] * h[3 + d] + ds[2] * h[6 + d];
    d2 += x * x;
  }
  double m = 2.0 * sqrt(d2) + reach * sqrt(e2);
  if (!(m == m)) m = 1e300;  // a NaN position or cell: search again, and let the search report it
  atomicMax(worst, (unsigned long long) __double_as_longlong(m));  // non-negative doubles order as their bits
}

// The smooth cutoff factor, argument and transcendentals in float as the reference
// evaluates them (include/pet/cutoff.hpp:17-26).
__device__ inline double cutoff_value(double d, double rc, double width, int kind) {
  const float pi = (float) 3.14159265358979323846;
  if (kind == 0) {
    const float x = (float) ((d - (rc - width)) / width);
    if (x <= 0.0f) return 1.0;
    if (x >= 1.0f) return 0.0;
    return 0.5 * (1.0 + (double) tanhf(1.0f / tanf(pi * x)));
  }
  const float x = fminf(fmaxf((float) ((d - (rc - width)) / width), 0.0f), 1.0f);
  return 0.5 * (1.0 + (double) cosf(pi * x));
}

// One warp per centre atom: its kept-edge count (d <= rc), and the largest count.
// An edge's own cutoff: the model's, or the mean of its two atoms' adaptive cutoffs (src/device_neighbors.cpp:243-246).
__device__ __forceinline__ double edge_cutoff(const double* acut, const int* nbr, int a, int e, double rc) {
  return acut ? 0.5 * (acut[a] + acut[nbr[e]]) : rc;
}

__global__ void k_keep_count(int NC, const int* __restrict__ roff, const double* __restrict__ dist, double rc,
                             int* __restrict__ kcnt, int* __restrict__ maxm, unsigned long long* __restrict__ pairs,
                             const double* __restrict__ acut, const int* __restrict__ nbr) {
  const int a = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (a >= NC) return;
  int c = 0;
  for (int e = roff[a] + lane; e < roff[a + 1]; e += 32) c += dist[e] <= edge_cutoff(acut, nbr, a, e, rc);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if (lane == 0) {
    kcnt[a] = c;
    atomicMax(maxm, c);
    atomicAdd(pairs, (unsigned long long) (c + 1) * (unsigned long long) (c + 1));  // tokens^2, an integer sum
  }
}

// One warp per centre atom: its kept edges to their packed rows, in raw order.
__global__ void k_pack(int NC, RawEdges re, PackedEdges pk, CutoffSpec cs) {
  const int a = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (a >= NC) return;
  int row = pk.off[a];
  const int row_end = pk.off[a + 1];  // with fixed shapes an atom's rows may be fewer than its kept edges (overflow)
  const int e1 = re.off[a + 1];
  for (int e0 = re.off[a]; e0 < e1; e0 += 32) {
    const int e = e0 + lane;
    const double rc = e < e1 ? edge_cutoff(pk.adaptive.acut, re.j, a, e, cs.cutoff) : 0.0;
    const bool keep = e < e1 && re.dist[e] <= rc;
    const unsigned m = __ballot_sync(0xffffffffu, keep);
    if (e < e1) {
      const int p = row + __popc(m & ((1u << lane) - 1u));
      if (keep && p < row_end) {
        const int j = re.j[e];
        pk.packed_of_raw[e] = p;
        pk.raw_of[p] = e;
        pk.center[p] = a;
        pk.nbr[p] = j;
        pk.species[p] = pk.atom_species[j];
        pk.vec[3 * p] = re.vec[3 * e], pk.vec[3 * p + 1] = re.vec[3 * e + 1], pk.vec[3 * p + 2] = re.vec[3 * e + 2];
        pk.dist[p] = re.dist[e];
        pk.cut[p] = (float) cutoff_value(re.dist[e], rc, cs.width, cs.kind);
        if (pk.rc) pk.rc[p] = rc;
      } else {
        pk.packed_of_raw[e] = -1;
      }
    }
    row += __popc(m);
  }
}

__global__ void k_pack_reverse(PackedEdges pk, const int* __restrict__ raw_reverse) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= pk.E) return;
  if (p >= pk.off[pk.N]) {  // a capacity's dead row: no atom's, no partner
    pk.reverse[p] = -1;
    return;
  }
  const int r = raw_reverse[pk.raw_of[p]];
  pk.reverse[p] = r >= 0 ? pk.packed_of_raw[r] : -1;
}

// Fixed shapes: more kept edges than rows, or more of one atom's than the attention kernels were sized for.
__global__ void k_check_capacity(const int* __restrict__ off, int NC, const int* __restrict__ maxm, int e_cap, int m_cap,
                                 int* __restrict__ overflow) {
  if (off[NC] > e_cap || *maxm > m_cap) *overflow = 1;
}
// A step that does not fit still has to stay inside its buffers until the host sees the flag and redoes it: no atom
// keeps more than m_cap rows, and no row lies past e_cap.
__global__ void k_clamp_counts(int* __restrict__ kcnt, int NC, int m_cap) {
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a < NC && kcnt[a] > m_cap) kcnt[a] = m_cap;
}
__global__ void k_clamp_offsets(int* __restrict__ off, int NC, int e_cap) {
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a <= NC && off[a] > e_cap) off[a] = e_cap;
}

}  // namespace

void wrap_positions(Stream& st, const Geom& g, double* posw) {
  if (g.Ntot == 0) return;
  k_wrap<<<cdiv(g.Ntot, 256), 256, 0, st.s>>>(g, posw);
  PETB_LAUNCH_CHECK(st);
}

RawEdges cell_list_search(Stream& st, Arena& arena, const Geom& g, const double* posw, double cutoff) {
  const int N = g.Ntot, nbins = g.nbins > 0 ? g.nbins : 1;
  // 52 bytes per raw edge and 56 per atom: the reference's own count (tools/roofline.py:308-309).
  const ProfScope ps(st, PC_GEOMETRY, 0.0, 56.0 * N);
  RawEdges re;
  re.off = arena.alloc<int>(N + 1);
  if (N == 0) {
    PETB_CUDA(cudaMemsetAsync(re.off, 0, sizeof(int), st.s));
    return re;
  }
  int* abin = arena.alloc<int>(N);
  int* bcnt = arena.alloc<int>(2 * size_t(nbins));  // counts, then fill cursors
  int* fill = bcnt + nbins;
  int* bstart = arena.alloc<int>(nbins + 1);
  int* unsorted = arena.alloc<int>(N);
  int* batom = arena.alloc<int>(N);
  int* ecnt = arena.alloc<int>(N);
  PETB_CUDA(cudaMemsetAsync(bcnt, 0, 2 * size_t(nbins) * sizeof(int), st.s));
  k_assign_bins<<<cdiv(N, 256), 256, 0, st.s>>>(g, posw, abin, bcnt);
  PETB_LAUNCH_CHECK(st);
  exclusive_scan(st, arena, bcnt, bstart, nbins);
  k_fill_bins<<<cdiv(N, 256), 256, 0, st.s>>>(N, abin, bstart, fill, unsorted);
  PETB_LAUNCH_CHECK(st);
  k_sort_bins<<<cdiv(size_t(nbins) * 32, 128), 128, 0, st.s>>>(nbins, bstart, unsorted, batom);
  PETB_LAUNCH_CHECK(st);

  const Walk w{g, posw, abin, bstart, batom, cutoff * cutoff};
  k_walk<false><<<cdiv(size_t(N) * 32, 128), 128, 0, st.s>>>(w, ecnt, nullptr, re);
  PETB_LAUNCH_CHECK(st);
  exclusive_scan(st, arena, ecnt, re.off, N);
  int E = 0;
  PETB_CUDA(cudaMemcpyAsync(&E, re.off + N, sizeof(int), cudaMemcpyDeviceToHost, st.s));
  PETB_CUDA(cudaStreamSynchronize(st.s));
  re.E = E;
  const size_t Ea = E > 0 ? E : 1;
  re.i = arena.alloc<int>(Ea);
  re.j = arena.alloc<int>(Ea);
  re.shift = arena.alloc<int>(3 * Ea);
  re.vec = arena.alloc<double>(3 * Ea);
  re.dist = arena.alloc<double>(Ea);
  re.reverse = arena.alloc<int>(Ea);
  // The count and the fill are the same instantiated walk over the same inputs with
  // contraction off, so they agree on every candidate.
  k_walk<true><<<cdiv(size_t(N) * 32, 128), 128, 0, st.s>>>(w, nullptr, re.off, re);
  PETB_LAUNCH_CHECK(st);
  return re;
}

void find_reverse(Stream& st, const RawEdges& re, int) {
  if (re.E == 0) return;
  const ProfScope ps(st, PC_GEOMETRY, 0.0, 52.0 * re.E);
  k_reverse<<<cdiv(re.E, 256), 256, 0, st.s>>>(re);
  PETB_LAUNCH_CHECK(st);
}

void edge_vectors(Stream& st, const RawEdges& re, const double* pos, const double* cell9) {
  if (re.E == 0) return;
  k_edge_vectors<<<cdiv(re.E, 256), 256, 0, st.s>>>(re, pos, cell9);
  PETB_LAUNCH_CHECK(st);
}

void edge_vectors_batch(Stream& st, const RawEdges& re, const Geom& g) {
  if (re.E == 0) return;
  const ProfScope ps(st, PC_GEOMETRY, 0.0, 52.0 * re.E);
  k_edge_vectors_batch<<<cdiv(re.E, 256), 256, 0, st.s>>>(re, g);
  PETB_LAUNCH_CHECK(st);
}

void unwrap_shifts(Stream& st, const RawEdges& re, const Geom& g, int* out) {
  if (re.E == 0) return;
  k_unwrap_shifts<<<cdiv(re.E, 256), 256, 0, st.s>>>(re, g, out);
  PETB_LAUNCH_CHECK(st);
}

void verlet_check(Stream& st, const Geom& g, const double* pos0, const double* cinv0, double reach, double* worst) {
  PETB_CUDA(cudaMemsetAsync(worst, 0, sizeof(double), st.s));
  if (g.Ntot == 0) return;
  k_verlet_check<<<cdiv(g.Ntot, 256), 256, 0, st.s>>>(g, pos0, cinv0, reach, reinterpret_cast<unsigned long long*>(worst));
  PETB_LAUNCH_CHECK(st);
}

PackedEdges pack_edges(Stream& st, Arena& arena, const RawEdges& re, int NC, const int* atom_species,
                       const CutoffSpec& cs, int* pinned, const AdaptiveCut& ad) {
  PackedEdges pk;
  pk.N = NC;
  pk.adaptive = ad;
  pk.atom_species = atom_species;
  pk.off = arena.alloc<int>(NC + 1);
  const ProfScope ps(st, PC_GEOMETRY, 0.0, 60.0 * double(re.E) + 8.0 * NC);
  int* kcnt = arena.alloc<int>(NC + 4);
  int* maxm = kcnt + NC;
  unsigned long long* pairs = reinterpret_cast<unsigned long long*>(arena.alloc_bytes(8));
  PETB_CUDA(cudaMemsetAsync(maxm, 0, sizeof(int), st.s));
  PETB_CUDA(cudaMemsetAsync(pairs, 0, 8, st.s));
  if (NC > 0) {
    k_keep_count<<<cdiv(size_t(NC) * 32, 256), 256, 0, st.s>>>(NC, re.off, re.dist, cs.cutoff, kcnt, maxm, pairs, ad.acut, re.j);
    PETB_LAUNCH_CHECK(st);
  }
  exclusive_scan(st, arena, kcnt, pk.off, NC);
  PETB_CUDA(cudaMemcpyAsync(pinned, pk.off + NC, sizeof(int), cudaMemcpyDeviceToHost, st.s));
  PETB_CUDA(cudaMemcpyAsync(pinned + 1, maxm, sizeof(int), cudaMemcpyDeviceToHost, st.s));
  PETB_CUDA(cudaMemcpyAsync(pinned + 2, pairs, 8, cudaMemcpyDeviceToHost, st.s));
  PETB_CUDA(cudaStreamSynchronize(st.s));
  pk.E = pinned[0];
  pk.M = pinned[1] > 1 ? pinned[1] : 1;
  pk.pairs = double(*reinterpret_cast<unsigned long long*>(pinned + 2));
  const size_t Ea = pk.E > 0 ? pk.E : 1, Er = re.E > 0 ? re.E : 1;
  pk.center = arena.alloc<int>(Ea);
  pk.nbr = arena.alloc<int>(Ea);
  pk.species = arena.alloc<int>(Ea);
  pk.reverse = arena.alloc<int>(Ea);
  pk.vec = arena.alloc<double>(3 * Ea);
  pk.dist = arena.alloc<double>(Ea);
  pk.cut = arena.alloc<float>(Ea);
  if (ad.acut) pk.rc = arena.alloc<double>(Ea);
  pk.raw_of = arena.alloc<int>(Ea);
  pk.packed_of_raw = arena.alloc<int>(Er);
  if (NC > 0 && re.E > 0) {
    k_pack<<<cdiv(size_t(NC) * 32, 256), 256, 0, st.s>>>(NC, re, pk, cs);
    PETB_LAUNCH_CHECK(st);
    // Edges whose centre is not a centre atom here (ghost rows of an exchanged list) keep no row.
    if (pk.E > 0) {
      k_pack_reverse<<<cdiv(pk.E, 256), 256, 0, st.s>>>(pk, re.reverse);
      PETB_LAUNCH_CHECK(st);
    }
  }
  return pk;
}

// The same with the shapes given: E_cap rows (the kept edges packed into the first of them, the rest dead: zero
// geometry, zero weight, no partner, in no atom's range) and M_cap as the most edges of an atom, so that nothing
// is read back and a stepping loop keeps one set of shapes (the reference's edge_capacity, src/model.cpp:549-567).
// *overflow is set on the device when the step does not fit; the caller reads it with the results.
PackedEdges pack_edges_fixed(Stream& st, Arena& arena, const RawEdges& re, int NC, const int* atom_species, const CutoffSpec& cs,
                             int e_cap, int m_cap, double pairs, int* overflow, const AdaptiveCut& ad) {
  PackedEdges pk;
  pk.N = NC, pk.E = e_cap, pk.M = m_cap, pk.pairs = pairs;
  pk.adaptive = ad;
  pk.atom_species = atom_species;
  pk.off = arena.alloc<int>(NC + 1);
  const ProfScope ps(st, PC_GEOMETRY, 0.0, 60.0 * double(re.E) + 8.0 * NC);
  int* kcnt = arena.alloc<int>(NC + 4);
  int* maxm = kcnt + NC;
  unsigned long long* pr = reinterpret_cast<unsigned long long*>(arena.alloc_bytes(8));
  PETB_CUDA(cudaMemsetAsync(maxm, 0, sizeof(int), st.s));
  PETB_CUDA(cudaMemsetAsync(pr, 0, 8, st.s));
  k_keep_count<<<cdiv(size_t(NC) * 32, 256), 256, 0, st.s>>>(NC, re.off, re.dist, cs.cutoff, kcnt, maxm, pr, ad.acut, re.j);
  PETB_LAUNCH_CHECK(st);
  k_clamp_counts<<<cdiv(NC, 256), 256, 0, st.s>>>(kcnt, NC, m_cap);  // maxm already holds the unclamped maximum
  PETB_LAUNCH_CHECK(st);
  exclusive_scan(st, arena, kcnt, pk.off, NC);
  k_check_capacity<<<1, 1, 0, st.s>>>(pk.off, NC, maxm, e_cap, m_cap, overflow);
  PETB_LAUNCH_CHECK(st);
  k_clamp_offsets<<<cdiv(NC + 1, 256), 256, 0, st.s>>>(pk.off, NC, e_cap);
  PETB_LAUNCH_CHECK(st);
  const size_t Ea = e_cap > 0 ? e_cap : 1, Er = re.E > 0 ? re.E : 1;
  // one block for the row arrays, cleared in one go: dead rows read as zeros
  const size_t bytes = Ea * (4 * 4 + 3 * 8 + 8 + 4 + 4);
  char* block = static_cast<char*>(arena.alloc_bytes(bytes + 64));
  PETB_CUDA(cudaMemsetAsync(block, 0, bytes + 64, st.s));
  pk.vec = reinterpret_cast<double*>(block), block += 24 * Ea;
  pk.dist = reinterpret_cast<double*>(block), block += 8 * Ea;
  pk.center = reinterpret_cast<int*>(block), block += 4 * Ea;
  pk.nbr = reinterpret_cast<int*>(block), block += 4 * Ea;
  pk.species = reinterpret_cast<int*>(block), block += 4 * Ea;
  pk.raw_of = reinterpret_cast<int*>(block), block += 4 * Ea;
  pk.cut = reinterpret_cast<float*>(block), block += 4 * Ea;
  pk.reverse = reinterpret_cast<int*>(block);
  if (ad.acut) {
    pk.rc = arena.alloc<double>(Ea);
    PETB_CUDA(cudaMemsetAsync(pk.rc, 0, 8 * Ea, st.s));
  }
  pk.packed_of_raw = arena.alloc<int>(Er);
  if (re.E > 0) {
    k_pack<<<cdiv(size_t(NC) * 32, 256), 256, 0, st.s>>>(NC, re, pk, cs);
    PETB_LAUNCH_CHECK(st);
  }
  if (e_cap > 0) {
    k_pack_reverse<<<cdiv(e_cap, 256), 256, 0, st.s>>>(pk, re.reverse);
    PETB_LAUNCH_CHECK(st);
  }
  return pk;
}

}  // namespace petb
