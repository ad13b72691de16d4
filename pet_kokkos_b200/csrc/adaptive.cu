// The adaptive cutoff: each atom's own cutoff radius from the smoothed count of its neighbours, and the
// gradient that flows back through it to every raw edge of the atom (kept by the network or not).
//
// Forward (the reference's solver_cutoffs / grid_cutoffs, src/device_neighbors.cpp:26-136): both schemes
// taper the neighbour count with the bump function whatever the model's own cutoff function.
//   solver  Newton-bisection for the r where n(r) = sum_j bump(d_j, r) + target (r / rmax)^3 reaches target,
//           then one implicit-function step; the root r and the slope dn there are kept for the backward;
//   grid    eff(a, p) = sum_j bump(d_j, probe_p); the cutoff is the softmax-weighted mean of the probes,
//           weighted by how close each probe's count is to target; eff is kept for the backward.
// An edge is kept when it is within the mean of its two atoms' cutoffs (src/device_neighbors.cpp:243-252).
// Backward (adaptive_part / adaptive_backward, src/forces.cpp:80-260,308-341): each kept edge's pair-cutoff
// adjoint goes half to each end; each atom's cutoff adjoint becomes a radial gradient on all its raw edges;
// those are folded into forces and virial over the raw list, a warp per atom in a fixed order.
// Geometry arithmetic is fp64 with the transcendentals in float, as the reference evaluates them.
#include "neighbors.h"
#include "ops.h"

namespace petb {

namespace {

constexpr double kMinCutoffFactor = 1.0 / 16.0, kSlopeFloor = 1e-6;  // include/pet/cutoff.hpp:53-57
constexpr int kSolverIters = 10;

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ inline double bump(double d, double rc, double width) {
  const float pi = (float) 3.14159265358979323846;
  const float x = (float) ((d - (rc - width)) / width);
  if (x <= 0.0f) return 1.0;
  if (x >= 1.0f) return 0.0;
  return 0.5 * (1.0 + (double) tanhf(1.0f / tanf(pi * x)));
}
// d(bump)/d(rc)  (dev_bump_dcutoff_dr, include/pet/cutoff.hpp:44-51)
__device__ inline double bump_drc(double d, double rc, double width) {
  const float pi = (float) 3.14159265358979323846;
  const float x = (float) ((d - (rc - width)) / width);
  if (x <= 0.0f || x >= 1.0f) return 0.0;
  const float ps = pi * fminf(fmaxf(x, 1e-6f), 1.0f - 1e-6f);
  const float si = sinf(ps);
  const float tt = tanhf(cosf(ps) / si);
  return 0.5 * (1.0 - (double) (tt * tt)) * (double) ((pi / (si * si)) / (float) width);
}
// d(bump)/d(d)  (bump_ddist, src/forces.cpp:22-29)
__device__ inline double bump_dd(double d, double rc, double width) {
  const float pi = (float) 3.14159265358979323846;
  const float x = (float) ((d - (rc - width)) / width);
  if (x <= 0.f || x >= 1.f) return 0.0;
  const float si = sinf(pi * x);
  const float t = tanhf(cosf(pi * x) / si);
  const float du = (-pi / (si * si)) / (float) width;
  return 0.5 * (1.0 - (double) (t * t)) * (double) du;
}

// One warp per atom.
__global__ void __launch_bounds__(256) k_solver(int N, const int* __restrict__ roff, const double* __restrict__ dist,
                                                double rmax, double width, double target, double* __restrict__ acut,
                                                double* __restrict__ root, double* __restrict__ slope) {
  const int a = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (a >= N) return;
  const int e0 = roff[a], e1 = roff[a + 1];
  const double inv_rmax = 1.0 / rmax;
  auto count = [&](double r, double& n, double& dn) {
    double sn = 0.0, sdn = 0.0;
    for (int e = e0 + lane; e < e1; e += 32) sn += bump(dist[e], r, width), sdn += bump_drc(dist[e], r, width);
    sn = warp_sum_d(sn), sdn = warp_sum_d(sdn);
    const double x = r * inv_rmax;
    n = sn + target * x * x * x;
    dn = sdn + 3.0 * target * x * x * inv_rmax;
  };
  double r_lo = 0.0, r_hi = rmax, r = 0.5 * rmax, n, dn;
  for (int it = 0; it < kSolverIters; ++it) {
    count(r, n, dn);
    const double f = n - target;
    if (f <= 0.0) r_lo = r;
    else r_hi = r;
    const double newton = r - f / fmax(dn, kSlopeFloor);
    r = (newton >= r_lo && newton <= r_hi) ? newton : 0.5 * (r_lo + r_hi);
  }
  count(r, n, dn);
  const double dn_root = fmax(dn, kSlopeFloor), lo_bound = rmax * kMinCutoffFactor;
  const double adapted = fmin(fmax(r - (n - target) / dn_root, lo_bound), rmax);
  if (lane == 0) {
    acut[a] = adapted;
    root[a] = r;
    slope[a] = (adapted > lo_bound && adapted < rmax) ? dn_root : 0.0;
  }
}

// One warp per atom, lanes striding the probes: each walks the atom's edges in order (a serial sweep's sums).
__global__ void __launch_bounds__(256) k_grid_eff(int N, int P, const int* __restrict__ roff, const double* __restrict__ dist,
                                                  const double* __restrict__ probes, double width, double* __restrict__ eff) {
  const int a = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (a >= N) return;
  for (int p = lane; p < P; p += 32) {
    const double pr = probes[p];
    double s = 0.0;
    for (int e = roff[a]; e < roff[a + 1]; ++e) s += bump(dist[e], pr, width);
    eff[size_t(a) * P + p] = s;
  }
}

__device__ inline double grid_diff(const double* eff, int p, int P, double target) {
  const double x = P > 1 ? (double) p / (P - 1) : 0.0;
  return eff[p] - target + target * x * x * x;
}
__device__ inline double grid_stencil(const double* eff, int p, int P, double target) {  // torch.gradient
  if (p == 0) return grid_diff(eff, 1, P, target) - grid_diff(eff, 0, P, target);
  if (p == P - 1) return grid_diff(eff, P - 1, P, target) - grid_diff(eff, P - 2, P, target);
  return 0.5 * (grid_diff(eff, p + 1, P, target) - grid_diff(eff, p - 1, P, target));
}

// One thread per atom: the softmax-weighted mean of the probes.
__global__ void k_grid_cutoff(int N, int P, const double* __restrict__ eff_all, const double* __restrict__ probes, double target,
                              double* __restrict__ acut) {
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= N) return;
  const double* eff = eff_all + size_t(a) * P;
  auto logw = [&](int p) {
    const double d = grid_diff(eff, p, P, target);
    const double g = P == 1 ? fabs(d) * 0.5 + 1e-12 : fmax(fabs(grid_stencil(eff, p, P, target)), 1e-12);
    const double r = d / g;
    return -0.5 * r * r;
  };
  double mx = -1e300, sum = 0.0, acc = 0.0;
  for (int p = 0; p < P; ++p) mx = fmax(mx, logw(p));
  for (int p = 0; p < P; ++p) {
    const double w = exp(logw(p) - mx);
    sum += w, acc += probes[p] * w;
  }
  acut[a] = acc / sum;
}

// adapted_adj(a) = sum over a's kept edges of half the edge's and half its partner's pair-cutoff adjoint.
__global__ void k_adapted_adj(PackedEdges pk, const double* __restrict__ pc_adj, double* __restrict__ adapted_adj) {
  const int a = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (a >= pk.n_atoms) return;
  double s = 0.0;
  if (a < pk.N)
    for (int k = pk.off[a] + lane; k < pk.off[a + 1]; k += 32) {
      s += 0.5 * pc_adj[k];
      const int r = pk.reverse[k];
      if (r >= 0) s += 0.5 * pc_adj[r];
    }
  s = warp_sum_d(s);
  if (lane == 0) adapted_adj[a] = s;
}

// Solver: d(cutoff)/d(d_j) = -(1/dn) dn_total/dd_j with r and dn held constant  (src/forces.cpp:93-110).
__global__ void k_gmag_solver(int E, const int* __restrict__ center, const double* __restrict__ dist,
                              const double* __restrict__ root, const double* __restrict__ slope,
                              const double* __restrict__ adapted_adj, double width, double scale, double* __restrict__ gmag) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  const int c = center[e];
  const double d = dist[e];
  gmag[e] = (d <= 0.0 || slope[c] <= 0.0) ? 0.0 : scale * adapted_adj[c] * (-bump_dd(d, root[c], width) / slope[c]) / d;
}

// Grid: the adjoint of the softmax-weighted mean through the weights and the gradient stencil back to eff
// (src/forces.cpp:111-196). One thread per atom writes diff_adj(a, :).
__global__ void k_grid_backward(int N, int P, const double* __restrict__ eff_all, const double* __restrict__ probes,
                                double target, const double* __restrict__ adapted_adj, double* __restrict__ diff_adj_all,
                                double* __restrict__ cq_all) {
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= N) return;
  const double* eff = eff_all + size_t(a) * P;
  double* diff_adj = diff_adj_all + size_t(a) * P;
  double* cq = cq_all + size_t(a) * P;
  auto grad_of = [&](int p, double& gs) {
    const double g = grid_stencil(eff, p, P, target), ag = fabs(g);
    gs = ag >= 1e-12 ? (g > 0.0 ? 1.0 : (g < 0.0 ? -1.0 : 0.0)) : 0.0;
    return ag > 1e-12 ? ag : 1e-12;
  };
  double mx = -1e300, sum = 0.0, cutoff = 0.0, gs;
  for (int p = 0; p < P; ++p) {
    const double r = grid_diff(eff, p, P, target) / grad_of(p, gs);
    mx = fmax(mx, -0.5 * r * r);
  }
  for (int p = 0; p < P; ++p) {
    const double r = grid_diff(eff, p, P, target) / grad_of(p, gs);
    sum += exp(-0.5 * r * r - mx);
  }
  for (int p = 0; p < P; ++p) {
    const double r = grid_diff(eff, p, P, target) / grad_of(p, gs);
    cutoff += probes[p] * (exp(-0.5 * r * r - mx) / sum);
  }
  for (int p = 0; p < P; ++p) {
    const double d = grid_diff(eff, p, P, target), gd = grad_of(p, gs), r = d / gd;
    const double w = exp(-0.5 * r * r - mx) / sum;
    const double A = adapted_adj[a] * w * (probes[p] - cutoff);
    diff_adj[p] = A * (-(d / (gd * gd)));
    cq[p] = A * (d * d / (gd * gd * gd)) * gs;
  }
  for (int r = 0; r < P; ++r) {  // the adjoint of the gradient stencil
    double B = 0.0;
    if (r - 1 >= 1 && r - 1 <= P - 2) B += 0.5 * cq[r - 1];
    if (r + 1 >= 1 && r + 1 <= P - 2) B += -0.5 * cq[r + 1];
    if (r == 1) B += cq[0];
    if (r == 0) B += -cq[0];
    if (r == P - 1) B += cq[P - 1];
    if (r == P - 2) B += -cq[P - 1];
    diff_adj[r] += B;
  }
}

// bump_dd(d, probe) is 0 unless the probe lies in (d, d + width): a few probes of the uniform grid.
__global__ void k_gmag_grid(int E, int P, const int* __restrict__ center, const double* __restrict__ dist,
                            const double* __restrict__ probes, const double* __restrict__ diff_adj, double width, double scale,
                            double* __restrict__ gmag) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  const double d = dist[e];
  if (d <= 0.0) {
    gmag[e] = 0.0;
    return;
  }
  const double p0 = probes[0], dp = P > 1 ? probes[1] - probes[0] : 1.0;
  const int lo = max((int) floor((d - p0) / dp), 0), hi = min((int) ceil((d + width - p0) / dp) + 1, P);
  double da = 0.0;
  for (int p = lo; p < hi; ++p) da += diff_adj[size_t(center[e]) * P + p] * bump_dd(d, probes[p], width);
  gmag[e] = scale * da / d;
}

// The same gather as the main fold, over the raw list: the partner's vector is minus this edge's and it enters with
// a minus sign, so it adds. A warp per atom, a fixed combination order.
__global__ void __launch_bounds__(256) k_raw_fold(int N, RawEdges re, const double* __restrict__ gmag, double* __restrict__ forces,
                                                  double* __restrict__ vir_atom) {
  const int a = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (a >= N) return;
  double s[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
  for (int e = re.off[a] + lane; e < re.off[a + 1]; e += 32) {
    const double ge = gmag[e], gr = re.reverse[e] >= 0 ? gmag[re.reverse[e]] : 0.0;
    const double* v = re.vec + 3 * size_t(e);
    for (int c = 0; c < 3; ++c) s[c] += (ge + gr) * v[c];
    for (int x = 0; x < 3; ++x)
      for (int y = 0; y < 3; ++y) s[3 + x * 3 + y] += v[x] * ge * v[y];
  }
  for (int t = 0; t < 12; ++t) s[t] = warp_sum_d(s[t]);
  if (lane == 0) {
    for (int c = 0; c < 3; ++c) forces[3 * size_t(a) + c] += s[c];
    for (int t = 0; t < 9; ++t) vir_atom[9 * size_t(a) + t] += s[3 + t];
  }
}

}  // namespace

AdaptiveCut adaptive_cutoffs(Stream& st, Arena& arena, const RawEdges& re, int n_atoms, const CutoffSpec& cs) {
  AdaptiveCut ad;
  if (cs.adaptive == 0 || n_atoms == 0) return ad;
  const ProfScope ps(st, PC_GEOMETRY, 0.0, 16.0 * double(re.E) + 24.0 * n_atoms);
  ad.n_atoms = n_atoms, ad.raw = re, ad.probes = cs.probes, ad.P = cs.n_probes;
  double* acut = arena.alloc<double>(n_atoms);
  ad.acut = acut;
  if (cs.adaptive == 2) {
    double* root = arena.alloc<double>(n_atoms);
    double* slope = arena.alloc<double>(n_atoms);
    k_solver<<<cdiv(size_t(n_atoms) * 32, 256), 256, 0, st.s>>>(n_atoms, re.off, re.dist, cs.cutoff, cs.width_adaptive, cs.target,
                                                               acut, root, slope);
    PETB_LAUNCH_CHECK(st);
    ad.root = root, ad.slope = slope;
  } else {
    if (cs.n_probes < 2) throw Error(1, "pet: the grid adaptive cutoff needs at least two probe radii");
    double* eff = arena.alloc<double>(size_t(n_atoms) * cs.n_probes);
    k_grid_eff<<<cdiv(size_t(n_atoms) * 32, 256), 256, 0, st.s>>>(n_atoms, cs.n_probes, re.off, re.dist, cs.probes,
                                                                 cs.width_adaptive, eff);
    PETB_LAUNCH_CHECK(st);
    k_grid_cutoff<<<cdiv(n_atoms, 128), 128, 0, st.s>>>(n_atoms, cs.n_probes, eff, cs.probes, cs.target, acut);
    PETB_LAUNCH_CHECK(st);
    ad.eff = eff;
  }
  return ad;
}

void adaptive_backward(Stream& st, Arena& arena, const PackedEdges& pk, const CutoffSpec& cs, const double* pc_adj, double scale,
                       double* forces, double* vir_atom, double** gmag_out) {
  const AdaptiveCut& ad = pk.adaptive;
  const int N = pk.n_atoms, E = ad.raw.E;
  *gmag_out = nullptr;
  if (!ad.acut || E == 0 || N == 0) return;
  const ProfScope ps(st, PC_FORCES, 60.0 * E, 120.0 * double(E));
  double* adapted_adj = arena.alloc<double>(N);
  double* gmag = arena.alloc<double>(E);
  k_adapted_adj<<<cdiv(size_t(N) * 32, 256), 256, 0, st.s>>>(pk, pc_adj, adapted_adj);
  PETB_LAUNCH_CHECK(st);
  if (cs.adaptive == 2) {
    k_gmag_solver<<<cdiv(E, 256), 256, 0, st.s>>>(E, ad.raw.i, ad.raw.dist, ad.root, ad.slope, adapted_adj, cs.width_adaptive, scale,
                                                 gmag);
    PETB_LAUNCH_CHECK(st);
  } else {
    double* diff_adj = arena.alloc<double>(size_t(N) * ad.P);
    double* cq = arena.alloc<double>(size_t(N) * ad.P);
    k_grid_backward<<<cdiv(N, 128), 128, 0, st.s>>>(N, ad.P, ad.eff, ad.probes, cs.target, adapted_adj, diff_adj, cq);
    PETB_LAUNCH_CHECK(st);
    k_gmag_grid<<<cdiv(E, 256), 256, 0, st.s>>>(E, ad.P, ad.raw.i, ad.raw.dist, ad.probes, diff_adj, cs.width_adaptive, scale, gmag);
    PETB_LAUNCH_CHECK(st);
  }
  k_raw_fold<<<cdiv(size_t(N) * 32, 256), 256, 0, st.s>>>(N, ad.raw, gmag, forces, vir_atom);
  PETB_LAUNCH_CHECK(st);
  *gmag_out = gmag;
}

}  // namespace petb
