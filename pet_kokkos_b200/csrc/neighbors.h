// The device neighbour pipeline: staged geometry -> wrapped positions -> cell-list
// raw edges (ordered, deterministic) -> reverse map -> packed model edges.
//
// It replaces the reference's stage_systems / wrap_positions / search
// (src/device_geometry.cpp:72-161,368-401), build_raw_edges_cells
// (src/device_cell_list.cpp:108-292), edge_topology / edge_geometry
// (src/device_neighbors.cpp:140-324) and pack_edges (src/model.cpp:499-584).
// The edge set, each atom's edge order and the fp64 vectors are the reference's:
// the distance test is evaluated in the same association order without fused
// multiply-adds (this file's kernels are compiled with -fmad=false).
#pragma once

#include "common.h"

namespace petb {

// One batch of B structures, Ntot atoms, staged on the device (the reference's DeviceGeom).
struct Geom {
  int Ntot = 0, B = 0;
  double* pos = nullptr;    // [Ntot,3] unwrapped
  int* sid = nullptr;       // [Ntot] owning structure
  int* spec = nullptr;      // [Ntot] species index
  int* soff = nullptr;      // [B+1] first atom of each structure
  int* sper = nullptr;      // [B] periodic bits
  double* scell = nullptr;  // [B,9]
  double* cinv = nullptr;   // [B,9]
  int* gnc = nullptr;       // [B,3] bins per axis
  int* gnr = nullptr;       // [B,3] search reach in bins
  int* goff = nullptr;      // [B+1] first bin of each structure
  int nbins = 0;
};

// Directed edges grouped by centre atom, in the search's fixed order.
struct RawEdges {
  int E = 0;
  int* i = nullptr;        // [E]
  int* j = nullptr;        // [E]
  int* shift = nullptr;    // [E,3]
  double* vec = nullptr;   // [E,3]
  double* dist = nullptr;  // [E]
  int* off = nullptr;      // [N+1]
  int* reverse = nullptr;  // [E] partner (j,i,-shift) or -1
};

// What an adaptive cutoff's forward leaves for its backward (device pointers; all null for a fixed cutoff).
struct AdaptiveCut {
  const double* acut = nullptr;    // [n_atoms] each atom's cutoff
  const double* root = nullptr;    // [n_atoms] solver: the root r of the neighbour-count equation
  const double* slope = nullptr;   // [n_atoms] solver: dn/dr there, 0 for a clamped cutoff
  const double* eff = nullptr;     // [n_atoms, P] grid: each probe's smoothed neighbour count
  const double* probes = nullptr;  // [P] grid: the probe radii
  int P = 0;
  int n_atoms = 0;
  RawEdges raw;                    // the list the cutoffs were computed from: every edge of it carries gradient
};

// The kept edges as the network reads them (the reference's PackedEdges).
struct PackedEdges {
  int N = 0;          // centre atoms (token rows 0..N-1)
  int n_atoms = 0;    // all atoms, ghosts included
  int n_local = 0;    // atoms whose energy counts
  int E = 0;          // kept edges
  int M = 0;          // most kept edges of any atom
  int B = 1;          // structures
  double pairs = 0.0; // sum over centre atoms of (kept edges + 1)^2: the attention's pair count
  int* off = nullptr;       // [N+1]
  int* center = nullptr;    // [E]
  int* nbr = nullptr;       // [E] neighbour atom
  int* species = nullptr;   // [E] neighbour species
  int* reverse = nullptr;   // [E] packed partner or -1
  double* vec = nullptr;    // [E,3]
  double* dist = nullptr;   // [E]
  float* cut = nullptr;     // [E] smooth cutoff factor
  double* rc = nullptr;     // [E] each edge's own cutoff (the mean of its atoms' adaptive cutoffs); null: the model's
  AdaptiveCut adaptive;
  int* raw_of = nullptr;    // [E] the raw edge this row came from
  int* packed_of_raw = nullptr;  // [E_raw] or -1
  const int* atom_species = nullptr;  // [n_atoms]
  const int* sid = nullptr;           // [n_atoms]
  const int* soff = nullptr;          // [B+1]
  // Over several ranks with an exchange (the reference's remote_map, src/model.cpp:459-497): the kept edges from
  // an owned atom to a ghost ("live"), whose partner rows another rank holds.
  int n_live = 0;
  const int* live_packed = nullptr;  // [n_live] packed row of each live edge, in the engine's order
  const int* remote_of = nullptr;    // [E] live index of a packed row, or -1
  const void* exchange = nullptr;    // the engine's pet_exchange (host pointer), null without one
};

struct CutoffSpec {
  double cutoff, width;
  int kind;  // 0 bump, 1 cosine
  // The adaptive cutoff (Hypers::adaptive, include/pet/config.hpp): 0 none, 1 grid, 2 solver.
  int adaptive = 0;
  double target = 0.0, width_adaptive = 0.5;
  const double* probes = nullptr;  // [n_probes] device, the grid scheme's radii
  int n_probes = 0;
};

// Host-side grid choice for one structure (bins per axis, reach), the reference's cl_grid.
void grid_for_cell(const double cell[9], int periodic_bits, int n_atoms, double cutoff, int nc[3], int nr[3]);
// Host-side inverse cell (rows = lattice vectors), the reference's pet_cellinv.
void invert_cell(const double c[9], double inv[9]);

// The Verlet cache's kernels (the reference's NefCache, src/device_geometry.cpp:165-352): vectors of cached pairs
// from a batch's current positions and cells; a searched list's shifts in terms of the unwrapped positions;
// the test whether a pair outside the cached list could have come inside the cutoff (worst [1], device).
void edge_vectors_batch(Stream& st, const RawEdges& re, const Geom& g);
void unwrap_shifts(Stream& st, const RawEdges& re, const Geom& g, int* out);
void verlet_check(Stream& st, const Geom& g, const double* pos0, const double* cinv0, double reach, double* worst);

// Wrapped positions for the search: posw [Ntot,3].
void wrap_positions(Stream& st, const Geom& g, double* posw);
// The cell-list search. Allocates from `arena`; reads back the edge count once.
RawEdges cell_list_search(Stream& st, Arena& arena, const Geom& g, const double* posw, double cutoff);
// Each raw edge's partner, by a search of the neighbour's own range.
void find_reverse(Stream& st, const RawEdges& re, int N);
// Edge vectors of an engine-supplied list from positions, shifts and the cell (the reference's md_vectors).
void edge_vectors(Stream& st, const RawEdges& re, const double* pos, const double* cell9);
// Keep test, cutoff factors, slots and packing. n_centres <= n_atoms atoms have edges.
PackedEdges pack_edges(Stream& st, Arena& arena, const RawEdges& re, int n_centres, const int* atom_species,
                       const CutoffSpec& cs, int* pinned_scratch, const AdaptiveCut& ad = AdaptiveCut());

// int exclusive scan: out[0..n] (n+1 values, out[n] = total).
void exclusive_scan(Stream& st, Arena& arena, const int* in, int* out, int n);
// Each atom's adaptive cutoff from the raw list (adaptive.cu); an empty result for a model without one.
AdaptiveCut adaptive_cutoffs(Stream& st, Arena& arena, const RawEdges& re, int n_atoms, const CutoffSpec& cs);
PackedEdges pack_edges_fixed(Stream& st, Arena& arena, const RawEdges& re, int NC, const int* atom_species, const CutoffSpec& cs,
                             int e_cap, int m_cap, double pairs, int* overflow, const AdaptiveCut& ad = AdaptiveCut());

}  // namespace petb
