/* pet_b200.h -- C ABI of the B200-native PET energy/forces/virial evaluator.
 *
 * A drop-in for the evaluation path behind the reference's pet::Calculator
 * (include/pet/calculator.hpp:174-319 in peterspackman/pet-kokkos).  The
 * reference has no C ABI of its own: its callers bind the C++ class directly
 * (python/core.cpp:366-390 via nanobind, lammps/ML-PET/pair_pet.cpp:140-167,
 * apps/pet_eval.cpp:561-584).  Every entry point below names the C++ member it
 * replaces; include/pet/calculator.hpp in this repository is a header-only C++
 * facade with the reference's class and struct names over these calls.
 *
 * Conventions (the reference's, calculator.hpp:4-7,120-126): Angstrom, eV,
 * eV/A; forces[Ntot*3] row-major, F = -dE/dx; virial[B*6] is the symmetric
 * W = V*stress in Voigt order xx yy zz xy xz yz; cell is 9 doubles, lattice
 * vectors as rows.  All pointers in these structs are HOST pointers unless a
 * field says "device".  Every function returns 0 on success, a PET_ERR_* code
 * otherwise; pet_last_error() returns the message.  One calculator owns one
 * CUDA device, one stream and its scratch pool; it is not re-entrant
 * (the reference's is not either: calculator.hpp:9-11, gemm.hpp:88-94).
 * There is no CPU fallback: creation fails if no CUDA device is present.
 */
#ifndef PET_B200_H
#define PET_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct pet_calc pet_calc;

enum {
  PET_OK = 0,
  PET_ERR_RUNTIME = 1,       /* std::runtime_error in the reference  */
  PET_ERR_INVALID = 2,       /* std::invalid_argument                */
  PET_ERR_LOGIC = 3,         /* std::logic_error                     */
  PET_ERR_ALLOC = 4,         /* std::bad_alloc / out of device memory */
  PET_ERR_CUDA = 5           /* a CUDA runtime call failed           */
};

/* GemmMode / AttentionMode of the reference (include/pet/gemm.hpp:65). */
enum { PET_GEMM_NATIVE = 0, PET_GEMM_TF32 = 1, PET_GEMM_BF16 = 2, PET_GEMM_TF32X3 = 3 };

/* pet::Options (calculator.hpp:32-117), the subset this path uses. A negative
 * value means "unset": environment (PET_GEMM, PET_GRAPHS, PET_MD_FIXED) then the
 * default. */
typedef struct pet_options {
  int device;               /* CUDA device ordinal; -1: the current device          */
  int gemm_mode;            /* PET_GEMM_*; -1 unset (default native fp32)             */
  int graphs;               /* replay repeated evaluations as a CUDA graph; -1 unset  */
  int md_fixed_shapes;      /* Options::md_fixed_shapes; -1 unset                     */
  size_t memory_budget_bytes; /* 0: ask the device                                     */
  int max_batch_atoms;      /* 0: none                                                */
  int cache_neighbors;      /* Options::cache_neighbors (calculator.hpp:39-40): 1 keeps a staged batch's pairs within
                               cutoff + 1 A between evaluations; 0: PET_CACHE_NEIGHBORS, then off */
  int recompute;            /* Options::recompute (include/pet/config.hpp:19-24): 0 auto (PET_RECOMPUTE, then the first
                               tier that fits the memory budget), 1 never, 2 wide, 3 layers */
  int reserved[6];
} pet_options;

/* pet::System (include/pet/neighbors.hpp:15-25). */
typedef struct pet_system {
  int n_atoms;
  const int* atomic_numbers;   /* [n_atoms]     */
  const double* positions;     /* [n_atoms * 3] */
  double cell[9];
  int pbc[3];
  int charge, spin_multiplicity;
} pet_system;

/* pet::Results (calculator.hpp:120-142). Caller-allocated; a null pointer skips
 * that output. edge_gradient is filled by pet_compute_edges/pet_compute_step
 * when asked for. */
typedef struct pet_results {
  double* energy;           /* [B]        */
  double* per_atom_energy;  /* [Ntot]     */
  double* forces;           /* [Ntot * 3] */
  double* virial;           /* [B * 6]    */
  int* struct_id;           /* [Ntot]     */
  double* edge_gradient;    /* [n_pairs * 3] */
} pet_results;

/* pet::Exchange (include/pet/exchange.hpp:19-41): what an engine supplies when it runs PET over several
 * ranks with ghosts only one cutoff deep. Ghosts then have no pairs of their own; an edge from an owned atom to a
 * ghost reads its partner edge's row from the rank that owns the ghost, once per message-passing layer in the
 * forward and once in the backward. Every pointer handed to the callbacks is a DEVICE pointer; `stream` is the
 * calculator's cudaStream_t. A callback either enqueues its transfers on that stream (NCCL send/recv, peer
 * copies) or synchronizes it, does the transfer its own way and returns once `in` is filled. (The calculator's
 * stream is non-blocking. Work a callback left on the legacy default stream, such as the tail of a blocking
 * cudaMemcpy from pageable memory, is ordered before the calculator's next kernel by the library; work left on any
 * other stream is the callback's to finish.) Every rank makes the
 * same sequence of calls, also with n_live = 0. Return 0, or non-zero to fail the evaluation.
 * (atoms_forward / atoms_reverse of the reference move per-atom values for the adaptive cutoff and D3; they are not
 * part of these callbacks, and an adaptive-cutoff model over an exchange is refused.) */
typedef struct pet_exchange {
  void* user;
  /* Exchange::set_live: once per evaluation, the kept edges to ghosts: live[n_live], ascending indices into the
   * list's owned-atom -> ghost pairs counted in list order (atom by atom, each atom's pairs in turn). */
  int (*set_live)(void* user, const int* live, int n_live, void* stream);
  /* Exchange::edges: out[n_live * width] holds one row per live edge, in set_live's order; send each to the rank
   * owning that ghost and fill in[n_live * width] with the partner edges' rows in the same order. */
  int (*edges)(void* user, const float* out, float* in, int n_live, int width, void* stream);
} pet_exchange;

/* pet::EdgeListView (include/pet/device_geometry.hpp:93-110): an MD engine's own
 * neighbour list. n_local < 0: every atom is owned. */
typedef struct pet_edge_list {
  int n_atoms, n_local;
  const double* positions;      /* [n_atoms * 3]              */
  const int* atomic_numbers;    /* [n_atoms]                  */
  const int* offsets;           /* [n_atoms + 1]              */
  const int* neighbors;         /* [offsets[n_atoms]]         */
  const int* shifts;            /* [offsets[n_atoms] * 3], optional */
  const double* cell;           /* [9], with shifts           */
  int half;
  const pet_exchange* exchange; /* EdgeListView::exchange; null: one rank, or ghosts ghost_cutoff deep. A full list. */
} pet_edge_list;

/* Calculator::DeviceArrays / Totals (calculator.hpp:248-259): DEVICE pointers,
 * [n,3] row-major doubles; forces, per_atom_energy and per_atom_virial are
 * added into. */
typedef struct pet_device_arrays {
  const double* positions;
  double* forces;
  double* per_atom_energy;
  double* per_atom_virial;
  double virial_scale;
} pet_device_arrays;
typedef struct pet_totals {
  double energy;
  double virial[6];
} pet_totals;

/* pet::DeviceEdgeListView (include/pet/device_geometry.hpp:113-135): an engine's full list already in DEVICE
 * memory (LAMMPS's KOKKOS package). Centre ilist[ii], ii < n_centres, has numneigh[i] neighbours
 * neighbors[i * stride_i + k * stride_k] & mask (either layout of the engine's 2-D array; the mask drops the bits the
 * engine keeps above the index). The pairs are taken in atom order, each atom's in list order. With image_of
 * (periodic images instead of ghosts) a neighbour j becomes the owned atom image_of[j] and the lattice shift between
 * them, worked out from positions and cell as they are at the call. Every pointer is device memory except cell. */
typedef struct pet_device_edge_list {
  int n_atoms, n_local, n_centres;
  const int* ilist;
  const int* numneigh;          /* indexed by atom */
  const int* neighbors;
  long stride_i, stride_k;      /* stride_k 0: 1 */
  int mask;                     /* 0: all bits */
  const int* atomic_numbers;    /* [n_atoms] */
  const int* image_of;          /* [n_atoms], optional */
  const double* positions;      /* [n_atoms * 3], with image_of */
  const double* cell;           /* HOST [9], with image_of */
  const pet_exchange* exchange; /* as pet_edge_list's */
} pet_device_edge_list;

/* pet::DevicePairListView (include/pet/device_geometry.hpp:137-154): an engine's pairs as a flat list in DEVICE
 * memory, in any order, as metatomic hands them over. Pair k is atom pairs[k * stride_pair] ->
 * pairs[k * stride_pair + stride_col], shifted by the next three columns (lattice vectors, as pet_edge_list's
 * shifts). A full list. With renumber (device, [n_atoms]) the engine's atom a is atom renumber[a] here, the positions
 * of every step are permuted the same way, and the results come back in this numbering. Each atom's pairs keep
 * their order in the list. */
typedef struct pet_pair_list {
  int n_atoms, n_local, n_pairs;
  const int* pairs;             /* device */
  long stride_pair, stride_col; /* 0, 0: 5 and 1 */
  const int* atomic_numbers;    /* device [n_atoms], the engine's numbering */
  const int* renumber;          /* device [n_atoms], optional */
} pet_pair_list;

/* pet::BatchResult of one structure (calculator.hpp:144-165): DEVICE pointers into the calculator's own buffers,
 * valid until its next evaluation. forces and virial are null when forces were not asked for. */
typedef struct pet_device_results {
  int n_atoms;
  const double* energy;          /* [1]           */
  const double* per_atom_energy; /* [n_atoms]     */
  const double* forces;          /* [n_atoms * 3] */
  const double* virial;          /* [6]           */
} pet_device_results;

/* The raw neighbour list of a batch as the device search lists it
 * (pet::RawEdges, include/pet/device_cell_list.hpp:52-59). Caller-allocated with
 * capacity `capacity` edges; n_edges receives the count (the call fails with
 * PET_ERR_INVALID and sets n_edges if capacity is too small). */
typedef struct pet_raw_edges {
  int capacity, n_edges;
  int* i;          /* [E] centre, global atom index    */
  int* j;          /* [E] neighbour, global atom index */
  int* shift;      /* [E * 3]                          */
  double* vec;     /* [E * 3] r_j + shift.cell - r_i   */
  double* dist;    /* [E]                              */
  int* reverse;    /* [E] the (j, i, -shift) edge or -1 (optional) */
  float* cutoff;   /* [E] smooth cutoff factor (optional)           */
} pet_raw_edges;

/* Calculator::Calculator(model_json, model_weights, opts) (calculator.hpp:179). */
int pet_calc_create(const char* model_json, const char* model_weights, const pet_options* opts, pet_calc** out);
/* Calculator::~Calculator. */
void pet_calc_destroy(pet_calc* c);
/* The message of the last failed call on `c` (or of a failed create when c is null). */
const char* pet_last_error(const pet_calc* c);

/* Calculator::compute(const System&, bool) and compute(const std::vector<System>&, bool)
 * (calculator.hpp:187,192; the batched form is what python/core.cpp:376 exposes as compute_batch). */
int pet_compute(pet_calc* c, const pet_system* systems, int n_systems, int compute_forces, pet_results* out);

/* Calculator::stage (calculator.hpp:214) and compute_device (:219): structures
 * staged once in device memory, evaluated there; results stay on the device
 * until pet_fetch_results. */
int pet_stage(pet_calc* c, const pet_system* systems, int n_systems);
int pet_compute_staged(pet_calc* c, int compute_forces);
int pet_fetch_results(pet_calc* c, pet_results* out);
/* pet::DeviceGeom (include/pet/device_geometry.hpp; Calculator::stage, calculator.hpp:210-213): where the staged
 * batch lies on the device. A caller that steps the structures there (a relaxation, MD) writes new positions into
 * `positions` on the calculator's stream or after synchronizing with it, then calls pet_compute_staged. Cells change
 * through pet_update_staged, which also refreshes the inverse cells and the search grid derived from them. */
typedef struct pet_device_geom {
  int n_structures, n_atoms;
  double* positions;         /* [n_atoms * 3] device */
  const double* cells;       /* [n_structures * 9] device */
  const int* struct_id;      /* [n_atoms] device */
  void* stream;              /* the calculator's cudaStream_t */
} pet_device_geom;
int pet_staged_geometry(pet_calc* c, pet_device_geom* out);
/* A staged batch that shrinks (a batched relaxation whose structures finish one by one): keep[n_keep] names the
 * staged structures that stay, in the order they have from now on; they keep the positions they have on the device,
 * and under Options::cache_neighbors their cached pairs follow them, renumbered, without a new search. The
 * reference's compute_device with a smaller DeviceGeom and its `staged` map (calculator.hpp:214-218;
 * cache_reassemble, src/device_geometry.cpp:203-246). */
int pet_keep_staged(pet_calc* c, const int* keep, int n_keep);
/* Moves the staged positions (and cells when non-null) on the device from host arrays. */
int pet_update_staged(pet_calc* c, const double* positions, const double* cells);

/* Calculator::compute_edges (calculator.hpp:227). */
int pet_compute_edges(pet_calc* c, const pet_edge_list* list, int compute_forces, int edge_gradients, pet_results* out);
/* Calculator::set_neighbors(const EdgeListView&) (calculator.hpp:235). */
int pet_set_neighbors(pet_calc* c, const pet_edge_list* list);
/* Calculator::compute_step(positions, cell, forces, edge_gradients) (calculator.hpp:238). With out == NULL the
 * results are left on the device (pet_device_results_of) and nothing is copied back or waited for. */
int pet_compute_step(pet_calc* c, const double* positions, const double* cell, int compute_forces,
                     int edge_gradients, pet_results* out);
/* Calculator::compute_step(const DeviceArrays&, cell) (calculator.hpp:259). */
int pet_compute_step_device(pet_calc* c, const pet_device_arrays* arrays, const double* cell, pet_totals* totals);
/* Calculator::set_neighbors(const DeviceEdgeListView&) (calculator.hpp:236): the list is set once, then stepped
 * with pet_compute_step / pet_compute_step_device. */
int pet_set_neighbors_device(pet_calc* c, const pet_device_edge_list* list);
/* Calculator::compute_pairs (calculator.hpp:260-268): a flat pair list set and evaluated in one call. positions
 * [n_atoms * 3] is device memory in the engine's order, cell [9] host memory (needed with shifts). The results stay
 * on the device (pet_fetch_results copies them out), in the list's numbering. It replaces any list
 * pet_set_neighbors holds; pet_compute_step / pet_compute_step_device then step the same list (a renumbered list
 * takes device positions). */
int pet_compute_pairs(pet_calc* c, const pet_pair_list* pairs, const double* positions, const double* cell,
                      int compute_forces, pet_device_results* out);

/* The device neighbour search alone: build_nef_device's raw list
 * (src/device_geometry.cpp:356-366, src/device_cell_list.cpp:108-292). */
int pet_neighbor_list(pet_calc* c, const pet_system* systems, int n_systems, pet_raw_edges* out);

/* Calculator::cutoff, ghost_cutoff, exchange_ghost_cutoff, energy_scale (calculator.hpp:272-288). */
double pet_cutoff(const pet_calc* c);
double pet_ghost_cutoff(const pet_calc* c);
double pet_exchange_ghost_cutoff(const pet_calc* c);
double pet_energy_scale(const pet_calc* c);
/* Calculator::supports (calculator.hpp:284). */
int pet_supports(const pet_calc* c, int atomic_number);
/* Calculator::workspace_bytes (calculator.hpp:303). */
size_t pet_workspace_bytes(const pet_calc* c);

/* Shapes of the latest evaluation: atoms, kept edges, max neighbours
 * (Calculator::memory_plan, calculator.hpp:307). */
int pet_last_shapes(const pet_calc* c, int* n_atoms, int* n_edges, int* max_neighbors);

/* The latest evaluation's memory decision (Calculator::memory_plan / MemoryPlan, include/pet/model.hpp:23-28,
 * calculator.hpp:305-308): shapes, the recompute tier it ran under (1 never, 2 wide, 3 layers), the bytes estimated
 * for that tier, the budget given (0: what the device has) and what the scratch pools hold now.
 * pet_memory_report writes the same as text with the device's free and total memory (Calculator::memory_report).
 * pet_recommended_batch_atoms: atoms per batch the device can afford, the smaller of what memory allows and where
 * throughput stops improving, known once something has been evaluated (Calculator::recommended_batch_atoms,
 * src/calculator.cpp:921-938). */
typedef struct pet_memory_plan_info {
  int atoms, max_neighbors;
  long edges;
  int tier;
  size_t estimate_bytes, budget_bytes, pool_bytes;
} pet_memory_plan_info;
int pet_memory_plan(const pet_calc* c, pet_memory_plan_info* out);
int pet_memory_report(const pet_calc* c, char* buf, size_t len);
int pet_recommended_batch_atoms(const pet_calc* c);

/* Kernels launched by this library on this calculator since creation, and the
 * device time in milliseconds of the latest evaluation (CUDA events on the
 * calculator's stream). */
long long pet_kernel_launches(const pet_calc* c);
/* Evaluations served by replaying a recorded CUDA graph (Options::graphs; the reference's GraphCache,
 * include/pet/graph.hpp:68-146: eager first, capture second, replay after). */
long long pet_graph_replays(const pet_calc* c);
/* Batches that pet_compute ran as several consecutive pieces to fit Options::memory_budget_bytes /
 * Options::max_batch_atoms (src/calculator.cpp:326-345). */
long long pet_batch_splits(const pet_calc* c);
/* Evaluations that ran out of device memory and were retried with the pools released and the batch cut smaller
 * (the reference's recovery, src/model.cpp:952-971). pet_debug_fail_alloc(k) is the test hook for it: the k-th
 * device allocation of the scratch pools from now (0 = the next) reports out of memory once; k < 0 disarms. */
long long pet_oom_recoveries(const pet_calc* c);
void pet_debug_fail_alloc(long k);
/* Times this calculator has asked the driver how much device memory is free (for the recompute tier and the batch
 * pieces it chooses by itself). The call goes into the kernel-mode driver and waits behind its other clients, so
 * the answer is kept for as long as the calculator's pools keep their size: a steady loop stops asking. */
long long pet_driver_memory_queries(const pet_calc* c);
/* Neighbour searches run for staged batches under Options::cache_neighbors, and the evaluations the cached
 * pairs served instead (the reference's NefCache, include/pet/device_geometry.hpp:198-228). */
long long pet_neighbor_searches(const pet_calc* c);
long long pet_neighbor_reuses(const pet_calc* c);
double pet_last_device_ms(const pet_calc* c);

/* Per-class device timing of evaluations (no counterpart in the reference's API; its
 * kernels are timed through Kokkos Tools labels, tools/roofline.py:431-441).
 * pet_profile(c, 1) starts bracketing launches with CUDA events on the calculator's
 * stream, pet_profile(c, 0) stops; pet_profile_read synchronizes and returns, per
 * kernel class, the brackets seen, their summed milliseconds and the algorithmic flops
 * and bytes of the work inside them, then clears the record. */
typedef struct pet_profile_entry {
  char name[32];
  int launches;
  double ms, flops, bytes;
} pet_profile_entry;
int pet_profile(pet_calc* c, int enable);
int pet_profile_read(pet_calc* c, pet_profile_entry* out, int capacity, int* n);

/* Copies a named intermediate of the latest evaluation to the host as float32
 * (testing aid; names follow the reference's workspace keys). Returns the
 * element count through n; fails if the name is unknown or capacity is short. */
int pet_debug_fetch(pet_calc* c, const char* name, float* out, size_t capacity, size_t* n);

/* One weight GEMM, C[m,n] = A[m,k] . W^T (W is [n,k]) or A . W (W is [k,n]) in the
 * given PET_GEMM_* mode, on host arrays (weight_gemm, src/ops.cpp:18-24; pins
 * tests/test_gemm_modes.cpp:63-103). */
int pet_gemm_host(pet_calc* c, int mode, int w_transposed, int m, int n, int k, const float* A, const float* W, float* C);

/* A ready-made pet_exchange over NCCL: what an MD engine's pair style does around pet::Exchange
 * (lammps/ML-PET/pair_pet.cpp:268-360 routing, :396-472 exchange_rows, :479-555 set_live / edges), inside the
 * library. Rows of edges to ghosts are packed by a kernel, cross with ncclSend / ncclRecv on the calculator's own
 * stream and are unpacked by a kernel: nothing synchronizes the host inside a pass. NCCL is taken from the process at
 * run time (libnccl.so.2), so a program without it still links and runs on one GPU.
 *   pet_nccl_unique_id          rank 0 makes the 128-byte id; the caller hands it to every rank (MPI, a file, ...)
 *   pet_nccl_exchange_create    collective over all ranks. dest[n_remote][2]: for each of this rank's edges from an
 *                               owned atom to a ghost, in list order, (rank, index among that rank's edges to ghosts) of
 *                               its partner edge. owner[n_listed] (optional, with n_total): the atom of the whole cell
 *                               that each listed atom is (itself or its ghost image), for pet_nccl_exchange_reduce.
 *   pet_nccl_exchange_callbacks the pet_exchange to put into pet_edge_list.exchange (valid until destroy)
 *   pet_nccl_exchange_reduce    after an evaluation: folds this rank's forces (device, [n_listed,3]) onto the cell's
 *                               atoms in list order, adds energy and virial, sums over the ranks with one
 *                               ncclAllReduce and copies [energy, virial(6), forces(3 n_total)] to out_host
 *   pet_nccl_exchange_timing    CUDA-event time spent inside edges() since the last call, and how many calls
 * All return PET_OK or an error code; pet_nccl_last_error() has the message (per host thread). */
typedef struct pet_nccl_exchange pet_nccl_exchange;
const char* pet_nccl_last_error(void);
/* The static schedule pet_nccl_exchange_create derives from a rank's routing, as host arrays (no GPU, no NCCL
 * needed): count[world] rows to and from each rank, send_slot[n_remote] / recv_slot[n_remote] each edge's row in the
 * send buffer and its partner's row in the receive buffer, both laid out as one block per rank in rank order. */
int pet_exchange_schedule(const int* dest, int n_remote, int world, int* count, int* send_slot, int* recv_slot);
int pet_nccl_unique_id(char* id128);
int pet_nccl_exchange_create(const char* id128, int rank, int world, int device, const int* dest, int n_remote,
                             const int* owner, int n_listed, int n_total, pet_nccl_exchange** out);
void pet_nccl_exchange_destroy(pet_nccl_exchange* x);
const pet_exchange* pet_nccl_exchange_callbacks(pet_nccl_exchange* x);
int pet_nccl_exchange_reduce(pet_nccl_exchange* x, const double* forces, const double* energy, const double* virial6,
                             void* stream, double* out_host);
int pet_nccl_exchange_timing(pet_nccl_exchange* x, int enable, double* ms, int* calls);
/* The latest evaluation's results where they lie on the device (forces [n_atoms,3], energy [B], virial [B,6]; null
 * before any evaluation or without forces) and the calculator's cudaStream_t: what pet_nccl_exchange_reduce reads. */
int pet_device_results_of(pet_calc* c, pet_device_results* out, void** stream);

/* C[m,n] = A[m,k] . W^T, W [n,k], fp32 on the CUDA cores, on host arrays, WITHOUT allocating
 * device memory. It has no counterpart in the reference. It exists for callers that cannot
 * call cudaMalloc: plug-ins of a host program that owns all device memory through its own
 * pool, code that runs while another thread of the process has a stream capture open (where
 * cudaMalloc is an error), loops that may not take the driver's allocation lock. Operands are
 * staged in a fixed 12 MiB array inside the library image (resident on every GPU that loads the
 * library until the process exits), on the current device; the copies and the kernel run on the
 * calling thread's own stream (cudaStreamPerThread), which the call waits for before it returns.
 * Limits and rules:
 *   - round64(m*k) + round64(n*k) + round64(m*n) floats must fit 3 Mi floats, n % 4 == 0 and
 *     k % 4 == 0; a larger problem is refused with PET_ERR_INVALID and a message in errbuf;
 *   - the first call on each device resolves the array's device address (cudaGetSymbolAddress):
 *     make that first call before any stream capture starts;
 *   - the operands are ordinary (pageable) host arrays, and CUDA refuses copies from such memory in every thread
 *     while any thread has a stream capture open in the global mode; for the length of the call the calling thread
 *     therefore switches its own capture mode to relaxed (cudaThreadExchangeStreamCaptureMode) and restores it after;
 *   - every call uses the same array, which keeps the previous call's contents (the kernel
 *     overwrites all of C, so nothing needs clearing); calls that overlap on one GPU (two host
 *     threads) race.
 * errbuf (optional) receives the message of a failure. */
int pet_gemm_host_static(int m, int n, int k, const float* A, const float* W, float* C, char* errbuf, size_t errbuf_len);

#ifdef __cplusplus
}
#endif
#endif /* PET_B200_H */
