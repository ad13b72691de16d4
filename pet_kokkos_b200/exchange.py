"""Exchange-mode domain decomposition of one periodic cell: ghosts one cutoff deep, edge rows swapped per layer.

The reference's protocol (include/pet/exchange.hpp:1-41; lammps/ML-PET/pair_pet.cpp:268-360,479-555): every rank
evaluates its owned atoms; a ghost is a neighbour only. An edge i -> g from an owned atom to a ghost reads its
partner edge's row (g's owner's edge to its image of i) once per message-passing layer, forward and backward.
What is here:

* `exchange_domain`  one rank's atoms, ghosts and full pair list, with a global description of every edge to a ghost;
* `route`            which edge of which rank is the partner of each edge to a ghost (matched by the two atoms and
                     the edge vector, as the reference's (tag, tag, vector) key does);
* `ThreadExchange`   the callbacks for ranks played as threads of one process on one GPU (the reference's
                     ImageExchange test, tests/test_edges.cpp:385-439): rows cross through host memory;
* `NcclExchange`     the callbacks for one process per GPU: rows cross with torch.distributed all-to-all over NCCL.
"""
from __future__ import annotations

import ctypes
import threading

import numpy as np

from .calculator import EdgeListView
from .domain import _pairs_within, rank_grid


def exchange_domain(system, rank, world, cutoff):
    """Rank `rank`'s share: (EdgeListView fields as a dict, owner [n_listed] global atom of every listed atom,
    image [n_listed, 3] lattice image of every listed atom, remote [n_remote, 2] (local centre, local ghost) of its
    edges to ghosts in list order)."""
    cell = np.asarray(system["cell"], dtype=np.float64).reshape(3, 3)
    pos = np.asarray(system["positions"], dtype=np.float64)
    z = np.asarray(system["atomic_numbers"])
    inv = np.linalg.inv(cell)
    frac = pos @ inv
    wrap = np.floor(frac)
    frac = frac - wrap
    wrapped = frac @ cell
    grid = rank_grid(world)
    coord = np.array(np.unravel_index(rank, grid))
    lo_f, hi_f = coord / np.array(grid), (coord + 1) / np.array(grid)
    mine = ((frac >= lo_f) & (frac < hi_f)).all(1)
    owned = np.nonzero(mine)[0]
    spacing = 1.0 / np.linalg.norm(inv, axis=0)
    margin = cutoff / spacing
    reach = np.ceil(margin).astype(int)
    gpos, gown, gimg = [], [], []
    for a in range(-reach[0], reach[0] + 1):
        for b in range(-reach[1], reach[1] + 1):
            for c in range(-reach[2], reach[2] + 1):
                f = frac + np.array([a, b, c])
                inside = ((f >= lo_f - margin) & (f < hi_f + margin)).all(1)
                if (a, b, c) == (0, 0, 0):
                    inside &= ~mine
                idx = np.nonzero(inside)[0]
                gpos.append(wrapped[idx] + np.array([a, b, c]) @ cell), gown.append(idx)
                gimg.append(np.tile([a, b, c], (len(idx), 1)))
    lpos = np.concatenate([wrapped[owned]] + gpos)
    owner = np.concatenate([owned] + gown)
    image = np.concatenate([np.zeros((len(owned), 3), int)] + gimg).astype(int)
    n_local = len(owned)
    ii, jj = _pairs_within(lpos, cutoff)
    keep = ii < n_local                      # ghosts have no pairs of their own
    ii, jj = ii[keep], jj[keep]
    # a ghost nobody lists is dropped from nothing: it simply has no edge
    off = np.concatenate([[0], np.cumsum(np.bincount(ii, minlength=len(lpos)))]).astype(np.int32)
    to_ghost = jj >= n_local
    remote = np.stack([ii[to_ghost], jj[to_ghost]], 1)
    fields = dict(positions=lpos, atomic_numbers=z[owner].astype(np.int32), offsets=off, neighbors=jj.astype(np.int32),
                  n_local=n_local)
    return fields, owner, image, remote


def route(domains):
    """For every rank p and every edge r of its edges to ghosts: (rank q, index r' among q's edges to ghosts) of the
    partner edge. The partner of i -> g (g an image of atom j) is, on j's owner, j -> its image of i with the opposite
    vector; the vector (rounded to 1e-4 A) tells several images of one atom apart."""
    n_atoms = 1 + max(int(d[1].max()) for d in domains if len(d[1]))
    keys, partners, label = [], [], []
    for q, (fields, owner, image, remote) in enumerate(domains):
        x = fields["positions"]
        i, g = remote[:, 0], remote[:, 1]
        v = np.rint((x[g] - x[i]) * 1e4).astype(np.int64)
        oi, og = owner[i].astype(np.int64), owner[g].astype(np.int64)
        pack = lambda w: ((w[:, 0] + (1 << 20)) << 42) | ((w[:, 1] + (1 << 20)) << 21) | (w[:, 2] + (1 << 20))
        keys.append(np.stack([oi * n_atoms + og, pack(v)], 1))
        partners.append(np.stack([og * n_atoms + oi, pack(-v)], 1))
        label.append(np.stack([np.full(len(remote), q), np.arange(len(remote))], 1))
    keys, partners, label = np.concatenate(keys), np.concatenate(partners), np.concatenate(label)
    n = len(keys)
    _, inv = np.unique(np.concatenate([keys, partners]), axis=0, return_inverse=True)
    inv = inv.reshape(-1)
    edge_of_id = np.full(inv.max() + 1 if n else 1, -1, np.int64)
    edge_of_id[inv[:n]] = np.arange(n)
    match = edge_of_id[inv[n:]]
    if (match < 0).any():
        bad = int(np.nonzero(match < 0)[0][0])
        raise RuntimeError(f"rank {label[bad, 0]}: edge {label[bad, 1]} to a ghost has no partner on the ghost's rank")
    dest = label[match]
    out, at = [], 0
    for d in domains:
        out.append(dest[at:at + len(d[3])])
        at += len(d[3])
    return out


_cudart = None


def _rt():
    """The CUDA runtime the process already uses (loaded by the library and by torch)."""
    global _cudart
    if _cudart is None:
        import ctypes.util
        for name in ("libcudart.so.12", "libcudart.so", ctypes.util.find_library("cudart")):
            if not name:
                continue
            try:
                _cudart = ctypes.CDLL(name)
                break
            except OSError:
                continue
        if _cudart is None:
            import glob
            import os
            import torch
            hits = glob.glob(os.path.join(os.path.dirname(torch.__file__), "..", "nvidia", "cuda_runtime", "lib", "libcudart.so*"))
            _cudart = ctypes.CDLL(hits[0])
        _cudart.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
        _cudart.cudaMemcpyAsync.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
        _cudart.cudaStreamSynchronize.argtypes = [ctypes.c_void_p]
    return _cudart


def _d2h(ptr, n, dtype):
    a = np.empty(n, dtype)
    if n:
        rc = _rt().cudaMemcpy(a.ctypes.data, ptr, a.nbytes, 2)
        if rc:
            raise RuntimeError(f"cudaMemcpy D2H failed: {rc}")
    return a


def _h2d(ptr, a, stream):
    """Host rows into the calculator's buffer, on the calculator's stream. A blocking cudaMemcpy from pageable memory
    returns once the rows are staged, before they have landed, and it runs on the legacy stream, which the
    calculator's non-blocking stream does not wait for: the kernels launched next could read the buffer too early."""
    if a.size:
        rc = _rt().cudaMemcpyAsync(ptr, a.ctypes.data, a.nbytes, 1, stream) or _rt().cudaStreamSynchronize(stream)
        if rc:
            raise RuntimeError(f"cudaMemcpy H2D failed: {rc}")


class ThreadHub:
    """What the ranks of one process share: the routing, each rank's live list and posted rows, and a barrier."""

    def __init__(self, dest):
        self.dest = dest
        self.world = len(dest)
        self.barrier = threading.Barrier(self.world)
        self.live = [None] * self.world
        self.rows = [None] * self.world
        self.mute = False  # a test sets this to see that the result depends on the exchange


class ThreadExchange:
    """One rank's callbacks when the ranks are threads of one process (rows cross through host memory)."""

    def __init__(self, hub: ThreadHub, rank: int):
        self.hub, self.rank = hub, rank

    def set_live(self, live_ptr, n_live, stream):
        _rt().cudaStreamSynchronize(stream)
        self.hub.live[self.rank] = _d2h(live_ptr, n_live, np.int32)
        self.hub.barrier.wait()
        # where each of this rank's live rows comes from: (rank q, row of q's live list)
        mine = self.hub.live[self.rank]
        d = self.hub.dest[self.rank][mine] if n_live else np.zeros((0, 2), int)
        self.src_rank = d[:, 0]
        self.src_row = np.zeros(n_live, int)
        for q in range(self.hub.world):
            m = self.src_rank == q
            if m.any():
                pos = np.searchsorted(self.hub.live[q], d[m, 1])
                if (pos >= len(self.hub.live[q])).any() or (self.hub.live[q][pos] != d[m, 1]).any():
                    raise RuntimeError("a live edge's partner is not live on its rank")
                self.src_row[m] = pos
        self.hub.barrier.wait()

    def edges(self, out_ptr, in_ptr, n_live, width, stream):
        _rt().cudaStreamSynchronize(stream)
        self.hub.rows[self.rank] = _d2h(out_ptr, n_live * width, np.float32).reshape(n_live, width)
        self.hub.barrier.wait()
        got = np.zeros((n_live, width), np.float32)
        if not self.hub.mute:
            for q in range(self.hub.world):
                m = self.src_rank == q
                if m.any():
                    got[m] = self.hub.rows[q][self.src_row[m]]
        _h2d(in_ptr, got, stream)
        self.hub.barrier.wait()


class _DeviceArray:
    """A device buffer as something torch.as_tensor can wrap without copying."""

    def __init__(self, ptr, n, typestr):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (int(ptr), False), "version": 2}


class NcclExchange:
    """One rank's callbacks with one process per GPU: torch.distributed all-to-all over NCCL.

    `dest` is this rank's routing ([n_remote, 2] from `route`); every rank built it from the same structure."""

    def __init__(self, dest, group=None):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.group = torch, dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.dest = np.asarray(dest).reshape(-1, 2)

    def set_live(self, live_ptr, n_live, stream):
        torch, dist = self.torch, self.dist
        _rt().cudaStreamSynchronize(stream)
        live = _d2h(live_ptr, n_live, np.int32)
        d = self.dest[live] if n_live else np.zeros((0, 2), int)
        order = np.argsort(d[:, 0], kind="stable")          # rows grouped by destination rank, list order within
        self.send_order = torch.as_tensor(order, device="cuda", dtype=torch.long)
        self.send_counts = np.bincount(d[:, 0], minlength=self.world).tolist()
        counts = torch.tensor(self.send_counts, device="cuda", dtype=torch.int64)
        got = torch.empty_like(counts)
        dist.all_to_all_single(got, counts, group=self.group)
        self.recv_counts = got.tolist()
        # tell each destination which of its edges to ghosts every row is the partner of
        tags = torch.as_tensor(d[order, 1], device="cuda", dtype=torch.int64)
        arrived = torch.empty(sum(self.recv_counts), device="cuda", dtype=torch.int64)
        dist.all_to_all_single(arrived, tags, self.recv_counts, self.send_counts, group=self.group)
        pos = np.searchsorted(live, arrived.cpu().numpy())
        if n_live and ((pos >= n_live).any() or (live[np.minimum(pos, n_live - 1)] != arrived.cpu().numpy()).any()):
            raise RuntimeError("a row arrived for an edge that is not live here")
        self.arrive_row = torch.as_tensor(pos, device="cuda", dtype=torch.long)

    def edges(self, out_ptr, in_ptr, n_live, width, stream):
        torch, dist = self.torch, self.dist
        _rt().cudaStreamSynchronize(stream)
        out = torch.as_tensor(_DeviceArray(out_ptr, max(n_live * width, 1), "<f4"), device="cuda")[:n_live * width].view(n_live, width)
        inn = torch.as_tensor(_DeviceArray(in_ptr, max(n_live * width, 1), "<f4"), device="cuda")[:n_live * width].view(n_live, width)
        send = out.index_select(0, self.send_order).contiguous()
        recv = torch.empty((sum(self.recv_counts), width), device="cuda", dtype=torch.float32)
        dist.all_to_all_single(recv, send, self.recv_counts, self.send_counts, group=self.group)
        inn.zero_()
        inn.index_copy_(0, self.arrive_row, recv)
        torch.cuda.current_stream().synchronize()


def view_of(fields, exchange):
    return EdgeListView(fields["positions"], fields["atomic_numbers"], fields["offsets"], fields["neighbors"],
                        n_local=fields["n_local"], exchange=exchange)


class NativeNcclExchange:
    """One rank's exchange with everything inside the library (csrc/nccl_exchange.cu): pack and unpack kernels and
    ncclSend / ncclRecv on the calculator's stream, ghost forces folded on the device, one ncclAllReduce. Python only
    hands over the routing and carries NCCL's id from rank 0 to the others (here with torch.distributed; an MD engine
    would use MPI).

    `dest` is this rank's routing ([n_remote, 2] from `route`), `owner` the global atom of every listed atom."""

    def __init__(self, dest, owner, n_total, device, group=None, single=False):
        import torch  # noqa: F401  before the library looks for NCCL: it then finds the copy PyTorch bundles, not another
        from .calculator import load_library
        self._lib = load_library()
        self._h = None
        idbuf = ctypes.create_string_buffer(128)
        if single:  # one rank, no job around it: every ghost is an image of one of this rank's own atoms
            rank, world = 0, 1
            if self._lib.pet_nccl_unique_id(idbuf):
                raise RuntimeError(self._lib.pet_nccl_last_error().decode())
        else:
            import torch
            import torch.distributed as dist
            rank, world = dist.get_rank(group), dist.get_world_size(group)
            if rank == 0 and self._lib.pet_nccl_unique_id(idbuf):
                raise RuntimeError(self._lib.pet_nccl_last_error().decode())
            t = torch.frombuffer(bytearray(idbuf.raw), dtype=torch.uint8).clone()
            t = t.cuda() if dist.get_backend(group) == "nccl" else t
            dist.broadcast(t, src=0, group=group)
            idbuf = ctypes.create_string_buffer(bytes(t.cpu().numpy().tobytes()), 128)
        d = np.ascontiguousarray(np.asarray(dest).reshape(-1, 2), dtype=np.int32)
        o = np.ascontiguousarray(owner, dtype=np.int32)
        h = ctypes.c_void_p()
        ip = lambda a: a.ctypes.data_as(ctypes.POINTER(ctypes.c_int))
        rc = self._lib.pet_nccl_exchange_create(idbuf, rank, world, int(device), ip(d), len(d), ip(o), len(o), int(n_total),
                                                ctypes.byref(h))
        if rc:
            raise RuntimeError(self._lib.pet_nccl_last_error().decode())
        self._h, self.n_total = h, int(n_total)
        self.native_callbacks = self._lib.pet_nccl_exchange_callbacks(h)

    def reduce(self, calc):
        """After an evaluation of `calc`: the whole cell's [energy, virial(6), forces(3 n_total)] on every rank."""
        r, stream = calc.device_results()
        out = np.empty(7 + 3 * self.n_total)
        rc = self._lib.pet_nccl_exchange_reduce(self._h, r.forces, r.energy, r.virial, stream,
                                                out.ctypes.data_as(ctypes.POINTER(ctypes.c_double)))
        if rc:
            raise RuntimeError(self._lib.pet_nccl_last_error().decode())
        return out

    def timing(self, enable=True):
        """(milliseconds inside edges() since the last call, number of calls); switches the CUDA-event brackets on or off."""
        ms, n = ctypes.c_double(), ctypes.c_int()
        if self._lib.pet_nccl_exchange_timing(self._h, int(enable), ctypes.byref(ms), ctypes.byref(n)):
            raise RuntimeError(self._lib.pet_nccl_last_error().decode())
        return ms.value, n.value

    def close(self):
        if self._h is not None:
            self._lib.pet_nccl_exchange_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def make_exchange(calc, routing, owner=None, n_total=0, device=0, group=None, native=True):
    """The exchange a rank of a torch.distributed job hands to its Calculator: the library's own over NCCL, or (with
    native=False) the torch.distributed one that the tests keep as a second opinion."""
    if native:
        return NativeNcclExchange(routing, owner, n_total, device, group)
    return NcclExchange(routing, group)


def fold_to_owners(results, owner, n_atoms):
    """This rank's share of the whole cell: (energy, forces [n_atoms, 3] with ghost forces added onto their owners,
    virial [6])."""
    F = np.zeros((n_atoms, 3))
    np.add.at(F, owner, results.forces)
    return float(results.energy[0]), F, np.asarray(results.virial[0], dtype=np.float64).copy()


def compute_threads(calcs, system, cutoff, mute=False):
    """Plays len(calcs) ranks as threads of this process, one Calculator each (they may share a GPU): the whole cell's
    (energy, forces, virial). With `mute` the rows that cross between ranks arrive as zeros (a test's control)."""
    world = len(calcs)
    domains = [exchange_domain(system, r, world, cutoff) for r in range(world)]
    hub = ThreadHub(route(domains))
    hub.mute = mute
    out, err = [None] * world, [None] * world

    def run(r):
        try:
            fields, owner, _, _ = domains[r]
            res = calcs[r].compute_edges(view_of(fields, ThreadExchange(hub, r)), True, False)
            out[r] = fold_to_owners(res, owner, system["n_atoms"])
        except BaseException as e:  # a rank that fails must not leave the others waiting at the barrier
            err[r] = e
            hub.barrier.abort()
    threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    [t.start() for t in threads]
    [t.join(timeout=600) for t in threads]
    if any(t.is_alive() for t in threads):
        hub.barrier.abort()
        raise RuntimeError("exchange: a rank thread did not finish")
    for e in err:
        if e is not None and not isinstance(e, threading.BrokenBarrierError):
            raise e
    for e in err:
        if e is not None:
            raise e
    E = sum(o[0] for o in out)
    F = sum(o[1] for o in out)
    W = sum(o[2] for o in out)
    return E, F, W, hub


def compute_distributed(calc, system, cutoff, group=None, steps=1, positions=None, native=False):
    """One process per GPU (torch.distributed initialised, NCCL): this rank evaluates its domain of `system` with
    ghosts one cutoff deep and an exchange over NCCL; returns the whole cell's (energy, forces, virial) on every rank.
    With steps > 1 the list is set once and compute_step runs `steps` times (an MD engine between list rebuilds).
    native: the library's own exchange and device-side reduction instead of the torch.distributed ones."""
    import torch
    import torch.distributed as dist
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    domains = [exchange_domain(system, r, world, cutoff) for r in range(world)]
    fields, owner, _, _ = domains[rank]
    if native:
        ex = NativeNcclExchange(route(domains)[rank], owner, system["n_atoms"], torch.cuda.current_device(), group)
        calc.set_neighbors(view_of(fields, ex))
        for _ in range(steps):
            calc.compute_step_on_device(fields["positions"], None, True)
            out = ex.reduce(calc)
        ex.close()
        return out[0], out[7:].reshape(-1, 3), out[1:7]
    ex = NcclExchange(route(domains)[rank], group)
    view = view_of(fields, ex)
    if steps == 1:
        res = calc.compute_edges(view, True, False)
    else:
        calc.set_neighbors(view)
        for _ in range(steps):
            res = calc.compute_step(fields["positions"], None, True, False)
    e, F, W = fold_to_owners(res, owner, system["n_atoms"])
    buf = torch.from_numpy(np.concatenate([[e], W, F.ravel()])).cuda()
    dist.all_reduce(buf, group=group)
    out = buf.cpu().numpy()
    return out[0], out[7:].reshape(-1, 3), out[1:7]
