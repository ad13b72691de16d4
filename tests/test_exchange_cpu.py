"""Exchange-mode decomposition, host logic: domains, ghosts one cutoff deep, the routing of edges to ghosts."""
import numpy as np
import pytest

from pet_kokkos_b200 import exchange, structures as st


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("n", [2, 3])
def test_domains_partition_the_cell_and_route_is_an_involution(world, n):
    s = st.diamond(n, jitter=0.05, seed=4)
    domains = [exchange.exchange_domain(s, r, world, 4.5) for r in range(world)]
    owned = np.concatenate([d[1][:d[0]["n_local"]] for d in domains])
    assert sorted(owned.tolist()) == list(range(s["n_atoms"]))
    for fields, owner, image, remote in domains:
        nl = fields["n_local"]
        assert fields["offsets"][-1] == fields["offsets"][nl], "ghosts have no pairs of their own"
        assert (remote[:, 0] < nl).all() and (remote[:, 1] >= nl).all()
    dest = exchange.route(domains)
    total = 0
    for p, d in enumerate(dest):
        for r, (q, rr) in enumerate(d):
            assert tuple(dest[q][rr]) == (p, r), "the partner's partner is the edge itself"
            fp, fq = domains[p][0], domains[q][0]
            i, g = domains[p][3][r]
            j, h = domains[q][3][rr]
            np.testing.assert_allclose(fp["positions"][g] - fp["positions"][i], -(fq["positions"][h] - fq["positions"][j]), atol=1e-9)
            assert domains[p][1][i] == domains[q][1][h] and domains[p][1][g] == domains[q][1][j]
        total += len(d)
    # every directed pair of the periodic cell is some rank's edge, once
    from oracle import neighbors_oracle as nbo
    idx, _, _ = nbo.brute_force_edges(s, 4.5)
    assert sum(len(d[0]["neighbors"]) for d in domains) == len(idx)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_static_schedule_delivers_every_partner_row(world, lib_path):
    """The library's NCCL exchange sends fixed blocks between ranks, laid out from the routing alone
    (pet_exchange_schedule: host arithmetic, no GPU). Played here with numpy: every rank packs a row per edge to a
    ghost into its send buffer, the blocks are copied rank to rank as ncclSend / ncclRecv would, and every edge must
    find its partner's row in its receive slot. Rows to images of a rank's own atoms stay on the rank."""
    import ctypes as C
    from pet_kokkos_b200.calculator import load_library
    lib = load_library()
    s = st.diamond(3, jitter=0.05, seed=4)
    domains = [exchange.exchange_domain(s, r, world, 4.5) for r in range(world)]
    dest = exchange.route(domains)
    ip = lambda a: a.ctypes.data_as(C.POINTER(C.c_int))
    count, send_slot, recv_slot, sendbuf = [], [], [], []
    for p in range(world):
        d = np.ascontiguousarray(dest[p], dtype=np.int32)
        n = len(d)
        c, ss, rs = np.zeros(world, np.int32), np.zeros(n, np.int32), np.zeros(n, np.int32)
        assert lib.pet_exchange_schedule(ip(d), n, world, ip(c), ip(ss), ip(rs)) == 0
        assert c.sum() == n and sorted(ss.tolist()) == list(range(n)) and sorted(rs.tolist()) == list(range(n))
        buf = np.full((n, 2), -1, np.int64)
        buf[ss] = np.stack([np.full(n, p), np.arange(n)], 1)  # the row of edge r of rank p says (p, r)
        count.append(c), send_slot.append(ss), recv_slot.append(rs), sendbuf.append(buf)
    for p in range(world):
        for q in range(world):
            assert count[p][q] == count[q][p], "a rank sends to a peer as many rows as it gets from it"
    off = [np.concatenate([[0], np.cumsum(c)]) for c in count]
    for p in range(world):
        recv = np.full((len(dest[p]), 2), -1, np.int64)
        for q in range(world):  # the block rank q sends to p lands where p expects rank q's rows
            recv[off[p][q]:off[p][q + 1]] = sendbuf[q][off[q][p]:off[q][p + 1]]
        got = recv[recv_slot[p]]
        assert np.array_equal(got, np.asarray(dest[p])), "every edge reads the row of its partner edge"
