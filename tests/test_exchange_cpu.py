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
