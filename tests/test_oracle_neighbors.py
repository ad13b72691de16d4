"""The neighbour-list oracle against the reference's own model-free tests.

Each test restates a Catch2 case of the reference (file:line in the docstring)
on the numpy restatement in oracle/neighbors_oracle.py; these are the vectors
that pin the oracle's edge sets and order.
"""
import numpy as np
import pytest

from oracle import neighbors_oracle as nbo
from pet_kokkos_b200 import structures as st

K_CUTOFF = 7.5  # tests/test_cell_list.cpp:113


def edge_set(idx):
    return set(map(tuple, idx.tolist()))


@pytest.mark.parametrize("name,systems", [
    ("box narrower than the cutoff", [st.diamond(2)]),
    ("two bins per axis", [st.diamond(3)]),
    ("many bins", [st.diamond(5)]),
    ("strongly skewed cell", [st.diamond(6, shear=0.5)]),
    ("mixed batch", [st.diamond(2), st.diamond(4), st.diamond(3)]),
])
def test_cell_list_equals_brute_force(name, systems):
    """tests/test_cell_list.cpp:119-150: same edge set, none listed twice."""
    for s in systems:
        ci, _, _ = nbo.cell_list_edges(s, K_CUTOFF)
        bi, _, _ = nbo.brute_force_edges(s, K_CUTOFF)
        assert len(ci) == len(edge_set(ci))
        assert edge_set(ci) == edge_set(bi)


def test_small_structure_gets_brute_force_order():
    """tests/test_cell_list.cpp:192-212: below the cell-list thresholds the order is (i, sa, sb, sc, j)."""
    for s in [st.diamond(1), st.diamond(1, shear=0.3)]:
        ci, _, _ = nbo.cell_list_edges(s, 4.5)
        bi, _, _ = nbo.brute_force_edges(s, 4.5)
        order = sorted(map(tuple, bi.tolist()), key=lambda e: (e[0], e[2], e[3], e[4], e[1]))
        assert [tuple(x) for x in ci.tolist()] == order


def test_simple_cubic_coordination():
    """tests/test_neighbors.cpp:52-73: spacing 2.0, cutoff 2.5 -> 6 neighbours, each one spacing away."""
    s = st.simple_cubic(4, 2.0)
    ed = nbo.build_edges([s], list(range(10)), 2.5, 0.5, search="brute")
    counts = np.diff(ed["off"])
    assert (counts == 6).all()
    np.testing.assert_allclose(ed["dist"], 2.0, rtol=1e-12)


def test_reverse_map_is_an_involution():
    """tests/test_neighbors.cpp:102-128: every edge has a partner, partner's partner is itself, vectors negate."""
    s = st.simple_cubic(3, 2.0)
    for search in ("brute", "cells"):
        ed = nbo.build_edges([s], list(range(10)), 2.5, 0.5, search=search)
        rev = ed["reverse"]
        assert len(rev) == 27 * 6
        assert (rev >= 0).all()
        assert (rev[rev] == np.arange(len(rev))).all()
        np.testing.assert_allclose(ed["vec"][rev], -ed["vec"], atol=1e-12)


def test_padding_free_molecule():
    """tests/test_neighbors.cpp:75-100,179-194: a non-periodic cluster is not wrapped; the far atom has no edges."""
    s = st.make_system([1, 1, 1], [[0, 0, 0], [1, 0, 0], [10, 0, 0]], np.zeros((3, 3)), (False, False, False))
    ed = nbo.build_edges([s], list(range(10)), 3.0, 0.5)
    assert np.diff(ed["off"]).tolist() == [1, 1, 0]
    w = st.make_system([8, 1, 1], [[0, 0, 0.11926], [0, 0.76323, -0.47704], [0, -0.76323, -0.47704]],
                       np.zeros((3, 3)), (False, False, False))
    ed = nbo.build_edges([w], list(range(10)), 5.0, 0.5)
    oh = np.sqrt(0.76323 ** 2 + 0.5963 ** 2)
    assert np.diff(ed["off"])[0] == 2
    np.testing.assert_allclose(ed["dist"][:2], oh, atol=1e-4)


def test_cutoff_function_values():
    """tests/test_neighbors.cpp:130-150: 1 inside, 0 at and beyond the cutoff, monotone across the taper."""
    rc, w = 5.0, 0.5
    f = lambda d: float(nbo.bump_cutoff_f32(np.array([d]), np.array([rc]), w)[0])
    assert f(1.0) == 1.0 and f(rc - w - 0.01) == 1.0 and f(rc) == 0.0 and f(rc + 1.0) == 0.0
    vals = [f(d) for d in np.arange(rc - w, rc + 1e-9, w / 50.0)]
    assert all(b <= a + 1e-7 for a, b in zip(vals, vals[1:]))
    g = lambda d: float(nbo.cosine_cutoff_f32(np.array([d]), np.array([rc]), w)[0])
    assert g(1.0) == 1.0 and abs(g(rc)) < 1e-7 and g(rc + 1.0) == 0.0


def test_batch_edges_never_cross_structures():
    """tests/test_neighbors.cpp:196-230: concatenation keeps structures apart and the reverse map valid."""
    a, b = st.simple_cubic(2, 2.0), st.simple_cubic(3, 2.0)
    ed = nbo.build_edges([a, b], list(range(10)), 2.5, 0.5)
    na = a["n_atoms"]
    assert ((ed["center"] < na) == (ed["neighbor"] < na)).all()
    assert (ed["reverse"][ed["reverse"]] == np.arange(len(ed["reverse"]))).all()
    assert (ed["struct_id"][:na] == 0).all() and (ed["struct_id"][na:] == 1).all()


def test_benchmark_shapes():
    """The synthetic 64-atom diamond has the edge count and neighbour maximum the workload table states."""
    ed = nbo.build_edges([st.diamond(2, jitter=0.05, seed=0)], list(range(-1, 85)), 4.5, 0.5)
    assert len(ed["center"]) == 4478 and ed["max_neighbors"] == 72
