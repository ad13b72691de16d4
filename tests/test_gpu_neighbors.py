"""The CUDA neighbour pipeline against the oracle: bit-exact edges, order, vectors and distances."""
import numpy as np
import pytest

from oracle import neighbors_oracle as nbo
from pet_kokkos_b200 import structures as st

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def calc(lib_path, models):
    from pet_kokkos_b200 import Calculator
    c = Calculator(*models("tiny"))
    yield c
    c.close()


def oracle_list(systems, cutoff):
    n0, ii, vv, dd = 0, [], [], []
    for s in systems:
        idx, vec, dist = nbo.cell_list_edges(s, cutoff)
        idx = idx.copy()
        idx[:, :2] += n0
        n0 += s["n_atoms"]
        ii.append(idx), vv.append(vec), dd.append(dist)
    return np.concatenate(ii), np.concatenate(vv), np.concatenate(dd)


SETUPS = {
    # the reference's cell-list cases (tests/test_cell_list.cpp:119-136) at the model's cutoff
    "narrow box": lambda: [st.diamond(2)],
    "two bins": lambda: [st.diamond(3)],
    "many bins": lambda: [st.diamond(5)],
    "skewed cell": lambda: [st.diamond(6, shear=0.5)],
    "mixed batch": lambda: [st.diamond(2), st.diamond(4), st.diamond(3), st.diamond(1), st.diamond(1, shear=0.3)],
    # the benchmark's inputs
    "diamond64 jitter": lambda: [st.diamond(2, jitter=0.05, seed=0)],
    "water648": lambda: [st.water_box(216, 18.64, seed=0)],
    "mixture batch": lambda: st.mixture_batch(16, 64, 9.0, seed=0),
    "molecule": lambda: [st.make_system([8, 1, 1], [[0, 0, 0.11926], [0, 0.76323, -0.47704], [0, -0.76323, -0.47704]],
                                        np.zeros((3, 3)), (False, False, False))],
    "diamond1728 jitter": lambda: [st.diamond(6, jitter=0.05, seed=0)],
}


@pytest.mark.parametrize("name", sorted(SETUPS))
def test_edges_bit_exact(calc, name):
    systems = SETUPS[name]()
    nl = calc.neighbor_list(systems)
    idx, vec, dist = oracle_list(systems, calc.cutoff)
    assert len(nl["i"]) == len(idx)
    assert (nl["i"] == idx[:, 0]).all() and (nl["j"] == idx[:, 1]).all() and (nl["shift"] == idx[:, 2:]).all()
    # fp64 vectors and distances: identical bit patterns, not merely close
    assert (nl["vec"].view(np.int64) == vec.view(np.int64)).all()
    assert (nl["dist"].view(np.int64) == dist.view(np.int64)).all()
    assert (nl["reverse"] == nbo.reverse_edges(idx, None)).all()
    cut = nbo.bump_cutoff_f32(dist, np.full_like(dist, calc.cutoff), 0.5).astype(np.float32)
    np.testing.assert_allclose(nl["cutoff"], cut, rtol=0, atol=2e-6)  # float tanh/tan differ by an ulp or two between libms


def test_edge_set_equals_host_brute_force(calc):
    """tests/test_cell_list.cpp:138-150 through the CUDA path, on unwrapped-safe inputs."""
    for s in [st.diamond(2), st.diamond(3), st.diamond(6, shear=0.5)]:
        nl = calc.neighbor_list([s])
        bi, _, _ = nbo.brute_force_edges(s, calc.cutoff)
        got = set(zip(nl["i"].tolist(), nl["j"].tolist(), *nl["shift"].T.tolist()))
        assert len(got) == len(nl["i"])
        assert got == set(map(tuple, bi.tolist()))


def test_reproducible_run_to_run(calc):
    """tests/test_cell_list.cpp:152-157: bins fill through atomics, the per-bin sort fixes the order."""
    systems = [st.diamond(4, jitter=0.05), st.diamond(3)]
    first = calc.neighbor_list(systems)
    for _ in range(3):
        again = calc.neighbor_list(systems)
        for k in first:
            assert (first[k] == again[k]).all(), k


def test_empty_and_single_atom(calc):
    one = st.make_system([6], [[0.1, 0.2, 0.3]], np.eye(3) * 20.0)
    assert len(calc.neighbor_list([one])["i"]) == 0
    lone = st.make_system([6], [[0.0, 0.0, 0.0]], np.eye(3) * 3.0)  # sees its own images
    nl = calc.neighbor_list([lone])
    idx, _, _ = oracle_list([lone], calc.cutoff)
    assert len(nl["i"]) == len(idx) > 0 and (nl["shift"] == idx[:, 2:]).all()
