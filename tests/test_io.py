"""Extended XYZ in and out (the reference's tests/test_io.cpp: symbols, frames, lattice and pbc rules, extra
columns, malformed files, a write/read round trip). No model and no GPU needed."""
import io

import numpy as np
import pytest

from pet_kokkos_b200 import io as pio, structures as st


def test_symbols_and_numbers():
    assert pio.element_number("H") == 1 and pio.element_number("Si") == 14 and pio.element_number("Og") == 118
    assert pio.element_symbol(1) == "H" and pio.element_symbol(79) == "Au" and pio.element_symbol(118) == "Og"
    assert pio.element_number("cl") == 17 and pio.element_number("CL") == 17  # case is normalised
    assert pio.element_number("47") == 47  # a numeric species column
    assert pio.element_number("Qq") == 0 and pio.element_number("") == 0
    assert [pio.element_symbol(z) for z in (0, -3, 119, 10 ** 6)] == ["X"] * 4
    assert all(pio.element_number(pio.element_symbol(z)) == z for z in range(1, 119))


def test_a_cluster_frame():
    frames = pio.read_extxyz('4\nProperties=species:S:1:pos:R:3 pbc="F F F"\n'
                             "N 0.0 0.0 0.1\nH 0.9 0.0 -0.3\nH -0.45 0.8 -0.3\nH -0.45 -0.8 -0.3\n")
    assert len(frames) == 1
    s = frames[0]
    assert s["n_atoms"] == 4 and s["atomic_numbers"].tolist() == [7, 1, 1, 1]
    assert s["positions"][1].tolist() == [0.9, 0.0, -0.3]
    assert not s["pbc"].any()


def test_lattice_rows_and_the_periodic_default():
    s = pio.read_extxyz('1\nlattice="2 0.5 0 0 3 0.25 0.125 0 4" Properties=species:S:1:pos:R:3\nGe 0.5 0.25 0.125\n')[0]
    assert s["cell"].tolist() == [[2, 0.5, 0], [0, 3, 0.25], [0.125, 0, 4]]  # rows, not columns
    assert s["pbc"].all()  # no pbc entry, a lattice: periodic
    s = pio.read_extxyz('1\nLattice="8 0 0 0 8 0 0 0 30" pbc="T T F"\nC 0 0 0\n')[0]
    assert s["pbc"].tolist() == [True, True, False]
    s = pio.read_extxyz("1\nenergy=-3.5\nAr 0 0 0\n")[0]
    assert not s["pbc"].any() and not s["cell"].any()
    s = pio.read_extxyz("1\nsublattice=\"1 2 3\" Lattice='5 0 0 0 5 0 0 0 5'\nAr 0 0 0\n")[0]  # a whole key only
    assert s["cell"].tolist() == np.diag([5.0, 5, 5]).tolist()


def test_several_frames_extra_columns_and_blank_lines():
    text = ("2\nProperties=species:S:1:pos:R:3:forces:R:3\nO 0 0 0 0.5 0.25 -1\nO 0 0 1.2 -0.5 -0.25 1\n"
            "\n\n1\nProperties=species:S:1:pos:R:3\n10 2 2 2\n")
    frames = pio.read_extxyz(io.StringIO(text))
    assert [f["n_atoms"] for f in frames] == [2, 1]
    assert frames[1]["atomic_numbers"].tolist() == [10]
    assert frames[0]["positions"][1].tolist() == [0, 0, 1.2]


@pytest.mark.parametrize("text,what", [
    ("3\nc\nH 0 0 0\nH 0 0 1\n", "ends after 2 of 3"),
    ("1\nc\nH 0 0\n", "cannot parse atom line"),
    ("1\nc\nH 0 zero 0\n", "cannot parse atom line"),
    ("1\nc\nQq 0 0 0\n", "unknown species"),
    ('1\nLattice="4 0 0 0 4"\nH 0 0 0\n', "Lattice needs 9 numbers, found 5"),
    ("2\n", "ends after the atom count"),
    ("atoms\nc\n", "expected an atom count"),
    ("-2\nc\n", "expected an atom count"),
])
def test_malformed_files_are_refused_with_a_message(text, what):
    with pytest.raises(RuntimeError, match=what):
        pio.read_extxyz(io.StringIO(text))


def test_a_missing_file():
    with pytest.raises(RuntimeError, match="cannot open"):
        pio.read_extxyz("no/such/file.xyz")


def test_write_then_read(tmp_path):
    s = st.make_system([8, 1, 26], [[0.0, 0.5, 1.25], [2.0, -1.5, 0.125], [1 / 3, 2 / 3, 1e-7]],
                       [[5.1, 0, 0], [0, 5.2, 0], [0.1, 0, 5.3]], pbc=(True, False, True))
    forces = np.array([[0.1, -0.2, 0.3], [-0.1, 0.2, -0.3], [0, 0, 0]])
    path = tmp_path / "frames.xyz"
    with open(path, "w") as f:
        pio.write_extxyz(f, s, forces, energy=-12.5)
        pio.write_extxyz(f, st.make_system([2], [[0, 0, 0]], np.zeros((3, 3)), pbc=(False, False, False)))
    text = path.read_text()
    assert "forces:R:3" in text and "energy=-12.5" in text and text.count("Lattice") == 1
    back = pio.read_extxyz(path)
    assert len(back) == 2
    b = back[0]
    assert b["atomic_numbers"].tolist() == [8, 1, 26] and b["pbc"].tolist() == [True, False, True]
    assert np.abs(b["positions"] - s["positions"]).max() <= 1e-10 and np.abs(b["cell"] - s["cell"]).max() <= 1e-10
    assert back[1]["n_atoms"] == 1 and not back[1]["pbc"].any()


def test_frames_feed_the_structure_helpers():
    """A frame read back is the same kind of dict the calculators take."""
    s = st.diamond(1, jitter=0.01, seed=0)
    buf = io.StringIO()
    pio.write_extxyz(buf, s)
    b = pio.read_extxyz(buf.getvalue())[0]
    assert set(b) == set(s) and b["positions"].dtype == np.float64 and b["atomic_numbers"].dtype == np.int32
