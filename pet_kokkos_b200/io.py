"""Structures in and out as extended XYZ: the reference's pet::read_extxyz / write_extxyz / element_symbol /
element_number (include/pet/io.hpp:12-27, src/io/extxyz.cpp).

A frame is an atom count, a comment line of key=value entries, then one line per atom: species, x, y, z and any
further columns (ignored). Lattice="ax ay az bx by bz cx cy cz" gives the cell's vectors as rows; pbc="T T F"
the periodic axes, which default to all three exactly when a lattice is given (as ASE writes). Keys match without
regard to case. The species column holds a symbol in any case, or an atomic number.
"""
import io as _io
import os

import numpy as np

from .structures import make_system

SYMBOLS = (
    "X H He Li Be B C N O F Ne Na Mg Al Si P S Cl Ar K Ca Sc Ti V Cr Mn Fe Co Ni Cu Zn Ga Ge As Se Br Kr Rb Sr Y Zr "
    "Nb Mo Tc Ru Rh Pd Ag Cd In Sn Sb Te I Xe Cs Ba La Ce Pr Nd Pm Sm Eu Gd Tb Dy Ho Er Tm Yb Lu Hf Ta W Re Os Ir Pt "
    "Au Hg Tl Pb Bi Po At Rn Fr Ra Ac Th Pa U Np Pu Am Cm Bk Cf Es Fm Md No Lr Rf Db Sg Bh Hs Mt Ds Rg Cn Nh Fl Mc Lv "
    "Ts Og").split()
_NUMBER = {s: z for z, s in enumerate(SYMBOLS) if z > 0}


def element_symbol(atomic_number):
    """'X' for anything outside 1..118."""
    z = int(atomic_number)
    return SYMBOLS[z] if 1 <= z < len(SYMBOLS) else SYMBOLS[0]


def element_number(symbol):
    """0 for an unknown symbol; 'he' and 'HE' are He; a numeric species is its own number."""
    s = str(symbol)
    if not s:
        return 0
    if s[0].isdigit():
        digits = s[:len(s) - len(s.lstrip("0123456789"))]  # the leading digits, as std::from_chars reads them
        return int(digits)
    return _NUMBER.get(s[0].upper() + s[1:].lower(), 0)


def _entry(comment, key):
    """key="quoted value", key='quoted' or key=bare from a comment line; '' when absent."""
    low, k = comment.lower(), key.lower()
    p = 0
    while True:
        p = low.find(k, p)
        if p < 0:
            return ""
        eq = p + len(k)
        whole = p == 0 or comment[p - 1].isspace()
        if whole and eq < len(comment) and comment[eq] == "=":
            v = eq + 1
            if v < len(comment) and comment[v] in "\"'":
                end = comment.find(comment[v], v + 1)
                return "" if end < 0 else comment[v + 1:end]
            return comment[v:].split(None, 1)[0] if comment[v:].strip() else ""
        p = eq


def read_extxyz(source):
    """Every frame of a file (a path), an open text file, or the text itself (when it holds a newline)."""
    if hasattr(source, "readline"):
        f, close = source, False
    elif isinstance(source, str) and "\n" in source:
        f, close = _io.StringIO(source), False
    else:
        try:
            f, close = open(os.fspath(source)), True
        except OSError as e:
            raise RuntimeError(f"extxyz: cannot open '{source}'") from e
    try:
        frames = []
        while True:
            line = f.readline()
            if not line:
                return frames
            if not line.strip():
                continue
            head = line.split()
            try:
                n = int(head[0])
            except ValueError:
                n = -1
            if n < 0:
                raise RuntimeError(f"extxyz: expected an atom count, got '{line.rstrip()}'")
            comment = f.readline()
            if not comment:
                raise RuntimeError("extxyz: file ends after the atom count")
            cell, has_cell = np.zeros((3, 3)), False
            lattice = _entry(comment, "Lattice")
            if lattice:
                try:
                    numbers = [float(t) for t in lattice.split()[:9]]
                except ValueError:
                    numbers = []
                if len(numbers) != 9:
                    raise RuntimeError(f"extxyz: Lattice needs 9 numbers, found {len(numbers)}")
                cell, has_cell = np.array(numbers).reshape(3, 3), True
            pbc_text = _entry(comment, "pbc")
            if pbc_text:
                tokens = pbc_text.split()[:3]
                pbc = [bool(t) and t[0] in "Tt1" for t in tokens] + [False] * (3 - len(tokens))
            else:
                pbc = [has_cell] * 3
            numbers, positions = [], []
            for a in range(n):
                line = f.readline()
                if not line:
                    raise RuntimeError(f"extxyz: file ends after {a} of {n} atoms")
                cols = line.split()
                try:
                    xyz = [float(c) for c in cols[1:4]]
                except ValueError:
                    xyz = []
                if len(xyz) != 3:
                    raise RuntimeError(f"extxyz: cannot parse atom line '{line.rstrip()}'")
                z = element_number(cols[0])
                if z == 0:
                    raise RuntimeError(f"extxyz: unknown species '{cols[0]}'")
                numbers.append(z)
                positions.append(xyz)
            frames.append(make_system(np.array(numbers, dtype=np.int32), np.array(positions, dtype=np.float64).reshape(n, 3),
                                      cell, pbc=tuple(pbc)))
    finally:
        if close:
            f.close()


def write_extxyz(out, system, forces=None, energy=None):
    """One frame to an open text file: 12 significant digits, the lattice only for a periodic structure."""
    n = int(system["n_atoms"])
    pbc = [bool(p) for p in system.get("pbc", (True, True, True))]
    fmt = lambda v: f"{float(v):.12g}"
    parts = []
    if any(pbc):
        parts.append('Lattice="' + " ".join(fmt(v) for v in np.asarray(system["cell"], dtype=np.float64).reshape(9)) + '"')
    parts.append("Properties=species:S:1:pos:R:3" + (":forces:R:3" if forces is not None else ""))
    parts.append('pbc="' + " ".join("T" if p else "F" for p in pbc) + '"')
    if energy is not None:
        parts.append("energy=" + fmt(energy))
    out.write(f"{n}\n" + " ".join(parts) + "\n")
    x = np.asarray(system["positions"], dtype=np.float64).reshape(n, 3)
    g = None if forces is None else np.asarray(forces, dtype=np.float64).reshape(n, 3)
    for a in range(n):
        cols = [element_symbol(system["atomic_numbers"][a])] + [fmt(v) for v in x[a]]
        if g is not None:
            cols += [fmt(v) for v in g[a]]
        out.write(" ".join(cols) + "\n")
