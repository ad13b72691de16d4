"""The C-ABI library: it builds for sm_100a, loads, and exports exactly what include/pet_b200.h declares."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "pet_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pet_[a-z_0-9]+)\s*\(", text)))


def test_header_and_binding_agree():
    from pet_kokkos_b200.calculator import SIGNATURES
    assert declared_symbols() == sorted(SIGNATURES)


def test_library_exports_every_declared_symbol(lib_path):
    lib = ctypes.CDLL(str(lib_path))
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_create_fails_loudly_without_a_model(lib_path):
    from pet_kokkos_b200.calculator import Calculator
    with pytest.raises((RuntimeError, ValueError)):
        Calculator("/nonexistent/model.json", "/nonexistent/model.safetensors")


def test_no_cpu_fallback(lib_path, models, has_gpu):
    """Without a CUDA device creation must fail, not fall back."""
    if has_gpu:
        pytest.skip("a GPU is present")
    from pet_kokkos_b200.calculator import Calculator
    with pytest.raises(RuntimeError):
        Calculator(*models("tiny"))


def test_product_does_not_import_the_oracle():
    pat = re.compile(r"^\s*(from|import)\s+\.*oracle|import_module\(.oracle", re.M)
    for p in (ROOT / "pet_kokkos_b200").rglob("*.py"):
        assert not pat.search(p.read_text()), p


def test_named_models_are_found_through_the_search_path(tmp_path, monkeypatch):
    """resolve_model (the reference's src/calculator.cpp:131-166): a name is looked up in $PET_MODEL_DIR first; a path
    prefix is taken as it is; a name nobody has raises with the places that were searched."""
    import pytest
    from pet_kokkos_b200 import calculator as calc
    (tmp_path / "a").mkdir(), (tmp_path / "b").mkdir()
    for ext in (".json", ".safetensors"):
        (tmp_path / "b" / ("pet-test" + ext)).write_text("x")
    (tmp_path / "a" / "half.json").write_text("x")  # without its weights a directory does not count
    monkeypatch.setenv("PET_MODEL_DIR", f"{tmp_path / 'a'}:{tmp_path / 'b'}")
    assert calc.model_search_dirs()[:2] == [str(tmp_path / "a"), str(tmp_path / "b")]
    assert calc.resolve_model("pet-test") == (str(tmp_path / "b" / "pet-test.json"), str(tmp_path / "b" / "pet-test.safetensors"))
    assert calc.resolve_model("/x/y/model") == ("/x/y/model.json", "/x/y/model.safetensors")
    with pytest.raises(RuntimeError, match="not found in"):
        calc.resolve_model("half")
    with pytest.raises(ValueError):
        calc.resolve_model("")
