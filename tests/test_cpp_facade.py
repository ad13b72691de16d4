"""The header-only C++ facade compiles and links against the C-ABI library with plain g++ (no CUDA headers needed)."""
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

SRC = r'''
#include "pet/calculator.hpp"
#include <cstdio>
int main(int argc, char** argv) {
  try {
    pet::Calculator c(argc > 1 ? argv[1] : "/nonexistent.json", argc > 2 ? argv[2] : "/nonexistent.safetensors");
    pet::System s;
    (void) c.compute(s, true);
  } catch (const std::exception& e) {
    std::printf("caught: %s\n", e.what());
    return 0;
  }
  return 0;
}
'''


def test_facade_compiles_links_and_reports_errors(lib_path, tmp_path):
    src = tmp_path / "driver.cpp"
    src.write_text(SRC)
    exe = tmp_path / "driver"
    subprocess.run(["g++", "-std=c++17", f"-I{ROOT / 'include'}", str(src), "-o", str(exe), f"-L{lib_path.parent}",
                    "-lpet_b200", f"-Wl,-rpath,{lib_path.parent}"], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout
    assert "caught:" in out
