"""Builds the CUDA library in-tree: pet_kokkos_b200/libpet_b200.so (sm_100a only).

Usage: python -m pet_kokkos_b200.build [--force] [--verbose]
nvcc cross-compiles without a GPU; the built .so travels with the source tree.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "libpet_b200.so"
OBJ = HERE / "build"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-ffp-contract=off",
          "--expt-relaxed-constexpr", "-Xcudafe", "--diag_suppress=177"]
# neighbour kernels: every fp64 product and sum rounded on its own (bit-exact edge decisions)
PER_FILE = {"neighbors.cu": ["-fmad=false"]}
SOURCES = ["checkpoint.cpp", "neighbors.cu", "ops.cu", "adaptive.cu", "attention.cu", "attention_tile.cu", "attention_mma.cu", "gemm_simt.cu", "gemm_tc.cu", "model.cu", "static_gemm.cu", "nccl_exchange.cu",
           "engine.cu", "capi.cu"]


def nvcc():
    return os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "pet_b200.h"]
    jobs = []
    for src in SOURCES:
        s, o = CSRC / src, OBJ / (src + ".o")
        if force or _stale(o, [s] + headers):
            cmd = [nvcc(), *ARCH, *COMMON, *PER_FILE.get(src, []), "-c", str(s), "-o", str(o)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError("nvcc failed on " + cmd[-3])

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(run, jobs))
    objs = [str(OBJ / (s + ".o")) for s in SOURCES]
    if jobs or force or not OUT.exists():
        cmd = [nvcc(), *ARCH, "-shared", "-o", str(OUT), *objs, "-lcudart", "-lcuda", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
