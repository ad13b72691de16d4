#!/bin/bash
# Compiles the reference's own evaluation path, from its sources where they lie,
# into two host libraries under oracle/_ref/:
#   libpet_ref.so       its GEMMs are the reference's own portable loop -- every line that
#                       computes is the reference's; the parity tests and the fixtures use it;
#   libpet_ref_blas.so  its PET_HAVE_CBLAS build (the reference's PET_USE_BLAS option), GEMMs
#                       through the optimised BLAS of this image -- the timed CPU baseline.
# g++ alone, against the host stand-in for Kokkos in oracle/kokkos_host/ and the
# nlohmann/json header that ships inside the cudnn-frontend Python package of this
# image. Nothing is copied out of the reference tree; only objects and the two
# libraries are written, under oracle/_ref/.
#
#   oracle/build_ref.sh <reference-root>
#
# TEST INFRASTRUCTURE ONLY (the checker of the parity tests and the CPU baseline).
set -euo pipefail
REF=${1:?usage: build_ref.sh <reference-root>}
HERE=$(cd "$(dirname "$0")" && pwd)
OUT=$HERE/_ref
JSON_INC=$(python - <<'PY'
import os, sysconfig, glob
for root in {sysconfig.get_paths()["purelib"], sysconfig.get_paths()["platlib"]}:
    for p in glob.glob(os.path.join(root, "include", "cudnn_frontend", "thirdparty")):
        if os.path.exists(os.path.join(p, "nlohmann", "json.hpp")):
            print(p); raise SystemExit
raise SystemExit("no nlohmann/json.hpp in this image")
PY
)
# d3.cpp / d3_data.cpp (DFT-D3, outside the evaluated path) are left out; ref_driver.cpp stubs what refers to them.
SRCS="model ops neighbors device_neighbors attention feedforward residual forces hvp device_geometry
      device_cell_list calculator checkpoint ozaki gemm_lowp vesin_neighbors fused_gemm fused_gemm_hip"
BASE="-std=c++17 -O2 -fPIC -fopenmp -march=x86-64-v3 -ffp-contract=off -w -I$HERE/kokkos_host -I$REF/include -I$JSON_INC"

build_variant() {  # <object dir> <library> <extra flags>
  local obj=$OUT/$1 lib=$OUT/$2 extra=$3 pids=() objs=""
  mkdir -p "$obj"
  for s in $SRCS; do
    g++ $BASE $extra -c "$REF/src/$s.cpp" -o "$obj/$s.o" &
    pids+=($!)
    objs="$objs $obj/$s.o"
  done
  g++ $BASE $extra -c "$HERE/ref_driver.cpp" -o "$obj/ref_driver.o" &
  pids+=($!)
  for p in "${pids[@]}"; do wait "$p"; done
  g++ -shared -fopenmp -o "$lib" $objs "$obj/ref_driver.o" -ldl -Wl,--no-undefined
  echo "built $lib"
}
build_variant obj libpet_ref.so ""
build_variant obj_blas libpet_ref_blas.so "-DPET_HAVE_CBLAS"
