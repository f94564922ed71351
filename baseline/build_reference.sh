#!/usr/bin/env bash
# Builds lumia431/photon_infer, unmodified, with its own CMake project into baseline/_ref, and the small
# harness beside this script against it.  Usage: baseline/build_reference.sh /path/to/photon_infer
#
# * glog is not installed here: find_package(glog) is pointed at baseline/glog_shim, a header in which LOG
#   and VLOG swallow their arguments (the reference logs progress lines only).  Eigen and GTest are optional
#   in the reference's CMakeLists.txt and stay off.
# * The reference's Release flags are -O3 -march=native.  The binary is built on one machine and run on
#   another, so the build type is RelWithDebInfo with its flags set to -O3 -DNDEBUG: the same optimisation
#   without instructions of the build machine's CPU.
# * CUDA architecture 100 (B200) instead of the reference's list of 75;80;86.
set -euo pipefail
REF="${1:?path of a checkout of lumia431/photon_infer}"
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
CUDA="${CUDA_HOME:-/usr/local/cuda}"
mkdir -p "$OUT/bin"
cmake -S "$REF" -B "$OUT/build" -G Ninja -DCMAKE_CUDA_ARCHITECTURES=100 -DPHOTON_BUILD_TESTS=OFF \
  -Dglog_DIR="$HERE/glog_shim" -DCMAKE_BUILD_TYPE=RelWithDebInfo \
  -DCMAKE_CXX_FLAGS_RELWITHDEBINFO="-O3 -DNDEBUG" -DCMAKE_CUDA_FLAGS_RELWITHDEBINFO="-O3 -DNDEBUG" > "$OUT/configure.log" 2>&1
cmake --build "$OUT/build" --target photon_core > "$OUT/build.log" 2>&1
g++ -std=c++20 -O2 -DPHOTON_USE_CUDA -I"$REF/include" -I"$HERE/glog_shim" -I"$CUDA/include" \
  "$HERE/reference_bench.cpp" "$OUT/build/lib/libphoton_core.a" -L"$CUDA/lib64" -Wl,-rpath,"$CUDA/lib64" -lcublas -lcudart -lpthread \
  -o "$OUT/bin/photon_ref_bench"
echo "built $OUT/bin/photon_ref_bench"
