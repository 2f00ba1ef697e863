#!/bin/bash
# Builds the UNMODIFIED reference CUDA kernel library (its own CMake project, `kernels/`) for sm_100a into baseline/_ref/
# and links the static library into one shared object that blaze_b200.benchmarks.reference_kernels loads through ctypes.
# Needs only cmake, ninja, nvcc and cuBLAS; no Rust.  Usage: baseline/build_reference_kernels.sh <path to the reference checkout>
# (or BLAZE_REFERENCE_DIR in the environment)
set -euo pipefail
REF="${1:-${BLAZE_REFERENCE_DIR:-}}"
[ -n "$REF" ] && [ -d "$REF/kernels" ] || { echo "usage: $0 <path to the reference checkout>" >&2; exit 2; }
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
mkdir -p "$OUT/build"
cd "$OUT/build"
cmake "$REF/kernels" -G Ninja -DCMAKE_CUDA_ARCHITECTURES=100a -DBLAZE_BUILD_TESTS=OFF -DCMAKE_BUILD_TYPE=Release > cmake.log 2>&1
ninja blaze_kernels > build.log 2>&1
CUDA_LIB="$(dirname "$(dirname "$(command -v nvcc)")")/lib64"
g++ -shared -o "$OUT/libblaze_ref_kernels.so" -Wl,--whole-archive libblaze_kernels.a -Wl,--no-whole-archive \
    -L"$CUDA_LIB" -lcudart -lcublas -Wl,-rpath,"$CUDA_LIB"
cp cmake.log build.log "$OUT/" && cd "$OUT" && rm -rf "$OUT/build"   # only the shared object and the logs travel to a GPU box
echo "built $OUT/libblaze_ref_kernels.so"
