#!/bin/bash
# Builds the reference's native CUDA runtime, unmodified, for sm_100 and installs the binary where
# baseline/reference_arm.py looks for it (baseline/_ref/bin/mfq-runtime).
#
#   baseline/build_reference_runtime.sh [path to the reference checkout] [build directory]
#
# The reference tree is copied first because CMake writes into its source tree's sibling paths; the copy is
# configured with the reference's own CMakeLists (cpp_runtime/CMakeLists.txt; CUDA back end
# cpp_runtime/backends/cuda/CMakeLists.txt, which takes its target from MFQ_CUDA_ARCHITECTURES) and only the
# `mfq-runtime` target is built.  Needs cmake >= 3.26, nvcc and a host compiler; NCCL is picked up when present.
set -euo pipefail
SRC="${1:-/root/reference}"
BUILD="${2:-/tmp/mfq-reference-build}"
HERE="$(cd "$(dirname "$0")" && pwd)"
rm -rf "$BUILD/src"
mkdir -p "$BUILD/src" "$BUILD/out" "$HERE/_ref/bin"
cp -r "$SRC/." "$BUILD/src/"
cmake -S "$BUILD/src/cpp_runtime" -B "$BUILD/out" -G Ninja \
      -DCMAKE_BUILD_TYPE=Release \
      -DMFQ_BUILD_CUDA_RUNTIME=ON -DMFQ_BUILD_HIP_RUNTIME=OFF -DMFQ_BUILD_METAL_RUNTIME=OFF \
      -DMFQ_CUDA_ARCHITECTURES=100 \
      -DCMAKE_CUDA_COMPILER="${NVCC:-/usr/local/cuda/bin/nvcc}"
cmake --build "$BUILD/out" --target mfq-runtime -j "$(nproc)"
BIN="$(find "$BUILD/out" -type f -name mfq-runtime -perm -u+x | head -n 1)"
cp "$BIN" "$HERE/_ref/bin/mfq-runtime"
echo "installed $HERE/_ref/bin/mfq-runtime"
