#!/usr/bin/env bash
# Builds libw4gemm.so (CUDA kernels + C ABI + host-side weight preparation) in-tree for sm_100a.
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
out="$here/../libw4gemm.so"
nvcc -std=c++17 -O3 -lineinfo -gencode arch=compute_100a,code=sm_100a \
     -Xcompiler -fPIC,-O3,-pthread ${W4_NVCC_EXTRA:-} \
     -shared "$here/w4_lib.cu" "$here/w4_preprocess.cpp" -o "$out"
echo "built $out"
