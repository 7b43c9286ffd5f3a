#!/usr/bin/env bash
# Builds libtrtllm_ops.so: the C++ torch.ops.trtllm registrations (trtllm_ops.cpp) against the headers
# of the installed torch wheel, linked to libw4gemm.so (which build.sh must have produced first).
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
pkg="$here/.."
read -r tinc tlib abi < <(python - <<'PY'
import os, torch
from torch.utils import cpp_extension as ce
print(" ".join("-I" + p for p in ce.include_paths()).replace(" ", ","), os.path.join(os.path.dirname(torch.__file__), "lib"),
      int(torch._C._GLIBCXX_USE_CXX11_ABI))
PY
)
cuda_inc="${CUDA_HOME:-/usr/local/cuda}/include"
g++ -std=c++17 -O2 -fPIC -shared -D_GLIBCXX_USE_CXX11_ABI="$abi" ${tinc//,/ } -I"$cuda_inc" \
    "$here/trtllm_ops.cpp" -o "$pkg/libtrtllm_ops.so" \
    -L"$pkg" -lw4gemm -L"$tlib" -lc10 -lc10_cuda -ltorch_cpu -ltorch \
    -Wl,-rpath,'$ORIGIN' -Wl,-rpath,"$tlib" -Wl,--no-as-needed
echo "built $pkg/libtrtllm_ops.so"
