#!/usr/bin/env bash
# Test infrastructure only. Builds oracle/_ref/libwoq_ref.so from the reference project's own
# integer weight path (symmetric_quantize + preprocess_weights_for_mixed_gemm and their helpers),
# compiled from the sources where they lie. Nothing is copied into this repository and nothing
# is written outside oracle/_ref/.
#
#   usage: oracle/build_ref.sh [REFERENCE_ROOT]      (default: $WOQ_REFERENCE_ROOT, else the reference checkout next to this repository)
#
# The reference needs CUTLASS headers for a handful of type traits only (half_t, uint4b_t,
# sizeof_bits, arch tags, layout tags); its own copy is an un-vendored git submodule, so the
# headers are taken from any CUTLASS include tree found in the Python environment. The script
# exits 0 without building when the reference or CUTLASS headers are absent, so callers can
# treat the cross-check as optional.
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ref="${1:-${WOQ_REFERENCE_ROOT:-$here/../../reference}}"
out="$here/_ref"
src="$ref/cpp/tensorrt_llm"

if [ ! -f "$src/kernels/cutlass_kernels/cutlass_preprocessors.cpp" ]; then
    echo "build_ref: reference sources not found under $ref - skipped"
    exit 0
fi

cutlass_inc="${CUTLASS_INCLUDE:-}"
if [ -z "$cutlass_inc" ]; then
    site="$(python -c 'import sysconfig; print(sysconfig.get_paths()["purelib"])' 2>/dev/null || true)"
    for cand in "$site/flashinfer/data/cutlass/include" "$site/tilelang/3rdparty/cutlass/include" \
                "$site/cutlass_library/source/include" /opt/cutlass/include; do
        if [ -f "$cand/cutlass/numeric_types.h" ]; then cutlass_inc="$cand"; break; fi
    done
fi
if [ -z "$cutlass_inc" ]; then
    echo "build_ref: no CUTLASS include tree found - skipped"
    exit 0
fi

cuda_inc="${CUDA_HOME:-/usr/local/cuda}/include"
mkdir -p "$out"
# -Bsymbolic: the CUDA runtime stubs in ref_shim.cpp must win over a real libcudart that the
# host process (torch) may already have loaded.
g++ -std=c++17 -O2 -fPIC -shared -w -Wl,-Bsymbolic -DENABLE_BF16 \
    -I "$ref/cpp" -I "$ref/cpp/include" \
    -I "$src/cutlass_extensions/include" -I "$cutlass_inc" -I "$cuda_inc" \
    "$here/ref_shim.cpp" \
    "$src/kernels/cutlass_kernels/cutlass_preprocessors.cpp" \
    "$src/common/stringUtils.cpp" "$src/common/tllmException.cpp" \
    "$src/common/logger.cpp" "$src/common/assert.cpp" \
    -o "$out/libwoq_ref.so"
echo "build_ref: built $out/libwoq_ref.so (CUTLASS headers: $cutlass_inc)"
