// Host-side creation of TMA tensor maps. cuTensorMapEncodeTiled lives in the driver library; it
// is looked up at run time through the runtime API so that the shared object has no link-time
// dependency on libcuda (it must load on a machine without a driver for the CPU-only checks).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace w4
{

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, cuuint64_t const*,
    cuuint64_t const*, cuuint32_t const*, cuuint32_t const*, CUtensorMapInterleave, CUtensorMapSwizzle,
    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn)
    {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess
            && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D row-major tensor: `cols` elements per row (innermost), `rows` rows, `row_stride_bytes`
// between rows; box = box_cols x box_rows elements. Out-of-range elements read as zero.
inline bool make_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dtype, void const* base, uint64_t cols,
    uint64_t rows, uint64_t row_stride_bytes, uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle swizzle)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn)
        return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
        == CUDA_SUCCESS;
}

} // namespace w4
