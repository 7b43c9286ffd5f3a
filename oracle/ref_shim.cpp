// Test infrastructure only (never linked into the product library).
//
// C entry points over the reference's own integer weight path, compiled from the reference
// sources where they lie (see build_ref.sh). The reference asks the CUDA runtime for the
// device's compute capability before choosing a layout
// (cpp/tensorrt_llm/kernels/cutlass_kernels/cutlass_preprocessors.cpp:567 through
// cpp/include/tensorrt_llm/common/cudaUtils.h:285-294); there is no GPU on a build host, so
// the runtime calls it makes are answered here with "device 0, compute capability
// REF_SM_MAJOR.REF_SM_MINOR" (10.0 = B200 by default).
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <exception>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include "tensorrt_llm/kernels/cutlass_kernels/cutlass_preprocessors.h"

static int g_sm_major = 10, g_sm_minor = 0;

// Failures of the reference's own shape checks come back as exceptions; report them as a status
// and, when WOQ_REF_VERBOSE is set, print what the reference said.
static int report(std::exception const& e)
{
    if (std::getenv("WOQ_REF_VERBOSE"))
        std::fprintf(stderr, "reference raised: %s\n", e.what());
    return -1;
}

extern "C"
{
    cudaError_t cudaGetDevice(int* device)
    {
        *device = 0;
        return cudaSuccess;
    }

    cudaError_t cudaDeviceGetAttribute(int* value, enum cudaDeviceAttr attr, int)
    {
        if (attr == cudaDevAttrComputeCapabilityMajor)
            *value = g_sm_major;
        else if (attr == cudaDevAttrComputeCapabilityMinor)
            *value = g_sm_minor;
        else
            *value = 0;
        return cudaSuccess;
    }

    char const* cudaGetErrorString(cudaError_t)
    {
        return "stubbed CUDA runtime (no device on this host)";
    }

    cudaError_t cudaGetLastError(void)
    {
        return cudaSuccess;
    }

    // Referenced by inline helpers of the reference's cudaUtils.h that this path never calls.
    cudaError_t cudaDeviceSynchronize(void)
    {
        return cudaSuccess;
    }

    cudaError_t cudaMemcpy(void*, void const*, size_t, enum cudaMemcpyKind)
    {
        return cudaErrorNoDevice;
    }

    cudaError_t cudaPointerGetAttributes(struct cudaPointerAttributes*, void const*)
    {
        return cudaErrorNoDevice;
    }
}

namespace ck = tensorrt_llm::kernels::cutlass_kernels;

static ck::QuantType qt(int bits)
{
    return bits == 8 ? ck::QuantType::W8_A16 : ck::QuantType::W4_A16;
}

extern "C"
{
    void ref_set_sm(int major, int minor)
    {
        g_sm_major = major;
        g_sm_minor = minor;
    }

    // rows = K, cols = N (element counts). Buffers hold rows*cols*bits/8 bytes.
    int ref_preprocess_weights_for_mixed_gemm(int8_t* out, int8_t const* in, size_t rows, size_t cols, int bits)
    {
        try
        {
            ck::preprocess_weights_for_mixed_gemm(out, in, {rows, cols}, qt(bits), false);
        }
        catch (std::exception const& e)
        {
            return report(e);
        }
        return 0;
    }

    // int4 weights laid out for fp8 activations (W4A8).
    int ref_preprocess_weights_w4a8(int8_t* out, int8_t const* in, size_t rows, size_t cols)
    {
        try
        {
            ck::preprocess_weights_for_mixed_gemm(out, in, {rows, cols}, ck::QuantType::W4_AFP8, false);
        }
        catch (std::exception const& e)
        {
            return report(e);
        }
        return 0;
    }

    int ref_permute_B_rows(int8_t* out, int8_t const* in, size_t rows, size_t cols, int bits)
    {
        try
        {
            ck::permute_B_rows_for_mixed_gemm(out, in, {rows, cols}, qt(bits), 80);
        }
        catch (std::exception const& e)
        {
            return report(e);
        }
        return 0;
    }

    int ref_subbyte_transpose(int8_t* out, int8_t const* in, size_t rows, size_t cols, int bits)
    {
        try
        {
            ck::subbyte_transpose(out, in, {rows, cols}, qt(bits));
        }
        catch (std::exception const& e)
        {
            return report(e);
        }
        return 0;
    }

    int ref_add_bias_and_interleave_inplace(int8_t* buf, size_t num_elts, int bits)
    {
        try
        {
            ck::add_bias_and_interleave_quantized_tensor_inplace(buf, num_elts, qt(bits));
        }
        catch (std::exception const& e)
        {
            return report(e);
        }
        return 0;
    }

    // weight fp32 [rows, cols]; scale_kind: 0 = fp32 scales, 1 = fp16, 2 = bf16 (the
    // <ComputeType, float> instantiations the reference ships).
    int ref_symmetric_quantize_f32(int8_t* processed, int8_t* unprocessed, void* scales, float const* weight,
        size_t rows, size_t cols, int bits, int scale_kind)
    {
        try
        {
            std::vector<size_t> shape{rows, cols};
            if (scale_kind == 1)
                ck::symmetric_quantize<half, float>(
                    processed, unprocessed, reinterpret_cast<half*>(scales), weight, shape, qt(bits), false);
            else if (scale_kind == 2)
                ck::symmetric_quantize<__nv_bfloat16, float>(
                    processed, unprocessed, reinterpret_cast<__nv_bfloat16*>(scales), weight, shape, qt(bits), false);
            else
            {
                // Only the 6-argument <float, float> form is instantiated by the reference.
                ck::symmetric_quantize<float, float>(
                    processed, reinterpret_cast<float*>(scales), weight, shape, qt(bits), false);
                if (unprocessed)
                    return -2;
            }
        }
        catch (std::exception const& e)
        {
            return report(e);
        }
        return 0;
    }

    int ref_symmetric_quantize_f16(int8_t* processed, int8_t* unprocessed, void* scales, void const* weight,
        size_t rows, size_t cols, int bits)
    {
        try
        {
            ck::symmetric_quantize<half, half>(processed, unprocessed, reinterpret_cast<half*>(scales),
                reinterpret_cast<half const*>(weight), {rows, cols}, qt(bits), false);
        }
        catch (std::exception const& e)
        {
            return report(e);
        }
        return 0;
    }

    int ref_symmetric_quantize_bf16(int8_t* processed, int8_t* unprocessed, void* scales, void const* weight,
        size_t rows, size_t cols, int bits)
    {
        try
        {
            ck::symmetric_quantize<__nv_bfloat16, __nv_bfloat16>(processed, unprocessed,
                reinterpret_cast<__nv_bfloat16*>(scales), reinterpret_cast<__nv_bfloat16 const*>(weight), {rows, cols},
                qt(bits), false);
        }
        catch (std::exception const& e)
        {
            return report(e);
        }
        return 0;
    }
}
