// Allocation-free variant of the prefill GEMM with an AWQ pre-quant scale.
//
// w4_gemm_launch needs the caller to hand it a workspace for the scaled copy of the activations
// (m * k elements). Some callers cannot provide one: code that runs where device allocation is
// forbidden or already finished - inside a framework's "no allocation from here on" region, in a
// plugin whose host owns all device memory and offered no workspace, or in a process that must
// not touch the allocator because another component has reserved the rest of the GPU. For those
// callers the scratch lives in a fixed array inside the library image instead.
//
// The array costs W4_STATIC_SCRATCH_BYTES of device memory on every GPU that loads the library,
// from load until the process exits, whether or not this entry point is ever called.
#include <mutex>

#include "w4_common.cuh"
#include "w4_internal.h"

namespace w4
{
namespace
{

// The scratch itself. In host code this name is only a handle for the runtime's symbol table, not a
// device address: the address a kernel can use is obtained below with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[W4_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch per device, resolved once per device with that device current.
void* static_scratch_address(int* status)
{
    static void* ptrs[64] = {};
    static std::mutex mu;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    {
        *status = W4_ERR_CUDA;
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev])
    {
        void* p = nullptr;
        cudaError_t const rc = cudaGetSymbolAddress(&p, g_static_scratch);
        if (rc != cudaSuccess || !p)
        {
            *status = W4_ERR_CUDA;
            return nullptr;
        }
        ptrs[dev] = p;
    }
    *status = W4_OK;
    return ptrs[dev];
}

} // namespace
} // namespace w4

extern "C" size_t w4_gemm_static_scratch_bytes(void)
{
    return W4_STATIC_SCRATCH_BYTES;
}

extern "C" int w4_gemm_launch_static_scratch(const W4GemmParams* p, void* stream)
{
    if (!p)
        return W4_ERR_NULL_POINTER;
    // The tensor-core kernel is the one that needs scratch; run it whatever m is. The caller's
    // workspace fields are ignored.
    W4GemmParams q = *p;
    q.regime = W4_REGIME_GEMM;
    q.workspace = nullptr;
    q.workspace_bytes = 0;
    size_t const need = q.act_scale ? size_t(q.m > 0 ? q.m : 0) * size_t(q.k > 0 ? q.k : 0) * 2 : 0;
    if (need > W4_STATIC_SCRATCH_BYTES)
        return W4_ERR_STATIC_SCRATCH; // m * k * 2 bytes do not fit the built-in scratch
    if (need > 0)
    {
        int status = W4_OK;
        void* scratch = w4::static_scratch_address(&status);
        if (status != W4_OK)
            return status;
        q.workspace = scratch;
        q.workspace_bytes = W4_STATIC_SCRATCH_BYTES;
    }
    int const rc = w4_gemm_validate(&q);
    if (rc != W4_OK)
        return rc;
    if (q.m == 0)
        return W4_OK;
    return w4::launch_gemm_tc(q, static_cast<cudaStream_t>(stream));
}
