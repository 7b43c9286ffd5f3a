// Prefill-regime tensor-core kernel (placeholder until the tcgen05 path lands).
#include "w4_common.cuh"
#include "w4_internal.h"

namespace w4
{

size_t gemm_tc_workspace_bytes(int m, int n, int k, int has_act_scale)
{
    (void) n;
    return has_act_scale ? size_t(m) * k * 2 : 0;
}

int launch_gemm_tc(W4GemmParams const& p, cudaStream_t stream)
{
    (void) p;
    (void) stream;
    return W4_ERR_UNSUPPORTED;
}

} // namespace w4
