// Single translation unit of the device library: the kernels share one device-side status word
// and are compiled together for sm_100a only.
#include "w4_gemv.cu"
#include "w4_gemm_tc.cu"
#include "w4_api.cu"
#include "w4_static_scratch.cu"
#include "w4_prep_gpu.cu"
#include "w4_allreduce.cu"
