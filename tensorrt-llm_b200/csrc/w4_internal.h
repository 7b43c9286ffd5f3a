// Internal interfaces between the C ABI (w4_api.cu) and the kernel translation units.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/w4_gemm.h"

namespace w4
{

struct DeviceInfo
{
    int device = -1;
    int num_sms = 0;
    int max_smem_optin = 0;
};

// Cached per-device properties of the current device (thread-safe, no allocation).
DeviceInfo const& current_device_info();

// Streaming decode kernel: handles any m by passes of at most 8 rows. Returns a W4Status.
// Where the decode kernel's epilogue sends its results when the all-reduce is fused into it: the
// packet inbox (slot `rank`) in every rank's all-reduce workspace. world == 0: no push.
struct PushTarget
{
    uint8_t* ws[W4_MAX_RANKS];
    int rank;
    int world;
    size_t pkt_slot;   // bytes of one sender's packet slot
    size_t copy_bytes; // bytes of one copy of the workspace's data areas
    size_t header_bytes;
    // gather != 0: the kernel also collects the peers' packets and writes the reduced result (one
    // kernel for GEMM and all-reduce); it then advances the workspace's call number itself.
    int gather;
    void const* bias;            // added after the sum when gathering
    unsigned long long timeout_ns;
};
int launch_gemv(W4GemmParams const& p, cudaStream_t stream, PushTarget const* push = nullptr);
// Fills `t` for the one-shot packet protocol of this all-reduce call; false when the call would not
// use that protocol (size, mode) or its arguments are not valid.
bool allreduce_push_target(W4AllReduceParams const& r, PushTarget* t);

// tcgen05 tensor-core kernel. Returns a W4Status.
int launch_gemm_tc(W4GemmParams const& p, cudaStream_t stream);
// Workspace: the minimum the kernel needs (scaled activation copy), and what also allows split-k.
size_t gemm_tc_workspace_min(int m, int k, int has_act_scale);
size_t gemm_tc_workspace_bytes(int m, int n, int k, int has_act_scale, int bits);
int gemm_tc_splits(int m, int n, int k, int num_sms, int bits);
// Activation-row tile the tensor-core kernel uses for this problem, and its estimated duration
// (microseconds, measured per-step costs); shared by the launcher and the regime heuristic.
int gemm_tc_row_tile(int m, int n, int num_sms, int bits);
double gemm_tc_estimate_us(int m, int n, int k, int num_sms, int bits);

// out[m, k] = act[m, k] * scale[k], rounded to the element type (the reference's
// apply_per_channel_scale, cpp/tensorrt_llm/kernels/preQuantScaleKernel.cu:43-95).
int launch_pre_quant_scale(void* out, void const* act, void const* scale, int m, int k, int act_dtype,
    cudaStream_t stream);

} // namespace w4
