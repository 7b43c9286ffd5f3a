// One-shot all-reduce over peer memory for the row-parallel weight-only GEMM: every rank's GEMM
// writes its [m, n] partial sums into a buffer that the other GPUs of the node have mapped
// (NVLink 5 through NVSwitch); this kernel, next on the same stream, tells the peers that the
// partial is complete, waits for theirs, and then every CTA pulls its slice of all partials with
// ordinary 16-byte loads, adds them in rank order in fp32 (the same order on every rank, so all
// ranks hold bit-identical results), adds the layer bias and stores the local output.
//
// It takes the place of the ncclAllReduce that follows the plugin in the reference
// (cpp/tensorrt_llm/plugins/ncclPlugin/allreducePlugin.cpp:407) for messages small enough that the
// collective is latency-bound; it follows the idea of the reference's own one-shot kernel for dense
// layers (cpp/tensorrt_llm/kernels/customAllReduceKernels.cu:1307), which the reference never
// applies to this path. No multicast objects and no cluster multicast: plain peer loads and stores.
//
// Synchronisation. Each rank owns kMaxRanks flag words; rank s announces call number `epoch` by
// storing it (release, system scope) into word s of every peer's flags.
// A CTA starts reducing once all words of its own rank's flags have reached `epoch`. Call numbers
// only grow, so flags are never reset. Callers alternate between two partial buffers: a rank can
// only reach call e + 2 after every peer has announced call e + 1, which a peer does after its call
// e (and with it all its reads of the buffers of call e) has finished.
// The wait is bounded in time; when it expires the kernel records W4_ERR_DEVICE_TIMEOUT in the
// device status word and returns without touching the output (a peer that never arrives must not
// hang this GPU).
#include "w4_common.cuh"
#include "w4_internal.h"

namespace w4
{
namespace ar
{

constexpr int kMaxRanks = W4_MAX_RANKS;
constexpr int kThreads = 256;

struct Args
{
    void const* partials[kMaxRanks];
    uint32_t* flags[kMaxRanks];
    void const* bias;
    void* out;
    size_t count;
    int n;
    int rank, world;
    uint32_t epoch;
    unsigned long long timeout_ns;
};

__device__ __forceinline__ unsigned long long global_timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(uint32_t const* p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Peer data is read around L1: the same addresses are rewritten by another GPU every second call.
__device__ __forceinline__ uint4 ld_peer(void const* p)
{
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

template <typename T>
__global__ void __launch_bounds__(kThreads) oneshot_kernel(Args const a)
{
    using P = Pair<T>;
    __shared__ int failed;
    if (threadIdx.x == 0)
        failed = 0;
    __syncthreads();

    // 1. announce: this rank's partial was written by the kernel before this one on the stream, so
    // it is already visible; the release store keeps the flag behind it for the peers
    if (blockIdx.x == 0 && threadIdx.x < a.world)
        st_release_sys(a.flags[threadIdx.x] + a.rank, a.epoch);
    // 2. wait for every rank (own word included: it is written by the CTA above)
    if (threadIdx.x < a.world)
    {
        uint32_t const* word = a.flags[a.rank] + threadIdx.x;
        unsigned long long const t0 = global_timer_ns();
        uint32_t polls = 0;
        while (int32_t(ld_acquire_sys(word) - a.epoch) < 0)
        {
            if ((++polls & 63u) == 0 && global_timer_ns() - t0 > a.timeout_ns)
            {
                failed = 1;
                atomicExch(&g_device_status, kDeviceTimeout);
                break;
            }
        }
    }
    __syncthreads();
    if (failed)
        return;

    // 3. pull and add, eight elements per thread and step
    size_t const vecs = a.count / 8;
    int const n_vec = a.n / 8;
    for (size_t i = size_t(blockIdx.x) * kThreads + threadIdx.x; i < vecs; i += size_t(gridDim.x) * kThreads)
    {
        // All peers' vectors are requested before the first is used: one NVLink round trip, not
        // `world` of them back to back.
        uint4 v[kMaxRanks];
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
            if (r < a.world)
                v[r] = ld_peer(static_cast<uint4 const*>(a.partials[r]) + i);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
        {
            if (r < a.world)
            {
                uint32_t const w[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
                for (int j = 0; j < 4; ++j)
                {
                    float lo, hi;
                    P::unpack2(w[j], lo, hi);
                    acc[2 * j] += lo;
                    acc[2 * j + 1] += hi;
                }
            }
        }
        if (a.bias)
        {
            uint4 const b = __ldg(static_cast<uint4 const*>(a.bias) + (i % n_vec));
            uint32_t const w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
            {
                float lo, hi;
                P::unpack2(w[j], lo, hi);
                acc[2 * j] += lo;
                acc[2 * j + 1] += hi;
            }
        }
        uint4 o;
        o.x = uint32_t(P::from_float(acc[0])) | (uint32_t(P::from_float(acc[1])) << 16);
        o.y = uint32_t(P::from_float(acc[2])) | (uint32_t(P::from_float(acc[3])) << 16);
        o.z = uint32_t(P::from_float(acc[4])) | (uint32_t(P::from_float(acc[5])) << 16);
        o.w = uint32_t(P::from_float(acc[6])) | (uint32_t(P::from_float(acc[7])) << 16);
        static_cast<uint4*>(a.out)[i] = o;
    }
}

} // namespace ar
} // namespace w4

extern "C" int w4_allreduce_oneshot(const W4AllReduceParams* p, void* stream)
{
    using namespace w4::ar;
    if (!p || !p->out)
        return W4_ERR_NULL_POINTER;
    if (p->world < 1 || p->world > kMaxRanks || p->rank < 0 || p->rank >= p->world)
        return W4_ERR_BAD_SHAPE;
    if (p->act_dtype != W4_DTYPE_FP16 && p->act_dtype != W4_DTYPE_BF16)
        return W4_ERR_BAD_DTYPE;
    if (p->count == 0)
        return W4_OK;
    if (p->count % 8 != 0 || p->n <= 0 || p->n % 8 != 0 || p->count % size_t(p->n) != 0)
        return W4_ERR_BAD_SHAPE;
    if (p->count * 2 > size_t(W4_ONESHOT_MAX_BYTES))
        return W4_ERR_UNSUPPORTED; // bandwidth-bound sizes belong to the library collective
    Args a{};
    for (int r = 0; r < p->world; ++r)
    {
        if (!p->partials[r] || !p->flags[r])
            return W4_ERR_NULL_POINTER;
        if (reinterpret_cast<uintptr_t>(p->partials[r]) & 15u)
            return W4_ERR_MISALIGNED;
        a.partials[r] = p->partials[r];
        a.flags[r] = p->flags[r];
    }
    if ((reinterpret_cast<uintptr_t>(p->out) | reinterpret_cast<uintptr_t>(p->bias)) & 15u)
        return W4_ERR_MISALIGNED;
    a.bias = p->bias;
    a.out = p->out;
    a.count = p->count;
    a.n = p->n;
    a.rank = p->rank;
    a.world = p->world;
    a.epoch = p->epoch;
    a.timeout_ns = p->timeout_ms > 0 ? (unsigned long long) (p->timeout_ms) * 1000000ull : 2000000000ull;
    w4::DeviceInfo const& dev = w4::current_device_info();
    if (dev.num_sms <= 0)
        return W4_ERR_CUDA;
    size_t const vecs = p->count / 8;
    size_t blocks = (vecs + kThreads - 1) / kThreads;
    if (blocks > size_t(dev.num_sms))
        blocks = size_t(dev.num_sms);
    cudaStream_t const s = static_cast<cudaStream_t>(stream);
    if (p->act_dtype == W4_DTYPE_FP16)
        oneshot_kernel<__half><<<unsigned(blocks), kThreads, 0, s>>>(a);
    else
        oneshot_kernel<__nv_bfloat16><<<unsigned(blocks), kThreads, 0, s>>>(a);
    return cudaGetLastError() == cudaSuccess ? W4_OK : W4_ERR_CUDA;
}
