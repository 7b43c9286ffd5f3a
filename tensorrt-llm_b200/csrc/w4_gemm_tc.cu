// Prefill-regime kernel: weight-only GEMM on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// Replaces CutlassFpAIntBGemmRunner::gemm of the reference project
// (cpp/tensorrt_llm/kernels/cutlass_kernels/fpA_intB_gemm/fpA_intB_gemm_template.h:394-465), which
// on compute capability 10.x runs an Ampere mma.sync kernel. Same math as that kernel: every
// weight is dequantised to T as round_T(fma(q, scale, zero))
// (cpp/tensorrt_llm/cutlass_extensions/include/cutlass_extensions/gemm/warp/mma_tensorop_dequantizer.h:247-262),
// products are accumulated in fp32, alpha and bias are applied in the epilogue.
//
// Orientation. The output tile is computed transposed: D[n, m] = sum_k W[n, k] * A[m, k]. The
// dequantised weights are the MMA's "A" operand and live in tensor memory (one TMEM lane per
// output column n, 128 per tile), written there straight from registers by the conversion warps,
// so they never travel through shared memory; the activations are the "B" operand, brought by TMA
// into 128-byte-swizzled shared memory and consumed by the MMA unmodified. One tile is 128 columns
// of W times up to 256 rows of the activation matrix, so each weight is converted once per 256
// activation rows.
//
// Warp roles (320 threads, one CTA per SM, persistent over tiles):
//   warp 0      TMA producer: activation tile [BM x 64] + packed weight tile per k step
//   warp 1      allocates TMEM, issues tcgen05.mma (one elected lane), commits to mbarriers
//   warps 2..9  conversion, two warps per TMEM lane quadrant taking alternate k steps: shared memory
//               -> registers -> exact int->T conversion, scale/zero -> tcgen05.st into the TMEM ring
//               of A stages; after the last k step the same warps run the epilogue (tcgen05.ld,
//               alpha/bias, convert, store), each on its share of the accumulator columns.
// All waits are bounded; a timeout sets the device status word and the CTA drains and exits.
#include <type_traits>

#include "w4_common.cuh"
#include "w4_internal.h"
#include "w4_tma.h"

namespace w4
{
namespace tc
{

constexpr int BN = 128;       // weight columns per tile (MMA M, TMEM lanes)
constexpr int BK = 64;        // k per pipeline step (one 128-byte swizzle span of T)
constexpr int kAStages = 4;   // TMEM ring of converted-weight stages (32 columns each)
constexpr int kACol0 = 256;   // first TMEM column of that ring; the accumulator uses [0, 256)
constexpr int kTmemCols = 512;
constexpr int kConvGroups = 2;   // groups of 4 conversion warps; group g converts k steps with ks % 2 == g
constexpr int kThreads = 64 + 128 * kConvGroups;
constexpr int kMaxStages = 8;

struct Args
{
    void const* scales;
    void const* zeros;
    void const* bias;
    void* out;
    float alpha;
    int m, n, k;
    int group_shift; // log2(group size), 31 = per-channel
    int tiles_n, tiles_m;
    int num_stages;
};

struct __align__(8) Barriers
{
    uint64_t full[kMaxStages];    // TMA landed (tx bytes)
    uint64_t empty[kMaxStages];   // MMA finished with the activations + 4 conversion warps read the weights
    uint64_t a_full[kAStages];    // 4 conversion warps stored the stage into TMEM
    uint64_t a_empty[kAStages];   // MMA finished reading the stage
    uint64_t d_full;              // accumulator complete
    uint64_t d_empty;             // 4 epilogue warps drained the accumulator
    uint32_t tmem_base;
    int abort_flag;
};

#ifdef W4_DBG_TRACE
// Debug build only: cycles CTA 0 spent in each kind of wait, per role.
__device__ long long g_tc_trace[64];
#define W4_TC_TIMED(slot_, expr_)                                                                                     \
    do                                                                                                                 \
    {                                                                                                                  \
        long long t0_ = clock64();                                                                                     \
        expr_;                                                                                                         \
        dbg_acc[(slot_) & 3] += clock64() - t0_;                                                                       \
    } while (0)
#define W4_TC_FLUSH(base_)                                                                                             \
    do                                                                                                                 \
    {                                                                                                                  \
        if (blockIdx.x == 0 && lane == 0)                                                                              \
            for (int i_ = 0; i_ < 4; ++i_)                                                                             \
                g_tc_trace[(base_) + i_] = dbg_acc[i_];                                                                \
    } while (0)
#else
#define W4_TC_TIMED(slot_, expr_) expr_
#define W4_TC_FLUSH(base_)
#endif

__device__ __forceinline__ bool wait_flag(uint64_t* bar, uint32_t parity, volatile int* abort_flag)
{
    for (uint32_t i = 0; i < kMaxWaitPolls; ++i)
    {
        if (mbar_try_wait(bar, parity))
            return true;
        if ((i & 255u) == 255u && *abort_flag)
            return false;
    }
    *abort_flag = 1;
    atomicExch(&g_device_status, kDeviceTimeout);
    return false;
}

__device__ __forceinline__ void tc_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem descriptor]; A is 128 lanes x 16 k of T (8 columns).
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate)
{
    uint32_t const acc = accumulate ? 1u : 0u;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
}

__device__ __forceinline__ void tc_st16(uint32_t taddr, uint32_t const (&v)[16])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(
            taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}

__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
        "%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major, 128-byte-swizzled tile of T whose rows are 128
// bytes (64 elements) wide: 8-row groups are 1024 bytes apart, descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr)
{
    uint64_t d = uint64_t((smem_addr & 0x3ffffu) >> 4);
    d |= uint64_t(1024 >> 4) << 32; // stride between 8-row groups
    d |= uint64_t(1) << 46;         // version
    d |= uint64_t(2) << 61;         // SWIZZLE_128B
    return d;
}

template <typename T, int BITS, int BM, bool HAS_ZERO>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_kernel(Args const a, __grid_constant__ CUtensorMap const tm_act, __grid_constant__ CUtensorMap const tm_w)
{
    using P = Pair<T>;
    constexpr int IL = BITS == 4 ? 4 : 2;
    constexpr int ACT_BYTES = BM * 128;          // BM rows x 64 k of T
    constexpr int W_BYTES = (BN / IL) * 128;     // interleaved rows x one 128-byte line each
    constexpr int STAGE_BYTES = ACT_BYTES + W_BYTES;
    constexpr int SEG = 128 / IL;                // bytes of one column inside a line
    constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u; // 0 = fp16, 1 = bf16
    constexpr uint32_t kIdesc = (1u << 4)                                   // fp32 accumulator
        | (kFmt << 7)                                                       // A type
        | (kFmt << 10)                                                      // B type (both K-major)
        | (uint32_t(BM >> 3) << 17)                                         // MMA N = activation rows
        | (uint32_t(BN >> 4) << 24);                                        // MMA M = weight columns

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Barriers* bars = reinterpret_cast<Barriers*>(smem + size_t(a.num_stages) * STAGE_BYTES);
    volatile int* abort_flag = &bars->abort_flag;

    int const warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef W4_DBG_TRACE
    long long dbg_acc[4] = {0, 0, 0, 0};
    if (blockIdx.x == 0 && threadIdx.x == 0)
    {
        for (int i = 0; i < 32; ++i)
            g_tc_trace[i] = 0;
        g_tc_trace[33] = clock64();
    }
    __syncthreads();
#endif
    int const num_tiles = a.tiles_n * a.tiles_m;
    int const ksteps = a.k / BK;

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < a.num_stages; ++s)
        {
            mbar_init(&bars->full[s], 1);
            mbar_init(&bars->empty[s], 5);
        }
        for (int s = 0; s < kAStages; ++s)
        {
            mbar_init(&bars->a_full[s], 4);
            mbar_init(&bars->a_empty[s], 1);
        }
        mbar_init(&bars->d_full, 1);
        mbar_init(&bars->d_empty, 4 * kConvGroups);
        bars->abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&bars->tmem_base)),
                     "r"(uint32_t(kTmemCols))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t const tmem = bars->tmem_base;

    if (warp == 0)
    {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0)
        {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_act) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w) : "memory");
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
#ifdef W4_DBG_MMA_ONLY
            ok = false; // timing experiment: nothing is loaded
#endif
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x)
            {
                int const tn = tile % a.tiles_n, tm = tile / a.tiles_n;
                for (int ks = 0; ks < ksteps; ++ks)
                {
                    W4_TC_TIMED(0, ok = wait_flag(&bars->empty[s], ph ^ 1, abort_flag));
                    if (!ok)
                        break;
                    uint8_t* stage = smem + size_t(s) * STAGE_BYTES;
#ifdef W4_DBG_HALF_ACT
                    // timing experiment only (wrong results): fetch the activation tile on even steps only
                    if (ks & 1)
                    {
                        mbar_expect_tx(&bars->full[s], W_BYTES);
                        tma_load_2d(stage + ACT_BYTES, &tm_w, ks * 128, tn * (BN / IL), &bars->full[s]);
                    }
                    else
#endif
                    {
                        mbar_expect_tx(&bars->full[s], STAGE_BYTES);
                        tma_load_2d(stage, &tm_act, ks * BK, tm * BM, &bars->full[s]);
                        tma_load_2d(stage + ACT_BYTES, &tm_w, ks * 128, tn * (BN / IL), &bars->full[s]);
                    }
                    if (++s == a.num_stages)
                    {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    }
    else if (warp == 1)
    {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0)
        {
            int s = 0, t = 0;
            uint32_t ph = 0, aph = 0, dph = 0;
            bool ok = true;
            for (int tile = blockIdx.x, it = 0; tile < num_tiles && ok; tile += gridDim.x, ++it)
            {
                if (it > 0)
                {
                    W4_TC_TIMED(3, ok = wait_flag(&bars->d_empty, dph, abort_flag));
                    if (!ok)
                        break;
                    dph ^= 1;
                    tc_fence_after();
                }
                for (int ks = 0; ks < ksteps; ++ks)
                {
#ifndef W4_DBG_MMA_ONLY
                    W4_TC_TIMED(1, ok = wait_flag(&bars->full[s], ph, abort_flag));
                    if (!ok)
                        break;
                    W4_TC_TIMED(2, ok = wait_flag(&bars->a_full[t], aph, abort_flag));
                    if (!ok)
                        break;
#endif
                    tc_fence_after();
                    uint32_t const b_addr = smem_u32(smem + size_t(s) * STAGE_BYTES);
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk)
                        tc_mma_ts(tmem, tmem + kACol0 + t * 32 + kk * 8, smem_desc_sw128(b_addr + kk * 32), kIdesc,
                            (ks | kk) != 0);
                    tc_commit(&bars->empty[s]);
                    tc_commit(&bars->a_empty[t]);
                    if (++s == a.num_stages)
                    {
                        s = 0;
                        ph ^= 1;
                    }
                    if (++t == kAStages)
                    {
                        t = 0;
                        aph ^= 1;
                    }
                }
                if (ok)
                    tc_commit(&bars->d_full);
            }
        }
    }
    else
    {
        // ------------------------------------------------------------------ conversion + epilogue
        int const quad = warp & 3;             // TMEM lane quadrant this warp may touch
        int const cgroup = (warp - 2) >> 2;    // which k steps this warp converts
        int const n_local = quad * 32 + lane;  // weight column inside the tile = TMEM lane
        uint32_t const lane_addr = tmem + (uint32_t(quad * 32) << 16);
        uint16_t const* scales = static_cast<uint16_t const*>(a.scales);
        uint16_t const* zeros = static_cast<uint16_t const*>(a.zeros);
        uint16_t const* bias = static_cast<uint16_t const*>(a.bias);
        uint16_t* out = static_cast<uint16_t*>(a.out);
        int const gsh = a.group_shift >= 31 ? 30 : a.group_shift - 6; // log2(k steps per scale group)
        // Column segment of this thread inside a stage's weight lines (two or four 16-byte chunks).
        int const w_off = (n_local / IL) * 128 + (n_local % IL) * SEG;

        int s = 0, t = 0;
        uint32_t ph = 0, aph = 0, dph = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x)
        {
            int const tn = tile % a.tiles_n, tm = tile / a.tiles_n;
            int const n = tn * BN + n_local;
            bool const n_ok = n < a.n;
            uint32_t s2 = 0, z2 = 0, s2_next = 0, z2_next = 0;
            if (n_ok)
            {
                s2_next = scales[n];
                if (HAS_ZERO)
                    z2_next = zeros[n];
            }
#ifdef W4_DBG_MMA_ONLY
            for (int ks = 0; ks < 0; ++ks)
#else
            for (int ks = 0; ks < ksteps; ++ks)
#endif
            {
                if ((ks & ((1 << gsh) - 1)) == 0)
                {
                    // new scale group: take the prefetched pair, start fetching the next one
                    s2 = s2_next | (s2_next << 16);
                    z2 = z2_next | (z2_next << 16);
                    int const gnext = (ks >> gsh) + 1;
                    if (n_ok && (gnext << gsh) < ksteps)
                    {
                        s2_next = scales[size_t(gnext) * a.n + n];
                        if (HAS_ZERO)
                            z2_next = zeros[size_t(gnext) * a.n + n];
                    }
                }
                if ((ks % kConvGroups) == cgroup)
                {
                    W4_TC_TIMED(4 + 4 * quad, ok = wait_flag(&bars->full[s], ph, abort_flag));
                    if (!ok)
                        break;
                    uint8_t const* wsm = smem + size_t(s) * STAGE_BYTES + ACT_BYTES + w_off;
                    constexpr int CHUNKS = SEG / 16; // 2 (int4) or 4 (int8)
                    uint4 raw[CHUNKS];
    #pragma unroll
                    for (int c = 0; c < CHUNKS; ++c)
                        raw[c] = *reinterpret_cast<uint4 const*>(wsm + c * 16);
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(&bars->empty[s]);
                    W4_TC_TIMED(5 + 4 * quad, ok = wait_flag(&bars->a_empty[t], aph ^ 1, abort_flag));
                    if (!ok)
                        break;
                    tc_fence_after();
                    uint32_t const a_addr = lane_addr + kACol0 + t * 32;
                    if (BITS == 4)
                    {
    #pragma unroll
                        for (int c = 0; c < 2; ++c)
                        {
                            uint32_t const r[4] = {raw[c].x, raw[c].y, raw[c].z, raw[c].w};
                            uint32_t v[16];
    #pragma unroll
                            for (int j = 0; j < 4; ++j)
                            {
                                uint32_t q[4];
                                cvt_int4x8<T>(r[j], q);
    #pragma unroll
                                for (int p = 0; p < 4; ++p) // pair p of register j holds k = 2j + 8p (+1)
                                    v[j + 4 * p] = HAS_ZERO ? P::fma(q[p], s2, z2) : P::mul(q[p], s2);
                            }
                            tc_st16(a_addr + 16 * c, v); // the TMEM address is warp-uniform
                        }
                    }
                    else
                    {
    #pragma unroll
                        for (int h = 0; h < 2; ++h)
                        {
                            uint32_t v[16];
    #pragma unroll
                            for (int cc = 0; cc < 2; ++cc)
                            {
                                uint4 const x = raw[2 * h + cc];
                                uint32_t const r[4] = {x.x, x.y, x.z, x.w};
    #pragma unroll
                                for (int j = 0; j < 4; ++j)
                                {
                                    uint32_t q[2];
                                    cvt_int8x4<T>(r[j], q);
    #pragma unroll
                                    for (int p = 0; p < 2; ++p) // pair p of register j holds k = 2j + 8p (+1)
                                        v[8 * cc + j + 4 * p] = HAS_ZERO ? P::fma(q[p], s2, z2) : P::mul(q[p], s2);
                                }
                            }
                            tc_st16(a_addr + 16 * h, v);
                        }
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(&bars->a_full[t]);
                }
                if (++s == a.num_stages)
                {
                    s = 0;
                    ph ^= 1;
                }
                if (++t == kAStages)
                {
                    t = 0;
                    aph ^= 1;
                }
            }
            if (!ok)
                break;

            // ---- epilogue: this thread owns output column n for all BM rows of the tile
            W4_TC_TIMED(6 + 4 * quad, ok = wait_flag(&bars->d_full, dph, abort_flag));
            if (!ok)
                break;
            dph ^= 1;
            tc_fence_after();
            float const bias_f = (bias && n_ok) ? P::to_float(bias[n]) : 0.f;
            int const m0 = tm * BM;
#pragma unroll 1
            for (int c0 = cgroup * 32; c0 < BM; c0 += 32 * kConvGroups)
            {
                if (m0 + c0 >= a.m)
                    break; // warp-uniform
                uint32_t v[32];
                tc_ld32(lane_addr + c0, v);
                if (n_ok)
                {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                    {
                        int const mrow = m0 + c0 + j;
                        if (mrow < a.m)
                            out[size_t(mrow) * a.n + n] = P::from_float(fmaf(a.alpha, __uint_as_float(v[j]), bias_f));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&bars->d_empty);
        }
    }

#ifdef W4_DBG_TRACE
    if (blockIdx.x == 0 && threadIdx.x == 0)
        g_tc_trace[32] = clock64();
#endif
    if (warp == 0)
        W4_TC_FLUSH(40);
    else if (warp == 1)
        W4_TC_FLUSH(0);
    else if (warp < 6)
        W4_TC_FLUSH(4 + 4 * (warp & 3));
    // Teardown: everyone meets here (also after a timeout), then the allocating warp frees TMEM.
    tc_fence_before();
    __syncthreads();
    if (warp == 1)
    {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(uint32_t(kTmemCols))
                     : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
template <typename T, int BITS, int BM, bool HAS_ZERO>
static int launch_one(W4GemmParams const& p, void const* act, DeviceInfo const& dev, cudaStream_t stream)
{
    constexpr int IL = BITS == 4 ? 4 : 2;
    constexpr int STAGE_BYTES = BM * 128 + (BN / IL) * 128;
    auto kernel = gemm_kernel<T, BITS, BM, HAS_ZERO>;

    Args a{};
    a.scales = p.scales;
    a.zeros = p.zeros;
    a.bias = p.bias;
    a.out = p.out;
    a.alpha = p.alpha;
    a.m = p.m;
    a.n = p.n;
    a.k = p.k;
    a.group_shift = p.group_size == 64 ? 6 : (p.group_size == 128 ? 7 : 31);
    a.tiles_n = (p.n + BN - 1) / BN;
    a.tiles_m = (p.m + BM - 1) / BM;
    size_t const fixed = sizeof(Barriers) + 1024; // + slack to align the ring to 1024 bytes
    int stages = int((size_t(dev.max_smem_optin) - fixed) / STAGE_BYTES);
    if (stages < 2)
        return W4_ERR_CUDA;
    a.num_stages = stages > kMaxStages ? kMaxStages : stages;
    size_t const smem = size_t(a.num_stages) * STAGE_BYTES + fixed;

    // Activations [m, k] of T, boxes of 64 k x BM rows, 128-byte swizzle (rows past m read as 0).
    // Weights as bytes: [n / IL interleaved rows, 2k bytes], boxes of one 128-byte line x BN/IL rows.
    CUtensorMap tm_act, tm_w;
    CUtensorMapDataType const dt
        = std::is_same<T, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (!make_tensor_map_2d(&tm_act, dt, act, uint64_t(p.k), uint64_t(p.m), uint64_t(p.k) * 2, BK, BM,
            CU_TENSOR_MAP_SWIZZLE_128B))
        return W4_ERR_CUDA;
    if (!make_tensor_map_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.weight, uint64_t(p.k) * 2, uint64_t(p.n / IL),
            uint64_t(p.k) * 2, 128, BN / IL, CU_TENSOR_MAP_SWIZZLE_NONE))
        return W4_ERR_CUDA;

    static bool configured[64] = {};
    if (dev.device < 0 || dev.device >= 64 || !configured[dev.device])
    {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dev.max_smem_optin)
            != cudaSuccess)
            return W4_ERR_CUDA;
        if (dev.device >= 0 && dev.device < 64)
            configured[dev.device] = true;
    }
    int const tiles = a.tiles_n * a.tiles_m;
    int const grid = tiles < dev.num_sms ? tiles : dev.num_sms;
    kernel<<<grid, kThreads, smem, stream>>>(a, tm_act, tm_w);
    return cudaGetLastError() == cudaSuccess ? W4_OK : W4_ERR_CUDA;
}

template <typename T, int BITS, bool HAS_ZERO>
static int dispatch_bm(W4GemmParams const& p, void const* act, DeviceInfo const& dev, cudaStream_t stream)
{
    if (p.m <= 64)
        return launch_one<T, BITS, 64, HAS_ZERO>(p, act, dev, stream);
    if (p.m <= 128)
        return launch_one<T, BITS, 128, HAS_ZERO>(p, act, dev, stream);
    return launch_one<T, BITS, 256, HAS_ZERO>(p, act, dev, stream);
}

template <typename T>
static int dispatch(W4GemmParams const& p, void const* act, DeviceInfo const& dev, cudaStream_t stream)
{
    bool const z = p.zeros != nullptr;
    if (p.weight_bits == 4)
        return z ? dispatch_bm<T, 4, true>(p, act, dev, stream) : dispatch_bm<T, 4, false>(p, act, dev, stream);
    return z ? dispatch_bm<T, 8, true>(p, act, dev, stream) : dispatch_bm<T, 8, false>(p, act, dev, stream);
}

} // namespace tc

#ifdef W4_DBG_TRACE
extern "C" int w4_dbg_read_tc_trace(long long* out)
{
    return cudaMemcpyFromSymbol(out, tc::g_tc_trace, sizeof(long long) * 64) == cudaSuccess ? 0 : -1;
}
#endif

size_t gemm_tc_workspace_bytes(int m, int n, int k, int has_act_scale)
{
    (void) n;
    // the pre-quant scale is applied to a copy of the activations, as the reference plugin does
    // (weightOnlyGroupwiseQuantMatmulPlugin.cpp:444-458 of the reference project)
    return has_act_scale ? size_t(m) * k * 2 : 0;
}

int launch_gemm_tc(W4GemmParams const& p, cudaStream_t stream)
{
    DeviceInfo const& dev = current_device_info();
    if (dev.num_sms <= 0)
        return W4_ERR_CUDA;
    void const* act = p.act;
    if (p.act_scale)
    {
        int const rc = launch_pre_quant_scale(p.workspace, p.act, p.act_scale, p.m, p.k, p.act_dtype, stream);
        if (rc != W4_OK)
            return rc;
        act = p.workspace;
    }
    return p.act_dtype == W4_DTYPE_FP16 ? tc::dispatch<__half>(p, act, dev, stream)
                                        : tc::dispatch<__nv_bfloat16>(p, act, dev, stream);
}

} // namespace w4
