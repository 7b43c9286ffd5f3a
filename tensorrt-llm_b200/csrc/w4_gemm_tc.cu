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
// of W times 64..256 rows of the activation matrix; a pipeline step covers 128 k (two 64-wide
// swizzled halves, eight tcgen05.mma of K = 16).
//
// Warp roles (320 threads, one CTA per SM, persistent over tiles, n-fastest tile order):
//   warp 0      TMA producer: two activation half-tiles [BM x 64] + the packed weight lines per step
//   warp 1      allocates TMEM, issues tcgen05.mma and tcgen05.commit (whole warp, warp-uniform
//               operands, one elected lane per instruction)
//   warps 2..9  conversion, two warps per TMEM lane quadrant taking alternate k steps: shared memory
//               -> registers -> exact int->T conversion, scale/zero -> tcgen05.st into the TMEM ring
//               of A stages; after the last k step the same warps run the epilogue (tcgen05.ld,
//               alpha/bias, convert, store), each on its share of the accumulator columns.
// Hand-offs: `full` (TMA -> conversion), per-warp step counters polled with acquire loads
// (conversion -> MMA), `done` (tcgen05.commit -> producer and conversion: the shared-memory stage
// and the TMEM stage of a step are released together), `d_full` / `d_empty` (accumulator).
// What was measured while tuning (B200): the pipeline has a cost per k step of roughly 900-1100
// cycles that does not depend on the row tile, so the step is made as fat as shared memory allows
// (128 k); issuing tcgen05.mma from a divergent single lane costs ~70 cycles per instruction
// against ~40 from a converged warp; scale/zero loads need several groups of lookahead because a
// step is shorter than an L2 round trip.
// All waits are bounded; a timeout sets the device status word and the CTA drains and exits.
#include <mutex>
#include <type_traits>

#include "w4_common.cuh"
#include "w4_internal.h"
#include "w4_tma.h"

namespace w4
{
namespace tc
{

constexpr int BN = 128;       // weight columns per tile (MMA M, TMEM lanes)
constexpr int BK = 128;       // k per pipeline step: two 64-wide halves (one 128-byte swizzle span of T each)
constexpr int kHalves = BK / 64;
constexpr int kMaxAStages = 4; // TMEM ring of converted-weight stages (64 columns each): columns 256..511
constexpr int kACol0 = 256;   // first TMEM column of that ring; the accumulator uses [0, 256)
constexpr int kTmemCols = 512;
constexpr int kConvGroups = 2;   // groups of 4 conversion warps; group g converts k steps with ks % 2 == g
constexpr int kThreads = 64 + 128 * kConvGroups;
constexpr int kMaxStages = kMaxAStages; // one ring index for the shared-memory stage and its TMEM stage

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
    // Split-k: an output tile's k range is cut into `splits` work items that run on different SMs;
    // each stores its fp32 partial tile and a second small kernel adds them in split order.
    int splits;       // 1 = off
    int ksteps_split; // k steps per work item
    float* partial;   // [splits, m, n] fp32 (workspace)
};

struct __align__(16) Barriers
{
    // TMA landed (tx bytes), one barrier per (conversion group, stage): the copy of a k step signals the
    // barrier of the group that converts that step. A group therefore sees every phase of every
    // barrier it waits on, whatever the number of stages and of k steps per tile (with one barrier
    // per stage a group would meet a subset of the phases and could take a lagging copy of the other
    // group's step for its own).
    uint64_t full[kConvGroups][kMaxStages];
    uint64_t done[kMaxStages];    // the MMAs of the step completed: smem stage and TMEM stage are free
    uint64_t d_full;              // accumulator complete
    uint64_t d_empty;             // the epilogue warps drained the accumulator
    // Steps each conversion warp has finished storing into TMEM, [group][quadrant]. The MMA warp
    // polls these with plain acquire loads: an mbarrier test issued by the MMA warp right after its
    // tcgen05.commit is held back until the committed MMAs finish, which costs a full step.
    alignas(16) uint32_t ready[kConvGroups][4];
    uint32_t tmem_base;
    int abort_flag;
};


__device__ __forceinline__ bool wait_flag(uint64_t* bar, uint32_t parity, volatile int* abort_flag)
{
    // Spin on the non-blocking test: the blocking try_wait form parks the thread for a
    // hardware-defined interval, which costs about a microsecond per hand-off in this pipeline.
    for (uint32_t i = 0; i < kMaxSpinPolls; ++i)
    {
        if (mbar_test_wait(bar, parity))
            return true;
        if ((i & 1023u) == 1023u && *abort_flag)
            return false;
    }
    *abort_flag = 1;
    atomicExch(&g_device_status, kDeviceTimeout);
    return false;
}

// Warp-wide wait: one lane polls, the result is broadcast (keeps 31 lanes off the barrier word).
__device__ __forceinline__ bool wait_flag_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int lane)
{
    int ok = 1;
    if (lane == 0)
        ok = wait_flag(bar, parity, abort_flag) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

__device__ __forceinline__ void tc_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ bool mbar_test_wait_addr(uint32_t bar_addr, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar_addr), "r"(parity)
        : "memory");
    return ok != 0;
}


// The following are executed by a whole (converged) warp; one elected lane performs the operation.
// Keeping the surrounding control flow warp-uniform lets the compiler hold addresses and
// descriptors in uniform registers, which is what the tensor-core and TMA instructions consume;
// issued from inside a divergent `if (lane == 0)` every operand has to be moved across first and
// one tcgen05.mma costs ~70 cycles to issue.
__device__ __forceinline__ void tc_mma_ts_elect(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc)
{
    asm volatile(
        "{\n"
        ".reg .pred p, pe;\n"
        "elect.sync _|pe, 0xffffffff;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
}

__device__ __forceinline__ void tc_commit_elect(uint32_t bar_addr)
{
    asm volatile(
        "{\n"
        ".reg .pred pe;\n"
        "elect.sync _|pe, 0xffffffff;\n"
        "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
        "}\n" ::"r"(bar_addr)
        : "memory");
}

// Warp-uniform bounded spin on an mbarrier phase (every lane polls the same word).
__device__ __forceinline__ bool spin_wait(uint32_t bar_addr, uint32_t parity, volatile int* abort_flag)
{
    uint32_t polls = 0;
    while (!mbar_test_wait_addr(bar_addr, parity))
    {
        if ((++polls & 0xffffu) == 0 && (*abort_flag || polls >= kMaxSpinPolls))
        {
            *abort_flag = 1;
            atomicExch(&g_device_status, kDeviceTimeout);
            return false;
        }
    }
    return true;
}

// Spins until all four conversion warps of a group have published at least `needed` steps.
__device__ __forceinline__ bool spin_ready(uint32_t addr, uint32_t needed, volatile int* abort_flag)
{
    uint32_t polls = 0;
    for (;;)
    {
        uint32_t a, b, c, d;
        asm volatile("ld.acquire.cta.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(a), "=r"(b), "=r"(c), "=r"(d)
                     : "r"(addr)
                     : "memory");
        // counters only grow and stay within a few steps of each other: compare as signed distance
        if (int(a - needed) >= 0 && int(b - needed) >= 0 && int(c - needed) >= 0 && int(d - needed) >= 0)
            return true;
        if ((++polls & 0xffffu) == 0 && (*abort_flag || polls >= kMaxSpinPolls))
        {
            *abort_flag = 1;
            atomicExch(&g_device_status, kDeviceTimeout);
            return false;
        }
    }
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

template <typename T, int BITS, int BM, bool HAS_ZERO, bool SPLITK>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_kernel(Args const a, __grid_constant__ CUtensorMap const tm_act, __grid_constant__ CUtensorMap const tm_w)
{
    using P = Pair<T>;
    constexpr int IL = BITS == 4 ? 4 : 2;
    constexpr int ACT_HALF = BM * 128;                      // BM rows x 64 k of T (one swizzled tile)
    constexpr int ACT_BYTES = kHalves * ACT_HALF;
    constexpr int W_BYTES = (BN / IL) * 128 * kHalves;      // interleaved rows x two adjacent 128-byte lines
    constexpr int STAGE_BYTES = ACT_BYTES + W_BYTES;
    constexpr int SEG = 128 / IL;                // bytes of one column inside a line
    constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u; // 0 = fp16, 1 = bf16
    constexpr uint32_t kIdesc = (1u << 4)                                   // fp32 accumulator
        | (kFmt << 7)                                                       // A type
        | (kFmt << 10)                                                      // B type (both K-major)
        | (uint32_t(BM >> 3) << 17)                                         // MMA N = activation rows
        | (uint32_t(BN >> 4) << 24);                                        // MMA M = weight columns

    // The 128-byte swizzle of the TMA copies and of the MMA descriptors is a function of the
    // shared-memory address: the ring starts on a 1024-byte boundary (declared, and checked below).
    extern __shared__ __align__(1024) uint8_t smem[];
    if ((smem_u32(smem) & 1023u) != 0) // never seen; nothing has been allocated or initialised yet
    {
        if (threadIdx.x == 0)
            atomicExch(&g_device_status, kDeviceTimeout);
        return;
    }
    Barriers* bars = reinterpret_cast<Barriers*>(smem + size_t(a.num_stages) * STAGE_BYTES);
    volatile int* abort_flag = &bars->abort_flag;

    int const warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int const num_tiles = a.tiles_n * a.tiles_m * (SPLITK ? a.splits : 1); // work items: (tile, split), splits adjacent
    int const ksteps_all = (a.k + BK - 1) / BK; // a trailing 64-wide half reads as zeros (TMA fill)

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < a.num_stages; ++s)
        {
            for (int g = 0; g < kConvGroups; ++g)
                mbar_init(&bars->full[g][s], 1);
            mbar_init(&bars->done[s], 1);
        }
        mbar_init(&bars->d_full, 1);
        mbar_init(&bars->d_empty, 4 * kConvGroups);
        bars->abort_flag = 0;
        for (int i = 0; i < kConvGroups * 4; ++i)
            (&bars->ready[0][0])[i] = 0;
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
        // (whole warp, warp-uniform; an elected lane issues the copies)
        if (lane == 0)
        {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_act) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w) : "memory");
        }
        __syncwarp();
        {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            uint32_t const smem_base = smem_u32(smem);
            uint32_t const full0 = smem_u32(&bars->full[0][0]), done0 = smem_u32(&bars->done[0]);
            for (int item = blockIdx.x; item < num_tiles && ok; item += gridDim.x)
            {
                int const tile = SPLITK ? item / a.splits : item, split = SPLITK ? item - tile * a.splits : 0;
                int const tn = tile % a.tiles_n, tm = tile / a.tiles_n;
                int const ks0 = SPLITK ? split * a.ksteps_split : 0, ks1 = SPLITK ? min(ksteps_all, ks0 + a.ksteps_split) : ksteps_all;
                for (int ks = ks0; ks < ks1; ++ks)
                {
                    ok = spin_wait(done0 + 8 * s, ph ^ 1, abort_flag);
                    if (!ok)
                        break;
                    uint32_t const stage = smem_base + uint32_t(s) * STAGE_BYTES;
                    uint32_t const full = full0 + 8 * ((uint32_t(ks) % kConvGroups) * kMaxStages + s);
                    elect_expect_tx(full, STAGE_BYTES);
                    elect_tma_load_2d(stage, &tm_act, ks * BK, tm * BM, full);
                    elect_tma_load_2d(stage + ACT_HALF, &tm_act, ks * BK + 64, tm * BM, full);
                    elect_tma_load_2d(stage + ACT_BYTES, &tm_w, ks * 128 * kHalves, tn * (BN / IL), full);
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
        // One thread feeds the tensor core; its queue is only about one instruction deep, so this
        // loop has to come back with the next MMA within ~100 cycles: descriptors and addresses are
        // advanced incrementally, there is one wait and one commit per k step, and the wait spins
        // on the non-blocking test.
        {
            uint64_t const desc0 = smem_desc_sw128(smem_u32(smem));
            constexpr uint64_t kDescStage = uint64_t(STAGE_BYTES >> 4); // address field is in 16-byte units
            uint32_t const done0 = smem_u32(&bars->done[0]);
            uint32_t const d_empty = smem_u32(&bars->d_empty), d_full = smem_u32(&bars->d_full);
            uint64_t desc = desc0;
            uint32_t a_col = tmem + kACol0;
            uint32_t done = done0;
            uint32_t const ready0 = smem_u32(&bars->ready[0][0]);
            uint32_t issued[kConvGroups] = {}; // k steps issued so far per conversion group, over all tiles
            int s = 0;
            uint32_t ph = 0, dph = 0;
            bool ok = true;
            for (int item = blockIdx.x, it = 0; item < num_tiles && ok; item += gridDim.x, ++it)
            {
                int const tile = SPLITK ? item / a.splits : item, split = SPLITK ? item - tile * a.splits : 0;
                int const ks0 = SPLITK ? split * a.ksteps_split : 0, ks1 = SPLITK ? min(ksteps_all, ks0 + a.ksteps_split) : ksteps_all;
                if (it > 0)
                {
                    ok = spin_wait(d_empty, dph, abort_flag);
                    if (!ok)
                        break;
                    dph ^= 1;
                    tc_fence_after();
                }
                uint32_t accumulate = 0;
                for (int ks = ks0; ks < ks1; ++ks)
                {
                    // The conversion warps publish a step only after they have seen the stage's TMA
                    // barrier, so it covers the activations as well.
                    uint32_t const grp = uint32_t(ks) % kConvGroups; // the group that converts this step
                    uint32_t const needed = ++issued[grp];
                    ok = spin_ready(ready0 + 16 * grp, needed, abort_flag);
                    if (!ok)
                        break;
                    tc_fence_after();
                    tc_mma_ts_elect(tmem, a_col, desc, kIdesc, accumulate);
                    tc_mma_ts_elect(tmem, a_col + 8, desc + 2, kIdesc, 1u);
                    tc_mma_ts_elect(tmem, a_col + 16, desc + 4, kIdesc, 1u);
                    tc_mma_ts_elect(tmem, a_col + 24, desc + 6, kIdesc, 1u);
                    constexpr uint64_t kDescHalf = uint64_t(ACT_HALF >> 4); // second 64-wide half of the step
                    tc_mma_ts_elect(tmem, a_col + 32, desc + kDescHalf, kIdesc, 1u);
                    tc_mma_ts_elect(tmem, a_col + 40, desc + kDescHalf + 2, kIdesc, 1u);
                    tc_mma_ts_elect(tmem, a_col + 48, desc + kDescHalf + 4, kIdesc, 1u);
                    tc_mma_ts_elect(tmem, a_col + 56, desc + kDescHalf + 6, kIdesc, 1u);
                    accumulate = 1u;
                    tc_commit_elect(done); // frees the shared-memory stage and the TMEM stage
                    desc += kDescStage;
                    a_col += 32 * kHalves;
                    done += 8;
                    if (++s == a.num_stages)
                    {
                        s = 0;
                        ph ^= 1;
                        desc = desc0;
                        a_col = tmem + kACol0;
                        done = done0;
                    }
                }
                if (ok)
                    tc_commit_elect(d_full);
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
        int const gsh = a.group_shift >= 31 ? 30 : a.group_shift - 6; // log2(64-wide halves per scale group)
        // Column segment of this thread inside the first of a stage's two weight lines.
        int const w_off = (n_local / IL) * (128 * kHalves) + (n_local % IL) * SEG;

        int s_item = 0;          // ring position of the current work item's first k step
        uint32_t ph_item = 0, dph = 0;
        uint32_t my_steps = 0; // steps this warp has stored into TMEM (published by lane 0)
        uint32_t full_seen = 0; // bit s: phases of full[cgroup][s] this group has consumed, mod 2
        bool ok = true;
        for (int item = blockIdx.x; item < num_tiles && ok; item += gridDim.x)
        {
            int const tile = SPLITK ? item / a.splits : item, split = SPLITK ? item - tile * a.splits : 0;
            int const tn = tile % a.tiles_n, tm = tile / a.tiles_n;
            int const ks0 = SPLITK ? split * a.ksteps_split : 0, ks1 = SPLITK ? min(ksteps_all, ks0 + a.ksteps_split) : ksteps_all;
            int const n = tn * BN + n_local;
            bool const n_ok = n < a.n;
            // Scale / zero of this thread's column for the steps THIS group converts (every
            // kConvGroups-th k step), one pair per 64-k half. They come from global memory (L2 at
            // best, ~1 us under load, longer than a k step), so the pairs of a step are loaded two of
            // the group's own steps ahead, into one of two register sets that the twice-unrolled loop
            // below addresses statically. (A shift queue does not work here: shifting it reads the
            // newest entry one scale group after its load was issued, and with 64-wide groups that
            // is half a k step - the warp ends up waiting for every load.)
            int const num_groups = a.group_shift >= 31 ? 1 : (a.k >> a.group_shift);
            auto load_pairs = [&](int ks, uint32_t(&sp)[kHalves], uint32_t(&zp)[kHalves])
            {
#pragma unroll
                for (int h = 0; h < kHalves; ++h)
                {
                    int const g = (ks * kHalves + h) >> gsh;
                    uint32_t sv = 0, zv = 0;
                    if (n_ok && ks < ks1 && g < num_groups)
                    {
                        sv = scales[size_t(g) * a.n + n];
                        if (HAS_ZERO)
                            zv = zeros[size_t(g) * a.n + n];
                    }
                    sp[h] = sv | (sv << 16);
                    zp[h] = zv | (zv << 16);
                }
            };
            // position of the item's first step in the ring; own steps are reached from it
            int const first_own = ks0 + ((cgroup - ks0 % kConvGroups + kConvGroups) % kConvGroups);
            int s = s_item;
            uint32_t ph = ph_item;
            auto advance = [&](int steps)
            {
                s += steps;
                while (s >= a.num_stages)
                {
                    s -= a.num_stages;
                    ph ^= 1;
                }
            };
            advance(first_own - ks0);
            uint32_t sset[2][kHalves], zset[2][kHalves];
            load_pairs(first_own, sset[0], zset[0]);
            load_pairs(first_own + kConvGroups, sset[1], zset[1]);

            // One own step: wait for its weights, convert, store into the TMEM stage, publish.
            auto convert_step = [&](int ks, uint32_t const(&s2h)[kHalves], uint32_t const(&z2h)[kHalves]) -> bool
            {
                (void) ks;
                {
                    // parity of this group's next phase on the stage's barrier: one bit per stage
                    uint32_t const fph = (full_seen >> s) & 1u;
                    full_seen ^= 1u << s;
                    ok = wait_flag_warp(&bars->full[cgroup][s], fph, abort_flag, lane);
                    if (!ok)
                        return false;
                    uint8_t const* wsm = smem + size_t(s) * STAGE_BYTES + ACT_BYTES + w_off;
                    constexpr int CHUNKS = SEG / 16; // 16-byte chunks per half: 2 (int4) or 4 (int8)
                    uint4 raw[kHalves][CHUNKS];
#pragma unroll
                    for (int h = 0; h < kHalves; ++h)
#pragma unroll
                        for (int c = 0; c < CHUNKS; ++c)
                            raw[h][c] = *reinterpret_cast<uint4 const*>(wsm + h * 128 + c * 16);
                    // Convert into registers first; only the stores have to wait for the TMEM stage.
                    // v[2h + x] holds TMEM columns 32h + 16x .. +15 (k = 64h + 32x .. +31).
                    uint32_t v[2 * kHalves][16];
#pragma unroll
                    for (int h = 0; h < kHalves; ++h)
                    {
                        uint32_t const s2 = s2h[h], z2 = z2h[h];
                        if (BITS == 4)
                        {
#pragma unroll
                            for (int c = 0; c < 2; ++c)
                            {
                                uint32_t const r[4] = {raw[h][c].x, raw[h][c].y, raw[h][c].z, raw[h][c].w};
#pragma unroll
                                for (int j = 0; j < 4; ++j)
                                {
                                    uint32_t q[4];
                                    cvt_int4x8<T>(r[j], q);
#pragma unroll
                                    for (int p = 0; p < 4; ++p) // pair p of register j holds k = 32c + 2j + 8p (+1)
                                        v[2 * h + c][j + 4 * p] = HAS_ZERO ? P::fma(q[p], s2, z2) : P::mul(q[p], s2);
                                }
                            }
                        }
                        else
                        {
#pragma unroll
                            for (int x = 0; x < 2; ++x)
#pragma unroll
                                for (int cc = 0; cc < 2; ++cc)
                                {
                                    uint4 const w = raw[h][(2 * x + cc) % CHUNKS];
                                    uint32_t const r[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                                    for (int j = 0; j < 4; ++j)
                                    {
                                        uint32_t q[2];
                                        cvt_int8x4<T>(r[j], q);
#pragma unroll
                                        for (int p = 0; p < 2; ++p) // pair p of register j holds k = 16(2x+cc) + 2j + 8p (+1)
                                            v[2 * h + x][8 * cc + j + 4 * p]
                                                = HAS_ZERO ? P::fma(q[p], s2, z2) : P::mul(q[p], s2);
                                    }
                                }
                        }
                    }
                    ok = wait_flag_warp(&bars->done[s], ph ^ 1, abort_flag, lane);
                    if (!ok)
                        return false;
                    tc_fence_after();
                    uint32_t const a_addr = lane_addr + kACol0 + s * (32 * kHalves); // warp-uniform column address
#pragma unroll
                    for (int x = 0; x < 2 * kHalves; ++x)
                        tc_st16(a_addr + 16 * x, v[x]);
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0)
                    {
                        ++my_steps;
                        asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(smem_u32(&bars->ready[cgroup][quad])),
                                     "r"(my_steps)
                                     : "memory");
                    }
                }
                return true;
            };

            for (int ks = first_own; ks < ks1 && ok; ks += 2 * kConvGroups)
            {
#pragma unroll
                for (int u = 0; u < 2; ++u)
                {
                    int const kk = ks + u * kConvGroups;
                    if (kk < ks1 && ok)
                    {
                        uint32_t s2h[kHalves], z2h[kHalves];
#pragma unroll
                        for (int h = 0; h < kHalves; ++h)
                        {
                            s2h[h] = sset[u][h];
                            z2h[h] = zset[u][h];
                        }
                        load_pairs(kk + 2 * kConvGroups, sset[u], zset[u]);
                        if (convert_step(kk, s2h, z2h))
                            advance(kConvGroups);
                    }
                }
            }
            // the next item starts where this one's k range ends
            s = s_item;
            ph = ph_item;
            advance(ks1 - ks0);
            s_item = s;
            ph_item = ph;
            if (!ok)
                break;

            // ---- epilogue: this thread owns output column n for all BM rows of the tile
            ok = wait_flag_warp(&bars->d_full, dph, abort_flag, lane);
            if (!ok)
                break;
            dph ^= 1;
            tc_fence_after();
            float const bias_f = (bias && n_ok) ? P::to_float(bias[n]) : 0.f;
            int const m0 = tm * BM;
            if (!SPLITK)
            {
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
                                out[size_t(mrow) * a.n + n]
                                    = P::from_float(fmaf(a.alpha, __uint_as_float(v[j]), bias_f));
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&bars->d_empty);
            }
            else
            {
                // Split-k: store the fp32 partial tile; splitk_reduce_kernel, next on the stream,
                // adds the partial tiles in split order (deterministic) and writes the output.
                float* part = a.partial + size_t(split) * a.m * a.n;
#pragma unroll 1
                for (int c0 = cgroup * 32; c0 < BM; c0 += 32 * kConvGroups)
                {
                    if (m0 + c0 >= a.m)
                        break;
                    uint32_t v[32];
                    tc_ld32(lane_addr + c0, v);
                    if (n_ok)
                    {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                        {
                            int const mrow = m0 + c0 + j;
                            if (mrow < a.m)
                                __stcg(part + size_t(mrow) * a.n + n, __uint_as_float(v[j]));
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&bars->d_empty);
            }
        }
    }

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
static size_t split_align(size_t bytes)
{
    return (bytes + 255) & ~size_t(255);
}

// Workspace for split-k: `splits` fp32 copies of the output.
static size_t split_bytes(int m, int n, int splits)
{
    return size_t(splits) * m * n * sizeof(float);
}

// out[m, n] = alpha * sum over splits (in order) of partial[s, m, n] + bias[n]; four columns per thread.
template <typename T>
__global__ void __launch_bounds__(256)
    splitk_reduce_kernel(T* out, float const* partial, T const* bias, float alpha, size_t mn_vec, int n_vec, int splits)
{
    using P = Pair<T>;
    size_t const i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= mn_vec)
        return;
    float4 const* src = reinterpret_cast<float4 const*>(partial) + i;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    int sp = 0;
    for (; sp + 4 <= splits; sp += 4)
    {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            v[u] = __ldcg(src + size_t(sp + u) * mn_vec);
#pragma unroll
        for (int u = 0; u < 4; ++u)
        {
            acc.x += v[u].x;
            acc.y += v[u].y;
            acc.z += v[u].z;
            acc.w += v[u].w;
        }
    }
    for (; sp < splits; ++sp)
    {
        float4 const v = __ldcg(src + size_t(sp) * mn_vec);
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
    }
    float b[4] = {0.f, 0.f, 0.f, 0.f};
    if (bias)
    {
        uint2 const bw = *reinterpret_cast<uint2 const*>(bias + size_t(i % n_vec) * 4);
        P::unpack2(bw.x, b[0], b[1]);
        P::unpack2(bw.y, b[2], b[3]);
    }
    uint2 o;
    o.x = uint32_t(P::from_float(fmaf(alpha, acc.x, b[0]))) | (uint32_t(P::from_float(fmaf(alpha, acc.y, b[1]))) << 16);
    o.y = uint32_t(P::from_float(fmaf(alpha, acc.z, b[2]))) | (uint32_t(P::from_float(fmaf(alpha, acc.w, b[3]))) << 16);
    *reinterpret_cast<uint2*>(out + i * 4) = o;
}

template <typename T, int BITS, int BM, bool HAS_ZERO, bool SPLITK>
static int launch_one(W4GemmParams const& p, void const* act, DeviceInfo const& dev, cudaStream_t stream, int splits)
{
    constexpr int IL = BITS == 4 ? 4 : 2;
    constexpr int STAGE_BYTES = kHalves * (BM * 128 + (BN / IL) * 128);
    auto kernel = gemm_kernel<T, BITS, BM, HAS_ZERO, SPLITK>;

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
    {
        // Split-k (chosen by the caller of this function): partial tiles go to the workspace, behind
        // the scaled copy of the activations if there is one.
        int const ksteps = (p.k + BK - 1) / BK;
        size_t const act_copy = (act != p.act) ? split_align(size_t(p.m) * p.k * 2) : 0;
        a.ksteps_split = (ksteps + splits - 1) / splits;
        a.splits = (ksteps + a.ksteps_split - 1) / a.ksteps_split; // no empty work items
        if (SPLITK)
            a.partial = reinterpret_cast<float*>(static_cast<char*>(p.workspace) + act_copy);
    }
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
    if (!make_tensor_map_2d(&tm_act, dt, act, uint64_t(p.k), uint64_t(p.m), uint64_t(p.k) * 2, 64, BM,
            CU_TENSOR_MAP_SWIZZLE_128B))
        return W4_ERR_CUDA;
    if (!make_tensor_map_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.weight, uint64_t(p.k) * 2, uint64_t(p.n / IL),
            uint64_t(p.k) * 2, 128 * kHalves, BN / IL, CU_TENSOR_MAP_SWIZZLE_NONE))
        return W4_ERR_CUDA;

    {
        // per-function, per-device attribute: set once (this block is instantiated once per kernel)
        static std::mutex mu;
        static bool configured[64] = {};
        std::lock_guard<std::mutex> lock(mu);
        if (dev.device < 0 || dev.device >= 64 || !configured[dev.device])
        {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dev.max_smem_optin)
                != cudaSuccess)
                return W4_ERR_CUDA;
            if (dev.device >= 0 && dev.device < 64)
                configured[dev.device] = true;
        }
    }
    int const tiles = a.tiles_n * a.tiles_m * (SPLITK ? a.splits : 1);
    int const grid = tiles < dev.num_sms ? tiles : dev.num_sms;
    kernel<<<grid, kThreads, smem, stream>>>(a, tm_act, tm_w);
    if (SPLITK)
    {
        size_t const mn_vec = size_t(p.m) * p.n / 4; // n is a multiple of 32
        splitk_reduce_kernel<T><<<unsigned((mn_vec + 255) / 256), 256, 0, stream>>>(static_cast<T*>(p.out), a.partial,
            static_cast<T const*>(p.bias), p.alpha, mn_vec, p.n / 4, a.splits);
    }
    return cudaGetLastError() == cudaSuccess ? W4_OK : W4_ERR_CUDA;
}

template <typename T, int BITS, bool HAS_ZERO>
static int dispatch_bm(W4GemmParams const& p, void const* act, DeviceInfo const& dev, cudaStream_t stream)
{
    int const bm = gemm_tc_row_tile(p.m, p.n, dev.num_sms, p.weight_bits);
    // Split-k when the tiles alone would leave most SMs idle and the caller's workspace has room
    // for the partial tiles; the unsplit kernel is a separate instantiation without any of it.
    int splits = gemm_tc_splits(p.m, p.n, p.k, dev.num_sms, p.weight_bits);
    if (splits > 1)
    {
        size_t const act_copy = (act != p.act) ? split_align(size_t(p.m) * p.k * 2) : 0;
        if (!p.workspace || p.workspace_bytes < act_copy + split_bytes(p.m, p.n, splits))
            splits = 1;
    }
    if (splits > 1)
    {
        if (bm == 64)
            return launch_one<T, BITS, 64, HAS_ZERO, true>(p, act, dev, stream, splits);
        if (bm == 128)
            return launch_one<T, BITS, 128, HAS_ZERO, true>(p, act, dev, stream, splits);
        if (bm == 192)
            return launch_one<T, BITS, 192, HAS_ZERO, true>(p, act, dev, stream, splits);
        return launch_one<T, BITS, 256, HAS_ZERO, true>(p, act, dev, stream, splits);
    }
    if (bm == 64)
        return launch_one<T, BITS, 64, HAS_ZERO, false>(p, act, dev, stream, 1);
    if (bm == 128)
        return launch_one<T, BITS, 128, HAS_ZERO, false>(p, act, dev, stream, 1);
    if (bm == 192)
        return launch_one<T, BITS, 192, HAS_ZERO, false>(p, act, dev, stream, 1);
    return launch_one<T, BITS, 256, HAS_ZERO, false>(p, act, dev, stream, 1);
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


// Microseconds one CTA spends per 128-wide k step, by row tile (measured on B200, bf16, group 128).
// int4: up to 192 rows the step is bound by the conversion / hand-off pipeline, not by its tensor
// work; 256 rows leave shared memory for three stages only and the step turns latency-bound. int8
// stages carry 16 KB of weights instead of 8: four of them fit up to 128 rows, three at 192 rows
// (4096 x 14336 x 4096: 546 us with 128-row tiles against 623 us with 192), two at 256; with 64-row
// tiles the int8 step is shorter (4096 x 14336 at 32 and 64 rows: 25 us for 32 steps).
static double step_us(int bm, int bits)
{
    if (bits == 8)
        return bm <= 64 ? 0.56 : (bm <= 128 ? 0.70 : (bm == 192 ? 1.11 : 1.9));
    return bm <= 128 ? 0.57 : (bm == 192 ? 0.70 : 1.05);
}

// Split-k factor: used when the output tiles would occupy less than half of the SMs; every work
// item keeps at least four k steps; only for m <= 256, where the fp32 partial tiles stay small.
int gemm_tc_splits(int m, int n, int k, int num_sms, int bits)
{
    int const bm = gemm_tc_row_tile(m, n, num_sms, bits);
    long const tiles = long((n + tc::BN - 1) / tc::BN) * long((m + bm - 1) / bm);
    int const ksteps = (k + tc::BK - 1) / tc::BK;
    if (tiles * 2 > num_sms || m > 256)
        return 1;
    long s = num_sms / tiles;
    if (s > ksteps / 4)
        s = ksteps / 4;
    if (s > 16)
        s = 16;
    return s < 1 ? 1 : int(s);
}

static double waves(int m, int n, int bm, int num_sms, int splits = 1)
{
    long const tiles = long((n + tc::BN - 1) / tc::BN) * long((m + bm - 1) / bm) * splits;
    return double((tiles + num_sms - 1) / num_sms);
}

int gemm_tc_row_tile(int m, int n, int num_sms, int bits)
{
    if (m <= 64)
        return 64;
    if (m <= 128)
        return 128;
    if (m <= 192 && bits != 8) // int8 keeps only three stages at 192 rows: let the costs decide
        return 192;
    int const cand[3] = {128, 192, 256};
    int bm = 0;
    double best = 0;
    for (int i = 0; i < 3; ++i)
    {
        double const cost = waves(m, n, cand[i], num_sms) * step_us(cand[i], bits);
        if (!bm || cost < best)
        {
            bm = cand[i];
            best = cost;
        }
    }
    return bm;
}

double gemm_tc_estimate_us(int m, int n, int k, int num_sms, int bits)
{
    int const bm = gemm_tc_row_tile(m, n, num_sms, bits);
    int const splits = gemm_tc_splits(m, n, k, num_sms, bits);
    int const ksteps = (k + tc::BK - 1) / tc::BK;
    int const per = (ksteps + splits - 1) / splits;
    return 7.0 + (splits > 1 ? 3.0 : 0.0) + waves(m, n, bm, num_sms, splits) * step_us(bm, bits) * double(per);
}

size_t gemm_tc_workspace_min(int m, int k, int has_act_scale)
{
    // the pre-quant scale is applied to a copy of the activations, as the reference plugin does
    // (weightOnlyGroupwiseQuantMatmulPlugin.cpp:444-458 of the reference project)
    return has_act_scale ? size_t(m) * k * 2 : 0;
}

size_t gemm_tc_workspace_bytes(int m, int n, int k, int has_act_scale, int bits)
{
    // what lets the kernel use split-k as well; with less (but at least the minimum) it runs unsplit
    DeviceInfo const& dev = current_device_info();
    int const sms = dev.num_sms > 0 ? dev.num_sms : 148;
    int const splits = gemm_tc_splits(m, n, k, sms, bits);
    size_t bytes = gemm_tc_workspace_min(m, k, has_act_scale);
    if (splits > 1)
        bytes = tc::split_align(bytes) + tc::split_bytes(m, n, splits);
    return bytes;
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
