// Decode-regime kernel, second form (m <= 8 per pass, activations small enough to stay resident in
// shared memory): streams the packed int4/int8 weights exactly once.
//
// Replaces weight_only::kernel of the reference project
// (cpp/tensorrt_llm/kernels/weightOnlyBatchedGemv/kernel.h:31-120) like the first form in
// w4_gemv.cu, whose weight streaming it shares: one persistent CTA per SM owns a contiguous range
// of interleaved weight rows and a producer lane moves 16-column x KP tiles (with their scale /
// zero boxes) into a shared-memory ring by bulk copies. What differs:
//
//  * The activations are staged ONCE per CTA in shared memory, converted to fp16 whatever the
//    activation type is, and the consumer warps read their mma B fragments from there instead of
//    holding them in registers. A consumer thread needs about 50 registers instead of 112, and a CTA
//    needs half of an SM's shared memory, so the CTA of the next launch in the stream (programmatic
//    dependent launch) becomes resident beside the running one and fills its ring while the running
//    one computes: launch latency, barrier set-up and the first tiles' HBM latency leave the
//    critical path.
//  * fp16 has ten mantissa bits, so a nibble may sit in bits 0..3 or 4..7 of the magic constant:
//    8 nibbles cost 4 logic operations and 1 shift (7 for a bf16 mantissa). The nibble in bits 4..7
//    comes out as 1024 + 16 u; the activations it meets are stored divided by 16. bf16 activations
//    are scaled per (row, 128-k unit) by a power of two that brings the unit's largest magnitude
//    to 2^14, so the conversion to fp16 is exact for everything within 2^-28 of that maximum.
//
// Arithmetic (FOLDED, as in w4_gemv.cu): within one scale group
//   sum_k a_k (q_k s + z) = s * (f * S - P) + z * Q,
// where S = sum_k a'_k w'_k is what the tensor cores compute from the stored fp16 activations a'
// and the magic-biased integers w' (fp32 accumulation), f is the unit's power-of-two factor,
// P = f * 1024 * sum a' + bias * sum a (bias = 8 or 128: the unsigned storage offset) and
// Q = sum a. f, P, Q are computed once per (row, unit) from the very values the tensor cores see.
// The pre-quant scale product is rounded to T (utility.h:116 of the reference GEMV) and
// alpha * acc + bias is formed in fp32 (utility.h:256-266).
//
// Scope: int4 with group size 128 or per-column scales, int8 with any scale layout; m <= 8 per
// launch; m * (2 k + pad) bytes of activations must leave room for at least three ring slots.
// Everything else stays with w4_gemv.cu.
#include <mutex>
#include <type_traits>

#include "w4_common.cuh"
#include "w4_internal.h"
#include "w4_tma.h"

namespace w4
{
namespace gemv2
{

constexpr int kWarps = 16; // consumer warps
constexpr int kConsumerThreads = kWarps * 32;
constexpr int kThreads = kConsumerThreads + 64; // + the producer warp and the watcher warp (one lane of each works)
constexpr int kBoxCols = 16;                    // columns per scale/zero box = one column group
constexpr int kZeroBoxOff = 512;                // bytes from a slot's scale box to its zero box (16 groups x 32 B)
// Shared memory one CTA may use when two are to share an SM: half of 228 KB less the 1 KB the
// system reserves per CTA.
constexpr int kHalfSmSmem = 233472 / 2 - 1024;

template <int BITS>
struct Cfg
{
    static constexpr int IL = BITS == 4 ? 4 : 2;        // columns per interleaved row
    static constexpr int RPG = 16 / IL;                 // interleaved rows per 16-column group
    static constexpr int CK = 128 / BITS;               // k values in one 16-byte chunk
    static constexpr int UK = 4 * CK;                   // k values per warp unit (4 chunks): 128 / 64
    static constexpr int KP = kWarps * UK;              // k panel covered by one tile: 2048 / 1024
    static constexpr int ROW_STRIDE = 2 * KP;           // bytes of one interleaved row inside a tile
    static constexpr int TILE_BYTES = RPG * ROW_STRIDE; // 16 KB
    static constexpr int VECS = BITS == 4 ? 4 : 2;      // 16-byte vectors of fp16 activations behind one chunk
    // Activations in shared memory: the four chunks of a unit are 80 (int4) / 32 (int8) bytes apart,
    // which puts the 16-byte vectors that the lanes of one row read at once into distinct banks.
    static constexpr int BLOCK_STRIDE = BITS == 4 ? 80 : 32;
    static constexpr int UNIT_STRIDE = 4 * BLOCK_STRIDE;
    static constexpr float BIAS = BITS == 4 ? 8.f : 128.f; // unsigned storage offset of the weights
};

struct Args
{
    uint8_t const* weight;
    void const* act;
    void const* act_scale;
    void const* scales;
    void const* zeros;
    void const* bias;
    void* out;
    float alpha;
    int m; // rows handled by this launch (<= 8)
    int n;
    int k;
    int group_shift;      // log2(group size); 31 for per-channel
    int num_cgs;          // n / 16
    int num_slots;
    int slot_bytes;       // tile bytes + scale/zero boxes, multiple of 128
    int groups_per_panel; // scale rows delivered with every tile (1 for per-channel)
    int depth;            // tiles kept in flight ahead of the one being consumed
    int act_stride;       // bytes between activation rows in shared memory
    int off_act, off_zero, off_tab, off_red, off_bar; // shared-memory layout (bytes)
    int red_bytes;
    int weights_static; // weights / scales / zeros / act_scale were complete before the preceding kernel started
};

// Shared-memory loads through 32-bit addresses with immediate offsets.
template <int OFF>
__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(OFF));
    return v;
}

// The B-fragment vectors of one chunk, fetched only by the lanes whose activation row exists: a lane
// that does not load costs no shared-memory cycle (a quarter-warp without active lanes is skipped),
// its registers keep whatever they held and are zeroed by the caller with an integer multiply.
template <int VECS>
__device__ __forceinline__ void lds_b_fragments(uint4 (&v)[VECS], uint32_t addr, uint32_t active)
{
    static_assert(VECS == 2 || VECS == 4, "two or four 16-byte vectors per chunk");
    if (VECS == 4)
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.u32 p, %17, 0;\n"
            "@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%16];\n"
            "@p ld.shared.v4.u32 {%4,%5,%6,%7}, [%16+16];\n"
            "@p ld.shared.v4.u32 {%8,%9,%10,%11}, [%16+32];\n"
            "@p ld.shared.v4.u32 {%12,%13,%14,%15}, [%16+48];\n"
            "}\n"
            : "=r"(v[0].x), "=r"(v[0].y), "=r"(v[0].z), "=r"(v[0].w), "=r"(v[1].x), "=r"(v[1].y), "=r"(v[1].z),
            "=r"(v[1].w), "=r"(v[VECS - 2].x), "=r"(v[VECS - 2].y), "=r"(v[VECS - 2].z), "=r"(v[VECS - 2].w),
            "=r"(v[VECS - 1].x), "=r"(v[VECS - 1].y), "=r"(v[VECS - 1].z), "=r"(v[VECS - 1].w)
            : "r"(addr), "r"(active));
    else
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.u32 p, %9, 0;\n"
            "@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%8];\n"
            "@p ld.shared.v4.u32 {%4,%5,%6,%7}, [%8+16];\n"
            "}\n"
            : "=r"(v[0].x), "=r"(v[0].y), "=r"(v[0].z), "=r"(v[0].w), "=r"(v[1].x), "=r"(v[1].y), "=r"(v[1].z),
            "=r"(v[1].w)
            : "r"(addr), "r"(active));
#pragma unroll
    for (int i = 0; i < VECS; ++i)
    {
        // integer multiply by 0 / 1: runs on the FMA pipe, which this kernel leaves idle
        v[i].x *= active;
        v[i].y *= active;
        v[i].z *= active;
        v[i].w *= active;
    }
}

template <int OFF>
__device__ __forceinline__ uint2 lds64(uint32_t addr)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFF));
    return v;
}

template <int OFF>
__device__ __forceinline__ uint32_t lds32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
    return v;
}

template <int OFF>
__device__ __forceinline__ uint32_t lds16(uint32_t addr)
{
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1+%2];" : "=h"(v) : "r"(addr), "n"(OFF));
    return v;
}

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
    uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// d = a * b (no accumulator input: starts a chain without zeroing registers first)
__device__ __forceinline__ void mma_f16_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
    uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// Makes a value opaque to the optimiser so that it is computed once and held in a register.
__device__ __forceinline__ void keep_in_register(uint32_t& v)
{
    asm volatile("" : "+r"(v));
}

__device__ __forceinline__ void keep_in_register(int& v)
{
    asm volatile("" : "+r"(v));
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi)
{
    __half2 const h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t const*>(&h);
}

template <typename T, int BITS, bool HAS_ZERO>
__global__ void __launch_bounds__(kThreads, 2)
    gemv2_kernel(Args const a, __grid_constant__ CUtensorMap const tm_scales, __grid_constant__ CUtensorMap const tm_zeros)
{
    using C = Cfg<BITS>;
    using P = Pair<T>;
    extern __shared__ __align__(128) uint8_t smem[];

    uint8_t* const ring = smem;
    uint8_t* const act_sm = smem + a.off_act;
    // (f, P, Q) table: 24 bytes per (unit, row pair): {f0, f1, P0, P1, Q0, Q1}.
    float* const tab = reinterpret_cast<float*>(smem + a.off_tab);
    float* const red = reinterpret_cast<float*>(smem + a.off_red);
    // Synchronisation area: done[16] (tiles finished per consumer warp), landed, abort flag, then
    // one mbarrier per slot for the bulk copies.
    uint32_t* const sync_words = reinterpret_cast<uint32_t*>(smem + a.off_bar);
    uint32_t const done0 = smem_u32(sync_words), landed_addr = done0 + 64;
    volatile int* const abort_flag = reinterpret_cast<volatile int*>(sync_words + 17);
    uint64_t* const full_bar = reinterpret_cast<uint64_t*>(smem + a.off_bar + 128);

    int const tid = threadIdx.x;
    int const warp = tid >> 5, lane = tid & 31;

    // Column groups (16 output columns) of this CTA: a contiguous, balanced range.
    int const c0 = int((int64_t(a.num_cgs) * blockIdx.x) / gridDim.x);
    int const c1 = int((int64_t(a.num_cgs) * (blockIdx.x + 1)) / gridDim.x);
    int const num_cg = c1 - c0;
    int const num_panels = (a.k + C::KP - 1) / C::KP;
    int const units = a.k / C::UK;
    size_t const row_bytes = size_t(2) * a.k;
    // With a single k panel the rows of a column group are adjacent in memory as well: keep them
    // adjacent in the slot so that one bulk copy moves the whole tile.
    int const row_stride = num_panels == 1 ? int(row_bytes) : C::ROW_STRIDE;
    int const num_tiles = num_cg * num_panels;

    if (tid == 0)
    {
        for (int s = 0; s < a.num_slots; ++s)
            mbar_init(&full_bar[s], 1);
        for (int i = 0; i < 18; ++i)
            sync_words[i] = 0u;
        mbar_fence_init();
    }
    else if (tid == 32)
    {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_scales) : "memory");
        if (HAS_ZERO)
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_zeros) : "memory");
    }
    __syncthreads();
    // Programmatic dependent launch: the next kernel in the stream may become resident now (it fits
    // beside this CTA) and start filling its own ring.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // ---------------------------------------------------------------------- producer
    // Tile j (column group j / num_panels, panel j % num_panels) starts once every consumer warp has
    // released the tile that used its slot before and tile j - depth has fully arrived: only `depth`
    // tiles share the memory pipe, so they land in order.
    if (warp == kWarps)
    {
        if (lane == 0)
        {
            // Weights that the preceding kernel may still be writing must not be fetched early.
            if (!a.weights_static)
                asm volatile("griddepcontrol.wait;" ::: "memory");
            int slot = 0, cg = 0, panel = 0;
            uint32_t const box_bytes = uint32_t(a.groups_per_panel) * kBoxCols * 2;
            for (int j = 0; j < num_tiles; ++j)
            {
                if (j >= a.num_slots)
                {
                    // every consumer warp has finished the tile that used this slot before
                    if (!wait_all_counts(done0, uint32_t(j - a.num_slots + 1), abort_flag))
                        break;
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                if (j >= a.depth && !wait_count(landed_addr, uint32_t(j - a.depth + 1), abort_flag))
                    break;
                int const row_first = (c0 + cg) * C::RPG;
                int const kp_len = min(C::KP, a.k - panel * C::KP);
                uint32_t const bytes = 2u * kp_len;
                mbar_expect_tx(&full_bar[slot], bytes * C::RPG + box_bytes * (HAS_ZERO ? 2 : 1));
                uint8_t* dst = ring + size_t(slot) * a.slot_bytes;
                uint8_t const* src = a.weight + size_t(row_first) * row_bytes + size_t(panel) * C::ROW_STRIDE;
                if (num_panels == 1)
                    bulk_g2s(dst, src, bytes * C::RPG, &full_bar[slot]);
                else
                    for (int r = 0; r < C::RPG; ++r)
                        bulk_g2s(dst + r * C::ROW_STRIDE, src + r * row_bytes, bytes, &full_bar[slot]);
                // The scale / zero rows of this panel for the group's 16 columns travel with the tile.
                int const grow = a.group_shift >= 31 ? 0 : panel * a.groups_per_panel;
                tma_load_2d(dst + C::TILE_BYTES, &tm_scales, (c0 + cg) * 16, grow, &full_bar[slot]);
                if (HAS_ZERO)
                    tma_load_2d(dst + C::TILE_BYTES + kZeroBoxOff, &tm_zeros, (c0 + cg) * 16, grow, &full_bar[slot]);
                if (++panel == num_panels)
                {
                    panel = 0;
                    ++cg;
                }
                if (++slot == a.num_slots)
                    slot = 0;
            }
        }
        return;
    }
    // ---------------------------------------------------------------------- watcher
    // The only warp that waits on the copies' mbarriers: tiles land in order, so it walks the slots
    // and publishes how many tiles have arrived.
    if (warp == kWarps + 1)
    {
        if (lane == 0)
        {
            int slot = 0;
            uint32_t parity = 0;
            for (int j = 0; j < num_tiles; ++j)
            {
                if (!mbar_wait_or_abort(&full_bar[slot], parity, abort_flag))
                    break;
                publish_count(landed_addr, uint32_t(j + 1));
                if (++slot == a.num_slots)
                {
                    slot = 0;
                    parity ^= 1;
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumers
    int const g = lane >> 2, t = lane & 3;
    int const MT = (a.m + 1) >> 1; // activation row pairs that exist
    // Columns (inside a 16-column group) behind logical mma rows g and g + 8, and where their
    // 16-byte chunks sit inside a tile. int4: adjacent columns (one 32-bit scale load serves
    // both, and their chunks are 32 bytes apart); int8: columns g and g + 8.
    int const colA = BITS == 4 ? 2 * g : g;
    int const colB = BITS == 4 ? 2 * g + 1 : 8 + g;
    // k offset of this thread's chunk inside a tile -> 128-byte line kk/64, 16-byte piece (kk%64)/CK.
    int const kk = warp * C::UK + t * C::CK;
    int const woff = (kk >> 6) * 128 + ((kk & 63) / C::CK) * 16;
    uint32_t const ring32 = smem_u32(ring);
    uint32_t wA0 = ring32 + (colA / C::IL) * row_stride + (colA % C::IL) * (128 / C::IL) + woff;
    uint32_t wB0 = ring32 + (colB / C::IL) * row_stride + (colB % C::IL) * (128 / C::IL) + woff;
    // Scale group of this warp's unit inside the panel's box, then this thread's column(s).
    int const sgrp = a.group_shift >= 31 ? 0 : (warp * C::UK) >> a.group_shift;
    uint32_t sc0 = ring32 + C::TILE_BYTES + (sgrp * kBoxCols + colA) * 2;
    // B fragments: activation row g, chunk t of every unit; lanes whose row does not exist load
    // nothing and hold zeros.
    bool const row_ok = g < a.m;
    uint32_t act0 = smem_u32(act_sm) + (row_ok ? g : 0) * a.act_stride + t * C::BLOCK_STRIDE;
    uint32_t active = row_ok ? 1u : 0u;
    // (f, P, Q) entries of the activation rows 2t, 2t+1 behind this thread's accumulator columns.
    uint32_t tab0 = smem_u32(tab) + (t < MT ? t : MT - 1) * 24;
    int const tstride = MT * 24;
    uint32_t const my_done = done0 + 4 * warp;
    // These per-thread addresses are used once per tile; keep them in registers (the compiler would
    // otherwise recompute them from the thread index inside the loop, some thirty instructions per tile).
    keep_in_register(wA0);
    keep_in_register(wB0);
    keep_in_register(sc0);
    keep_in_register(act0);
    keep_in_register(active);
    keep_in_register(tab0);

    // ---- stage the activations: act * pre-quant scale (rounded to T) -> fp16, per (row, unit).
    // One warp per (row, unit) job, JB jobs at a time with all their global loads issued first. The
    // pre-quant scale is a weight-like constant: when the caller declared the weights static, the
    // first batch's scales are fetched before the wait for the preceding kernel.
    {
        T const* act = static_cast<T const*>(a.act);
        T const* ps = static_cast<T const*>(a.act_scale);
        if (tid < 16)
            reinterpret_cast<uint32_t*>(smem + a.off_zero)[tid] = 0u;
        int const jobs = a.m * units;
        constexpr int VPL = C::UK / 32; // values per lane: 4 (int4) or 2 (int8)
        constexpr int JB = 4;
        uint2 scv[JB];
        auto load_scales = [&](int job0)
        {
#pragma unroll
            for (int j = 0; j < JB; ++j)
            {
                int const job = job0 + j * kWarps;
                scv[j] = make_uint2(0u, 0u);
                if (job < jobs)
                {
                    int const u = job % units;
                    int const k0 = u * C::UK + lane * VPL;
                    if (VPL == 4)
                        scv[j] = __ldg(reinterpret_cast<uint2 const*>(ps + k0));
                    else
                        scv[j].x = __ldg(reinterpret_cast<uint32_t const*>(ps + k0));
                }
            }
        };
        bool const ps_early = ps != nullptr && a.weights_static;
        if (ps_early)
            load_scales(warp);

        // Activations (and, later, the output) belong to the preceding kernels: wait for them here.
        asm volatile("griddepcontrol.wait;" ::: "memory");

        for (int job0 = warp; job0 < jobs; job0 += kWarps * JB)
        {
            uint2 x[JB];
#pragma unroll
            for (int j = 0; j < JB; ++j)
            {
                int const job = job0 + j * kWarps;
                x[j] = make_uint2(0u, 0u);
                if (job < jobs)
                {
                    int const row = job / units, u = job - row * units;
                    int const k0 = u * C::UK + lane * VPL;
                    if (VPL == 4)
                        x[j] = __ldg(reinterpret_cast<uint2 const*>(act + size_t(row) * a.k + k0));
                    else
                        x[j].x = __ldg(reinterpret_cast<uint32_t const*>(act + size_t(row) * a.k + k0));
                }
            }
            if (ps)
            {
                if (!(ps_early && job0 == warp))
                    load_scales(job0);
#pragma unroll
                for (int j = 0; j < JB; ++j)
                {
                    x[j].x = P::mul(x[j].x, scv[j].x);
                    if (VPL == 4)
                        x[j].y = P::mul(x[j].y, scv[j].y);
                }
            }
#pragma unroll
            for (int j = 0; j < JB; ++j)
            {
                int const job = job0 + j * kWarps;
                if (job >= jobs)
                    break; // warp-uniform
                int const row = job / units, u = job - row * units;
                float v[4] = {0.f, 0.f, 0.f, 0.f};
                P::unpack2(x[j].x, v[0], v[1]);
                if (VPL == 4)
                    P::unpack2(x[j].y, v[2], v[3]);
                // Power-of-two factor of the unit: bf16 spans more exponents than fp16 holds.
                float mul = 1.f, f = 1.f;
                if (std::is_same<T, __nv_bfloat16>::value)
                {
                    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1)
                        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                    uint32_t e = __float_as_uint(amax) >> 23; // biased exponent of the largest magnitude
                    e = e < 15u ? 15u : (e > 254u ? 254u : e);
                    mul = __uint_as_float((268u - e) << 23); // 2^(141 - e): the maximum lands in [2^14, 2^15)
                    f = __uint_as_float((e - 14u) << 23);    // 2^(e - 141)
                }
                // int4: the activations behind the nibbles extracted from bits 4..7 (registers 4..7
                // and 12..15 of a chunk's 16) are stored divided by 16.
                bool const hi = BITS == 4 && ((lane >> 1) & 1);
                float const lmul = hi ? mul * 0.0625f : mul;
                uint32_t h[2];
                float part = 0.f;
#pragma unroll
                for (int i = 0; i < VPL / 2; ++i)
                {
                    h[i] = pack_half2(v[2 * i] * lmul, v[2 * i + 1] * lmul);
                    float2 const back = __half22float2(*reinterpret_cast<__half2 const*>(&h[i]));
                    part += back.x + back.y;
                }
                float const lo_sum = warp_sum(hi ? 0.f : part);
                float const hi_sum = BITS == 4 ? warp_sum(hi ? part : 0.f) : 0.f;
                if (lane == 0)
                {
                    float const sum_stored = lo_sum + hi_sum;            // sum of a'
                    float const sum_true = f * (lo_sum + 16.f * hi_sum); // sum of the activations themselves
                    float* e = tab + (u * MT + (row >> 1)) * 6 + (row & 1);
                    e[0] = f;
                    e[2] = f * 1024.f * sum_stored + C::BIAS * sum_true;
                    e[4] = sum_true;
                    if (row + 1 == a.m && (a.m & 1))
                    {
                        e[1] = 0.f;
                        e[3] = 0.f;
                        e[5] = 0.f;
                    }
                }
                // Register index i of the chunk (pair of k values) -> place inside the chunk's block:
                // int4: vector i % 4, word i / 4; int8: vector (i % 4) / 2, word 2 (i % 2) + i / 4.
                int const tq = lane >> 3; // chunk (lane t of the consumers) this lane's values belong to
                uint8_t* const blk = act_sm + row * a.act_stride + u * C::UNIT_STRIDE + tq * C::BLOCK_STRIDE;
                if (BITS == 4)
                {
                    int const i0 = 2 * (lane & 7);
#pragma unroll
                    for (int i = 0; i < 2; ++i)
                    {
                        int const reg = i0 + i;
                        *reinterpret_cast<uint32_t*>(blk + ((reg & 3) << 4) + ((reg >> 2) << 2)) = h[i];
                    }
                }
                else
                {
                    int const reg = lane & 7, jj = reg & 3;
                    *reinterpret_cast<uint32_t*>(blk + ((jj >> 1) << 4) + ((((jj & 1) << 1) + (reg >> 2)) << 2)) = h[0];
                }
            }
        }
    }
    named_bar_sync(1, kConsumerThreads);

    // ---- main loop over this CTA's tiles (column group outer, k panel inner)
    constexpr uint32_t kMagic = 0x64006400u;              // {1024, 1024}
    int const per_cg = kWarps * 16 * a.m;                 // floats of partial sums per column group
    int const batch = max(1, (a.red_bytes / 4) / per_cg); // column groups per reduction
    bool ok = true;
    int s = 0, panel = 0, cb = 0, cg = 0;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int tile = 0; tile < num_tiles; ++tile)
    {
        if (ok)
            ok = wait_count(landed_addr, uint32_t(tile + 1), abort_flag);
        uint32_t const so = uint32_t(s) * uint32_t(a.slot_bytes);
        int const u = panel * kWarps + warp;
        if (u < units)
        {
            uint4 const wa = lds128<0>(wA0 + so);
            uint4 const wb = BITS == 4 ? lds128<32>(wA0 + so) : lds128<0>(wB0 + so);
            uint32_t const ra[4] = {wa.x, wa.y, wa.z, wa.w};
            uint32_t const rb[4] = {wb.x, wb.y, wb.z, wb.w};
            uint32_t const au = act0 + u * C::UNIT_STRIDE;
            // scale / zero words of the thread's two columns and the unit's (f, P, Q) entries: fetched
            // up front so that their latency hides behind the nibble extraction
            uint32_t s_word, z_word = 0;
            if (BITS == 4)
            {
                s_word = lds32<0>(sc0 + so);
                if (HAS_ZERO)
                    z_word = lds32<kZeroBoxOff>(sc0 + so);
            }
            else
            {
                s_word = lds16<0>(sc0 + so) | (lds16<16>(sc0 + so) << 16);
                if (HAS_ZERO)
                    z_word = lds16<kZeroBoxOff>(sc0 + so) | (lds16<kZeroBoxOff + 16>(sc0 + so) << 16);
            }
            uint32_t const ta = tab0 + u * tstride;
            uint2 const f2 = lds64<0>(ta), p2 = lds64<8>(ta); // (f0, f1), (P0, P1)
            uint2 q2 = make_uint2(0u, 0u);                     // (Q0, Q1)
            if (HAS_ZERO)
                q2 = lds64<16>(ta);
            float S[2][4];
            if (BITS == 4)
            {
                uint4 bv[4];
                lds_b_fragments<4>(bv, au, active);
#pragma unroll
                for (int jj = 0; jj < 4; ++jj)
                {
                    uint4 const b = bv[jj];
                    uint32_t const a8 = ra[jj] >> 8, b8 = rb[jj] >> 8;
                    uint32_t const xa0 = lop3_and_or(ra[jj], 0x000f000fu, kMagic);
                    uint32_t const xa1 = lop3_and_or(ra[jj], 0x00f000f0u, kMagic);
                    uint32_t const xa2 = lop3_and_or(a8, 0x000f000fu, kMagic);
                    uint32_t const xa3 = lop3_and_or(a8, 0x00f000f0u, kMagic);
                    uint32_t const xb0 = lop3_and_or(rb[jj], 0x000f000fu, kMagic);
                    uint32_t const xb1 = lop3_and_or(rb[jj], 0x00f000f0u, kMagic);
                    uint32_t const xb2 = lop3_and_or(b8, 0x000f000fu, kMagic);
                    uint32_t const xb3 = lop3_and_or(b8, 0x00f000f0u, kMagic);
                    if (jj == 0)
                    {
                        mma_f16_first(S[0], xa0, xb0, xa1, xb1, b.x, b.y);
                        mma_f16_first(S[1], xa2, xb2, xa3, xb3, b.z, b.w);
                    }
                    else
                    {
                        mma_f16(S[0], xa0, xb0, xa1, xb1, b.x, b.y);
                        mma_f16(S[1], xa2, xb2, xa3, xb3, b.z, b.w);
                    }
                }
            }
            else
            {
                constexpr uint32_t kMagic8 = 0x64646464u; // prmt source: 0x64 high bytes -> 1024 + byte
                uint4 bv[2];
                lds_b_fragments<2>(bv, au, active);
#pragma unroll
                for (int v = 0; v < 2; ++v)
                {
                    uint4 const b = bv[v];
#pragma unroll
                    for (int e = 0; e < 2; ++e)
                    {
                        int const jj = 2 * v + e;
                        uint32_t const xa0 = prmt(ra[jj], kMagic8, 0x4240u), xa1 = prmt(ra[jj], kMagic8, 0x4341u);
                        uint32_t const xb0 = prmt(rb[jj], kMagic8, 0x4240u), xb1 = prmt(rb[jj], kMagic8, 0x4341u);
                        uint32_t const b0 = e ? b.z : b.x, b1 = e ? b.w : b.y;
                        if (v == 0)
                            mma_f16_first(S[e], xa0, xb0, xa1, xb1, b0, b1);
                        else
                            mma_f16(S[e], xa0, xb0, xa1, xb1, b0, b1);
                    }
                }
            }
            // scale, zero and the magic / storage-offset correction on the fp32 unit sums
            float sA, sB, zA = 0.f, zB = 0.f;
            P::unpack2(s_word, sA, sB);
            if (HAS_ZERO)
                P::unpack2(z_word, zA, zB);
            float const f0 = __uint_as_float(f2.x), f1 = __uint_as_float(f2.y);
            float const p0 = __uint_as_float(p2.x), p1 = __uint_as_float(p2.y);
            acc[0] = fmaf(sA, fmaf(S[0][0] + S[1][0], f0, -p0), acc[0]);
            acc[1] = fmaf(sA, fmaf(S[0][1] + S[1][1], f1, -p1), acc[1]);
            acc[2] = fmaf(sB, fmaf(S[0][2] + S[1][2], f0, -p0), acc[2]);
            acc[3] = fmaf(sB, fmaf(S[0][3] + S[1][3], f1, -p1), acc[3]);
            if (HAS_ZERO)
            {
                float const q0 = __uint_as_float(q2.x), q1 = __uint_as_float(q2.y);
                acc[0] = fmaf(zA, q0, acc[0]);
                acc[1] = fmaf(zA, q1, acc[1]);
                acc[2] = fmaf(zB, q0, acc[2]);
                acc[3] = fmaf(zB, q1, acc[3]);
            }
        }
        __syncwarp();
        if (lane == 0)
            publish_count(my_done, uint32_t(tile + 1));
        if (++s == a.num_slots)
            s = 0;
        if (++panel < num_panels)
            continue;

        // ---- a column group is complete: park its partial sums, [cb][warp][column half * 8 + g][row]
        panel = 0;
#pragma unroll
        for (int c = 0; c < 4; ++c)
        {
            int const row = 2 * t + (c & 1);
            if (row < a.m)
                red[((cb * kWarps + warp) * 16 + (c >> 1) * 8 + g) * a.m + row] = acc[c];
            acc[c] = 0.f;
        }
        ++cb;
        ++cg;
        if (cb < batch && cg < num_cg)
            continue;

        // ---- combine the 16 warps' partial sums in a fixed order and write this batch of columns
        named_bar_sync(1, kConsumerThreads);
        int const cg_first = c0 + cg - cb;
        for (int o = tid; o < cb * 16 * a.m; o += kConsumerThreads)
        {
            int const col_in = o & 15, rest = o >> 4;
            int const row = rest % a.m, b = rest / a.m;
            int const lg = BITS == 4 ? col_in >> 1 : col_in & 7;
            int const chalf = BITS == 4 ? col_in & 1 : col_in >> 3;
            float const* src = red + ((b * kWarps) * 16 + chalf * 8 + lg) * a.m + row;
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w)
                sum += src[w * 16 * a.m];
            int const col = (cg_first + b) * 16 + col_in;
            float v = a.alpha * sum;
            if (a.bias)
                v += P::to_float(static_cast<uint16_t const*>(a.bias)[col]);
            static_cast<uint16_t*>(a.out)[size_t(row) * a.n + col] = P::from_float(v);
        }
        cb = 0;
        if (cg < num_cg)
            named_bar_sync(1, kConsumerThreads);
    }
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
static int round_up(int v, int to)
{
    return (v + to - 1) / to * to;
}

// Shared-memory plan for one problem. Returns false when the activations leave too little room for
// the ring (the caller then uses the register-resident form of the kernel).
template <int BITS>
static bool plan(Args& a, DeviceInfo const& dev, int grid, size_t* smem_bytes)
{
    using C = Cfg<BITS>;
    a.groups_per_panel = a.group_shift >= 31 ? 1 : C::KP >> a.group_shift;
    a.slot_bytes = C::TILE_BYTES + 2 * kZeroBoxOff;
    int const units = a.k / C::UK;
    // Row stride: an odd multiple of 64 bytes (int4) / 16 bytes past a multiple of 128 (int8), so that
    // the two rows a quarter-warp reads together use distinct banks.
    a.act_stride = units * C::UNIT_STRIDE;
    if (BITS == 4)
        a.act_stride += (a.act_stride % 128 == 0) ? 64 : 0;
    else
        a.act_stride += 16;
    int const MT = (a.m + 1) / 2;
    int const act_bytes = round_up(a.m * a.act_stride, 128);
    int const fpq_bytes = round_up(units * MT * 24, 128);
    // Partial sums: all column groups of a CTA in one reduction when that stays small.
    int const cgs = (a.num_cgs + grid - 1) / grid;
    int const per_cg = kWarps * 16 * a.m * 4;
    int red = cgs * per_cg;
    int const red_cap = 16 * 1024 > per_cg ? 16 * 1024 : per_cg;
    if (red > red_cap)
        red = red_cap / per_cg * per_cg;
    a.red_bytes = red;
    int const fixed_front = act_bytes + 128 + fpq_bytes + round_up(red, 128);
    auto slots_for = [&](int budget) { return (budget - fixed_front - 384) / a.slot_bytes; };
    int slots = slots_for(kHalfSmSmem);
    if (slots >= 5)
        slots = slots > 6 ? 6 : slots; // two CTAs (of consecutive launches) per SM
    else
    {
        slots = slots_for(dev.max_smem_optin);
        if (slots > 12)
            slots = 12;
    }
    if (slots < 3)
        return false;
    a.num_slots = slots;
    int const depth = (72 * 1024 + a.slot_bytes / 2) / a.slot_bytes;
    a.depth = depth < 1 ? 1 : (depth > slots - 1 ? slots - 1 : depth);
    a.off_act = slots * a.slot_bytes;
    a.off_zero = a.off_act + act_bytes;
    a.off_tab = a.off_zero + 128;
    a.off_red = a.off_tab + fpq_bytes;
    a.off_bar = a.off_red + round_up(red, 128);
    *smem_bytes = size_t(a.off_bar) + 128 + size_t(slots) * 8;
    return true;
}

template <typename T, int BITS, bool HAS_ZERO>
static int launch_one(Args a, DeviceInfo const& dev, cudaStream_t stream)
{
    using C = Cfg<BITS>;
    auto kernel = gemv2_kernel<T, BITS, HAS_ZERO>;
    int const grid = a.num_cgs < dev.num_sms ? a.num_cgs : dev.num_sms;
    size_t smem = 0;
    if (!plan<BITS>(a, dev, grid, &smem))
        return W4_ERR_UNSUPPORTED;
    CUtensorMap tm_scales, tm_zeros;
    uint64_t const groups = a.group_shift >= 31 ? 1 : uint64_t(a.k >> a.group_shift);
    if (!make_tensor_map_2d(&tm_scales, CU_TENSOR_MAP_DATA_TYPE_UINT16, a.scales, uint64_t(a.n), groups,
            uint64_t(a.n) * 2, kBoxCols, uint32_t(a.groups_per_panel), CU_TENSOR_MAP_SWIZZLE_NONE))
        return W4_ERR_CUDA;
    tm_zeros = tm_scales;
    if (HAS_ZERO
        && !make_tensor_map_2d(&tm_zeros, CU_TENSOR_MAP_DATA_TYPE_UINT16, a.zeros, uint64_t(a.n), groups,
            uint64_t(a.n) * 2, kBoxCols, uint32_t(a.groups_per_panel), CU_TENSOR_MAP_SWIZZLE_NONE))
        return W4_ERR_CUDA;
    {
        // The opt-in shared-memory limit and the carve-out are per-function, per-device attributes:
        // set them once (this block is instantiated once per kernel).
        static std::mutex mu;
        static bool configured[64] = {};
        if (dev.device < 0 || dev.device >= 64)
            return W4_ERR_CUDA;
        std::lock_guard<std::mutex> lock(mu);
        if (!configured[dev.device])
        {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dev.max_smem_optin)
                    != cudaSuccess
                || cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                       cudaSharedmemCarveoutMaxShared)
                    != cudaSuccess)
                return W4_ERR_CUDA;
            configured[dev.device] = true;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kernel, a, tm_scales, tm_zeros) != cudaSuccess)
        return W4_ERR_CUDA;
    return cudaGetLastError() == cudaSuccess ? W4_OK : W4_ERR_CUDA;
}

template <typename T>
static int dispatch(Args const& a, int bits, DeviceInfo const& dev, cudaStream_t stream)
{
    bool const z = a.zeros != nullptr;
    if (bits == 4)
        return z ? launch_one<T, 4, true>(a, dev, stream) : launch_one<T, 4, false>(a, dev, stream);
    return z ? launch_one<T, 8, true>(a, dev, stream) : launch_one<T, 8, false>(a, dev, stream);
}

// True when this form of the kernel covers the problem (one pass of `rows` <= 8 rows).
bool supports(W4GemmParams const& p, int rows, DeviceInfo const& dev)
{
    if (rows < 1 || rows > 8)
        return false;
    if (p.weight_bits == 4 && (p.group_size == 64 || p.k % 128 != 0))
        return false; // a warp unit spans 128 k: one scale group per unit is needed
    Args a{};
    a.m = rows;
    a.k = p.k;
    a.group_shift = p.group_size == 64 ? 6 : (p.group_size == 128 ? 7 : 31);
    a.num_cgs = p.n / 16;
    int const grid = a.num_cgs < dev.num_sms ? a.num_cgs : dev.num_sms;
    size_t smem = 0;
    return p.weight_bits == 4 ? plan<4>(a, dev, grid, &smem) : plan<8>(a, dev, grid, &smem);
}

int launch(W4GemmParams const& p, int m0, int rows, DeviceInfo const& dev, cudaStream_t stream)
{
    size_t const elt = 2;
    Args a{};
    a.weight = static_cast<uint8_t const*>(p.weight);
    a.act = static_cast<char const*>(p.act) + size_t(m0) * p.k * elt;
    a.act_scale = p.act_scale;
    a.scales = p.scales;
    a.zeros = p.zeros;
    a.bias = p.bias;
    a.out = static_cast<char*>(p.out) + size_t(m0) * p.n * elt;
    a.alpha = p.alpha;
    a.m = rows;
    a.n = p.n;
    a.k = p.k;
    a.group_shift = p.group_size == 64 ? 6 : (p.group_size == 128 ? 7 : 31);
    a.num_cgs = p.n / 16;
    a.weights_static = (p.flags & W4_GEMM_WEIGHTS_STATIC) ? 1 : 0;
    return p.act_dtype == W4_DTYPE_FP16 ? dispatch<__half>(a, p.weight_bits, dev, stream)
                                        : dispatch<__nv_bfloat16>(a, p.weight_bits, dev, stream);
}

} // namespace gemv2
} // namespace w4
