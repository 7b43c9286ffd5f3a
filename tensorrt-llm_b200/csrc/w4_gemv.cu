// Decode-regime kernel (m = 1..8 or 9..16 per pass): streams the packed int4/int8 weights exactly once.
//
// Replaces weight_only::kernel of the reference project
// (cpp/tensorrt_llm/kernels/weightOnlyBatchedGemv/kernel.h:31-120) and, for m >= 5 / m >= 16, the
// small-M CUTLASS tactics it falls back to.
//
// Design (B200): one persistent CTA per SM owns a contiguous range of "interleaved rows" of the
// preprocessed weight (one interleaved row = IL adjacent output columns x all of K = 2K bytes, see
// below), so every CTA streams one contiguous slab of HBM. One lane of a producer warp group moves
// that slab into a shared-memory ring with bulk (TMA-engine) copies, one tile (16 columns x one k
// panel, with its scale/zero boxes) at a time (a flat copy when K fits one panel; with several
// panels int4 rows come through a tensor map whose swizzle removes the bank conflicts of the
// consumers' reads), a bounded number of tiles in flight so that they land in order; 16 consumer warps split K, pull 16-byte chunks out of the ring with 128-bit shared
// loads and feed mma.sync (weights as the 16-row A operand, the m <= 8 activation rows as the
// 8-column B operand, held in registers; a 16-row pass feeds two B fragments per weight fragment
// and covers half as much k per tile), accumulating in fp32. The producer group hands most of
// its registers to the consumers (setmaxnreg). Partial sums of the 16 warps are combined through
// shared memory in a fixed order (deterministic) once per batch of column groups, then alpha/bias
// are applied and the result stored. The kernel is launched as a programmatic dependent: weight
// copies start before the preceding kernel has finished, activations are read after it.
//
// Weight layout consumed (preprocess_weights_for_mixed_gemm on sm_100,
// cpp/tensorrt_llm/kernels/cutlass_kernels/cutlass_preprocessors.cpp:564-615): interleaved row R
// holds columns IL*R .. IL*R+IL-1 (IL = 4 for int4, 2 for int8); inside it every 128-byte line is
// one 64-wide k tile, split into IL column segments; every aligned 16-byte chunk holds CK = 32
// (int4) / 16 (int8) consecutive k of one column in the order
// { 2j+8q+e : register j = 0..3, pair q, element e }, with the nibbles/bytes of each 32-bit
// register pre-shuffled. Because a dot product does not care about the order of k, each thread
// treats the chunk it loaded as its own mma fragment and the activation fragment is simply loaded
// in the matching order.
//
// Arithmetic. Two variants, chosen per problem:
//  * EXACT (int4 with group size 64): as the reference's kernels, the dequantised weight is
//    round_T(fma(q, scale, zero)) (weightOnlyBatchedGemv/utility.h:157-162) and that is what is
//    multiplied; the sum is kept in fp32 (the reference GEMV keeps it in T).
//  * FOLDED (everything else): within one scale group sum_k a_k (q_k s + z) = s * sum_k a_k q_k +
//    z * sum_k a_k, so the tensor cores multiply the activations with the raw biased integers,
//    placed into the mantissa of a magic constant C by a single logic op (C + u, exact), and the
//    scale, the zero and the -(C + bias) * sum_k a_k correction are applied to the fp32 group sum.
//    No per-weight floating-point instruction is left. The weight is not rounded to T first, so
//    the result is closer to real arithmetic than the reference's; it stays far inside the 1e-2 *
//    max|ref| bound this path is held to.
// In both, the pre-quant scale product is rounded to T (utility.h:116) and alpha * acc + bias is
// formed in fp32 (utility.h:256-266).
#include <mutex>

#include "w4_common.cuh"
#include "w4_internal.h"
#include "w4_tma.h"

namespace w4
{
namespace gemv
{

// Consumer warps. With 8 (half the registers and shared memory, so that CTAs of consecutive launches
// share an SM) one CTA cannot keep up with the copies: 12.4 us against 10.4 us on a 4096 x 14336 int4
// matrix, 93 us against 63 us on 8192 x 57344.
constexpr int kWarps = 16;
constexpr int kConsumerThreads = kWarps * 32;
constexpr int kThreads = kConsumerThreads + 128; // + one producer warp group (one lane of it works)
// Registers: a fifth warp per scheduler would cap every thread at 96 registers; the producer group
// gives its share back (setmaxnreg) and the consumer groups take it.
constexpr int kProducerRegs = 24, kConsumerRegs = 112; // 128 * 24 + 512 * 112 <= 640 * 96 (the launch-time pool)
constexpr int kRedBytes = 64 * 1024;            // shared memory for cross-warp partial sums
constexpr int kRedBytes16 = 112 * 1024;         // the same for 16-row passes (7 column groups)
constexpr int kScaleBoxCols = 24;               // columns per scale/zero box: 16 + slack to start on a 16-byte boundary

template <int BITS, int MB>
struct Cfg
{
    static constexpr int IL = BITS == 4 ? 4 : 2;        // columns per interleaved row
    static constexpr int RPG = 16 / IL;                 // interleaved rows per 16-column group
    static constexpr int CK = 128 / BITS;               // k values in one 16-byte chunk
    static constexpr int UK = 4 * CK;                   // k values per warp unit (4 chunks)
    static constexpr int UPW = (MB == 1 || BITS == 8) ? 2 : 1; // units per warp per tile (int8 units are half as wide)
    static constexpr int KP = kWarps * UPW * UK;        // k panel covered by one tile
    static constexpr int ROW_STRIDE = 2 * KP;           // bytes of one interleaved row inside a tile
    static constexpr int TILE_BYTES = RPG * ROW_STRIDE; // 32 KB (MB = 1) or 16 KB (MB = 2)
    static constexpr int AREGS = CK / 2;                // activation pair registers per chunk
};

// Constants of the FOLDED variant. The biased integer u = q + BIAS is turned into the T value
// MAGIC + u. PLANES == 2 (bf16 + int8, whose 8-bit payload does not fit a bf16 mantissa) splits
// every byte into two nibbles: the low-nibble plane meets activations scaled by 1/16, so the unit
// sum is S = (1/16) sum a u + MAGIC (1 + 1/16) sum a.
template <typename T, int BITS>
struct Fold;
template <>
struct Fold<__half, 4>
{
    static constexpr uint32_t MAGIC2 = 0x64006400u; // {1024, 1024}
    static constexpr float SCALE = 1.f, CORR = 1024.f + 8.f;
    static constexpr int PLANES = 1;
};
template <>
struct Fold<__nv_bfloat16, 4>
{
    static constexpr uint32_t MAGIC2 = 0x43004300u; // {128, 128}
    static constexpr float SCALE = 1.f, CORR = 128.f + 8.f;
    static constexpr int PLANES = 1;
};
template <>
struct Fold<__half, 8>
{
    static constexpr uint32_t MAGIC2 = 0x64646464u; // prmt source: 0x64 high bytes -> 1024 + byte
    static constexpr float SCALE = 1.f, CORR = 1024.f + 128.f;
    static constexpr int PLANES = 1;
};
template <>
struct Fold<__nv_bfloat16, 8>
{
    static constexpr uint32_t MAGIC2 = 0x43004300u;
    static constexpr float SCALE = 16.f, CORR = 17.f * 128.f + 128.f;
    static constexpr int PLANES = 2;
};

template <typename T>
struct Consts;
template <>
struct Consts<__half>
{
    static constexpr uint32_t ONE2 = 0x3c003c00u, SIXTEENTH2 = 0x2c002c00u;
};
template <>
struct Consts<__nv_bfloat16>
{
    static constexpr uint32_t ONE2 = 0x3f803f80u, SIXTEENTH2 = 0x3d803d80u;
};

__host__ __device__ inline int num_panels_of(int k, int kp)
{
    return (k + kp - 1) / kp;
}

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
    int m;           // rows handled by this launch (<= 8 * MB)
    int n;
    int k;
    int group_shift; // log2(group size); 31 for per-channel (k >> 31 == 0)
    int num_groups;  // rows of the scale tensor (1 for per-channel)
    int num_rows;    // n / IL
    int num_slots;
    int slot_bytes;       // tile bytes + scale/zero boxes, multiple of 128
    int groups_per_panel; // scale rows delivered with every tile (1 for per-channel)
    int box_stride;       // bytes between the scale box and the zero box (multiple of 128)
    int depth;            // tiles kept in flight ahead of the one being consumed
    int red_bytes;        // shared memory for the cross-warp partial sums
    int weights_static;   // weights / scales / zeros were complete before the preceding kernel started
    PushTarget push;      // world > 0: the epilogue also sends the results to the peers as flagged packets
    int push_row0;        // row of the whole call that this pass's row 0 is
};

// Shared flag: once any wait in the CTA timed out, every later wait returns at once.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag)
{
    for (uint32_t i = 0; i < kMaxWaitPolls; ++i)
    {
        if (mbar_try_wait(bar, parity))
            return true;
        if ((i & 1023u) == 1023u && *abort_flag)
            return false;
    }
    *abort_flag = 1;
    atomicExch(&g_device_status, kDeviceTimeout);
    return false;
}

template <typename T, int BITS, int MB, bool HAS_ZERO, bool HAS_ACT_SCALE, bool FOLD, int CB, bool PUSH>
__global__ void __launch_bounds__(kThreads, 1)
    gemv_kernel(Args const a, __grid_constant__ CUtensorMap const tm_scales, __grid_constant__ CUtensorMap const tm_zeros,
        __grid_constant__ CUtensorMap const tm_w)
{
    using C = Cfg<BITS, MB>;
    using P = Pair<T>;
    using F = Fold<T, BITS>;
    constexpr int PLANES = FOLD ? F::PLANES : 1;
    // Slots start on 1024-byte boundaries: the swizzle of the int4 weight tiles is a function of the
    // shared-memory address.
    extern __shared__ __align__(1024) uint8_t smem[];

    if (BITS == 4 && num_panels_of(a.k, C::KP) > 1 && (smem_u32(smem) & 1023u) != 0) // never seen; tiles would be read wrongly
    {
        if (threadIdx.x == 0)
            atomicExch(&g_device_status, kDeviceTimeout);
        return;
    }
    uint8_t* ring = smem;
    float* red = reinterpret_cast<float*>(smem + size_t(a.num_slots) * a.slot_bytes);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + size_t(a.num_slots) * a.slot_bytes + a.red_bytes);
    uint64_t* empty_bar = full_bar + a.num_slots;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + a.num_slots);

    int const tid = threadIdx.x;
    int const warp = tid >> 5, lane = tid & 31;

    // Row range of this CTA (balanced to within one interleaved row).
    int const r0 = int((int64_t(a.num_rows) * blockIdx.x) / gridDim.x);
    int const r1 = int((int64_t(a.num_rows) * (blockIdx.x + 1)) / gridDim.x);
    int const num_cg = (r1 - r0 + C::RPG - 1) / C::RPG;
    int const num_panels = (a.k + C::KP - 1) / C::KP;
    size_t const row_bytes = size_t(2) * a.k;
    // With a single k panel the rows of a column group are adjacent in memory as well: keep them
    // adjacent in the slot so that one bulk copy moves the whole tile.
    int const row_stride = num_panels == 1 ? int(row_bytes) : C::ROW_STRIDE;

    int const num_tiles = num_cg * num_panels;

    // Partial sums in shared memory: [cg in batch][warp][mb][c][g * MT + t], only the lanes whose
    // rows exist (t < MT) are stored.
    int const MT = MB == 2 ? 4 : (a.m + 1) >> 1;
    int const per_cg = kWarps * MB * 4 * 8 * MT;
    int const red_cap = max(1, (a.red_bytes / 4) / per_cg); // column groups the reduction buffer holds
    // Column groups that share one activation load (only matters with several k panels); the
    // reduction batch is a whole number of such sub-batches.
    // CB == 0: no register sub-batches; the partial sums of a whole reduction batch accumulate in
    // shared memory across the k panels, so one activation load per panel serves the whole batch.
    constexpr bool RED_ACC = CB == 0;
    constexpr int CBR = RED_ACC ? 1 : CB;
    int const cbe = RED_ACC ? red_cap : min(CB, red_cap);
    int const batch = (red_cap / cbe) * cbe;


    // Starts the copies of tile i into its ring slot; called by the producer lane only.
    auto issue_tile = [&](int i, int slot)
    {
        // Tile order: column groups in sub-batches of `cbe`; inside a sub-batch the k panels are
        // the outer loop, so one activation load serves all its column groups.
        int const per_sb = cbe * num_panels;
        int const sb = i / per_sb, r = i - sb * per_sb;
        int const ncb = min(cbe, num_cg - sb * cbe);
        int const panel = r / ncb, cg = sb * cbe + (r - panel * ncb);
        int const row_first = r0 + cg * C::RPG;
        int const rows = min(C::RPG, r1 - row_first);
        int const kp_len = min(C::KP, a.k - panel * C::KP);
        uint32_t const bytes = 2u * kp_len;
        uint32_t const box_bytes = uint32_t(a.groups_per_panel) * kScaleBoxCols * 2;
        uint8_t* dst = ring + size_t(slot) * a.slot_bytes;
        if (BITS == 4 && num_panels > 1)
        {
            // int4 with several k panels: every row's panel is fetched as a box of 128-byte lines
            // through a tensor map with the 32-byte-atom swizzle, which spreads the two lines a
            // quarter-warp reads over all banks (+6 % on a 8192 x 57344 matrix; with a single panel
            // the one flat copy below is as fast, so it stays). A box always arrives whole: lines
            // past k hold the next row's weights (or zeros past the tensor's end) and only ever
            // meet zero activations.
            int const lpr = a.k >> 6; // lines per interleaved row
            mbar_expect_tx(&full_bar[slot], uint32_t(rows) * C::ROW_STRIDE + box_bytes * (HAS_ZERO ? 2 : 1));
            for (int r = 0; r < rows; ++r)
                tma_load_2d(dst + r * C::ROW_STRIDE, &tm_w, 0, (row_first + r) * lpr + panel * (C::KP >> 6),
                    &full_bar[slot]);
        }
        else
        {
            mbar_expect_tx(&full_bar[slot], bytes * rows + box_bytes * (HAS_ZERO ? 2 : 1));
            uint8_t const* src = a.weight + size_t(row_first) * row_bytes + size_t(panel) * C::ROW_STRIDE;
            if (num_panels == 1)
                bulk_g2s(dst, src, bytes * rows, &full_bar[slot]);
            else
                for (int r = 0; r < rows; ++r)
                    bulk_g2s(dst + r * C::ROW_STRIDE, src + r * row_bytes, bytes, &full_bar[slot]);
        }
        // The scale / zero rows of this panel for the group's columns travel with the tile, from
        // the 8-column boundary at or below the group's first column.
        int const col_aligned = (row_first * C::IL) & ~7;
        int const grow = a.group_shift >= 31 ? 0 : panel * a.groups_per_panel;
        tma_load_2d(dst + C::TILE_BYTES, &tm_scales, col_aligned, grow, &full_bar[slot]);
        if (HAS_ZERO)
            tma_load_2d(dst + C::TILE_BYTES + a.box_stride, &tm_zeros, col_aligned, grow, &full_bar[slot]);
    };

    if (tid == 0)
    {
        for (int s = 0; s < a.num_slots; ++s)
        {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], kWarps);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    else if (tid == 32)
    {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_scales) : "memory");
        if (BITS == 4)
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w) : "memory");
        if (HAS_ZERO)
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_zeros) : "memory");
    }
    __syncthreads();
    // Programmatic dependent launch: let the next kernel in the stream begin its own prologue as
    // SMs free up.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // ---------------------------------------------------------------------- producer
    // Tile j starts once (a) every consumer warp has released the tile that used its slot before
    // and (b) tile j - depth has fully arrived: only `depth` tiles share the memory pipe, so they
    // land in order and early enough to overlap with the arithmetic (the copy engine serves all
    // outstanding copies side by side: started together they would also all finish together).
    // The producer touches only weights, scales and zeros; it runs ahead of the preceding kernel
    // only when the caller declared them static (W4_GEMM_WEIGHTS_STATIC).
    if (warp >= kWarps)
    {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kProducerRegs));
        if (warp == kWarps && lane == 0)
        {
            // Weights that the preceding kernel may still be writing must not be fetched early.
            if (!a.weights_static)
                asm volatile("griddepcontrol.wait;" ::: "memory");
            int slot = 0, use = 0;
            for (int j = 0; j < num_tiles; ++j)
            {
                if (j >= a.num_slots)
                {
                    if (!wait_or_abort(&empty_bar[slot], (use - 1) & 1, abort_flag))
                        break;
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                if (j >= a.depth)
                {
                    int const sd = slot >= a.depth ? slot - a.depth : slot - a.depth + a.num_slots;
                    int const ud = slot >= a.depth ? use : use - 1;
                    if (!wait_or_abort(&full_bar[sd], ud & 1, abort_flag))
                        break;
                }
                issue_tile(j, slot);
                if (++slot == a.num_slots)
                {
                    slot = 0;
                    ++use;
                }
            }
        }
        return;
    }
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kConsumerRegs));

    // ---------------------------------------------------------------------- consumers
    int const g = lane >> 2, t = lane & 3;
    // Columns (inside a 16-column group) behind logical mma rows g and g + 8, and where their
    // 16-byte chunks sit inside a tile. int4: adjacent columns (one 32-bit scale load serves
    // both); int8: columns g and g + 8, which makes every 8-lane phase of the shared load read one
    // whole 128-byte line.
    int const colA = BITS == 4 ? 2 * g : g;
    int const colB = BITS == 4 ? 2 * g + 1 : 8 + g;
    int const segA = (colA / C::IL) * row_stride + (colA % C::IL) * (128 / C::IL);
    int const segB = (colB / C::IL) * row_stride + (colB % C::IL) * (128 / C::IL);
    // int4: byte offset of this thread's chunk of column A in a tile, per unit. In the swizzled tiles
    // of the multi-panel case line L keeps its 32-byte column segment s at position s ^ (L & 3).
    // Column B is the segment next to it: the offset with bit 5 flipped, swizzled or not.
    uint32_t woff[C::UPW];
#pragma unroll
    for (int j = 0; j < C::UPW; ++j)
    {
        int const kk = (j * kWarps + warp) * C::UK + t * C::CK;
        int const line = (colA / C::IL) * (row_stride >> 7) + (kk >> 6);
        int const swz = num_panels > 1 ? (line & 3) : 0;
        woff[j] = uint32_t(line * 128 + (((colA % C::IL) ^ swz) << 5) + ((kk & 63) / C::CK) * 16);
    }

    T const* act = static_cast<T const*>(a.act);
    T const* act_scale = static_cast<T const*>(a.act_scale);

    uint32_t afrag[C::UPW][MB][C::AREGS];
    uint32_t afrag_lo[PLANES == 2 ? C::UPW : 1][MB][PLANES == 2 ? C::AREGS : 1]; // activations / 16
    float asum[C::UPW][MB][2]; // FOLDED: sum of this unit's activations for rows 2t, 2t+1

    // (scale, zero) words of this thread's two columns (low half = column A) for unit j, read from
    // the boxes that arrived with the tile. FOLDED applies them to the unit's sum, so the group is
    // that of the unit; EXACT applies them to the thread's own chunk.
    auto read_scales = [&](int j, int cg, uint8_t const* tile, uint32_t& s, uint32_t& z)
    {
        int const kk = (j * kWarps + warp) * C::UK + (FOLD ? 0 : t * C::CK);
        int const col_base = (r0 + cg * C::RPG) * C::IL;
        int const coff = col_base - (col_base & ~7);
        uint16_t const* sc = reinterpret_cast<uint16_t const*>(tile + C::TILE_BYTES)
            + (kk >> a.group_shift) * kScaleBoxCols + coff;
        uint16_t const* zr = sc + a.box_stride / 2;
        z = 0;
        if (BITS == 4)
        {
            s = *reinterpret_cast<uint32_t const*>(sc + colA);
            if (HAS_ZERO)
                z = *reinterpret_cast<uint32_t const*>(zr + colA);
        }
        else
        {
            s = uint32_t(sc[colA]) | (uint32_t(sc[colB]) << 16);
            if (HAS_ZERO)
                z = uint32_t(zr[colA]) | (uint32_t(zr[colB]) << 16);
        }
    };

    // Activation fragments of this warp's units for one k panel, in chunk order; FOLDED also
    // needs the per-unit activation sums, obtained with an all-ones A fragment.
    auto load_act = [&](int panel)
    {
#pragma unroll
        for (int j = 0; j < C::UPW; ++j)
        {
            int const k0 = panel * C::KP + (j * kWarps + warp) * C::UK + t * C::CK;
#pragma unroll
            for (int mb = 0; mb < MB; ++mb)
            {
                int const row = mb * 8 + g;
                bool const valid = row < a.m && k0 < a.k;
#pragma unroll
                for (int v = 0; v < C::AREGS / 4; ++v)
                {
                    uint4 x = make_uint4(0, 0, 0, 0);
                    if (valid)
                    {
                        x = __ldg(reinterpret_cast<uint4 const*>(act + size_t(row) * a.k + k0) + v);
                        if (HAS_ACT_SCALE)
                        {
                            uint4 const ps = __ldg(reinterpret_cast<uint4 const*>(act_scale + k0) + v);
                            x.x = P::mul(x.x, ps.x);
                            x.y = P::mul(x.y, ps.y);
                            x.z = P::mul(x.z, ps.z);
                            x.w = P::mul(x.w, ps.w);
                        }
                    }
                    afrag[j][mb][4 * v + 0] = x.x;
                    afrag[j][mb][4 * v + 1] = x.y;
                    afrag[j][mb][4 * v + 2] = x.z;
                    afrag[j][mb][4 * v + 3] = x.w;
                }
                if (FOLD)
                {
                    constexpr uint32_t one = Consts<T>::ONE2;
                    uint32_t const ones[4] = {one, one, one, one};
                    float sum[2][4]; // two independent chains
#pragma unroll
                    for (int i = 0; i < C::AREGS / 2; ++i)
                    {
                        // same (b0, b1) pairing as the main loop; any pairing covers all of k once
                        int const lo = BITS == 4 ? (i >> 1) + 8 * (i & 1) : i;
                        if (i < 2)
                            P::mma0(sum[i & 1], ones, afrag[j][mb][lo], afrag[j][mb][lo + 4]);
                        else
                            P::mma(sum[i & 1], ones, afrag[j][mb][lo], afrag[j][mb][lo + 4]);
                    }
                    asum[j][mb][0] = sum[0][0] + sum[1][0];
                    asum[j][mb][1] = sum[0][1] + sum[1][1];
                    if (PLANES == 2)
                    {
#pragma unroll
                        for (int i = 0; i < C::AREGS; ++i)
                            afrag_lo[j][mb][i] = P::mul(afrag[j][mb][i], Consts<T>::SIXTEENTH2);
                    }
                }
            }
        }
    };

    float acc[CBR][MB][4]; // running sums of the column groups of the current sub-batch

    // One warp unit (16 columns x UK k) out of the tile in shared memory.
    auto process_unit = [&](int j, int cg, uint8_t const* tile, float(&acc)[MB][4])
    {
        uint32_t s_word, z_word;
        read_scales(j, cg, tile, s_word, z_word);
        // Chunk of this thread inside the row piece: k offset kk -> 128-byte line kk/64, 16-byte
        // slot (kk%64)/CK inside the column segment.
        int const kk = (j * kWarps + warp) * C::UK + t * C::CK;
        int const off = (kk >> 6) * 128 + ((kk & 63) / C::CK) * 16;
        uint4 const wa = *reinterpret_cast<uint4 const*>(tile + (BITS == 4 ? woff[j] : uint32_t(segA + off)));
        uint4 const wb = *reinterpret_cast<uint4 const*>(tile + (BITS == 4 ? woff[j] ^ 32u : uint32_t(segB + off)));
        uint32_t const ra[4] = {wa.x, wa.y, wa.z, wa.w};
        uint32_t const rb[4] = {wb.x, wb.y, wb.z, wb.w};

        if (FOLD)
        {
            constexpr uint32_t kMagic = F::MAGIC2;
            float S[2][MB][4]; // two independent accumulation chains, each started by an mma0
#pragma unroll
            for (int jj = 0; jj < 4; ++jj)
            {
                if (BITS == 4)
                {
                    uint32_t xa[4], xb[4];
#pragma unroll
                    for (int p = 0; p < 4; ++p)
                    {
                        xa[p] = lop3_and_or(ra[jj] >> (4 * p), 0x000f000fu, kMagic);
                        xb[p] = lop3_and_or(rb[jj] >> (4 * p), 0x000f000fu, kMagic);
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                    {
                        uint32_t const frag[4] = {xa[2 * h], xb[2 * h], xa[2 * h + 1], xb[2 * h + 1]};
#pragma unroll
                        for (int mb = 0; mb < MB; ++mb)
                        {
                            if (jj == 0)
                                P::mma0(S[h][mb], frag, afrag[j][mb][jj + 8 * h], afrag[j][mb][jj + 8 * h + 4]);
                            else
                                P::mma(S[h][mb], frag, afrag[j][mb][jj + 8 * h], afrag[j][mb][jj + 8 * h + 4]);
                        }
                    }
                }
                else if (PLANES == 1)
                {
                    uint32_t const frag[4] = {prmt(ra[jj], kMagic, 0x4240u), prmt(rb[jj], kMagic, 0x4240u),
                        prmt(ra[jj], kMagic, 0x4341u), prmt(rb[jj], kMagic, 0x4341u)};
#pragma unroll
                    for (int mb = 0; mb < MB; ++mb)
                    {
                        if (jj < 2)
                            P::mma0(S[jj & 1][mb], frag, afrag[j][mb][jj], afrag[j][mb][jj + 4]);
                        else
                            P::mma(S[jj & 1][mb], frag, afrag[j][mb][jj], afrag[j][mb][jj + 4]);
                    }
                }
                else
                {
                    // nibble planes of the bytes: (byte0, byte2) and (byte1, byte3) pairs
                    uint32_t const lo[4] = {lop3_and_or(ra[jj], 0x000f000fu, kMagic),
                        lop3_and_or(rb[jj], 0x000f000fu, kMagic), lop3_and_or(ra[jj] >> 8, 0x000f000fu, kMagic),
                        lop3_and_or(rb[jj] >> 8, 0x000f000fu, kMagic)};
                    uint32_t const hi[4] = {lop3_and_or(ra[jj] >> 4, 0x000f000fu, kMagic),
                        lop3_and_or(rb[jj] >> 4, 0x000f000fu, kMagic), lop3_and_or(ra[jj] >> 12, 0x000f000fu, kMagic),
                        lop3_and_or(rb[jj] >> 12, 0x000f000fu, kMagic)};
#pragma unroll
                    for (int mb = 0; mb < MB; ++mb)
                    {
                        int const jl = PLANES == 2 ? j : 0, ml = PLANES == 2 ? mb : 0;
                        int const i0 = PLANES == 2 ? jj : 0, i1 = PLANES == 2 ? jj + 4 : 0;
                        if (jj == 0)
                        {
                            P::mma0(S[0][mb], lo, afrag_lo[jl][ml][i0], afrag_lo[jl][ml][i1]);
                            P::mma0(S[1][mb], hi, afrag[j][mb][jj], afrag[j][mb][jj + 4]);
                        }
                        else
                        {
                            P::mma(S[0][mb], lo, afrag_lo[jl][ml][i0], afrag_lo[jl][ml][i1]);
                            P::mma(S[1][mb], hi, afrag[j][mb][jj], afrag[j][mb][jj + 4]);
                        }
                    }
                }
            }
            // scale, zero and magic-constant correction on the fp32 group sums
            float sA, sB, zA = 0.f, zB = 0.f;
            P::unpack2(s_word, sA, sB);
            if (HAS_ZERO)
                P::unpack2(z_word, zA, zB);
            float const cA = fmaf(-F::CORR, sA, zA), cB = fmaf(-F::CORR, sB, zB);
            float const mA = sA * F::SCALE, mB = sB * F::SCALE;
#pragma unroll
            for (int mb = 0; mb < MB; ++mb)
            {
                acc[mb][0] = fmaf(mA, S[0][mb][0] + S[1][mb][0], fmaf(cA, asum[j][mb][0], acc[mb][0]));
                acc[mb][1] = fmaf(mA, S[0][mb][1] + S[1][mb][1], fmaf(cA, asum[j][mb][1], acc[mb][1]));
                acc[mb][2] = fmaf(mB, S[0][mb][2] + S[1][mb][2], fmaf(cB, asum[j][mb][0], acc[mb][2]));
                acc[mb][3] = fmaf(mB, S[0][mb][3] + S[1][mb][3], fmaf(cB, asum[j][mb][1], acc[mb][3]));
            }
        }
        else
        {
            uint32_t const sA = prmt(s_word, s_word, 0x1010u), sB = prmt(s_word, s_word, 0x3232u);
            uint32_t const zA = prmt(z_word, z_word, 0x1010u), zB = prmt(z_word, z_word, 0x3232u);
#pragma unroll
            for (int jj = 0; jj < 4; ++jj)
            {
                if (BITS == 4)
                {
                    uint32_t qa[4], qb[4];
                    cvt_int4x8<T>(ra[jj], qa);
                    cvt_int4x8<T>(rb[jj], qb);
#pragma unroll
                    for (int p = 0; p < 4; ++p)
                    {
                        qa[p] = HAS_ZERO ? P::fma(qa[p], sA, zA) : P::mul(qa[p], sA);
                        qb[p] = HAS_ZERO ? P::fma(qb[p], sB, zB) : P::mul(qb[p], sB);
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                    {
                        uint32_t const frag[4] = {qa[2 * h], qb[2 * h], qa[2 * h + 1], qb[2 * h + 1]};
#pragma unroll
                        for (int mb = 0; mb < MB; ++mb)
                            P::mma(acc[mb], frag, afrag[j][mb][jj + 8 * h], afrag[j][mb][jj + 8 * h + 4]);
                    }
                }
                else
                {
                    uint32_t qa[2], qb[2];
                    cvt_int8x4<T>(ra[jj], qa);
                    cvt_int8x4<T>(rb[jj], qb);
#pragma unroll
                    for (int p = 0; p < 2; ++p)
                    {
                        qa[p] = HAS_ZERO ? P::fma(qa[p], sA, zA) : P::mul(qa[p], sA);
                        qb[p] = HAS_ZERO ? P::fma(qb[p], sB, zB) : P::mul(qb[p], sB);
                    }
                    uint32_t const frag[4] = {qa[0], qb[0], qa[1], qb[1]};
#pragma unroll
                    for (int mb = 0; mb < MB; ++mb)
                        P::mma(acc[mb], frag, afrag[j][mb][jj], afrag[j][mb][jj + 4]);
                }
            }
        }
    };

    // Activations (and, later, the output) belong to the preceding kernels: wait for them here.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (num_cg > 0)
        load_act(0);

    bool ok = true;
    int slot = 0, use = 0;
    bool first_act = true; // the first activation fragments were loaded above
    for (int cg0 = 0; cg0 < num_cg; cg0 += batch)
    {
        int const nb = min(batch, num_cg - cg0);
        if (RED_ACC)
        {
            for (int panel = 0; panel < num_panels; ++panel)
            {
                if (num_panels > 1 && !first_act)
                    load_act(panel);
                first_act = false;
                for (int cb = 0; cb < nb; ++cb)
                {
                    if (ok)
                        ok = wait_or_abort(&full_bar[slot], use & 1, abort_flag);
                    uint8_t const* tile = ring + size_t(slot) * a.slot_bytes;
#pragma unroll
                    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            acc[0][mb][c] = 0.f;
#pragma unroll
                    for (int j = 0; j < C::UPW; ++j)
                        process_unit(j, cg0 + cb, tile, acc[0]);
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(&empty_bar[slot]);
                    if (++slot == a.num_slots)
                    {
                        slot = 0;
                        ++use;
                    }
                    // every thread owns its entries of the buffer: plain read-modify-write
                    if (t < MT)
                    {
#pragma unroll
                        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
                            for (int c = 0; c < 4; ++c)
                            {
                                float* dst = red + (((cb * kWarps + warp) * MB + mb) * 4 + c) * (8 * MT) + g * MT + t;
                                *dst = panel == 0 ? acc[0][mb][c] : *dst + acc[0][mb][c];
                            }
                    }
                }
            }
        }
        for (int c0 = 0; !RED_ACC && c0 < nb; c0 += cbe)
        {
            int const ncb = min(cbe, nb - c0);
#pragma unroll
            for (int ci = 0; ci < CB; ++ci)
#pragma unroll
                for (int mb = 0; mb < MB; ++mb)
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        acc[ci][mb][c] = 0.f;

            for (int panel = 0; panel < num_panels; ++panel)
            {
                if (num_panels > 1 && !first_act)
                    load_act(panel);
                first_act = false;
#pragma unroll
                for (int ci = 0; ci < CB; ++ci)
                {
                    if (ci >= ncb)
                        break;
                    int const cg = cg0 + c0 + ci;
                    if (ok)
                    {
                        ok = wait_or_abort(&full_bar[slot], use & 1, abort_flag);
                    }
                    uint8_t const* tile = ring + size_t(slot) * a.slot_bytes;
#pragma unroll
                    for (int j = 0; j < C::UPW; ++j)
                        process_unit(j, cg, tile, acc[ci]);
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(&empty_bar[slot]);
                    if (++slot == a.num_slots)
                    {
                        slot = 0;
                        ++use;
                    }
                }
            }
            if (t < MT)
            {
#pragma unroll
                for (int ci = 0; ci < CB; ++ci)
                {
                    if (ci >= ncb)
                        break;
                    int const cb = c0 + ci;
#pragma unroll
                    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            red[(((cb * kWarps + warp) * MB + mb) * 4 + c) * (8 * MT) + g * MT + t] = acc[ci][mb][c];
                }
            }
        }

        // Combine the 16 warps' partial sums in a fixed order and write this batch of columns.
        named_bar_sync(1, kConsumerThreads);
        constexpr int MPAD = 8 * MB;
        for (int o = tid; o < nb * 16 * MPAD; o += kConsumerThreads)
        {
            int const col_in = o & 15, row = (o >> 4) & (MPAD - 1), cb = o / (16 * MPAD);
            int const lg = BITS == 4 ? col_in >> 1 : col_in & 7;
            int const chalf = BITS == 4 ? col_in & 1 : col_in >> 3;
            int const irow = r0 + (cg0 + cb) * C::RPG + col_in / C::IL;
            int const col = (r0 + (cg0 + cb) * C::RPG) * C::IL + col_in;
            uint32_t v16 = 0;
            bool valid = false;
            if (row < a.m && irow < r1)
            {
                int const mb = row >> 3, lt = (row & 7) >> 1, c = chalf * 2 + (row & 1);
                float const* src = red + ((cb * kWarps * MB + mb) * 4 + c) * (8 * MT) + lg * MT + lt;
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < kWarps; ++w)
                    sum += src[w * MB * 4 * 8 * MT];
                float v = a.alpha * sum;
                if (a.bias)
                    v += P::to_float(static_cast<uint16_t const*>(a.bias)[col]);
                v16 = P::from_float(v);
                if (!(PUSH && a.push.gather)) // when gathering, `out` receives the reduced values below
                    static_cast<uint16_t*>(a.out)[size_t(row) * a.n + col] = uint16_t(v16);
                valid = true;
            }
            if (PUSH)
            {
                // Fused all-reduce, first half: four neighbouring lanes hold four neighbouring
                // columns of one row (one interleaved row of this CTA, so all four are valid or none
                // is); the first of them sends them as one flagged 16-byte packet
                // {2 values, call number, 2 values, call number} into its slot of every peer's inbox.
                // (All 32 lanes are here: the loop bound is a multiple of the warp size.)
                uint32_t const pair = v16 | (__shfl_down_sync(0xffffffffu, v16, 1) << 16);
                uint32_t const pair1 = __shfl_down_sync(0xffffffffu, pair, 2);
                if (valid && (col_in & 3) == 0)
                {
                    uint32_t const epoch = *reinterpret_cast<volatile uint32_t const*>(a.push.ws[a.push.rank]) + 1u;
                    size_t const pkt = (size_t(a.push_row0 + row) * a.n + size_t(col)) >> 2;
                    size_t const off = a.push.header_bytes + size_t(epoch & 1u) * a.push.copy_bytes
                        + size_t(a.push.rank) * a.push.pkt_slot + pkt * 16;
                    // (when gathering, the own slot gets a copy too, so that the sum below treats all
                    // ranks alike)
#pragma unroll
                    for (int r = 0; r < W4_MAX_RANKS; ++r)
                        if (r < a.push.world && (r != a.push.rank || a.push.gather))
                            asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(a.push.ws[r] + off),
                                         "r"(pair), "r"(epoch), "r"(pair1), "r"(epoch)
                                         : "memory");
                }
            }
        }
        if (PUSH && a.push.gather)
        {
            // Fused all-reduce, second half: the same lanes poll their packet in every rank's slot of
            // the local inbox (bounded in time), add the values in rank order in fp32 (+ bias) and
            // write the reduced row segment. Every CTA of every rank has pushed before it waits, and
            // all CTAs of a launch are resident (one per SM), so nobody waits for a CTA that cannot run.
            for (int o = tid; o < nb * 16 * MPAD; o += kConsumerThreads)
            {
                int const col_in = o & 15, row = (o >> 4) & (MPAD - 1), cb = o / (16 * MPAD);
                int const irow = r0 + (cg0 + cb) * C::RPG + col_in / C::IL;
                int const col = (r0 + (cg0 + cb) * C::RPG) * C::IL + col_in;
                if (row >= a.m || irow >= r1 || (col_in & 3) != 0)
                    continue;
                uint32_t const epoch = *reinterpret_cast<volatile uint32_t const*>(a.push.ws[a.push.rank]) + 1u;
                size_t const pkt = (size_t(a.push_row0 + row) * a.n + size_t(col)) >> 2;
                uint8_t const* inbox = a.push.ws[a.push.rank] + a.push.header_bytes
                    + size_t(epoch & 1u) * a.push.copy_bytes + pkt * 16;
                uint4 pk[W4_MAX_RANKS];
                unsigned long long t0 = 0;
                bool got = false;
                for (uint32_t polls = 1; !got; ++polls)
                {
                    uint32_t bad = 0;
#pragma unroll
                    for (int r = 0; r < W4_MAX_RANKS; ++r)
                        if (r < a.push.world)
                        {
                            asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                                         : "=r"(pk[r].x), "=r"(pk[r].y), "=r"(pk[r].z), "=r"(pk[r].w)
                                         : "l"(inbox + size_t(r) * a.push.pkt_slot)
                                         : "memory");
                            bad |= (pk[r].y ^ epoch) | (pk[r].w ^ epoch);
                        }
                    got = bad == 0;
                    if (!got && (polls & 15u) == 0)
                    {
                        if (*abort_flag)
                            break;
                        unsigned long long now;
                        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                        if (t0 == 0)
                            t0 = now;
                        else if (now - t0 > a.push.timeout_ns)
                        {
                            *abort_flag = 1;
                            atomicExch(&g_device_status, kDeviceTimeout);
                            break;
                        }
                    }
                }
                if (!got)
                    continue;
                float acc4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int r = 0; r < W4_MAX_RANKS; ++r)
                    if (r < a.push.world)
                    {
                        float lo, hi;
                        P::unpack2(pk[r].x, lo, hi);
                        acc4[0] += lo;
                        acc4[1] += hi;
                        P::unpack2(pk[r].z, lo, hi);
                        acc4[2] += lo;
                        acc4[3] += hi;
                    }
                if (a.push.bias)
                {
                    uint2 const bv = *reinterpret_cast<uint2 const*>(static_cast<uint16_t const*>(a.push.bias) + col);
                    float lo, hi;
                    P::unpack2(bv.x, lo, hi);
                    acc4[0] += lo;
                    acc4[1] += hi;
                    P::unpack2(bv.y, lo, hi);
                    acc4[2] += lo;
                    acc4[3] += hi;
                }
                uint2 o2;
                o2.x = uint32_t(P::from_float(acc4[0])) | (uint32_t(P::from_float(acc4[1])) << 16);
                o2.y = uint32_t(P::from_float(acc4[2])) | (uint32_t(P::from_float(acc4[3])) << 16);
                *reinterpret_cast<uint2*>(static_cast<uint16_t*>(a.out) + size_t(row) * a.n + col) = o2;
            }
        }
        if (cg0 + batch < num_cg)
            named_bar_sync(1, kConsumerThreads);
    }
    if (PUSH && a.push.gather)
    {
        // This launch was a whole all-reduce call: the last CTA to get here advances the workspace's
        // call number (every CTA has read it before it takes its ticket; the next call is a later
        // kernel on the stream).
        named_bar_sync(1, kConsumerThreads);
        if (tid == 0)
        {
            uint32_t* ctrl = reinterpret_cast<uint32_t*>(a.push.ws[a.push.rank]);
            uint32_t const epoch = *reinterpret_cast<volatile uint32_t*>(ctrl) + 1u;
            if (atomicAdd(ctrl + 1, 1u) == gridDim.x - 1u)
            {
                ctrl[1] = 0u;
                *reinterpret_cast<volatile uint32_t*>(ctrl) = epoch;
            }
        }
    }
}

} // namespace gemv
} // namespace w4

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
namespace w4
{
namespace gemv
{

template <typename T, int BITS, int MB, bool HAS_ZERO, bool HAS_ACT_SCALE, bool FOLD, int CB, bool PUSH>
static int launch_one(Args const& a, DeviceInfo const& dev, cudaStream_t stream)
{
    using C = Cfg<BITS, MB>;
    auto kernel = gemv_kernel<T, BITS, MB, HAS_ZERO, HAS_ACT_SCALE, FOLD, CB, PUSH>;
    Args args = a;
    args.groups_per_panel = a.group_shift >= 31 ? 1 : C::KP >> a.group_shift;
    args.box_stride = (args.groups_per_panel * kScaleBoxCols * 2 + 127) & ~127;
    args.slot_bytes = (C::TILE_BYTES + 2 * args.box_stride + 1023) & ~1023;
    // 64 KB of partial sums (8 column groups at 8 rows, 32 at one): every reduction is a CTA-wide
    // barrier, and fewer of them measured faster than the two ring slots this costs (four slots
    // remain; ~72 KB are in flight at a time anyway).
    args.red_bytes = MB == 2 ? kRedBytes16 : kRedBytes;
    size_t const fixed = size_t(args.red_bytes) + 64 + 1024; // + slack to start the ring on a 1024-byte boundary
    // Shared memory per CTA: all a block may have.
    size_t const smem_budget = size_t(dev.max_smem_optin);
    int slots = int((smem_budget - fixed) / (args.slot_bytes + 16));
    if (slots < 2)
        return W4_ERR_CUDA;
    if (slots > 12)
        slots = 12;
    args.num_slots = slots;
    // Tiles in flight ahead of the consumers: about 72 KB per SM covers the HBM latency-bandwidth
    // product with margin.
    int depth = (72 * 1024 + args.slot_bytes / 2) / args.slot_bytes;
    args.depth = depth < 1 ? 1 : (depth > slots - 1 ? slots - 1 : depth);
    size_t const smem = size_t(slots) * args.slot_bytes + fixed + size_t(slots) * 16;

    // Scale / zero tensors as 2-D maps [groups, n]; every tile fetches a box of its panel's group
    // rows x kScaleBoxCols columns.
    CUtensorMap tm_scales, tm_zeros;
    uint64_t const groups = uint64_t(a.num_groups);
    if (!make_tensor_map_2d(&tm_scales, CU_TENSOR_MAP_DATA_TYPE_UINT16, a.scales, uint64_t(a.n), groups,
            uint64_t(a.n) * 2, kScaleBoxCols, uint32_t(args.groups_per_panel), CU_TENSOR_MAP_SWIZZLE_NONE))
        return W4_ERR_CUDA;
    tm_zeros = tm_scales;
    if (HAS_ZERO
        && !make_tensor_map_2d(&tm_zeros, CU_TENSOR_MAP_DATA_TYPE_UINT16, a.zeros, uint64_t(a.n), groups,
            uint64_t(a.n) * 2, kScaleBoxCols, uint32_t(args.groups_per_panel), CU_TENSOR_MAP_SWIZZLE_NONE))
        return W4_ERR_CUDA;
    // int4 weights with several k panels as [lines, 128 bytes]; box = the lines of one row's panel.
    CUtensorMap tm_w = tm_scales;
    if (BITS == 4 && a.k > C::KP)
    {
        uint64_t const lpr = uint64_t(a.k) >> 6;
        uint32_t const box_lines = uint32_t(C::KP >> 6); // used with several k panels only
        if (!make_tensor_map_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.weight, 128, uint64_t(args.num_rows) * lpr, 128, 128,
                box_lines, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B))
            return W4_ERR_CUDA;
    }

    // The opt-in shared-memory limit is a per-function, per-device attribute: set it once.
    {
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
    int const grid = args.num_rows < dev.num_sms ? args.num_rows : dev.num_sms;
    {
        // the kernel's tile counter is 16 bits wide
        long const rows_per_cta = (args.num_rows + grid - 1) / grid;
        long const tiles_per_cta = ((rows_per_cta + C::RPG - 1) / C::RPG + 1) * ((a.k + C::KP - 1) / C::KP);
        if (tiles_per_cta > 60000)
            return W4_ERR_BAD_SHAPE;
    }
    // Launched as a programmatic dependent of whatever precedes it in the stream (the kernel
    // orders itself with griddepcontrol.wait).
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
    if (cudaLaunchKernelEx(&cfg, kernel, args, tm_scales, tm_zeros, tm_w) != cudaSuccess)
        return W4_ERR_CUDA;
    return cudaGetLastError() == cudaSuccess ? W4_OK : W4_ERR_CUDA;
}

template <typename T, int BITS, int MB, bool FOLD, int CB, bool PUSH>
static int dispatch_inputs(Args const& a, DeviceInfo const& dev, cudaStream_t stream)
{
    bool const z = a.zeros != nullptr, s = a.act_scale != nullptr;
    if (z && s)
        return launch_one<T, BITS, MB, true, true, FOLD, CB, PUSH>(a, dev, stream);
    if (z)
        return launch_one<T, BITS, MB, true, false, FOLD, CB, PUSH>(a, dev, stream);
    if (s)
        return launch_one<T, BITS, MB, false, true, FOLD, CB, PUSH>(a, dev, stream);
    return launch_one<T, BITS, MB, false, false, FOLD, CB, PUSH>(a, dev, stream);
}

// The epilogue that sends the results to the peers (and may collect theirs) is an instantiation of
// its own, int4 only: compiled into the ordinary kernel it cost that kernel 10 % (11.2 against
// 10.0 us on a 4096 x 14336 matrix) although it never ran.
template <typename T, int BITS, int MB, bool FOLD, int CB>
static int dispatch_flags(Args const& a, DeviceInfo const& dev, cudaStream_t stream)
{
    if constexpr (BITS == 4)
    {
        if (a.push.world > 0)
            return dispatch_inputs<T, BITS, MB, FOLD, CB, true>(a, dev, stream);
    }
    return dispatch_inputs<T, BITS, MB, FOLD, CB, false>(a, dev, stream);
}

// 8-row passes: with more than one k panel the column groups are walked in sub-batches of 4 that
// share each activation load and keep their sums in registers, or, when a CTA has more than 4 of
// them, accumulate in shared memory like the 16-row passes; with a single panel there is nothing
// to share. 16-row passes hold half as much k per panel (their activation fragments are twice as
// large), so they always accumulate in shared memory and load the activations once per panel for all
// the column groups of a reduction batch.
template <typename T, int BITS, int MB, bool FOLD>
static int dispatch_panels(Args const& a, DeviceInfo const& dev, cudaStream_t stream)
{
    if constexpr (MB == 2)
        return dispatch_flags<T, BITS, MB, FOLD, 0>(a, dev, stream);
    else
    {
        if (a.k > Cfg<BITS, MB>::KP)
        {
            // more column groups per CTA than one register sub-batch holds: accumulate in shared
            // memory instead, and load the activations once per panel for all of them (8192 x 57344
            // int4, m = 1: 60.0 -> 54.1 us; with two groups per CTA the register form is the faster)
            int const ctas = a.num_rows < dev.num_sms ? a.num_rows : dev.num_sms;
            int const groups = (a.num_rows + Cfg<BITS, MB>::RPG - 1) / Cfg<BITS, MB>::RPG;
            if (groups > 4 * ctas)
                return dispatch_flags<T, BITS, MB, FOLD, 0>(a, dev, stream);
            return dispatch_flags<T, BITS, MB, FOLD, 4>(a, dev, stream);
        }
        return dispatch_flags<T, BITS, MB, FOLD, 1>(a, dev, stream);
    }
}

template <typename T>
static int dispatch_bits(Args const& a, int bits, int mb, DeviceInfo const& dev, cudaStream_t stream)
{
    if (bits == 4)
    {
        // A warp unit spans 128 k for int4: the folded arithmetic needs one scale group per unit.
        bool const fold = a.group_shift >= 7;
        if (mb == 2)
            return fold ? dispatch_panels<T, 4, 2, true>(a, dev, stream) : dispatch_panels<T, 4, 2, false>(a, dev, stream);
        return fold ? dispatch_panels<T, 4, 1, true>(a, dev, stream) : dispatch_panels<T, 4, 1, false>(a, dev, stream);
    }
    return mb == 2 ? dispatch_panels<T, 8, 2, true>(a, dev, stream) : dispatch_panels<T, 8, 1, true>(a, dev, stream);
}

} // namespace gemv

int launch_gemv(W4GemmParams const& p, cudaStream_t stream, PushTarget const* push)
{
    DeviceInfo const& dev = current_device_info();
    if (dev.num_sms <= 0)
        return W4_ERR_CUDA;
    size_t const elt = 2;
    // Passes over the weights: 16 rows at a time (two B fragments per weight fragment) while more
    // than 8 rows are left, then one pass of up to 8.
    for (int m0 = 0; m0 < p.m;)
    {
        int const left = p.m - m0;
        int const mb = left > 8 ? 2 : 1;
        int const rows = left < 8 * mb ? left : 8 * mb;
        gemv::Args a{};
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
        a.num_groups = p.group_size ? p.k / p.group_size : 1;
        a.num_rows = p.n / (p.weight_bits == 4 ? 4 : 2);
        a.weights_static = (p.flags & W4_GEMM_WEIGHTS_STATIC) ? 1 : 0;
        if (push && p.weight_bits == 4)
        {
            a.push = *push;
            // rows of a later pass land further down in the peers' inboxes: packet index counts from
            // the first row of the whole call
            a.push_row0 = m0;
        }
        int const rc = p.act_dtype == W4_DTYPE_FP16 ? gemv::dispatch_bits<__half>(a, p.weight_bits, mb, dev, stream)
                                                    : gemv::dispatch_bits<__nv_bfloat16>(a, p.weight_bits, mb, dev, stream);
        if (rc != W4_OK)
            return rc;
        m0 += rows;
    }
    return W4_OK;
}

} // namespace w4
