// Decode-regime kernel (m = 1..16 per pass): streams the packed int4/int8 weights exactly once.
//
// Replaces weight_only::kernel of the reference project
// (cpp/tensorrt_llm/kernels/weightOnlyBatchedGemv/kernel.h:31-120) and, for m >= 5 / m >= 16, the
// small-M CUTLASS tactics it falls back to. Same math: the dequantised weight is
// round_T(fma(q, scale, zero)) (utility.h:157-162), the pre-quant scale product is rounded to T
// (utility.h:116), alpha * acc + bias is formed in fp32 (utility.h:256-266). Unlike the reference
// the dot product itself is accumulated in fp32.
//
// Design (B200): one persistent CTA per SM owns a contiguous range of "interleaved rows" of the
// preprocessed weight (one interleaved row = IL adjacent output columns x all of K = 2K bytes, see
// below), so every CTA streams one contiguous slab of HBM. A producer warp moves that slab into a
// shared-memory ring with bulk (TMA-engine) copies, hundreds of KB in flight per SM from the first
// cycle; 16 consumer warps split K, pull 16-byte chunks out of the ring with 128-bit shared loads,
// convert and dequantise in registers and feed mma.sync (weights as the 16-row A operand, the m <= 8
// activation rows as the 8-column B operand), accumulating in fp32. Partial sums of the 16 warps
// are combined through shared memory in a fixed order (deterministic), then alpha/bias are applied
// and the result stored.
//
// Weight layout consumed (preprocess_weights_for_mixed_gemm on sm_100,
// cpp/tensorrt_llm/kernels/cutlass_kernels/cutlass_preprocessors.cpp:564-615): interleaved row R
// holds columns IL*R .. IL*R+IL-1 (IL = 4 for int4, 2 for int8); inside it every 128-byte line is
// one 64-wide k tile, split into IL column segments; every aligned 16-byte chunk holds CK = 32
// (int4) / 16 (int8) consecutive k of one column in the order
// { 2j+8q+e : register j = 0..3, pair q, element e }, with the nibbles/bytes of each 32-bit
// register pre-shuffled for the converters in w4_common.cuh. Because a dot product does not care
// about the order of k, each thread treats the chunk it loaded as its own mma fragment and the
// activation fragment is simply loaded in the matching order.
#include "w4_common.cuh"
#include "w4_internal.h"

namespace w4
{

namespace gemv
{

constexpr int kWarps = 16;                       // consumer warps
constexpr int kConsumerThreads = kWarps * 32;    // 512
constexpr int kThreads = kConsumerThreads + 32;  // + producer warp

template <int BITS, int MB>
struct Cfg
{
    static constexpr int IL = BITS == 4 ? 4 : 2;        // columns per interleaved row
    static constexpr int RPG = 16 / IL;                 // interleaved rows per 16-column group
    static constexpr int CK = 128 / BITS;               // k values in one 16-byte chunk
    static constexpr int UK = 4 * CK;                   // k values per warp unit (4 chunks)
    static constexpr int UPW = MB == 1 ? 2 : 1;         // units per warp per tile
    static constexpr int KP = kWarps * UPW * UK;        // k panel covered by one tile
    static constexpr int ROW_STRIDE = 2 * KP;           // bytes of one interleaved row inside a tile
    static constexpr int TILE_BYTES = RPG * ROW_STRIDE; // 32 KB (MB = 1) or 16 KB (MB = 2)
    static constexpr int AREGS = CK / 2;                // activation pair registers per chunk
    static constexpr int RED_FLOATS = 2 * kWarps * MB * 4 * 32;
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
    int m; // rows handled by this launch (<= 8 * MB)
    int n;
    int k;
    int group; // group size; k for per-channel
    int num_rows; // n / IL
    int num_slots;
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

template <typename T, int BITS, int MB, bool HAS_ZERO, bool HAS_ACT_SCALE>
__global__ void __launch_bounds__(kThreads, 1) gemv_kernel(Args const a)
{
    using C = Cfg<BITS, MB>;
    using P = Pair<T>;
    extern __shared__ __align__(128) uint8_t smem[];

    uint8_t* ring = smem;
    float* red = reinterpret_cast<float*>(smem + size_t(a.num_slots) * C::TILE_BYTES);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(red + C::RED_FLOATS);
    uint64_t* empty_bar = full_bar + a.num_slots;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + a.num_slots);

    int const tid = threadIdx.x;
    int const warp = tid >> 5, lane = tid & 31;

    // Row range of this CTA (balanced to within one interleaved row).
    int const r0 = int((int64_t(a.num_rows) * blockIdx.x) / gridDim.x);
    int const r1 = int((int64_t(a.num_rows) * (blockIdx.x + 1)) / gridDim.x);
    int const num_cg = (r1 - r0 + C::RPG - 1) / C::RPG;
    int const num_panels = (a.k + C::KP - 1) / C::KP;
    int const num_tiles = num_cg * num_panels;
    size_t const row_bytes = size_t(2) * a.k;

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
    __syncthreads();

    if (warp == kWarps)
    {
        // ------------------------------------------------------------------ producer
        if (lane == 0)
        {
            for (int i = 0; i < num_tiles; ++i)
            {
                int const slot = i % a.num_slots, use = i / a.num_slots;
                if (use > 0 && !wait_or_abort(&empty_bar[slot], (use - 1) & 1, abort_flag))
                    break;
                int const cg = i / num_panels, panel = i - cg * num_panels;
                int const row_first = r0 + cg * C::RPG;
                int const rows = min(C::RPG, r1 - row_first);
                int const kp_len = min(C::KP, a.k - panel * C::KP);
                uint32_t const bytes = 2u * kp_len;
                mbar_expect_tx(&full_bar[slot], bytes * rows);
                uint8_t* dst = ring + size_t(slot) * C::TILE_BYTES;
                uint8_t const* src = a.weight + size_t(row_first) * row_bytes + size_t(panel) * C::ROW_STRIDE;
                for (int r = 0; r < rows; ++r)
                    bulk_g2s(dst + r * C::ROW_STRIDE, src + r * row_bytes, bytes, &full_bar[slot]);
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumers
    int const g = lane >> 2, t = lane & 3;
    // Columns (inside a 16-column group) behind logical mma rows g and g + 8, and where their
    // 16-byte chunks sit inside a tile. int4: adjacent columns (one 32-bit scale load serves
    // both); int8: columns g and g + 8, which makes every 8-lane phase of the shared load read one
    // whole 128-byte line.
    int const colA = BITS == 4 ? 2 * g : g;
    int const colB = BITS == 4 ? 2 * g + 1 : 8 + g;
    int const segA = (colA / C::IL) * C::ROW_STRIDE + (colA % C::IL) * (128 / C::IL);
    int const segB = (colB / C::IL) * C::ROW_STRIDE + (colB % C::IL) * (128 / C::IL);

    uint16_t const* scales = static_cast<uint16_t const*>(a.scales);
    uint16_t const* zeros = static_cast<uint16_t const*>(a.zeros);
    T const* act = static_cast<T const*>(a.act);
    T const* act_scale = static_cast<T const*>(a.act_scale);

    uint32_t afrag[C::UPW][MB][C::AREGS];
    uint32_t s_cur[C::UPW], z_cur[C::UPW], s_nxt[C::UPW], z_nxt[C::UPW];

    // (scale, zero) words of this thread's two columns for tile i: low half = column A.
    auto load_scales = [&](int i, uint32_t(&s)[C::UPW], uint32_t(&z)[C::UPW])
    {
        int const cg = i / num_panels, panel = i - cg * num_panels;
        int const col_base = (r0 + cg * C::RPG) * C::IL;
        bool const va = (r0 + cg * C::RPG + colA / C::IL) < r1;
        bool const vb = (r0 + cg * C::RPG + colB / C::IL) < r1;
#pragma unroll
        for (int j = 0; j < C::UPW; ++j)
        {
            int const k0 = panel * C::KP + (j * kWarps + warp) * C::UK + t * C::CK;
            s[j] = 0;
            z[j] = 0;
            if (k0 < a.k)
            {
                size_t const base = size_t(k0 / a.group) * a.n + col_base;
                if (BITS == 4)
                {
                    if (va) // columns A and B share an interleaved row for int4
                    {
                        s[j] = __ldg(reinterpret_cast<uint32_t const*>(scales + base + colA));
                        if (HAS_ZERO)
                            z[j] = __ldg(reinterpret_cast<uint32_t const*>(zeros + base + colA));
                    }
                }
                else
                {
                    uint32_t sa = va ? __ldg(scales + base + colA) : 0u;
                    uint32_t sb = vb ? __ldg(scales + base + colB) : 0u;
                    s[j] = sa | (sb << 16);
                    if (HAS_ZERO)
                    {
                        uint32_t za = va ? __ldg(zeros + base + colA) : 0u;
                        uint32_t zb = vb ? __ldg(zeros + base + colB) : 0u;
                        z[j] = za | (zb << 16);
                    }
                }
            }
        }
    };

    // Activation fragments of this warp's units for one k panel, in chunk order.
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
            }
        }
    };

    if (num_tiles > 0)
    {
        load_scales(0, s_nxt, z_nxt);
        load_act(0);
    }

    bool ok = true;
    int i = 0;
    for (int cg = 0; cg < num_cg; ++cg)
    {
        float acc[MB][4];
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int c = 0; c < 4; ++c)
                acc[mb][c] = 0.f;

        for (int panel = 0; panel < num_panels; ++panel, ++i)
        {
#pragma unroll
            for (int j = 0; j < C::UPW; ++j)
            {
                s_cur[j] = s_nxt[j];
                z_cur[j] = z_nxt[j];
            }
            if (i + 1 < num_tiles)
                load_scales(i + 1, s_nxt, z_nxt);
            if (num_panels > 1 && i > 0)
                load_act(panel);

            int const slot = i % a.num_slots, use = i / a.num_slots;
            if (ok)
                ok = wait_or_abort(&full_bar[slot], use & 1, abort_flag);
            uint8_t const* tile = ring + size_t(slot) * C::TILE_BYTES;

#pragma unroll
            for (int j = 0; j < C::UPW; ++j)
            {
                // Chunk of this thread inside the row piece: k offset kk -> 128-byte line kk/64,
                // 16-byte slot (kk%64)/CK inside the column segment.
                int const kk = (j * kWarps + warp) * C::UK + t * C::CK;
                int const off = (kk >> 6) * 128 + ((kk & 63) / C::CK) * 16;
                uint4 const wa = *reinterpret_cast<uint4 const*>(tile + segA + off);
                uint4 const wb = *reinterpret_cast<uint4 const*>(tile + segB + off);
                uint32_t const ra[4] = {wa.x, wa.y, wa.z, wa.w};
                uint32_t const rb[4] = {wb.x, wb.y, wb.z, wb.w};
                uint32_t const sA = prmt(s_cur[j], s_cur[j], 0x1010u), sB = prmt(s_cur[j], s_cur[j], 0x3232u);
                uint32_t const zA = prmt(z_cur[j], z_cur[j], 0x1010u), zB = prmt(z_cur[j], z_cur[j], 0x3232u);
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
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&empty_bar[slot]);
        }

        // Combine the 16 warps' partial sums (fixed order) and write this column group.
        float* buf = red + (cg & 1) * (C::RED_FLOATS / 2);
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int c = 0; c < 4; ++c)
                buf[((warp * MB + mb) * 4 + c) * 32 + lane] = acc[mb][c];
        named_bar_sync(1, kConsumerThreads);
        if (tid < 128 * MB)
        {
            int const mb = tid >> 7, c = (tid >> 5) & 3, l = tid & 31;
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w)
                sum += buf[((w * MB + mb) * 4 + c) * 32 + l];
            int const lg = l >> 2, lt = l & 3;
            int const col_in = (c < 2) ? (BITS == 4 ? 2 * lg : lg) : (BITS == 4 ? 2 * lg + 1 : 8 + lg);
            int const row = mb * 8 + 2 * lt + (c & 1);
            int const irow = r0 + cg * C::RPG + col_in / C::IL;
            if (row < a.m && irow < r1)
            {
                int const col = (r0 + cg * C::RPG) * C::IL + col_in;
                float v = a.alpha * sum;
                if (a.bias)
                    v += P::to_float(static_cast<uint16_t const*>(a.bias)[col]);
                static_cast<uint16_t*>(a.out)[size_t(row) * a.n + col] = P::from_float(v);
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

template <typename T, int BITS, int MB, bool HAS_ZERO, bool HAS_ACT_SCALE>
static int launch_one(Args const& a, DeviceInfo const& dev, cudaStream_t stream)
{
    using C = Cfg<BITS, MB>;
    auto kernel = gemv_kernel<T, BITS, MB, HAS_ZERO, HAS_ACT_SCALE>;
    size_t const fixed = C::RED_FLOATS * sizeof(float) + 64;
    int slots = int((size_t(dev.max_smem_optin) - fixed) / (C::TILE_BYTES + 16));
    if (slots < 2)
        return W4_ERR_CUDA;
    if (slots > 12)
        slots = 12;
    size_t const smem = size_t(slots) * C::TILE_BYTES + fixed + size_t(slots) * 16;

    // The opt-in shared-memory limit is a per-function, per-device attribute: set it once.
    static bool configured[64] = {};
    if (dev.device < 0 || dev.device >= 64 || !configured[dev.device])
    {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dev.max_smem_optin)
            != cudaSuccess)
            return W4_ERR_CUDA;
        if (dev.device >= 0 && dev.device < 64)
            configured[dev.device] = true;
    }
    Args args = a;
    args.num_slots = slots;
    int const grid = args.num_rows < dev.num_sms ? args.num_rows : dev.num_sms;
    kernel<<<grid, kThreads, smem, stream>>>(args);
    return cudaGetLastError() == cudaSuccess ? W4_OK : W4_ERR_CUDA;
}

template <typename T, int BITS, int MB>
static int dispatch_flags(Args const& a, DeviceInfo const& dev, cudaStream_t stream)
{
    bool const z = a.zeros != nullptr, s = a.act_scale != nullptr;
    if (z && s)
        return launch_one<T, BITS, MB, true, true>(a, dev, stream);
    if (z)
        return launch_one<T, BITS, MB, true, false>(a, dev, stream);
    if (s)
        return launch_one<T, BITS, MB, false, true>(a, dev, stream);
    return launch_one<T, BITS, MB, false, false>(a, dev, stream);
}

template <typename T>
static int dispatch_bits(Args const& a, int bits, int mb, DeviceInfo const& dev, cudaStream_t stream)
{
    if (bits == 4)
        return mb == 1 ? dispatch_flags<T, 4, 1>(a, dev, stream) : dispatch_flags<T, 4, 2>(a, dev, stream);
    return mb == 1 ? dispatch_flags<T, 8, 1>(a, dev, stream) : dispatch_flags<T, 8, 2>(a, dev, stream);
}

} // namespace gemv

int launch_gemv(W4GemmParams const& p, cudaStream_t stream)
{
    DeviceInfo const& dev = current_device_info();
    if (dev.num_sms <= 0)
        return W4_ERR_CUDA;
    size_t const elt = 2;
    for (int m0 = 0; m0 < p.m; m0 += 16)
    {
        int const rows = p.m - m0 < 16 ? p.m - m0 : 16;
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
        a.group = p.group_size ? p.group_size : p.k;
        a.num_rows = p.n / (p.weight_bits == 4 ? 4 : 2);
        int const mb = rows <= 8 ? 1 : 2;
        int const rc = p.act_dtype == W4_DTYPE_FP16 ? gemv::dispatch_bits<__half>(a, p.weight_bits, mb, dev, stream)
                                                    : gemv::dispatch_bits<__nv_bfloat16>(a, p.weight_bits, mb, dev, stream);
        if (rc != W4_OK)
            return rc;
    }
    return W4_OK;
}

} // namespace w4
