// Device-side weight preparation: per-column symmetric quantisation and the layout transform the
// GEMM kernels consume, as CUDA kernels. The reference project does both on one CPU thread
// (cpp/tensorrt_llm/kernels/cutlass_kernels/cutlass_preprocessors.cpp:564-615 and 652-762); the
// bytes produced here are identical to its output on compute capability 10.x (and to the host
// functions w4_preprocess_weights / w4_symmetric_quantize of this library).
//
// HBM-bound byte work. One CTA turns a tile of 64 k rows x 256 input bytes (512 int4 or 256 int8
// columns) into 128 output lines of 128 bytes: the rows are read with coalesced 16-byte loads into
// shared memory; a thread then reads the 8 (int4) / 4 (int8) rows behind one output register as
// 32-bit words, transposes the block of elements in registers and owns that register of 8 / 4
// adjacent columns - the closed form of the four reference passes (row permutation inside 16/32-row
// blocks, sub-byte transpose, column interleave in 64-k tiles, bias + in-register shuffle).
#include <algorithm>

#include "w4_common.cuh"
#include "w4_internal.h"

namespace w4
{
namespace prep
{

constexpr int kTileK = 64;        // rows per tile: one interleave tile
constexpr int kTileBytes = 256;   // input bytes per row per tile
constexpr int kThreads = 256;
constexpr int kSmemPitch = kTileBytes + 16; // padded row pitch of the staged tile

// The reference's row permutations inside blocks of 16 (int8) / 32 (int4) rows,
//   {0, 1, 8, 9, 2, 3, 10, 11, 4, 5, 12, 13, 6, 7, 14, 15} and
//   {0, 1, 8, 9, 16, 17, 24, 25, 2, 3, 10, 11, 18, 19, 26, 27, 4, 5, ..., 22, 23, 30, 31},
// are used in closed form: perm[a * E + s] = 2 * a + 8 * (s / 2) + s % 2 for a = 0..3, s = 0..E-1
// (E = 4 / 8 elements per 32-bit register).

// Transposes in registers: w[d] holds element c of row d at position c; afterwards w[c] holds
// element d of column c at position d. int4: 8 x 8 nibbles (16-bit halves, bytes, then nibbles are
// exchanged between register pairs), int8: 4 x 4 bytes.
__device__ __forceinline__ void transpose_nibbles(uint32_t (&w)[8])
{
#pragma unroll
    for (int d = 0; d < 4; ++d)
    {
        uint32_t const a = w[d], b = w[d + 4];
        w[d] = __byte_perm(a, b, 0x5410);
        w[d + 4] = __byte_perm(a, b, 0x7632);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
    {
        int const d = (i & 1) + 4 * (i >> 1); // 0, 1, 4, 5
        uint32_t const a = w[d], b = w[d + 2];
        w[d] = __byte_perm(a, b, 0x6240);
        w[d + 2] = __byte_perm(a, b, 0x7351);
    }
#pragma unroll
    for (int d = 0; d < 8; d += 2)
    {
        uint32_t const a = w[d], b = w[d + 1];
        w[d] = (a & 0x0F0F0F0Fu) | ((b & 0x0F0F0F0Fu) << 4);
        w[d + 1] = ((a >> 4) & 0x0F0F0F0Fu) | (b & 0xF0F0F0F0u);
    }
}

__device__ __forceinline__ void transpose_bytes(uint32_t (&w)[4])
{
#pragma unroll
    for (int d = 0; d < 2; ++d)
    {
        uint32_t const a = w[d], b = w[d + 2];
        w[d] = __byte_perm(a, b, 0x5410);
        w[d + 2] = __byte_perm(a, b, 0x7632);
    }
#pragma unroll
    for (int d = 0; d < 4; d += 2)
    {
        uint32_t const a = w[d], b = w[d + 1];
        w[d] = __byte_perm(a, b, 0x6240);
        w[d + 1] = __byte_perm(a, b, 0x7351);
    }
}

// Output stage shared by both kernels: `tile` holds 64 rows of two's-complement weights (int4: two
// per byte, even column in the low nibble) for `cols` columns starting at column n0.
// A 32-bit word of the staged tile holds E = 8 (int4) / 4 (int8) adjacent columns of one row, an
// output register E rows of one column. A thread therefore takes the E rows behind register vr -
// in the register's element order - of one word position, transposes the E x E block in registers
// and owns E finished output registers (register vr of E adjacent columns); the bias (+8 / +128
// on two's complement) is one XOR per register. Lanes run over vr first, so a store instruction
// writes runs of VT consecutive registers.
template <int BITS>
__device__ __forceinline__ void emit_tile(uint32_t* out, uint8_t const* tile, int k_tile, int n0, int cols, int K)
{
    constexpr int E = 32 / BITS;           // elements per 32-bit register
    constexpr int VT = 64 / E;             // registers per 64-k tile of one column
    constexpr int IL = BITS == 8 ? 2 : 4;  // interleaved columns
    constexpr int GP = BITS == 8 ? 16 : 32;
    constexpr uint32_t kBias = BITS == 8 ? 0x80808080u : 0x88888888u;
    size_t const regs_per_irow = size_t(K / E) * IL;
    int const words = cols / E; // staged words per row (cols is a multiple of 32)
    for (int item = threadIdx.x; item < words * VT; item += kThreads)
    {
        int const vr = item % VT, wq = item / VT;
        uint32_t w[E];
#pragma unroll
        for (int d = 0; d < E; ++d)
        {
            // position d of the register holds source element s of the permuted column; the row of the
            // tile behind position kp = vr * E + s of it: both of the reference's permutations (blocks
            // of 16 / 32 rows) satisfy perm[(vr % 4) * E + s] = 2 * (vr % 4) + 8 * (s / 2) + s % 2
            int const s = BITS == 4 ? (d < 4 ? 2 * d : 2 * (d - 4) + 1) : (d == 1 ? 2 : (d == 2 ? 1 : d));
            int const kl = GP * (vr >> 2) + 2 * (vr & 3) + 8 * (s >> 1) + (s & 1);
            w[d] = *reinterpret_cast<uint32_t const*>(tile + kl * kSmemPitch + wq * 4);
        }
        if constexpr (BITS == 4)
            transpose_nibbles(w);
        else
            transpose_bytes(w);
#pragma unroll
        for (int c = 0; c < E; ++c)
        {
            int const nl = wq * E + c; // column inside the tile
            size_t const irow = size_t(n0 / IL + nl / IL);
            out[irow * regs_per_irow + size_t(k_tile) * 32 + (nl % IL) * VT + vr] = w[c] ^ kBias;
        }
    }
}

template <int BITS>
__global__ void __launch_bounds__(kThreads) preprocess_kernel(uint32_t* out, uint8_t const* in, int K, int N)
{
    __shared__ __align__(16) uint8_t tile[kTileK * kSmemPitch];
    int const row_bytes = N * BITS / 8;
    int const b0 = blockIdx.x * kTileBytes;
    int const nbytes = min(kTileBytes, row_bytes - b0);
    int const k_tile = blockIdx.y;
    // 64 rows x nbytes, 16 bytes per thread and step (row_bytes is a multiple of 32)
    for (int i = threadIdx.x; i < kTileK * (kTileBytes / 16); i += kThreads)
    {
        int const r = i / (kTileBytes / 16), c = (i % (kTileBytes / 16)) * 16;
        if (c < nbytes)
            *reinterpret_cast<uint4*>(tile + r * kSmemPitch + c)
                = *reinterpret_cast<uint4 const*>(in + size_t(k_tile * kTileK + r) * row_bytes + b0 + c);
    }
    __syncthreads();
    emit_tile<BITS>(out, tile, k_tile, b0 * 8 / BITS, nbytes * 8 / BITS, K);
}

// W4A8-layout registers (the reference's layout for fp8 activations, cutlass_preprocessors.cpp:114-116,
// 175-179 of the TensorRT-LLM tree: two interleaved columns, 128-row tiles, rows of a 32-block in the
// order {0..3, 16..19, 4..7, 20..23, ...}) -> the W4A16 registers the GEMM kernels consume. Both hold
// biased nibbles, so this is a pure permutation: one thread per output register gathers its eight
// nibbles from the two source registers that hold them (same column, same 32-row block) and a warp
// writes one whole 128-byte line.
__global__ void __launch_bounds__(kThreads) relayout_w4a8_kernel(uint32_t* out, uint32_t const* in, int K, int N)
{
    size_t const total = size_t(K) * size_t(N) / 8;
    size_t const regs_per_irow16 = size_t(K) / 2; // four columns of K / 8 registers
    size_t const regs_per_irow8 = size_t(K) / 4;  // two columns
    for (size_t reg = size_t(blockIdx.x) * kThreads + threadIdx.x; reg < total; reg += size_t(gridDim.x) * kThreads)
    {
        size_t const irow = reg / regs_per_irow16;
        int const vwr = int(reg - irow * regs_per_irow16);
        int const within = vwr & 31;
        int const n = int(irow) * 4 + (within >> 3);
        int const vr = (vwr >> 5) * 8 + (within & 7); // register of column n, counted over all of K
        uint32_t const* src = in + size_t(n >> 1) * regs_per_irow8 + 16 * (n & 1);
        uint32_t word = 0;
#pragma unroll
        for (int d = 0; d < 8; ++d)
        {
            int const s = d < 4 ? 2 * d : 2 * (d - 4) + 1;
            int const kp = vr * 8 + s;
            int const k = (kp & ~31) + 2 * (vr & 3) + 8 * (s >> 1) + (s & 1); // the int4 row permutation, closed form
            // position of row k in the W4A8 order: the inverse of its 32-row permutation in closed form
            int const k8 = (k & ~31) + ((k >> 2) & 3) * 8 + ((k >> 4) & 1) * 4 + (k & 3);
            int const e = k8 & 7;
            int const dd = (e & 1) ? 4 + (e >> 1) : e >> 1;
            uint32_t const w = __ldg(src + 32 * (k8 >> 7) + ((k8 & 127) >> 3));
            word |= ((w >> (4 * dd)) & 0xFu) << (4 * d);
        }
        out[reg] = word;
    }
}

// amax -> scale = amax * 2^-(bits-1), in place, plus the copy rounded to the activation type.
__global__ void finish_scales_kernel(float* scales, void* scales_t, int scales_dtype, int N, float range)
{
    int const c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= N)
        return;
    float const s = scales[c] * range;
    scales[c] = s;
    if (scales_t)
    {
        if (scales_dtype == W4_DTYPE_FP16)
            static_cast<__half*>(scales_t)[c] = __float2half_rn(s);
        else
            static_cast<__nv_bfloat16*>(scales_t)[c] = __float2bfloat16_rn(s);
    }
}

// Eight consecutive weights of one row as floats (one or two 16-byte loads).
template <typename W>
__device__ __forceinline__ void load8(W const* p, float (&x)[8]);
template <>
__device__ __forceinline__ void load8<float>(float const* p, float (&x)[8])
{
    float4 const a = __ldg(reinterpret_cast<float4 const*>(p)), b = __ldg(reinterpret_cast<float4 const*>(p) + 1);
    x[0] = a.x, x[1] = a.y, x[2] = a.z, x[3] = a.w, x[4] = b.x, x[5] = b.y, x[6] = b.z, x[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__half>(__half const* p, float (&x)[8])
{
    uint4 const v = __ldg(reinterpret_cast<uint4 const*>(p));
    uint32_t const w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
        Pair<__half>::unpack2(w[i], x[2 * i], x[2 * i + 1]);
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(__nv_bfloat16 const* p, float (&x)[8])
{
    uint4 const v = __ldg(reinterpret_cast<uint4 const*>(p));
    uint32_t const w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
        Pair<__nv_bfloat16>::unpack2(w[i], x[2 * i], x[2 * i + 1]);
}

// Per-column max |w| over a slab of rows. A CTA is 64 column vectors (eight columns, one 16-byte load
// each) x 4 row lanes: the lanes walk the slab four rows apart, four loads in flight per thread (with
// one the pass is bound by the memory latency), and are merged through shared memory, so a slab
// costs one atomic per column. Non-negative floats order like their bit patterns: the slabs are
// merged with an integer atomic max, and the result does not depend on the order.
constexpr int kAmaxVecs = 64, kAmaxLanes = 4, kAmaxRows = 128; // columns / 8, row lanes, rows per CTA

template <typename W>
__global__ void __launch_bounds__(kAmaxVecs* kAmaxLanes) column_amax_kernel(float* amax, W const* w, int K, int N)
{
    __shared__ float part[kAmaxLanes][kAmaxVecs * 8];
    int const cv = threadIdx.x % kAmaxVecs, lane = threadIdx.x / kAmaxVecs;
    int const c0 = (blockIdx.x * kAmaxVecs + cv) * 8;
    bool const inside = c0 < N; // n is a multiple of 32: a thread's eight columns are all inside or all outside
    int const r0 = blockIdx.y * kAmaxRows, r1 = min(K, r0 + kAmaxRows);
    float m[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (inside)
    {
        int r = r0 + lane;
        for (; r + 3 * kAmaxLanes < r1; r += 4 * kAmaxLanes)
        {
            float x[4][8];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                load8<W>(w + size_t(r + j * kAmaxLanes) * N + c0, x[j]);
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    m[e] = fmaxf(m[e], fabsf(x[j][e]));
        }
        for (; r < r1; r += kAmaxLanes)
        {
            float x[8];
            load8<W>(w + size_t(r) * N + c0, x);
#pragma unroll
            for (int e = 0; e < 8; ++e)
                m[e] = fmaxf(m[e], fabsf(x[e]));
        }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e)
        part[lane][cv * 8 + e] = m[e];
    __syncthreads();
    // one column per thread and step
    for (int c = threadIdx.x; c < kAmaxVecs * 8; c += kAmaxVecs * kAmaxLanes)
    {
        int const col = blockIdx.x * kAmaxVecs * 8 + c;
        if (col < N)
        {
            float v = part[0][c];
#pragma unroll
            for (int l = 1; l < kAmaxLanes; ++l)
                v = fmaxf(v, part[l][c]);
            atomicMax(reinterpret_cast<int*>(amax) + col, __float_as_int(v));
        }
    }
}

// Quantises a tile (q = clamp(int(round(w / scale))), round half away from zero, zero column -> 0),
// optionally stores it row-major (the reference's "unprocessed" output) and emits the kernel layout.
// Eight columns per thread and step: 16-byte loads of the weights and the scales, one 4- or 8-byte
// store of the packed result.
template <typename W, int BITS>
__global__ void __launch_bounds__(kThreads)
    quantize_kernel(uint32_t* out, uint8_t* unprocessed, W const* w, float const* scales, int K, int N)
{
    __shared__ __align__(16) uint8_t tile[kTileK * kSmemPitch];
    constexpr int kCols = kTileBytes * 8 / BITS; // columns per tile
    constexpr int kVecPerRow = kCols / 8;
    int const row_bytes = N * BITS / 8;
    int const n0 = blockIdx.x * kCols;
    int const cols = min(kCols, N - n0); // a multiple of 32
    int const k_tile = blockIdx.y;
    int const lo = BITS == 8 ? -128 : -8, hi = BITS == 8 ? 127 : 7;
    // A thread keeps its eight columns for the whole tile (kThreads is a multiple of kVecPerRow): the
    // scales are loaded once, the rows come two at a time so that both loads are in flight together.
    static_assert(kThreads % kVecPerRow == 0 && kTileK % (2 * (kThreads / kVecPerRow)) == 0, "row walk");
    constexpr int kRowStep = kThreads / kVecPerRow;
    int const c0 = (threadIdx.x % kVecPerRow) * 8;
    if (c0 < cols)
    {
        float4 const sa = __ldg(reinterpret_cast<float4 const*>(scales + n0 + c0));
        float4 const sb = __ldg(reinterpret_cast<float4 const*>(scales + n0 + c0) + 1);
        float const s[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};
        float inv[8]; // 1 / scale, 0 for a zero column (every q is 0 there)
#pragma unroll
        for (int e = 0; e < 8; ++e)
            inv[e] = s[e] != 0.f ? __fdiv_rn(1.f, s[e]) : 0.f;
        for (int rb = threadIdx.x / kVecPerRow; rb < kTileK; rb += 2 * kRowStep)
        {
            float x[2][8];
#pragma unroll
            for (int j = 0; j < 2; ++j)
                load8<W>(w + (size_t(k_tile) * kTileK + rb + j * kRowStep) * N + n0 + c0, x[j]);
#pragma unroll
            for (int j = 0; j < 2; ++j)
            {
                int const r = rb + j * kRowStep;
                size_t const row = size_t(k_tile) * kTileK + r;
                uint32_t qv[8];
#pragma unroll
                for (int e = 0; e < 8; ++e)
                {
                    // q = round-half-away(w / s) with an IEEE division, as the reference computes it. The
                    // product with the reciprocal is within 3 * 2^-24 * |w / s| <= 2.3e-5 of that
                    // quotient, so wherever it is not within 1e-4 of a rounding boundary both round to
                    // the same integer (and round-to-nearest-even equals round-half-away off the
                    // boundary); the rare value near a boundary takes the division.
                    float const r = x[j][e] * inv[e];
                    int q = __float2int_rn(r);
                    if (fabsf(r - float(q)) > 0.4999f)
                        q = s[e] != 0.f ? int(roundf(__fdiv_rn(x[j][e], s[e]))) : 0;
                    qv[e] = uint32_t(max(lo, min(hi, q)));
                }
                if (BITS == 4)
                {
                    uint32_t word = 0;
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        word |= (qv[e] & 0xFu) << (4 * e); // even column in the low nibble
                    *reinterpret_cast<uint32_t*>(tile + r * kSmemPitch + c0 / 2) = word;
                    if (unprocessed)
                        *reinterpret_cast<uint32_t*>(unprocessed + row * row_bytes + (n0 + c0) / 2) = word;
                }
                else
                {
                    uint2 word;
                    word.x = (qv[0] & 0xFFu) | ((qv[1] & 0xFFu) << 8) | ((qv[2] & 0xFFu) << 16) | (qv[3] << 24);
                    word.y = (qv[4] & 0xFFu) | ((qv[5] & 0xFFu) << 8) | ((qv[6] & 0xFFu) << 16) | (qv[7] << 24);
                    *reinterpret_cast<uint2*>(tile + r * kSmemPitch + c0) = word;
                    if (unprocessed)
                        *reinterpret_cast<uint2*>(unprocessed + row * row_bytes + n0 + c0) = word;
                }
            }
        }
    }
    __syncthreads();
    emit_tile<BITS>(out, tile, k_tile, n0, cols, K);
}

bool shape_ok(long k, long n, int bits)
{
    return k > 0 && n > 0 && k % 64 == 0 && (n * bits / 8) % 32 == 0 && (k * bits / 8) % 32 == 0
        && k < (1l << 31) && n < (1l << 31);
}

template <typename W>
int quantize_typed(void* processed, void* unprocessed, float* scales, void* scales_t, int scales_dtype, W const* w,
    int k, int n, int bits, cudaStream_t stream)
{
    if (cudaMemsetAsync(scales, 0, size_t(n) * sizeof(float), stream) != cudaSuccess)
        return W4_ERR_CUDA;
    dim3 const ga((n + kAmaxVecs * 8 - 1) / (kAmaxVecs * 8), (k + kAmaxRows - 1) / kAmaxRows);
    column_amax_kernel<W><<<ga, kAmaxVecs * kAmaxLanes, 0, stream>>>(scales, w, k, n);
    finish_scales_kernel<<<(n + 255) / 256, 256, 0, stream>>>(scales, scales_t, scales_dtype, n,
        1.f / float(1 << (bits - 1)));
    int const cols_per_tile = kTileBytes * 8 / bits;
    dim3 const gq((n + cols_per_tile - 1) / cols_per_tile, k / kTileK);
    if (bits == 4)
        quantize_kernel<W, 4><<<gq, kThreads, 0, stream>>>(static_cast<uint32_t*>(processed),
            static_cast<uint8_t*>(unprocessed), w, scales, k, n);
    else
        quantize_kernel<W, 8><<<gq, kThreads, 0, stream>>>(static_cast<uint32_t*>(processed),
            static_cast<uint8_t*>(unprocessed), w, scales, k, n);
    return cudaGetLastError() == cudaSuccess ? W4_OK : W4_ERR_CUDA;
}

} // namespace prep
} // namespace w4

extern "C"
{

    int w4_preprocess_weights_device(void* out, const void* in, size_t k, size_t n, int bits, void* stream)
    {
        using namespace w4::prep;
        if (!out || !in)
            return W4_ERR_NULL_POINTER;
        if (bits != 4 && bits != 8)
            return W4_ERR_BAD_DTYPE;
        if (!shape_ok(long(k), long(n), bits))
            return W4_ERR_BAD_SHAPE;
        if ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(in)) & 15u)
            return W4_ERR_MISALIGNED;
        if (out == in)
            return W4_ERR_UNSUPPORTED; // not an in-place transform
        cudaStream_t const s = static_cast<cudaStream_t>(stream);
        int const row_bytes = int(n) * bits / 8;
        dim3 const grid((row_bytes + kTileBytes - 1) / kTileBytes, unsigned(k) / kTileK);
        if (bits == 4)
            preprocess_kernel<4><<<grid, kThreads, 0, s>>>(static_cast<uint32_t*>(out),
                static_cast<uint8_t const*>(in), int(k), int(n));
        else
            preprocess_kernel<8><<<grid, kThreads, 0, s>>>(static_cast<uint32_t*>(out),
                static_cast<uint8_t const*>(in), int(k), int(n));
        return cudaGetLastError() == cudaSuccess ? W4_OK : W4_ERR_CUDA;
    }

    int w4_relayout_w4a8_to_w4a16_device(void* out, const void* in, size_t k, size_t n, void* stream)
    {
        using namespace w4::prep;
        if (!out || !in)
            return W4_ERR_NULL_POINTER;
        if (!shape_ok(long(k), long(n), 4) || k % 128 != 0 || n % 64 != 0)
            return W4_ERR_BAD_SHAPE;
        if ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(in)) & 15u)
            return W4_ERR_MISALIGNED;
        if (out == in)
            return W4_ERR_UNSUPPORTED; // not an in-place transform
        size_t const regs = k * n / 8;
        unsigned const grid = unsigned(std::min<size_t>((regs + kThreads - 1) / kThreads, size_t(148) * 32));
        relayout_w4a8_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint32_t*>(out),
            static_cast<uint32_t const*>(in), int(k), int(n));
        return cudaGetLastError() == cudaSuccess ? W4_OK : W4_ERR_CUDA;
    }

    int w4_symmetric_quantize_device(void* processed, void* unprocessed, float* scales, void* scales_t,
        int scales_dtype, const void* weight, int weight_dtype, size_t k, size_t n, int bits, void* stream)
    {
        using namespace w4::prep;
        if (!processed || !scales || !weight)
            return W4_ERR_NULL_POINTER;
        if (bits != 4 && bits != 8)
            return W4_ERR_BAD_DTYPE;
        if (scales_t && scales_dtype != W4_DTYPE_FP16 && scales_dtype != W4_DTYPE_BF16)
            return W4_ERR_BAD_DTYPE;
        if (!shape_ok(long(k), long(n), bits))
            return W4_ERR_BAD_SHAPE;
        if ((reinterpret_cast<uintptr_t>(processed) | reinterpret_cast<uintptr_t>(unprocessed)
                | reinterpret_cast<uintptr_t>(scales) | reinterpret_cast<uintptr_t>(weight))
            & 15u)
            return W4_ERR_MISALIGNED;
        cudaStream_t const s = static_cast<cudaStream_t>(stream);
        switch (weight_dtype)
        {
        case W4_DTYPE_FP32:
            return quantize_typed(processed, unprocessed, scales, scales_t, scales_dtype,
                static_cast<float const*>(weight), int(k), int(n), bits, s);
        case W4_DTYPE_FP16:
            return quantize_typed(processed, unprocessed, scales, scales_t, scales_dtype,
                static_cast<__half const*>(weight), int(k), int(n), bits, s);
        case W4_DTYPE_BF16:
            return quantize_typed(processed, unprocessed, scales, scales_t, scales_dtype,
                static_cast<__nv_bfloat16 const*>(weight), int(k), int(n), bits, s);
        default: return W4_ERR_BAD_DTYPE;
        }
    }

} // extern "C"
