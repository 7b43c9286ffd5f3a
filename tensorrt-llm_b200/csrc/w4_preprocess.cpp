// Host-side weight preparation: symmetric per-column quantisation and the layout transform the
// kernels consume. The reference does this on the CPU as well
// (cpp/tensorrt_llm/kernels/cutlass_kernels/cutlass_preprocessors.cpp:564-615, 652-762 of the
// TensorRT-LLM tree); the bytes produced here are identical to its output on compute capability
// 10.x. Instead of the reference's four passes over the matrix (row permute, sub-byte transpose,
// column interleave, bias + register shuffle) the transform is evaluated in closed form, one output
// 32-bit register at a time, and the registers are independent so the loop is split over threads.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "../../include/w4_gemm.h"

namespace
{

constexpr int kPerm8[16] = {0, 1, 8, 9, 2, 3, 10, 11, 4, 5, 12, 13, 6, 7, 14, 15};
constexpr int kPerm4[32] = {0, 1, 8, 9, 16, 17, 24, 25, 2, 3, 10, 11, 18, 19, 26, 27, 4, 5, 12, 13, 20, 21, 28, 29, 6,
    7, 14, 15, 22, 23, 30, 31};

bool shape_ok(size_t k, size_t n, int bits)
{
    if (bits != 4 && bits != 8)
        return false;
    // k: whole 64-wide tiles (interleave step). n: the reference's transpose wants both byte
    // extents to be multiples of 32, which is n % 64 == 0 for int4 and n % 32 == 0 for int8.
    return k > 0 && n > 0 && k % 64 == 0 && (n * bits / 8) % 32 == 0 && (k * bits / 8) % 32 == 0;
}

template <typename F>
void parallel_for(size_t count, size_t min_chunk, F&& body)
{
    unsigned hw = std::thread::hardware_concurrency();
    size_t const workers = std::max<size_t>(1, std::min<size_t>(hw ? hw : 1, count / std::max<size_t>(1, min_chunk)));
    if (workers <= 1)
    {
        body(size_t(0), count);
        return;
    }
    std::vector<std::thread> pool;
    size_t const step = (count + workers - 1) / workers;
    for (size_t w = 0; w < workers; ++w)
    {
        size_t const lo = w * step, hi = std::min(count, lo + step);
        if (lo < hi)
            pool.emplace_back([=, &body] { body(lo, hi); });
    }
    for (auto& t : pool)
        t.join();
}

// in: [k, n*bits/8] two's-complement, row-major. out: same byte count, kernel layout.
void transform(uint8_t* out, uint8_t const* in, size_t K, size_t N, int bits)
{
    size_t const E = 32 / bits;            // elements per 32-bit register
    size_t const VT = 64 / E;              // registers per 64-wide k tile of one column
    size_t const IL = bits == 8 ? 2 : 4;   // columns interleaved
    size_t const Gp = bits == 8 ? 16 : 32; // rows per permutation block
    int const* perm = bits == 8 ? kPerm8 : kPerm4;
    size_t const regs_per_irow = (K / E) * IL;
    size_t const num_regs = K * N / E;
    size_t const in_row_bytes = N * bits / 8;
    uint32_t* dst = reinterpret_cast<uint32_t*>(out);

    parallel_for(num_regs, size_t(1) << 16,
        [=](size_t lo, size_t hi)
        {
            for (size_t reg = lo; reg < hi; ++reg)
            {
                size_t const irow = reg / regs_per_irow, vwr = reg % regs_per_irow;
                size_t const tile = vwr / (VT * IL), within = vwr % (VT * IL);
                size_t const n = irow * IL + within / VT;
                size_t const vr = tile * VT + within % VT;
                uint32_t word = 0;
                for (size_t d = 0; d < E; ++d)
                {
                    // position d of the register holds source element s of the permuted column
                    size_t const s = bits == 4 ? (d < 4 ? 2 * d : 2 * (d - 4) + 1) : (d == 1 ? 2 : (d == 2 ? 1 : d));
                    size_t const kp = vr * E + s;
                    size_t const k = (kp / Gp) * Gp + size_t(perm[kp % Gp]);
                    uint32_t u;
                    if (bits == 8)
                        u = uint8_t(int(int8_t(in[k * in_row_bytes + n])) + 128);
                    else
                    {
                        uint8_t const b = in[k * in_row_bytes + n / 2];
                        int const v = (n & 1) ? (int8_t(b) >> 4) : (int8_t(b << 4) >> 4);
                        u = uint32_t(v + 8) & 0xFu;
                    }
                    word |= u << (bits * d);
                }
                dst[reg] = word;
            }
        });
}

// int4 weights as the reference lays them out for fp8 activations (W4A8;
// cutlass_preprocessors.cpp:114-116,175-179 with mixed_gemm_B_layout.h:105-117 for an 8-bit A type):
// two columns interleaved, 128-row tiles, its own row permutation inside every block of 32 rows.
// Register `reg` of the output holds, in nibble d, element e(d) of word j of tile t of column
// 2 * irow + c, where reg = irow * (K / 4) + 32 * t + 16 * c + j. One routine walks that map in
// either direction: FORWARD builds the W4A8 bytes from row-major two's-complement nibbles, the other
// direction recovers the row-major nibbles from W4A8 bytes.
constexpr int kPerm4A8[32] = {0, 1, 2, 3, 16, 17, 18, 19, 4, 5, 6, 7, 20, 21, 22, 23, 8, 9, 10, 11, 24, 25, 26, 27, 12, 13,
    14, 15, 28, 29, 30, 31};

template <bool FORWARD>
void walk_w4a8(uint8_t* laid_out, uint8_t* row_major, size_t K, size_t N)
{
    size_t const regs_per_irow = K / 4; // two columns of K / 8 registers
    size_t const num_irows = N / 2;
    size_t const row_bytes = N / 2;
    uint32_t* regs = reinterpret_cast<uint32_t*>(laid_out);
    // parallel over interleaved rows: a pair of columns touches its own bytes of every source row
    // (two nibbles of one byte), so the reverse direction has no write conflicts either
    parallel_for(num_irows, 16,
        [=](size_t lo, size_t hi)
        {
            for (size_t irow = lo; irow < hi; ++irow)
                for (size_t vwr = 0; vwr < regs_per_irow; ++vwr)
                {
                    size_t const t = vwr / 32, c = (vwr % 32) / 16, j = vwr % 16;
                    size_t const n = irow * 2 + c;
                    uint32_t word = FORWARD ? 0u : regs[irow * regs_per_irow + vwr];
                    for (size_t d = 0; d < 8; ++d)
                    {
                        size_t const e = d < 4 ? 2 * d : 2 * (d - 4) + 1;
                        size_t const kp = 128 * t + 8 * j + e;
                        size_t const k = (kp & ~size_t(31)) + size_t(kPerm4A8[kp & 31]);
                        uint8_t& b = row_major[k * row_bytes + n / 2];
                        if (FORWARD)
                        {
                            int const v = (n & 1) ? (int8_t(b) >> 4) : (int8_t(uint8_t(b << 4)) >> 4);
                            word |= (uint32_t(v + 8) & 0xFu) << (4 * d);
                        }
                        else
                        {
                            uint32_t const q = (((word >> (4 * d)) & 0xFu) - 8u) & 0xFu; // two's complement nibble
                            b = (n & 1) ? uint8_t((b & 0x0F) | (q << 4)) : uint8_t((b & 0xF0) | q);
                        }
                    }
                    if (FORWARD)
                        regs[irow * regs_per_irow + vwr] = word;
                }
        });
}

bool shape_ok_w4a8(size_t k, size_t n)
{
    return k > 0 && n > 0 && k % 128 == 0 && n % 64 == 0;
}

} // namespace

extern "C" int w4_preprocess_weights_w4a8(int8_t* out, const int8_t* in, size_t k, size_t n)
{
    if (!out || !in)
        return W4_ERR_NULL_POINTER;
    if (!shape_ok_w4a8(k, n))
        return W4_ERR_BAD_SHAPE;
    walk_w4a8<true>(reinterpret_cast<uint8_t*>(out), const_cast<uint8_t*>(reinterpret_cast<uint8_t const*>(in)), k, n);
    return W4_OK;
}

extern "C" int w4_relayout_w4a8_to_w4a16(int8_t* out, const int8_t* in, size_t k, size_t n)
{
    if (!out || !in)
        return W4_ERR_NULL_POINTER;
    if (!shape_ok_w4a8(k, n) || !shape_ok(k, n, 4))
        return W4_ERR_BAD_SHAPE;
    std::vector<uint8_t> row_major(k * n / 2);
    walk_w4a8<false>(const_cast<uint8_t*>(reinterpret_cast<uint8_t const*>(in)), row_major.data(), k, n);
    transform(reinterpret_cast<uint8_t*>(out), row_major.data(), k, n, 4);
    return W4_OK;
}

extern "C" int w4_preprocess_weights(int8_t* out, const int8_t* in, size_t k, size_t n, int bits)
{
    if (!out || !in)
        return W4_ERR_NULL_POINTER;
    if (bits != 4 && bits != 8)
        return W4_ERR_BAD_DTYPE;
    if (!shape_ok(k, n, bits))
        return W4_ERR_BAD_SHAPE;
    transform(reinterpret_cast<uint8_t*>(out), reinterpret_cast<uint8_t const*>(in), k, n, bits);
    return W4_OK;
}

extern "C" int w4_symmetric_quantize(int8_t* processed, int8_t* unprocessed, float* scales, const float* weight,
    size_t k, size_t n, int bits)
{
    if (!processed || !scales || !weight)
        return W4_ERR_NULL_POINTER;
    if (bits != 4 && bits != 8)
        return W4_ERR_BAD_DTYPE;
    if (!shape_ok(k, n, bits))
        return W4_ERR_BAD_SHAPE;
    size_t const row_bytes = n * bits / 8;
    std::vector<int8_t> tmp;
    int8_t* q = unprocessed;
    if (!q)
    {
        tmp.resize(k * row_bytes);
        q = tmp.data();
    }
    // per-column amax in fp32, then scale = amax / 2^(bits-1); the unrounded fp32 scale quantises.
    std::fill(scales, scales + n, 0.f);
    for (size_t r = 0; r < k; ++r)
    {
        float const* w = weight + r * n;
        for (size_t c = 0; c < n; ++c)
            scales[c] = std::max(scales[c], std::fabs(w[c]));
    }
    float const range = 1.f / float(1 << (bits - 1));
    for (size_t c = 0; c < n; ++c)
        scales[c] *= range;
    int const lo = bits == 8 ? -128 : -8, hi = bits == 8 ? 127 : 7;
    parallel_for(k, 64,
        [=](size_t r_lo, size_t r_hi)
        {
            for (size_t r = r_lo; r < r_hi; ++r)
            {
                float const* w = weight + r * n;
                int8_t* dst = q + r * row_bytes;
                if (bits == 4)
                    std::memset(dst, 0, row_bytes);
                for (size_t c = 0; c < n; ++c)
                {
                    float const s = scales[c];
                    // round half away from zero, as C round() does in the reference
                    float const v = s != 0.f ? std::round(w[c] / s) : 0.f;
                    int const iv = std::max(lo, std::min(hi, int(v)));
                    if (bits == 8)
                        dst[c] = int8_t(iv);
                    else
                        dst[c / 2] = int8_t(uint8_t(dst[c / 2]) | uint8_t((iv & 0xF) << (4 * (c & 1))));
                }
            }
        });
    transform(reinterpret_cast<uint8_t*>(processed), reinterpret_cast<uint8_t const*>(q), k, n, bits);
    return W4_OK;
}

extern "C" int w4_pack_int4(int8_t* packed, const int8_t* unpacked, size_t num_packed_bytes)
{
    if (!packed || !unpacked)
        return W4_ERR_NULL_POINTER;
    for (size_t i = 0; i < num_packed_bytes; ++i)
    {
        int const a = unpacked[2 * i], b = unpacked[2 * i + 1];
        if (a < -8 || a > 7 || b < -8 || b > 7)
            return W4_ERR_BAD_DTYPE;
        packed[i] = int8_t(uint8_t((a & 0xF) | ((b & 0xF) << 4)));
    }
    return W4_OK;
}

extern "C" void w4_unpack_int4(int8_t* unpacked, const int8_t* packed, size_t num_packed_bytes)
{
    for (size_t i = 0; i < num_packed_bytes; ++i)
    {
        int8_t const b = packed[i];
        unpacked[2 * i + 0] = int8_t(int8_t(uint8_t(b) << 4) >> 4);
        unpacked[2 * i + 1] = int8_t(b >> 4);
    }
}
