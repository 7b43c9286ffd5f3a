// Host-side weight preparation: symmetric per-column quantisation and the layout transform the
// kernels consume. The reference does this on the CPU as well
// (cpp/tensorrt_llm/kernels/cutlass_kernels/cutlass_preprocessors.cpp:564-615, 652-762 of the
// TensorRT-LLM tree); the bytes produced here are identical to its output on compute capability
// 10.x. Instead of the reference's four passes over the matrix (row permute, sub-byte transpose,
// column interleave, bias + register shuffle) the transform is evaluated in closed form: the rows
// behind an output register are read as 32-bit words and an 8 x 8 nibble (4 x 4 byte) block is
// transposed in registers; blocks are independent, so the loop is split over threads.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

#include "../../include/w4_gemm.h"

namespace
{

constexpr int kPerm8[16] = {0, 1, 8, 9, 2, 3, 10, 11, 4, 5, 12, 13, 6, 7, 14, 15};
constexpr int kPerm4[32] = {0, 1, 8, 9, 16, 17, 24, 25, 2, 3, 10, 11, 18, 19, 26, 27, 4, 5, 12, 13, 20, 21, 28, 29, 6,
    7, 14, 15, 22, 23, 30, 31};

// The closed form of both row permutations that the transforms below use.
constexpr bool closed_form_matches_tables()
{
    for (int a = 0; a < 4; ++a)
    {
        for (int s = 0; s < 8; ++s)
            if (kPerm4[a * 8 + s] != 2 * a + 8 * (s / 2) + s % 2)
                return false;
        for (int s = 0; s < 4; ++s)
            if (kPerm8[a * 4 + s] != 2 * a + 8 * (s / 2) + s % 2)
                return false;
    }
    return true;
}
static_assert(closed_form_matches_tables(), "perm[a * E + s] == 2 * a + 8 * (s / 2) + s % 2");

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

// w[d] holds element c of row d at position c; afterwards w[c] holds element d of column c at
// position d. 8 x 8 nibbles (16-bit halves, bytes, then nibbles exchanged between register pairs) or
// 4 x 4 bytes.
inline void transpose_nibbles(uint32_t (&w)[8])
{
    for (int d = 0; d < 4; ++d)
    {
        uint32_t const a = w[d], b = w[d + 4];
        w[d] = (a & 0x0000FFFFu) | (b << 16);
        w[d + 4] = (a >> 16) | (b & 0xFFFF0000u);
    }
    for (int i = 0; i < 4; ++i)
    {
        int const d = (i & 1) + 4 * (i >> 1); // 0, 1, 4, 5
        uint32_t const a = w[d], b = w[d + 2];
        w[d] = (a & 0x00FF00FFu) | ((b & 0x00FF00FFu) << 8);
        w[d + 2] = ((a >> 8) & 0x00FF00FFu) | (b & 0xFF00FF00u);
    }
    for (int d = 0; d < 8; d += 2)
    {
        uint32_t const a = w[d], b = w[d + 1];
        w[d] = (a & 0x0F0F0F0Fu) | ((b & 0x0F0F0F0Fu) << 4);
        w[d + 1] = ((a >> 4) & 0x0F0F0F0Fu) | (b & 0xF0F0F0F0u);
    }
}

inline void transpose_bytes(uint32_t (&w)[4])
{
    for (int d = 0; d < 2; ++d)
    {
        uint32_t const a = w[d], b = w[d + 2];
        w[d] = (a & 0x0000FFFFu) | (b << 16);
        w[d + 2] = (a >> 16) | (b & 0xFFFF0000u);
    }
    for (int d = 0; d < 4; d += 2)
    {
        uint32_t const a = w[d], b = w[d + 1];
        w[d] = (a & 0x00FF00FFu) | ((b & 0x00FF00FFu) << 8);
        w[d + 1] = ((a >> 8) & 0x00FF00FFu) | (b & 0xFF00FF00u);
    }
}

// One 64-row k tile x one 32-bit word column (E = 8 / 4 adjacent matrix columns): for every register
// index vr of the tile, the E rows behind it - in the register's element order - are read as words,
// the E x E block of elements is transposed and register vr of each of the E columns is written; the
// bias (+8 / +128 on two's complement) is one XOR. Row of the tile behind element s of register vr:
// both of the reference's row permutations (blocks of 16 / 32 rows, kPerm8 / kPerm4) satisfy
// perm[(vr % 4) * E + s] = 2 * (vr % 4) + 8 * (s / 2) + s % 2.
template <int BITS>
void transform_words(uint32_t* dst, uint8_t const* in, size_t K, size_t N, size_t k_tile, size_t wq_lo, size_t wq_hi)
{
    constexpr int E = 32 / BITS, VT = 64 / E, IL = BITS == 8 ? 2 : 4, GP = BITS == 8 ? 16 : 32;
    constexpr uint32_t kBias = BITS == 8 ? 0x80808080u : 0x88888888u;
    size_t const in_row_bytes = N * BITS / 8;
    size_t const regs_per_irow = (K / E) * IL;
    uint8_t const* tile = in + k_tile * 64 * in_row_bytes;
    for (size_t wq = wq_lo; wq < wq_hi; ++wq)
        for (int vr = 0; vr < VT; ++vr)
        {
            uint32_t w[E];
            for (int d = 0; d < E; ++d)
            {
                int const s = BITS == 4 ? (d < 4 ? 2 * d : 2 * (d - 4) + 1) : (d == 1 ? 2 : (d == 2 ? 1 : d));
                int const kl = GP * (vr >> 2) + 2 * (vr & 3) + 8 * (s >> 1) + (s & 1);
                std::memcpy(&w[d], tile + size_t(kl) * in_row_bytes + wq * 4, 4);
            }
            if constexpr (BITS == 4)
                transpose_nibbles(w);
            else
                transpose_bytes(w);
            for (int c = 0; c < E; ++c)
            {
                size_t const n = wq * E + size_t(c);
                dst[(n / IL) * regs_per_irow + k_tile * 32 + (n % IL) * VT + size_t(vr)] = w[c] ^ kBias;
            }
        }
}

// in: [k, n*bits/8] two's-complement, row-major. out: same byte count, kernel layout. Work items are
// (k tile, block of 16 words = one cache line per row), split over threads; every output register is
// written exactly once.
void transform(uint8_t* out, uint8_t const* in, size_t K, size_t N, int bits)
{
    size_t const words = N * size_t(bits) / 32; // 32-bit words per input row
    size_t const blocks = (words + 15) / 16;
    size_t const k_tiles = K / 64;
    uint32_t* dst = reinterpret_cast<uint32_t*>(out);
    parallel_for(k_tiles * blocks, 8,
        [=](size_t lo, size_t hi)
        {
            for (size_t item = lo; item < hi; ++item)
            {
                size_t const k_tile = item / blocks, b = item % blocks;
                size_t const wq_lo = b * 16, wq_hi = std::min(words, wq_lo + 16);
                if (bits == 4)
                    transform_words<4>(dst, in, K, N, k_tile, wq_lo, wq_hi);
                else
                    transform_words<8>(dst, in, K, N, k_tile, wq_lo, wq_hi);
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
    // (Row slabs in parallel, merged under a lock: a maximum does not depend on the order.)
    std::fill(scales, scales + n, 0.f);
    {
        std::mutex merge;
        parallel_for(k, 256,
            [&, n](size_t r_lo, size_t r_hi)
            {
                std::vector<float> local(n, 0.f);
                for (size_t r = r_lo; r < r_hi; ++r)
                {
                    float const* w = weight + r * n;
                    for (size_t c = 0; c < n; ++c)
                        local[c] = std::max(local[c], std::fabs(w[c]));
                }
                std::lock_guard<std::mutex> lock(merge);
                for (size_t c = 0; c < n; ++c)
                    scales[c] = std::max(scales[c], local[c]);
            });
    }
    float const range = 1.f / float(1 << (bits - 1));
    for (size_t c = 0; c < n; ++c)
        scales[c] *= range;
    int const lo = bits == 8 ? -128 : -8, hi = bits == 8 ? 127 : 7;
    // q = round-half-away(w / s) with an IEEE division, as C round() does in the reference. The product
    // with the reciprocal is within 3 * 2^-24 * |w / s| <= 2.3e-5 of that quotient, so unless it lies
    // within 1e-4 of a rounding boundary both round to the same integer (and round-to-nearest-even
    // equals round-half-away off the boundary); near a boundary, or for anything that is not a
    // number, the division decides.
    std::vector<float> inv(n);
    for (size_t c = 0; c < n; ++c)
        inv[c] = scales[c] != 0.f ? 1.f / scales[c] : 0.f;
    float const* inv_s = inv.data();
    auto quantise = [=](float w, size_t c) -> int
    {
        float const r = w * inv_s[c];
        int iv = int(std::lrintf(r));
        if (!(std::fabs(r - float(iv)) <= 0.4999f))
        {
            float const s = scales[c];
            iv = int(s != 0.f ? std::round(w / s) : 0.f);
        }
        return std::max(lo, std::min(hi, iv));
    };
    parallel_for(k, 64,
        [=](size_t r_lo, size_t r_hi)
        {
            for (size_t r = r_lo; r < r_hi; ++r)
            {
                float const* w = weight + r * n;
                int8_t* dst = q + r * row_bytes;
                if (bits == 8)
                    for (size_t c = 0; c < n; ++c)
                        dst[c] = int8_t(quantise(w[c], c));
                else
                    for (size_t c = 0; c < n; c += 2) // n is even: two columns per byte, even column low
                        dst[c / 2] = int8_t(uint8_t((quantise(w[c], c) & 0xF) | ((quantise(w[c + 1], c + 1) & 0xF) << 4)));
            }
        });
    transform(reinterpret_cast<uint8_t*>(processed), reinterpret_cast<uint8_t const*>(q), k, n, bits);
    return W4_OK;
}

extern "C" int w4_pack_int4(int8_t* packed, const int8_t* unpacked, size_t num_packed_bytes)
{
    if (!packed || !unpacked)
        return W4_ERR_NULL_POINTER;
    std::atomic<bool> out_of_range{false};
    parallel_for(num_packed_bytes, size_t(1) << 20,
        [&](size_t lo, size_t hi)
        {
            bool bad = false;
            for (size_t i = lo; i < hi; ++i)
            {
                int const a = unpacked[2 * i], b = unpacked[2 * i + 1];
                bad |= a < -8 || a > 7 || b < -8 || b > 7;
                packed[i] = int8_t(uint8_t((a & 0xF) | ((b & 0xF) << 4)));
            }
            if (bad)
                out_of_range.store(true, std::memory_order_relaxed);
        });
    return out_of_range.load() ? W4_ERR_BAD_DTYPE : W4_OK; // the packed bytes are unspecified then
}

extern "C" void w4_unpack_int4(int8_t* unpacked, const int8_t* packed, size_t num_packed_bytes)
{
    parallel_for(num_packed_bytes, size_t(1) << 20,
        [=](size_t lo, size_t hi)
        {
            for (size_t i = lo; i < hi; ++i)
            {
                int8_t const b = packed[i];
                unpacked[2 * i + 0] = int8_t(int8_t(uint8_t(b) << 4) >> 4);
                unpacked[2 * i + 1] = int8_t(b >> 4);
            }
        });
}
