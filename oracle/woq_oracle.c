/*
 * TEST INFRASTRUCTURE ONLY - CPU restatement of the reference's integer weight path.
 *
 * This file restates, step by step and in plain C, what TensorRT-LLM does on the host to turn a
 * floating-point [K, N] weight into the bytes its weight-only GEMM kernels consume. It is the
 * checker for the CUDA/host product code, never a part of it: only tests, the smoke check and the
 * benchmark's CPU-baseline leg may load it.
 *
 * Parity status: PINNED. Every function here is compared byte for byte with the reference's own
 * code compiled from its sources (oracle/build_ref.sh -> oracle/_ref/libwoq_ref.so) in
 * tests/test_oracle.py, and with golden vectors generated from that library
 * (tests/golden/make_golden.py).
 *
 * Reference file for every citation below:
 *   cpp/tensorrt_llm/kernels/cutlass_kernels/cutlass_preprocessors.cpp   ("pre.cpp")
 *   cpp/tensorrt_llm/thop/weightOnlyQuantOp.cpp                          ("op.cpp")
 *
 * Conventions: K = rows (reduction dim), N = columns (output features), bits in {4, 8}.
 * A quantised [K, N] matrix is K rows of N*bits/8 bytes; for int4 the element with the even
 * column index sits in the low nibble.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_OK 0
#define ORACLE_BAD_SHAPE -1
#define ORACLE_BAD_ARG -2

/* pre.cpp:163-184 - row permutations that line data up with the mma.sync fragment order. */
static const int kPerm8[16] = {0, 1, 8, 9, 2, 3, 10, 11, 4, 5, 12, 13, 6, 7, 14, 15};
static const int kPerm4[32] = {0, 1, 8, 9, 16, 17, 24, 25, 2, 3, 10, 11, 18, 19, 26, 27, 4, 5, 12, 13, 20, 21, 28, 29,
    6, 7, 14, 15, 22, 23, 30, 31};
/* pre.cpp:175-179 - the permutation for int4 weights under fp8 activations (W4A8). */
static const int kPerm4A8[32] = {0, 1, 2, 3, 16, 17, 18, 19, 4, 5, 6, 7, 20, 21, 22, 23, 8, 9, 10, 11, 24, 25, 26, 27,
    12, 13, 14, 15, 28, 29, 30, 31};

static int get_elt(const uint8_t* buf, size_t idx, int bits)
{
    if (bits == 8)
        return buf[idx];
    return (buf[idx >> 1] >> (4 * (idx & 1))) & 0xF;
}

static void set_elt(uint8_t* buf, size_t idx, int bits, int v)
{
    if (bits == 8)
    {
        buf[idx] = (uint8_t) v;
        return;
    }
    uint8_t* b = buf + (idx >> 1);
    int sh = 4 * (int) (idx & 1);
    *b = (uint8_t) ((*b & ~(0xF << sh)) | ((v & 0xF) << sh));
}

/* pre.cpp:186-244 permute_B_rows_for_mixed_gemm: inside every block of 16 (int8) or 32 (int4)
 * rows, destination row r receives source row perm[r]. Rows move whole. */
int oracle_permute_rows(uint8_t* out, const uint8_t* in, size_t K, size_t N, int bits)
{
    if (bits != 4 && bits != 8)
        return ORACLE_BAD_ARG;
    const int block = bits == 8 ? 16 : 32; /* B_ROWS_PER_MMA = 8 * (16 / bits), pre.cpp:199,208 */
    const int* perm = bits == 8 ? kPerm8 : kPerm4;
    if (K % block || N % 8) /* pre.cpp:212-217 */
        return ORACLE_BAD_SHAPE;
    const size_t row_bytes = N * bits / 8;
    for (size_t base = 0; base < K; base += block)
        for (int r = 0; r < block; ++r)
            memcpy(out + (base + r) * row_bytes, in + (base + perm[r]) * row_bytes, row_bytes);
    return ORACLE_OK;
}

/* pre.cpp:250-387 subbyte_transpose_impl: [K, N] row-major -> [N, K] row-major, element by
 * element, keeping the "even index in the low nibble" packing. The reference works in 64x64
 * tiles for speed and requires both byte extents to be multiples of 32 (pre.cpp:280-283). */
int oracle_subbyte_transpose(uint8_t* out, const uint8_t* in, size_t K, size_t N, int bits)
{
    if (bits != 4 && bits != 8)
        return ORACLE_BAD_ARG;
    const size_t col_bytes = N * bits / 8, col_bytes_t = K * bits / 8;
    if (col_bytes % 32 || col_bytes_t % 32)
        return ORACLE_BAD_SHAPE;
    for (size_t k = 0; k < K; ++k)
        for (size_t n = 0; n < N; ++n)
            set_elt(out, n * K + k, bits, get_elt(in, k * N + n, bits));
    return ORACLE_OK;
}

/* pre.cpp:512-562 interleave_column_major_tensor with the Ampere layout the reference selects
 * for compute capability >= 100 (pre.cpp:140-143): ThreadblockK = 64 and
 * ColumnsInterleaved = 128*8 / (bits*64) = 2 (int8) or 4 (int4)
 * (cutlass_extensions/include/cutlass_extensions/gemm/kernel/mixed_gemm_B_layout.h:89-117).
 * Input is the transposed matrix, N rows of K elements, viewed as 32-bit words. */
int oracle_interleave_columns(uint8_t* out, const uint8_t* in, size_t K, size_t N, int bits)
{
    if (bits != 4 && bits != 8)
        return ORACLE_BAD_ARG;
    const size_t elts_per_word = 32 / bits;
    const size_t rows_per_tile = 64;
    const size_t interleave = bits == 8 ? 2 : 4;
    if (K % elts_per_word || K % rows_per_tile) /* pre.cpp:529-536 */
        return ORACLE_BAD_SHAPE;
    const size_t words_per_col = K / elts_per_word;
    const size_t words_per_tile = rows_per_tile / elts_per_word;
    const uint32_t* src = (const uint32_t*) in;
    uint32_t* dst = (uint32_t*) out;
    for (size_t n = 0; n < N; ++n)
    {
        const size_t write_col = n / interleave;
        for (size_t w = 0; w < words_per_col; ++w)
        {
            const size_t base = w - w % words_per_tile;
            const size_t write_word = interleave * base + words_per_tile * (n % interleave) + w % words_per_tile;
            dst[write_col * words_per_col * interleave + write_word] = src[n * words_per_col + w]; /* :545-557 */
        }
    }
    return ORACLE_OK;
}

int oracle_add_bias_and_interleave(uint8_t* buf, size_t num_elts, int bits);

/* The int4 layout for fp8 activations (W4A8), pre.cpp:114-116 with
 * cutlass_extensions/.../mixed_gemm_B_layout.h:105-117 for an 8-bit A type: ThreadblockK = 128 and
 * ColumnsInterleaved = 256 / 128 = 2; rows permuted by kPerm4A8; the nibble step is the W4A16 one
 * (pre.cpp:498-505). */
int oracle_preprocess_weights_w4a8(uint8_t* out, const uint8_t* in, size_t K, size_t N)
{
    const int bits = 4;
    if (K % 128 || N % 8)
        return ORACLE_BAD_SHAPE;
    const size_t num_bytes = K * N / 2;
    uint8_t* a = (uint8_t*) malloc(num_bytes ? num_bytes : 1);
    uint8_t* b = (uint8_t*) malloc(num_bytes ? num_bytes : 1);
    if (!a || !b)
    {
        free(a);
        free(b);
        return ORACLE_BAD_ARG;
    }
    const size_t row_bytes = N / 2;
    for (size_t base = 0; base < K; base += 32)
        for (int r = 0; r < 32; ++r)
            memcpy(a + (base + r) * row_bytes, in + (base + kPerm4A8[r]) * row_bytes, row_bytes);
    int rc = oracle_subbyte_transpose(b, a, K, N, bits);
    if (rc == ORACLE_OK)
    {
        const size_t elts_per_word = 8, rows_per_tile = 128, interleave = 2;
        const size_t words_per_col = K / elts_per_word, words_per_tile = rows_per_tile / elts_per_word;
        const uint32_t* src = (const uint32_t*) b;
        uint32_t* dst = (uint32_t*) a;
        for (size_t n = 0; n < N; ++n)
            for (size_t w = 0; w < words_per_col; ++w)
            {
                const size_t base = w - w % words_per_tile;
                const size_t write_word = interleave * base + words_per_tile * (n % interleave) + w % words_per_tile;
                dst[(n / interleave) * words_per_col * interleave + write_word] = src[n * words_per_col + w];
            }
        rc = oracle_add_bias_and_interleave(a, K * N, bits);
    }
    if (rc == ORACLE_OK)
        memcpy(out, a, num_bytes);
    free(a);
    free(b);
    return rc;
}

/* pre.cpp:412-433 (int8) and :435-489 (int4): make the values unsigned (+128 / +8) and shuffle
 * the elements inside every 32-bit register so that the device converter needs no shifts. */
int oracle_add_bias_and_interleave(uint8_t* buf, size_t num_elts, int bits)
{
    if (bits == 8)
    {
        if (num_elts % 4)
            return ORACLE_BAD_SHAPE;
        for (size_t i = 0; i < num_elts; ++i)
            buf[i] = (uint8_t) ((int) (int8_t) buf[i] + 128);
        for (size_t b = 0; b < num_elts; b += 4)
        {
            uint8_t t = buf[b + 1];
            buf[b + 1] = buf[b + 2];
            buf[b + 2] = t;
        }
        return ORACLE_OK;
    }
    if (bits != 4)
        return ORACLE_BAD_ARG;
    const size_t num_bytes = num_elts / 2;
    if (num_bytes % 4)
        return ORACLE_BAD_SHAPE;
    for (size_t i = 0; i < num_bytes; ++i)
    {
        int lo = (int) (int8_t) (buf[i] << 4) >> 4; /* sign-extended low nibble */
        int hi = (int) (int8_t) buf[i] >> 4;        /* sign-extended high nibble */
        buf[i] = (uint8_t) (((lo + 8) & 0xF) | (((hi + 8) & 0xF) << 4));
    }
    uint32_t* reg = (uint32_t*) buf;
    for (size_t i = 0; i < num_bytes / 4; ++i)
    {
        const uint32_t cur = reg[i];
        uint32_t t = 0;
        for (int dest = 0; dest < 8; ++dest)
        {
            const int src = dest < 4 ? 2 * dest : 2 * (dest - 4) + 1; /* pre.cpp:480 */
            t |= ((cur >> (4 * src)) & 0xFu) << (4 * dest);
        }
        reg[i] = t;
    }
    return ORACLE_OK;
}

/* pre.cpp:564-615 preprocess_weights_for_mixed_gemm on compute capability 10.x:
 * permute rows -> transpose -> interleave columns -> bias + register shuffle. */
int oracle_preprocess_weights(uint8_t* out, const uint8_t* in, size_t K, size_t N, int bits)
{
    if (bits != 4 && bits != 8)
        return ORACLE_BAD_ARG;
    const size_t num_bytes = K * N * bits / 8;
    uint8_t* a = (uint8_t*) malloc(num_bytes ? num_bytes : 1);
    uint8_t* b = (uint8_t*) malloc(num_bytes ? num_bytes : 1);
    if (!a || !b)
    {
        free(a);
        free(b);
        return ORACLE_BAD_ARG;
    }
    int rc = oracle_permute_rows(a, in, K, N, bits);
    if (rc == ORACLE_OK)
        rc = oracle_subbyte_transpose(b, a, K, N, bits);
    if (rc == ORACLE_OK)
        rc = oracle_interleave_columns(a, b, K, N, bits);
    if (rc == ORACLE_OK)
        rc = oracle_add_bias_and_interleave(a, K * N, bits);
    if (rc == ORACLE_OK)
        memcpy(out, a, num_bytes);
    free(a);
    free(b);
    return rc;
}

/* pre.cpp:652-762 symmetric_quantize for one 2-D matrix with fp32 arithmetic.
 *  - per-column amax over all rows in fp32 (:696-703);
 *  - scale = amax * 2^-(bits-1), used unrounded for quantising, returned as fp32 so the caller can
 *    round it to fp16 / bf16 exactly as ComputeType(float) does (:707-711);
 *  - q = round-half-away(w / scale), clamped to [-128,127] or [-8,7]; a zero column gives q = 0
 *    (:721-750);
 *  - then the layout transform (:760-761).
 * unprocessed may be NULL. */
int oracle_symmetric_quantize(uint8_t* processed, uint8_t* unprocessed, float* scales, const float* weight, size_t K,
    size_t N, int bits)
{
    if (bits != 4 && bits != 8)
        return ORACLE_BAD_ARG;
    if (!processed || !scales || !weight)
        return ORACLE_BAD_ARG;
    const size_t bytes_per_row = N * bits / 8;
    uint8_t* q = unprocessed;
    if (!q)
        q = (uint8_t*) malloc(K * bytes_per_row + 1);
    if (!q)
        return ORACLE_BAD_ARG;
    const float range_scale = 1.f / (float) (1 << (bits - 1));
    for (size_t n = 0; n < N; ++n)
        scales[n] = 0.f;
    for (size_t k = 0; k < K; ++k)
        for (size_t n = 0; n < N; ++n)
        {
            const float a = fabsf(weight[k * N + n]);
            if (a > scales[n])
                scales[n] = a;
        }
    for (size_t n = 0; n < N; ++n)
        scales[n] *= range_scale;
    for (size_t k = 0; k < K; ++k)
    {
        uint8_t* row = q + k * bytes_per_row;
        const float* wrow = weight + k * N;
        if (bits == 8)
        {
            for (size_t n = 0; n < N; ++n)
            {
                const float s = scales[n];
                float v = s != 0.f ? roundf(wrow[n] / s) : 0.f;
                v = fmaxf(-128.f, fminf(127.f, v));
                row[n] = (uint8_t) (int8_t) v;
            }
        }
        else
        {
            for (size_t j = 0; j < bytes_per_row; ++j)
            {
                uint8_t packed = 0;
                for (int h = 0; h < 2; ++h)
                {
                    const size_t n = 2 * j + h;
                    if (n < N)
                    {
                        const float s = scales[n];
                        const float v = s != 0.f ? roundf(wrow[n] / s) : 0.f;
                        int iv = (int) v;
                        iv = iv < -8 ? -8 : (iv > 7 ? 7 : iv);
                        packed |= (uint8_t) ((iv & 0xF) << (4 * h));
                    }
                }
                row[j] = packed;
            }
        }
    }
    int rc = oracle_preprocess_weights(processed, q, K, N, bits);
    if (!unprocessed)
        free(q);
    return rc;
}

/* op.cpp:284-316 unpack_int4_packed_tensor_to_int8: low nibble first, sign-extended. */
void oracle_unpack_int4(int8_t* out, const uint8_t* packed, size_t num_bytes)
{
    for (size_t i = 0; i < num_bytes; ++i)
    {
        out[2 * i + 0] = (int8_t) ((int8_t) (packed[i] << 4) >> 4);
        out[2 * i + 1] = (int8_t) ((int8_t) packed[i] >> 4);
    }
}

/* op.cpp:318-353 pack_int8_tensor_to_packed_int4; returns ORACLE_BAD_ARG for a value outside
 * [-8, 7] where the reference raises. */
int oracle_pack_int4(uint8_t* packed, const int8_t* in, size_t num_bytes_out)
{
    for (size_t i = 0; i < num_bytes_out; ++i)
    {
        const int8_t a = in[2 * i], b = in[2 * i + 1];
        if (a < -8 || a > 7 || b < -8 || b > 7)
            return ORACLE_BAD_ARG;
        packed[i] = (uint8_t) ((a & 0xF) | ((b & 0xF) << 4));
    }
    return ORACLE_OK;
}

/* Inverse of oracle_preprocess_weights, used by the floating-point oracle to recover the signed
 * integers from the bytes the kernels consume. It evaluates the closed form of the four layout
 * steps position by position; there is no reference counterpart, so it is checked as a round
 * trip against the forward path above. out: K*N int8 values, row-major [K, N]. */
int oracle_unpreprocess_to_int8(int8_t* out, const uint8_t* processed, size_t K, size_t N, int bits)
{
    if (bits != 4 && bits != 8)
        return ORACLE_BAD_ARG;
    const size_t E = 32 / bits, VT = 64 / E, IL = bits == 8 ? 2 : 4, Gp = bits == 8 ? 16 : 32;
    const int* perm = bits == 8 ? kPerm8 : kPerm4;
    static const int swz8[4] = {0, 2, 1, 3};
    if (K % 64 || N % 8 || (N * bits / 8) % 32)
        return ORACLE_BAD_SHAPE;
    for (size_t p = 0; p < K * N; ++p)
    {
        const size_t d = p % E, reg = p / E;
        const size_t s = bits == 4 ? (d < 4 ? 2 * d : 2 * (d - 4) + 1) : (size_t) swz8[d];
        const size_t wcol = reg / ((K / E) * IL), vwr = reg % ((K / E) * IL);
        const size_t tile = vwr / (VT * IL), within = vwr % (VT * IL);
        const size_t n = wcol * IL + within / VT;
        const size_t vr = tile * VT + within % VT;
        const size_t kp = vr * E + s;
        const size_t k = (kp / Gp) * Gp + (size_t) perm[kp % Gp];
        const int u = get_elt(processed, p, bits);
        out[k * N + n] = (int8_t) (bits == 4 ? u - 8 : u - 128);
    }
    return ORACLE_OK;
}
