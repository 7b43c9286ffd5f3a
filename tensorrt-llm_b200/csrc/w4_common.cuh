// Shared device helpers for the sm_100a weight-only GEMM kernels: PTX wrappers (mbarrier, bulk
// copies, mma.sync), the integer -> fp16/bf16 converters for the interleaved weight layout, and
// the bounded-wait policy.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace w4
{

// Device-side status word. Kernels never trap or spin forever: a wait that runs out of polls
// records a code here and the kernel drains and returns. Read through w4_gemm_device_status().
// The library is built as one translation unit (w4_lib.cu), so this is the single instance.
static __device__ int g_device_status = 0;

constexpr int kDeviceTimeout = -10; // == W4_ERR_DEVICE_TIMEOUT

// Upper bound on polls of one mbarrier wait. One try_wait already blocks for a hardware-defined
// interval, so this is on the order of a second, far beyond any legitimate wait.
constexpr uint32_t kMaxWaitPolls = 1u << 20;
// Same bound for loops that spin on the non-blocking mbarrier test (tens of cycles per poll).
constexpr uint32_t kMaxSpinPolls = 1u << 26;

__device__ __forceinline__ uint32_t smem_u32(void const* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Non-blocking test of a phase.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait. Returns false (after recording the timeout) when the phase never completed.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity)
{
    for (uint32_t i = 0; i < kMaxWaitPolls; ++i)
    {
        if (mbar_try_wait(bar, parity))
            return true;
    }
    atomicExch(&g_device_status, kDeviceTimeout);
    return false;
}

// Contiguous global -> shared bulk copy (TMA engine, no tensor map). dst, src 16-byte aligned,
// bytes a multiple of 16. Completion is signalled on `bar` as transaction bytes.
__device__ __forceinline__ void bulk_g2s(void* dst, void const* src, uint32_t bytes, uint64_t* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// 2-D tiled TMA load (tensor map in kernel parameter / constant space). c0 = innermost coordinate
// (its byte offset must be a multiple of 16), c1 = row. Out-of-range parts of the box read as zero
// and still count towards the transaction bytes.
__device__ __forceinline__ void tma_load_2d(void* dst, void const* tensor_map, int c0, int c1, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
            "r"(smem_u32(dst)),
        "l"(tensor_map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
        : "memory");
}

// Variants for a converged warp: one elected lane performs the operation, operands are warp-uniform.
__device__ __forceinline__ void elect_expect_tx(uint32_t bar_addr, uint32_t bytes)
{
    asm volatile(
        "{\n"
        ".reg .pred pe;\n"
        "elect.sync _|pe, 0xffffffff;\n"
        "@pe mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n"
        "}\n" ::"r"(bar_addr),
        "r"(bytes)
        : "memory");
}

__device__ __forceinline__ void elect_tma_load_2d(uint32_t dst, void const* tensor_map, int c0, int c1, uint32_t bar_addr)
{
    asm volatile(
        "{\n"
        ".reg .pred pe;\n"
        "elect.sync _|pe, 0xffffffff;\n"
        "@pe cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        "}\n" ::"r"(dst),
        "l"(tensor_map), "r"(c0), "r"(c1), "r"(bar_addr)
        : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv)
{
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));
    return r;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// ---------------------------------------------------------------------------------------------
// Element-type traits: packed-pair arithmetic on raw 32-bit registers.
// ---------------------------------------------------------------------------------------------
template <typename T>
struct Pair;

template <>
struct Pair<__half>
{
    using T2 = __half2;
    static __device__ __forceinline__ T2 as(uint32_t v)
    {
        return *reinterpret_cast<T2*>(&v);
    }
    static __device__ __forceinline__ uint32_t bits(T2 v)
    {
        return *reinterpret_cast<uint32_t*>(&v);
    }
    static __device__ __forceinline__ uint32_t fma(uint32_t a, uint32_t b, uint32_t c)
    {
        return bits(__hfma2(as(a), as(b), as(c)));
    }
    static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b)
    {
        return bits(__hmul2(as(a), as(b)));
    }
    static __device__ __forceinline__ uint32_t sub(uint32_t a, uint32_t b)
    {
        return bits(__hsub2(as(a), as(b)));
    }
    static __device__ __forceinline__ float to_float(uint16_t h)
    {
        return __half2float(__ushort_as_half(h));
    }
    static __device__ __forceinline__ uint16_t from_float(float f)
    {
        return __half_as_ushort(__float2half_rn(f));
    }
    // Both halves of a packed pair as floats (low half first).
    static __device__ __forceinline__ void unpack2(uint32_t v, float& lo, float& hi)
    {
        float2 const f = __half22float2(as(v));
        lo = f.x;
        hi = f.y;
    }
    static __device__ __forceinline__ void mma(float (&d)[4], uint32_t const (&a)[4], uint32_t b0, uint32_t b1)
    {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    // d = a * b (no accumulator input: starts a chain without zeroing registers first)
    static __device__ __forceinline__ void mma0(float (&d)[4], uint32_t const (&a)[4], uint32_t b0, uint32_t b1)
    {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
    }
};

template <>
struct Pair<__nv_bfloat16>
{
    using T2 = __nv_bfloat162;
    static __device__ __forceinline__ T2 as(uint32_t v)
    {
        return *reinterpret_cast<T2*>(&v);
    }
    static __device__ __forceinline__ uint32_t bits(T2 v)
    {
        return *reinterpret_cast<uint32_t*>(&v);
    }
    static __device__ __forceinline__ uint32_t fma(uint32_t a, uint32_t b, uint32_t c)
    {
        return bits(__hfma2(as(a), as(b), as(c)));
    }
    static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b)
    {
        return bits(__hmul2(as(a), as(b)));
    }
    static __device__ __forceinline__ uint32_t sub(uint32_t a, uint32_t b)
    {
        return bits(__hsub2(as(a), as(b)));
    }
    static __device__ __forceinline__ float to_float(uint16_t h)
    {
        return __uint_as_float(static_cast<uint32_t>(h) << 16);
    }
    static __device__ __forceinline__ uint16_t from_float(float f)
    {
        return __bfloat16_as_ushort(__float2bfloat16_rn(f));
    }
    // Both halves of a packed pair as floats (low half first): two integer ops.
    static __device__ __forceinline__ void unpack2(uint32_t v, float& lo, float& hi)
    {
        lo = __uint_as_float(v << 16);
        hi = __uint_as_float(v & 0xffff0000u);
    }
    static __device__ __forceinline__ void mma(float (&d)[4], uint32_t const (&a)[4], uint32_t b0, uint32_t b1)
    {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    // d = a * b (no accumulator input: starts a chain without zeroing registers first)
    static __device__ __forceinline__ void mma0(float (&d)[4], uint32_t const (&a)[4], uint32_t b0, uint32_t b1)
    {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%10,%10,%10,%10};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
    }
};

// ---------------------------------------------------------------------------------------------
// Converters. Input: one 32-bit register of the preprocessed weight (values biased to unsigned and
// shuffled inside the register, cutlass_preprocessors.cpp:412-489 of the reference project).
// Output: the SIGNED integer values, exact, as packed pairs of T. Pair p of an int4 register
// holds the register's source elements (2p, 2p+1); pair p of an int8 register holds source
// elements (2p, 2p+1) as well (bytes 0,2 then 1,3 after the reference's byte swap).
// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void cvt_int4x8(uint32_t r, uint32_t (&q)[4]);

template <>
__device__ __forceinline__ void cvt_int4x8<__half>(uint32_t r, uint32_t (&q)[4])
{
    // 0x6400 = 1024.0: OR-ing a nibble into the low mantissa bits gives 1024 + u; a nibble four
    // bits higher gives 1024 + 16 u, folded back with one fma.
    constexpr uint32_t kMagic = 0x64006400u;
    constexpr uint32_t kSubLo = 0x64086408u;  // {1032, 1032} = 1024 + 8
    constexpr uint32_t kSixteenth = 0x2c002c00u; // {1/16, 1/16}
    constexpr uint32_t kNeg72 = 0xd480d480u;  // {-72, -72} = -(1024/16 + 8)
    uint32_t const r8 = r >> 8;
    q[0] = Pair<__half>::sub(lop3_and_or(r, 0x000f000fu, kMagic), kSubLo);
    q[1] = Pair<__half>::fma(lop3_and_or(r, 0x00f000f0u, kMagic), kSixteenth, kNeg72);
    q[2] = Pair<__half>::sub(lop3_and_or(r8, 0x000f000fu, kMagic), kSubLo);
    q[3] = Pair<__half>::fma(lop3_and_or(r8, 0x00f000f0u, kMagic), kSixteenth, kNeg72);
}

template <>
__device__ __forceinline__ void cvt_int4x8<__nv_bfloat16>(uint32_t r, uint32_t (&q)[4])
{
    // 0x4300 = 128.0 with a 7-bit mantissa: only a nibble in bits 0..3 stays exact, so shift.
    constexpr uint32_t kMagic = 0x43004300u;
    constexpr uint32_t kSub = 0x43084308u; // {136, 136} = 128 + 8
#pragma unroll
    for (int p = 0; p < 4; ++p)
        q[p] = Pair<__nv_bfloat16>::sub(lop3_and_or(r >> (4 * p), 0x000f000fu, kMagic), kSub);
}

template <typename T>
__device__ __forceinline__ void cvt_int8x4(uint32_t r, uint32_t (&q)[2]);

template <>
__device__ __forceinline__ void cvt_int8x4<__half>(uint32_t r, uint32_t (&q)[2])
{
    constexpr uint32_t kMagic = 0x64646464u;
    constexpr uint32_t kSub = 0x64806480u; // {1152, 1152} = 1024 + 128
    q[0] = Pair<__half>::sub(prmt(r, kMagic, 0x4240u), kSub);
    q[1] = Pair<__half>::sub(prmt(r, kMagic, 0x4341u), kSub);
}

template <>
__device__ __forceinline__ void cvt_int8x4<__nv_bfloat16>(uint32_t r, uint32_t (&q)[2])
{
    // bf16 cannot hold 8 payload bits under a magic exponent, so go through fp32 (2^23 + u) and
    // keep the high halves: integers in [-128, 127] are exact in bf16.
    constexpr uint32_t kMagic = 0x4B000000u;
    constexpr float kBias = 8388608.f + 128.f;
    float f[4];
#pragma unroll
    for (int b = 0; b < 4; ++b)
        f[b] = __uint_as_float(prmt(r, kMagic, 0x7540u | b)) - kBias;
    q[0] = prmt(__float_as_uint(f[0]), __float_as_uint(f[2]), 0x7632u);
    q[1] = prmt(__float_as_uint(f[1]), __float_as_uint(f[3]), 0x7632u);
}

} // namespace w4
