// The C ABI declared in include/w4_gemm.h: argument validation, the M-based regime choice and
// dispatch into the two kernel families. Nothing here allocates; only w4_gemm_run_host synchronises.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "w4_common.cuh"
#include "w4_internal.h"

namespace w4
{

DeviceInfo const& current_device_info()
{
    static DeviceInfo infos[64];
    static std::mutex mu;
    static DeviceInfo invalid;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
        return invalid;
    std::lock_guard<std::mutex> lock(mu);
    DeviceInfo& d = infos[dev];
    if (d.device != dev)
    {
        int sms = 0, smem = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess
            || cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess)
            return invalid;
        d.num_sms = sms;
        d.max_smem_optin = smem;
        d.device = dev;
    }
    return d;
}

// ------------------------------------------------------------------------------------------------
// act[m, k] * scale[k] -> out, rounded to the element type. Counterpart of the reference's
// apply_per_channel_scale (cpp/tensorrt_llm/kernels/preQuantScaleKernel.cu:43-95); used in front
// of the tensor-core kernel only (the decode kernel fuses the product into its activation load).
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void pre_quant_scale_kernel(uint4* out, uint4 const* act, uint4 const* scale, size_t total_vec, int k_vec)
{
    using P = Pair<T>;
    size_t const stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total_vec; i += stride)
    {
        uint4 a = act[i];
        uint4 const s = __ldg(scale + (i % k_vec));
        a.x = P::mul(a.x, s.x);
        a.y = P::mul(a.y, s.y);
        a.z = P::mul(a.z, s.z);
        a.w = P::mul(a.w, s.w);
        out[i] = a;
    }
}

int launch_pre_quant_scale(void* out, void const* act, void const* scale, int m, int k, int act_dtype,
    cudaStream_t stream)
{
    DeviceInfo const& dev = current_device_info();
    if (dev.num_sms <= 0)
        return W4_ERR_CUDA;
    size_t const total_vec = size_t(m) * k / 8;
    int const threads = 256;
    size_t blocks = (total_vec + threads - 1) / threads;
    size_t const cap = size_t(dev.num_sms) * 8;
    if (blocks > cap)
        blocks = cap;
    if (blocks == 0)
        return W4_OK;
    if (act_dtype == W4_DTYPE_FP16)
        pre_quant_scale_kernel<__half><<<unsigned(blocks), threads, 0, stream>>>(static_cast<uint4*>(out),
            static_cast<uint4 const*>(act), static_cast<uint4 const*>(scale), total_vec, k / 8);
    else
        pre_quant_scale_kernel<__nv_bfloat16><<<unsigned(blocks), threads, 0, stream>>>(static_cast<uint4*>(out),
            static_cast<uint4 const*>(act), static_cast<uint4 const*>(scale), total_vec, k / 8);
    return cudaGetLastError() == cudaSuccess ? W4_OK : W4_ERR_CUDA;
}

// Stages a small activation block from mapped pinned host memory into device memory: the loads cross
// PCIe, the kernel that follows on the stream may start at once (it waits for this one before it
// touches the activations) and fetch its weights meanwhile. Takes the place of a copy-engine transfer,
// whose fixed cost is several microseconds.
__global__ void stage_in_kernel(uint4* dst, uint4 const* src, size_t vecs)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    size_t const stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs; i += stride)
        dst[i] = src[i];
}

} // namespace w4

namespace
{

// Device-visible address of a host pointer when it is pinned, mapped and 16-byte aligned, else null.
void* mapped_device_pointer(void const* host)
{
    cudaPointerAttributes at{};
    if (cudaPointerGetAttributes(&at, host) != cudaSuccess)
    {
        (void) cudaGetLastError();
        return nullptr;
    }
    if (at.type != cudaMemoryTypeHost || !at.devicePointer || (reinterpret_cast<uintptr_t>(at.devicePointer) & 15u))
        return nullptr;
    return at.devicePointer;
}

bool aligned16(void const* p)
{
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

// Logger: the levels and level names of the reference's (cpp/include/tensorrt_llm/common/logger.h:41-48,
// cpp/tensorrt_llm/common/logger.cpp:30-46), read once from W4_LOG_LEVEL or, failing that, from the
// reference's own TLLM_LOG_LEVEL; ERROR when neither is set. Everything goes to stderr.
std::atomic<int> g_log_level{-1};

int level_from_name(char const* name)
{
    if (!name)
        return -1;
    if (!std::strcmp(name, "TRACE"))
        return W4_LOG_TRACE;
    if (!std::strcmp(name, "DEBUG") || !std::strcmp(name, "VERBOSE"))
        return W4_LOG_DEBUG;
    if (!std::strcmp(name, "INFO"))
        return W4_LOG_INFO;
    if (!std::strcmp(name, "WARNING"))
        return W4_LOG_WARNING;
    if (!std::strcmp(name, "ERROR"))
        return W4_LOG_ERROR;
    return -1;
}

int log_level()
{
    int level = g_log_level.load(std::memory_order_relaxed);
    if (level < 0)
    {
        level = level_from_name(std::getenv("W4_LOG_LEVEL"));
        if (level < 0)
            level = level_from_name(std::getenv("TLLM_LOG_LEVEL"));
        if (level < 0)
            level = W4_LOG_ERROR;
        g_log_level.store(level, std::memory_order_relaxed);
    }
    return level;
}

void log_line(int level, char const* fmt, ...)
{
    if (level < log_level())
        return;
    char const* name = level >= W4_LOG_ERROR ? "ERROR"
        : level >= W4_LOG_WARNING            ? "WARNING"
        : level >= W4_LOG_INFO               ? "INFO"
        : level >= W4_LOG_DEBUG              ? "DEBUG"
                                             : "TRACE";
    char text[512];
    va_list args;
    va_start(args, fmt);
    std::vsnprintf(text, sizeof text, fmt, args);
    va_end(args);
    std::fprintf(stderr, "[w4_gemm][%s] %s\n", name, text);
}

// W4_FORCE_REGIME = gemv | gemm overrides the cost model wherever the regime is left to the library
// (launches and workspace sizes alike); read once. For debugging and A/B timing, like the reference's
// FORCE_NCCL_ALL_REDUCE_STRATEGY (cpp/tensorrt_llm/plugins/ncclPlugin/allreducePlugin.cpp:333).
int forced_regime()
{
    static int const forced = []
    {
        char const* v = std::getenv("W4_FORCE_REGIME");
        if (v && !std::strcmp(v, "gemv"))
            return int(W4_REGIME_GEMV);
        if (v && !std::strcmp(v, "gemm"))
            return int(W4_REGIME_GEMM);
        if (v && *v)
            log_line(W4_LOG_WARNING, "W4_FORCE_REGIME=%s ignored (expected gemv or gemm)", v);
        return int(W4_REGIME_AUTO);
    }();
    return forced;
}

int auto_regime(int m, int n, int k, int group_size, int weight_bits, int act_dtype)
{
    int const f = forced_regime();
    return f != W4_REGIME_AUTO ? f : w4_gemm_select_regime_typed(m, n, k, group_size, weight_bits, act_dtype);
}

int resolve_regime(W4GemmParams const& p)
{
    if (p.regime == W4_REGIME_GEMV || p.regime == W4_REGIME_GEMM)
        return p.regime;
    return auto_regime(p.m, p.n, p.k, p.group_size, p.weight_bits, p.act_dtype);
}

void log_refusal(char const* entry, W4GemmParams const* p, int rc)
{
    if (log_level() > W4_LOG_WARNING)
        return;
    if (!p)
        log_line(W4_LOG_WARNING, "%s refused: %s", entry, w4_status_string(rc));
    else
        log_line(W4_LOG_WARNING, "%s refused: %s (m=%d n=%d k=%d bits=%d group=%d regime=%d)", entry,
            w4_status_string(rc), p->m, p->n, p->k, p->weight_bits, p->group_size, p->regime);
}

} // namespace

extern "C"
{

    int w4_gemm_version(void)
    {
        return 112;
    }

    const char* w4_status_string(int status)
    {
        switch (status)
        {
        case W4_OK: return "ok";
        case W4_ERR_NULL_POINTER: return "a mandatory pointer is null";
        case W4_ERR_BAD_SHAPE: return "unsupported shape (need k % 64 == 0 and n % 64 == 0 (int4) / n % 32 == 0 (int8))";
        case W4_ERR_BAD_GROUP: return "group_size must be 0, 64 or 128 and divide k";
        case W4_ERR_BAD_DTYPE: return "act_dtype must be fp16/bf16 and weight_bits 4 or 8";
        case W4_ERR_MISALIGNED: return "pointers must be 16-byte aligned";
        case W4_ERR_UNSUPPORTED: return "valid in the reference but not supported by this library";
        case W4_ERR_WORKSPACE: return "workspace missing or too small";
        case W4_ERR_CUDA: return "CUDA runtime error";
        case W4_ERR_BAD_REGIME: return "regime not valid for this problem";
        case W4_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait expired";
        case W4_ERR_STATIC_SCRATCH: return "m * k * 2 bytes exceed the built-in scratch of w4_gemm_launch_static_scratch";
        default: return "unknown status";
        }
    }

    int w4_gemm_validate(const W4GemmParams* p)
    {
        if (!p)
            return W4_ERR_NULL_POINTER;
        if (p->act_dtype != W4_DTYPE_FP16 && p->act_dtype != W4_DTYPE_BF16)
            return W4_ERR_BAD_DTYPE;
        if (p->weight_bits != 4 && p->weight_bits != 8)
            return W4_ERR_BAD_DTYPE;
        if (p->m < 0 || p->n <= 0 || p->k <= 0)
            return W4_ERR_BAD_SHAPE;
        // k: whole 64-wide tiles (fpA_intB_gemm_template.h:191-196 of the reference); n: what the
        // reference's own preprocessing accepts (cutlass_preprocessors.cpp:280-283).
        if (p->k % 64 != 0 || (p->n * p->weight_bits / 8) % 32 != 0)
            return W4_ERR_BAD_SHAPE;
        if (p->group_size != 0 && p->group_size != 64 && p->group_size != 128)
            return W4_ERR_BAD_GROUP;
        if (p->group_size != 0 && p->k % p->group_size != 0)
            return W4_ERR_BAD_GROUP;
        if (p->regime != W4_REGIME_AUTO && p->regime != W4_REGIME_GEMV && p->regime != W4_REGIME_GEMM)
            return W4_ERR_BAD_REGIME;
        if (p->m == 0)
            return W4_OK;
        if (!p->act || !p->weight || !p->scales || !p->out)
            return W4_ERR_NULL_POINTER;
        if (!aligned16(p->act) || !aligned16(p->weight) || !aligned16(p->scales) || !aligned16(p->out)
            || !aligned16(p->act_scale) || !aligned16(p->zeros) || !aligned16(p->bias) || !aligned16(p->workspace))
            return W4_ERR_MISALIGNED;
        // Mandatory part only (the scaled activation copy of the tensor-core path); the rest of
        // w4_gemm_workspace_bytes() enables split-k and is optional.
        size_t const need = resolve_regime(*p) == W4_REGIME_GEMM
            ? w4::gemm_tc_workspace_min(p->m, p->k, p->act_scale != nullptr)
            : 0;
        if (need > 0 && (!p->workspace || p->workspace_bytes < need))
            return W4_ERR_WORKSPACE;
        return W4_OK;
    }

    int w4_gemm_select_regime(int m, int n, int k, int group_size, int weight_bits)
    {
        return w4_gemm_select_regime_typed(m, n, k, group_size, weight_bits, W4_DTYPE_FP16);
    }

    int w4_gemm_select_regime_typed(int m, int n, int k, int group_size, int weight_bits, int act_dtype)
    {
        (void) group_size;
        if (m <= 8)
            return W4_REGIME_GEMV; // one pass over the weights
        // Cost model fitted to measurements on B200 (microseconds). The decode kernel passes over the
        // packed weights once per 16 rows while more than 8 rows are left, then once for up to 8:
        // an 8-row pass costs 4.2 us plus the weight bytes at 3.4 TB/s (config 2: 12.1 us; 4096 x 4096
        // int4: 6.6 us), a 16-row pass 6.3 us plus the bytes at 2.7 TB/s for int4 (config 2: 17.2 us;
        // 4096 x 1024: 6.8 us) and 3.5 us plus the bytes at 3.2 TB/s for int8, whose narrower units let
        // a 16-row tile cover as much k as an 8-row one (4096 x 4096: 7.8 us; 4096 x 14336: 20-23 us);
        // bf16 activations with int8 weights need two mma planes per byte: 5.0 us plus the bytes at
        // 3.1 TB/s (4096 x 1024: 6.4 us; 4096 x 4096: 9.6 us; 4096 x 14336: 23.6 us).
        // The tensor-core kernel's
        // estimate comes from its own per-step costs. The SM count is the current device's (148 when
        // no device is present).
        w4::DeviceInfo const& dev = w4::current_device_info();
        int const sms = dev.num_sms > 0 ? dev.num_sms : 148;
        double const weight_mb = double(n) * double(k) * weight_bits / 8.0 / 1.0e6;
        int passes16 = 0, left = m;
        while (left > 8)
        {
            ++passes16;
            left -= left < 16 ? left : 16;
        }
        double const pass16_us = weight_bits == 8
            ? (act_dtype == W4_DTYPE_BF16 ? weight_mb / 3.1 + 5.0 : weight_mb / 3.2 + 3.5)
            : weight_mb / 2.7 + 6.3;
        double const gemv_us = passes16 * pass16_us + (left > 0 ? weight_mb / 3.4 + 4.2 : 0.0);
        double const gemm_us = w4::gemm_tc_estimate_us(m, n, k, sms, weight_bits);
        return gemv_us <= gemm_us ? W4_REGIME_GEMV : W4_REGIME_GEMM;
    }

    size_t w4_gemm_workspace_bytes(int m, int n, int k, int group_size, int weight_bits, int act_dtype,
        int has_act_scale, int regime)
    {
        if (m <= 0)
            return 0;
        int r = regime;
        if (r != W4_REGIME_GEMV && r != W4_REGIME_GEMM)
            r = auto_regime(m, n, k, group_size, weight_bits, act_dtype);
        if (r == W4_REGIME_GEMV)
            return 0;
        return w4::gemm_tc_workspace_bytes(m, n, k, has_act_scale, weight_bits);
    }

    size_t w4_gemm_workspace_bytes_max(int max_m, int n, int k, int group_size, int weight_bits, int act_dtype,
        int has_act_scale)
    {
        size_t best = 0;
        // split-k is only used up to 256 rows; beyond that the size grows with m (or is zero)
        for (int m = 1; m <= max_m && m <= 256; ++m)
        {
            size_t const b = w4_gemm_workspace_bytes(m, n, k, group_size, weight_bits, act_dtype, has_act_scale,
                W4_REGIME_AUTO);
            best = b > best ? b : best;
        }
        if (max_m > 256)
        {
            size_t const b = w4_gemm_workspace_bytes(max_m, n, k, group_size, weight_bits, act_dtype, has_act_scale,
                W4_REGIME_GEMM);
            best = b > best ? b : best;
        }
        return best;
    }

    void w4_set_log_level(int level)
    {
        g_log_level.store(level < 0 ? -1 : level, std::memory_order_relaxed); // negative: back to the environment
    }

    int w4_get_log_level(void)
    {
        return log_level();
    }

    int w4_gemm_launch(const W4GemmParams* p, void* stream)
    {
        int rc = w4_gemm_validate(p);
        if (rc != W4_OK)
        {
            log_refusal("w4_gemm_launch", p, rc);
            return rc;
        }
        if (p->m == 0)
            return W4_OK;
        cudaStream_t const s = static_cast<cudaStream_t>(stream);
        bool const gemv = resolve_regime(*p) == W4_REGIME_GEMV;
        if (log_level() <= W4_LOG_DEBUG)
            log_line(W4_LOG_DEBUG, "w4_gemm_launch m=%d n=%d k=%d bits=%d group=%d zeros=%d bias=%d act_scale=%d alpha=%g %s%s",
                p->m, p->n, p->k, p->weight_bits, p->group_size, p->zeros != nullptr, p->bias != nullptr,
                p->act_scale != nullptr, double(p->alpha), gemv ? "decode kernel" : "tensor-core kernel",
                p->regime == W4_REGIME_AUTO ? " (chosen)" : " (requested)");
        rc = gemv ? w4::launch_gemv(*p, s) : w4::launch_gemm_tc(*p, s);
        if (rc != W4_OK)
            log_line(W4_LOG_ERROR, "w4_gemm_launch failed: %s (m=%d n=%d k=%d bits=%d group=%d)", w4_status_string(rc),
                p->m, p->n, p->k, p->weight_bits, p->group_size);
        return rc;
    }

    int w4_gemm_launch_push(const W4GemmParams* p, const W4AllReduceParams* r, void* stream)
    {
        if (!p || !r)
            return W4_ERR_NULL_POINTER;
        // Only the decode kernel on int4 weights has the pushing epilogue, and only the one-shot packet
        // protocol of the all-reduce takes packets from it; the bias belongs to the reduce. (Asked
        // before the validation, which would demand the tensor-core kernel's workspace.)
        if (p->m <= 0 || p->weight_bits != 4 || p->bias || resolve_regime(*p) != W4_REGIME_GEMV)
            return W4_ERR_UNSUPPORTED;
        int const rc = w4_gemm_validate(p);
        if (rc != W4_OK)
            return rc;
        if (p->out != r->partial || r->count != size_t(p->m) * size_t(p->n) || r->n != p->n
            || r->act_dtype != p->act_dtype)
            return W4_ERR_BAD_SHAPE;
        w4::PushTarget t{};
        if (!w4::allreduce_push_target(*r, &t))
            return W4_ERR_UNSUPPORTED;
        return w4::launch_gemv(*p, static_cast<cudaStream_t>(stream), &t);
    }

    int w4_gemm_allreduce(const W4GemmParams* p, const W4AllReduceParams* r, void* stream)
    {
        if (!p || !r)
            return W4_ERR_NULL_POINTER;
        // Up to 16 rows are one launch of the decode kernel: it can do the whole call itself - push
        // its results, collect the peers', add and write r->out - and advance the call number.
        if (p->m > 0 && p->m <= 16 && p->weight_bits == 4 && !p->bias && resolve_regime(*p) == W4_REGIME_GEMV
            && p->out == r->partial && r->count == size_t(p->m) * size_t(p->n) && r->n == p->n
            && r->act_dtype == p->act_dtype && r->out)
        {
            w4::PushTarget t{};
            if (w4::allreduce_push_target(*r, &t))
            {
                int const vrc = w4_gemm_validate(p);
                if (vrc != W4_OK)
                    return vrc;
                t.gather = 1;
                t.bias = r->bias;
                W4GemmParams g = *p;
                g.out = r->out;
                return w4::launch_gemv(g, static_cast<cudaStream_t>(stream), &t);
            }
        }
        int rc = w4_gemm_launch_push(p, r, stream);
        W4AllReduceParams q = *r;
        if (rc == W4_OK)
            q.mode = W4_ALLREDUCE_GATHER_ONLY;
        else if (rc == W4_ERR_UNSUPPORTED)
            rc = w4_gemm_launch(p, stream);
        if (rc != W4_OK)
            return rc;
        return w4_allreduce(&q, stream);
    }

    int w4_gemm_launch_experts(const W4GemmParams* p, int num_experts, const int* expert_first_row, void* stream)
    {
        if (!p || !expert_first_row)
            return W4_ERR_NULL_POINTER;
        if (num_experts < 1 || expert_first_row[0] != 0)
            return W4_ERR_BAD_SHAPE;
        for (int e = 0; e < num_experts; ++e)
            if (expert_first_row[e + 1] < expert_first_row[e])
                return W4_ERR_BAD_SHAPE;
        size_t const elt = 2;
        size_t const groups = p->group_size ? size_t(p->k) / size_t(p->group_size) : 1;
        size_t const weight_bytes = size_t(p->k) * p->n * p->weight_bits / 8;
        auto at = [](const void* base, size_t bytes) -> const void*
        { return base ? static_cast<const char*>(base) + bytes : nullptr; };
        for (int e = 0; e < num_experts; ++e)
        {
            int const row0 = expert_first_row[e], rows = expert_first_row[e + 1] - row0;
            if (rows == 0)
                continue;
            W4GemmParams q = *p;
            q.m = rows;
            q.act = at(p->act, size_t(row0) * p->k * elt);
            q.out = const_cast<void*>(at(p->out, size_t(row0) * p->n * elt));
            q.weight = at(p->weight, size_t(e) * weight_bytes);
            q.scales = at(p->scales, size_t(e) * groups * p->n * elt);
            q.zeros = at(p->zeros, size_t(e) * groups * p->n * elt);
            q.bias = at(p->bias, size_t(e) * p->n * elt);
            int const rc = w4_gemm_launch(&q, stream);
            if (rc != W4_OK)
                return rc;
        }
        return W4_OK;
    }

    int w4_gemm_run_host(const W4GemmParams* p, const void* host_act, void* host_out, void* stream)
    {
        int const rc = w4_gemm_validate(p);
        if (rc != W4_OK)
            return rc;
        if (p->m == 0)
            return W4_OK;
        if (!host_act || !host_out)
            return W4_ERR_NULL_POINTER;
        cudaStream_t const s = static_cast<cudaStream_t>(stream);
        size_t const elt = 2;
        size_t const in_bytes = size_t(p->m) * p->k * elt, out_bytes = size_t(p->m) * p->n * elt;
        // Decode-sized blocks in mapped pinned memory skip the copy engine in both directions: a small
        // kernel loads the activations across PCIe and the GEMM stores its result straight into the
        // host buffer. Anything else (pageable or unaligned host memory, large blocks) is copied.
        constexpr size_t kDirectMax = 256 * 1024;
        void* const in_dev = in_bytes <= kDirectMax ? mapped_device_pointer(host_act) : nullptr;
        void* const out_dev = out_bytes <= kDirectMax ? mapped_device_pointer(host_out) : nullptr;
        if (in_dev)
        {
            size_t const vecs = in_bytes / 16; // k % 64 == 0: whole vectors
            unsigned const blocks = unsigned((vecs + 255) / 256 < 64 ? (vecs + 255) / 256 : 64);
            w4::stage_in_kernel<<<blocks, 256, 0, s>>>(
                static_cast<uint4*>(const_cast<void*>(p->act)), static_cast<uint4 const*>(in_dev), vecs);
            if (cudaGetLastError() != cudaSuccess)
                return W4_ERR_CUDA;
        }
        else if (cudaMemcpyAsync(const_cast<void*>(p->act), host_act, in_bytes, cudaMemcpyHostToDevice, s) != cudaSuccess)
            return W4_ERR_CUDA;
        // The activations were just written by the work in front: an ordinary dependency, which the
        // kernels honour; the weights keep whatever the caller declared in `flags`.
        W4GemmParams q = *p;
        if (out_dev)
            q.out = out_dev;
        int const lrc = resolve_regime(q) == W4_REGIME_GEMV ? w4::launch_gemv(q, s) : w4::launch_gemm_tc(q, s);
        if (lrc != W4_OK)
            return lrc;
        if (!out_dev && cudaMemcpyAsync(host_out, p->out, out_bytes, cudaMemcpyDeviceToHost, s) != cudaSuccess)
            return W4_ERR_CUDA;
        return cudaStreamSynchronize(s) == cudaSuccess ? W4_OK : W4_ERR_CUDA;
    }

    int w4_gemm_device_status(void)
    {
        int v = 0, zero = 0;
        if (cudaMemcpyFromSymbol(&v, w4::g_device_status, sizeof(int)) != cudaSuccess)
            return W4_ERR_CUDA;
        if (v != 0 && cudaMemcpyToSymbol(w4::g_device_status, &zero, sizeof(int)) != cudaSuccess)
            return W4_ERR_CUDA;
        return v;
    }

} // extern "C"
