/*
 * C ABI of the B200 weight-only quantised GEMM (W4A16 / W8A16).
 *
 * Every entry point is plain C: pointers, sizes, ints. Nothing here allocates device memory,
 * keeps a caller's pointer after the call returns, synchronises the stream (w4_gemm_run_host apart,
 * whose job that is) or throws; every
 * function that can fail returns a W4Status (0 = success, negative = error) and
 * w4_status_string() names it.
 *
 * What each entry point stands in for in TensorRT-LLM (paths inside that project):
 *   w4_gemm_launch           - weight_only::kernel_launcher(arch, Params&, stream)
 *                              (cpp/tensorrt_llm/kernels/weightOnlyBatchedGemv/kernelLauncher.h:31)
 *                              and CutlassFpAIntBGemmRunnerInterface::gemm(...)
 *                              (cpp/tensorrt_llm/kernels/cutlass_kernels/fpA_intB_gemm/fpA_intB_gemm.h:62-79),
 *                              i.e. the body of WeightOnlyQuantMatmulPlugin::enqueue
 *                              (cpp/tensorrt_llm/plugins/weightOnlyQuantMatmulPlugin/weightOnlyQuantMatmulPlugin.cpp:283-339)
 *                              and WeightOnlyGroupwiseQuantMatmulPlugin::enqueue
 *                              (cpp/tensorrt_llm/plugins/weightOnlyGroupwiseQuantMatmulPlugin/weightOnlyGroupwiseQuantMatmulPlugin.cpp:407-495).
 *   W4GemmParams             - weight_only::Params
 *                              (cpp/tensorrt_llm/kernels/weightOnlyBatchedGemv/common.h:64-102).
 *   w4_gemm_workspace_bytes  - CutlassFpAIntBGemmRunner::getWorkspaceSize (fpA_intB_gemm_template.h:577-581)
 *                              plus the smoothed-activation buffer the groupwise plugin adds
 *                              (weightOnlyGroupwiseQuantMatmulPlugin.cpp:377-379).
 *   w4_gemm_workspace_bytes_max
 *                            - the same, maximised over the optimisation profile's m range, which is
 *                              what getWorkspaceSize reports at configure time
 *                              (m_workspaceMaxSize in configurePlugin, weightOnlyGroupwiseQuantMatmulPlugin.cpp:377-379).
 *   w4_gemm_select_regime    - GemmPluginProfiler::getBestConfig, the reference's per-M choice
 *                              between its CUDA-core GEMV and a CUTLASS tactic
 *                              (cpp/tensorrt_llm/plugins/common/gemmPluginProfiler.cpp:221-250).
 *   w4_symmetric_quantize    - symmetric_quantize<ComputeType, WeightType>
 *                              (cpp/tensorrt_llm/kernels/cutlass_kernels/cutlass_preprocessors.cpp:652-762).
 *   w4_preprocess_weights    - preprocess_weights_for_mixed_gemm (cutlass_preprocessors.cpp:564-615).
 *   w4_preprocess_weights_device / w4_symmetric_quantize_device
 *                            - the same two functions as CUDA kernels on device buffers (the
 *                              reference runs them on one CPU thread only,
 *                              cutlass_preprocessors.cpp:685-758); byte-identical results.
 *   w4_allreduce             - the ncclAllReduce that follows the plugin in a row-parallel layer
 *                              (cpp/tensorrt_llm/plugins/ncclPlugin/allreducePlugin.cpp:407), as a
 *                              peer-memory kernel in the manner of the reference's one-shot / two-shot
 *                              kernels (cpp/tensorrt_llm/kernels/customAllReduceKernels.cu:1307,1426).
 *   w4_gemm_launch_push / w4_gemm_allreduce
 *                            - the decode GEMM with the first half of that all-reduce in its epilogue;
 *                              the reference fuses a GEMM with its all-reduce for dense layers on sm_90
 *                              only (cpp/tensorrt_llm/plugins/gemmAllReducePlugin), never on this path.
 *   w4_preprocess_weights_w4a8 / w4_relayout_w4a8_to_w4a16 / w4_relayout_w4a8_to_w4a16_device
 *                            - preprocess_weights_for_mixed_gemm with QuantType::W4_AFP8
 *                              (cutlass_preprocessors.cpp:114-116) and its conversion into the layout
 *                              the kernels consume (W4A8-AWQ layers).
 *   w4_gemm_launch_experts   - one GEMM per expert over 3-D weights
 *                              (cpp/tensorrt_llm/thop/weightOnlyQuantOp.cpp:136-147 lays them out).
 *   w4_gemm_run_host, w4_gemm_launch_static_scratch
 *                            - no counterpart: host buffers in and out; no workspace from the caller.
 *   w4_pack_int4 / w4_unpack_int4
 *                            - pack_int8_tensor_to_packed_int4 / unpack_int4_packed_tensor_to_int8
 *                              (cpp/tensorrt_llm/thop/weightOnlyQuantOp.cpp:284-353).
 */
#ifndef W4_GEMM_H
#define W4_GEMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C"
{
#endif

    typedef enum W4Status
    {
        W4_OK = 0,
        W4_ERR_NULL_POINTER = -1,   /* a mandatory pointer is null */
        W4_ERR_BAD_SHAPE = -2,      /* m/n/k violate the layout's divisibility rules */
        W4_ERR_BAD_GROUP = -3,      /* group_size not in {0, 64, 128} or does not divide k */
        W4_ERR_BAD_DTYPE = -4,      /* act_dtype / weight_bits not supported */
        W4_ERR_MISALIGNED = -5,     /* a pointer misses the alignment the kernels need */
        W4_ERR_UNSUPPORTED = -6,    /* valid in the reference, not built here (e.g. W4A8 in the C++ plugin classes) */
        W4_ERR_WORKSPACE = -7,      /* workspace missing or smaller than w4_gemm_workspace_bytes() */
        W4_ERR_CUDA = -8,           /* a CUDA runtime call failed; see cudaGetLastError() */
        W4_ERR_BAD_REGIME = -9,     /* regime not valid for this shape */
        W4_ERR_DEVICE_TIMEOUT = -10, /* a bounded device-side wait expired (reported by w4_gemm_device_status) */
        W4_ERR_STATIC_SCRATCH = -11  /* problem too large for w4_gemm_launch_static_scratch's built-in scratch */
    } W4Status;

    /* Activation / scale / output element type (one type for all of them, as in the plugins). */
    enum
    {
        W4_DTYPE_FP16 = 0,
        W4_DTYPE_BF16 = 1,
        W4_DTYPE_FP32 = 2 /* only as the source type of w4_symmetric_quantize_device */
    };

    /* Which kernel family runs. AUTO applies w4_gemm_select_regime(). */
    enum
    {
        W4_REGIME_AUTO = 0,
        W4_REGIME_GEMV = 1, /* streaming decode kernel, any m (re-streams the weights every 8 rows) */
        W4_REGIME_GEMM = 2  /* tcgen05 tensor-core kernel */
    };

    /* quant_algo bits of the groupwise plugin (weightOnlyGroupwiseQuantMatmulPlugin.cpp:33-37). */
    enum
    {
        W4_ALGO_BIAS = 1,
        W4_ALGO_ZERO = 2,
        W4_ALGO_PRE_QUANT_SCALE = 4,
        W4_ALGO_FP8_ALPHA = 8,
        W4_ALGO_INT8_WEIGHT = 16
    };

    /*
     * W4GemmParams.flags.
     * W4_GEMM_WEIGHTS_STATIC: weight, scales, zeros and act_scale were completely written before the
     * kernel that precedes this GEMM on the stream was launched (true for inference weights, which
     * are written once at load time). The decode kernel is a programmatic dependent launch: with
     * this bit it starts fetching those tensors while the preceding kernel is still running and
     * waits for that kernel only before it reads `act` and writes `out`. Without the bit it waits
     * before its first fetch, which is always safe - set it only when the statement above holds
     * (it does NOT hold for a GEMM enqueued right behind w4_symmetric_quantize_device,
     * w4_preprocess_weights_device or any other kernel that writes the weights).
     */
    enum
    {
        W4_GEMM_WEIGHTS_STATIC = 1
    };

    /*
     * out[m, n] = alpha * sum_k (act[m, k] * act_scale[k]) * (q[k, n] * scales[g(k), n] + zeros[g(k), n]) + bias[n]
     *
     *   act        [m, k] row-major, fp16 or bf16 (act_dtype)            device, mandatory
     *   act_scale  [k] same type, AWQ pre-quant scale                     device, optional (NULL = ones)
     *   weight     the bytes produced by w4_preprocess_weights / w4_symmetric_quantize
     *              ([k, n*weight_bits/8] int8)                             device, mandatory
     *   scales     [k/group_size, n] (group_size 64/128) or [n] (group_size 0), same type as act
     *   zeros      same shape as scales, already multiplied by the scale as the reference expects
     *              (tensorrt_llm/quantization/functional.py:1010-1014)    device, optional
     *   bias       [n]                                                    device, optional
     *   out        [m, n] row-major, same type as act                     device, mandatory
     *   n          the real number of output features (not the packed extent)
     *   workspace  scratch of w4_gemm_workspace_bytes(); may be NULL when that is 0. Mandatory only when
     *              act_scale is set and the tensor-core kernel runs (m*k*2 bytes); the rest lets that
     *              kernel split k over idle SMs and is optional (smaller: it runs unsplit)
     */
    typedef struct W4GemmParams
    {
        const void* act;
        const void* act_scale;
        const void* weight;
        const void* scales;
        const void* zeros;
        const void* bias;
        void* out;
        float alpha;
        int m;
        int n;
        int k;
        int group_size;  /* 0 (per output column), 64 or 128 */
        int weight_bits; /* 4 or 8 */
        int act_dtype;   /* W4_DTYPE_* */
        int regime;      /* W4_REGIME_* */
        void* workspace;
        size_t workspace_bytes;
        unsigned flags; /* W4_GEMM_* bits, 0 = none */
    } W4GemmParams;

    int w4_gemm_version(void);
    const char* w4_status_string(int status);

    /* Validates p without touching the device; the same checks w4_gemm_launch runs first. */
    int w4_gemm_validate(const W4GemmParams* p);

    /* Enqueues the GEMM on `stream` (a cudaStream_t; NULL = default stream). m == 0 is a no-op. */
    int w4_gemm_launch(const W4GemmParams* p, void* stream);

    /* w4_gemm_launch for a caller whose activations and result live in host memory (pinned, for the
     * copies to be asynchronous): one call in place of copy-in, enqueue, copy-out and synchronise. No
     * counterpart in the reference, whose plugins only ever see device tensors.
     * Enqueues on `stream`: host_act [m, k] -> p->act, the GEMM, p->out -> host_out [m, n]; returns
     * once the stream has drained, so host_out is valid on return. p->act and p->out are device buffers
     * of the caller, used as staging (their contents afterwards are unspecified: blocks of up to 256 KiB
     * in mapped pinned memory are read and written by kernels directly, without the copy engine);
     * everything else in p as for w4_gemm_launch. Allocates nothing. */
    int w4_gemm_run_host(const W4GemmParams* p, const void* host_act, void* host_out, void* stream);

    /*
     * One GEMM per expert of a mixture-of-experts layer over 3-D weights, enqueued back to back on
     * `stream`. p describes expert 0: weight is [E][K, N*bits/8], every expert's matrix laid out on its
     * own - what preprocess_weights_for_mixed_gemm does with a 3-D tensor
     * (cpp/tensorrt_llm/thop/weightOnlyQuantOp.cpp:136-147, force_interleave); scales / zeros are
     * [E][K/G, N] (or [E][N]), bias [E][N]; act_scale [K] is shared. The rows of act and out are sorted
     * by expert: expert e owns rows expert_first_row[e] .. expert_first_row[e + 1] - 1 (host array of
     * num_experts + 1 non-decreasing ints starting at 0; the running totals the reference's MoE GEMM
     * takes as total_tokens_including_expert,
     * cpp/tensorrt_llm/kernels/internal_cutlass_kernels/include/moe_gemm_kernels.h:236, kept on the host). p->m is ignored; the
     * workspace must cover the largest per-expert row count (w4_gemm_workspace_bytes_max) and is
     * reused by every expert. Experts without rows are skipped. Returns the first error.
     */
    int w4_gemm_launch_experts(const W4GemmParams* p, int num_experts, const int* expert_first_row, void* stream);

    /* Bytes of scratch w4_gemm_launch needs for this problem in the regime it would pick. */
    size_t w4_gemm_workspace_bytes(int m, int n, int k, int group_size, int weight_bits, int act_dtype,
        int has_act_scale, int regime);

    /* The largest w4_gemm_workspace_bytes() over m = 1..max_m: what a plugin reserves at configure
     * time (getWorkspaceSize), since the optional split-k part peaks at small m, not at max_m. */
    size_t w4_gemm_workspace_bytes_max(int max_m, int n, int k, int group_size, int weight_bits, int act_dtype,
        int has_act_scale);

    /* W4_REGIME_GEMV or W4_REGIME_GEMM for this shape: the cost model alone, a pure function of its
     * arguments and the device's SM count. Wherever the library resolves W4_REGIME_AUTO itself (launches
     * and workspace sizes alike) the environment variable W4_FORCE_REGIME = gemv | gemm, read once,
     * overrides it - a debugging and A/B switch in the manner of the reference's
     * FORCE_NCCL_ALL_REDUCE_STRATEGY (cpp/tensorrt_llm/plugins/ncclPlugin/allreducePlugin.cpp:333). */
    int w4_gemm_select_regime(int m, int n, int k, int group_size, int weight_bits);

    /* The same with the activation type (W4_DTYPE_FP16 / W4_DTYPE_BF16), which is what the launches and
     * the workspace sizes use: decode passes over int8 weights cost more with bf16 activations (a
     * byte does not fit a bf16 mantissa and is multiplied as two nibble planes), so the switch to the
     * tensor-core kernel comes earlier there. w4_gemm_select_regime answers for float16. */
    int w4_gemm_select_regime_typed(int m, int n, int k, int group_size, int weight_bits, int act_dtype);

    /* Logging. Levels and names are the reference logger's
     * (cpp/include/tensorrt_llm/common/logger.h:41-48); the level is read once from W4_LOG_LEVEL or,
     * when that is unset, from the reference's TLLM_LOG_LEVEL (TRACE, DEBUG / VERBOSE, INFO, WARNING,
     * ERROR; cpp/tensorrt_llm/common/logger.cpp:30-46), default ERROR. Lines go to stderr:
     * ERROR - a launch failed; WARNING - w4_gemm_launch refused its arguments; DEBUG - one line per
     * w4_gemm_launch with the shape and the kernel taken. w4_set_log_level(level < 0) returns to
     * the environment's setting. */
    enum
    {
        W4_LOG_TRACE = 0,
        W4_LOG_DEBUG = 10,
        W4_LOG_INFO = 20,
        W4_LOG_WARNING = 30,
        W4_LOG_ERROR = 40
    };
    void w4_set_log_level(int level);
    int w4_get_log_level(void);

    /* Reads and clears the device-side status word of the current device (synchronises the
     * device). 0, or W4_ERR_DEVICE_TIMEOUT when a kernel gave up a bounded wait. */
    int w4_gemm_device_status(void);

/* Size of the scratch array built into the library for w4_gemm_launch_static_scratch. */
#define W4_STATIC_SCRATCH_BYTES (8u * 1024u * 1024u)

    /*
     * Same contract as w4_gemm_launch, for callers that can neither allocate device memory nor
     * pass a workspace (allocation-free regions of a serving loop, plugin hosts that granted no
     * workspace, processes in which another component owns the allocator). It always runs the
     * tensor-core kernel and keeps that kernel's scratch - the activations multiplied by the AWQ
     * pre-quant scale, m * k * 2 bytes, and, for shapes with few output tiles when the rest of the
     * array has room, the fp32 partial tiles of its split-k behind them - in a
     * W4_STATIC_SCRATCH_BYTES (8 MiB) array that is part of the library image. This entry point has no counterpart in the reference.
     *   - p->workspace / p->workspace_bytes are ignored; nothing is allocated or freed, here or
     *     in any library it calls.
     *   - m * k * 2 > W4_STATIC_SCRATCH_BYTES with act_scale set returns W4_ERR_STATIC_SCRATCH
     *     (for example m = 512, k = 8192 still fits; m = 4096, k = 4096 does not).
     *   - The first call on each device resolves the array's device address; make that call
     *     before starting any stream capture on that device.
     *   - All calls on a device share the one array, which still holds the previous call's data;
     *     the kernel overwrites everything it reads, so nothing needs clearing, but two calls
     *     whose execution overlaps on the GPU (different streams) would race on it: serialise
     *     them.
     *   - Every GPU that loads the library gives up 8 MiB for the array until the process exits.
     */
    int w4_gemm_launch_static_scratch(const W4GemmParams* p, void* stream);
    size_t w4_gemm_static_scratch_bytes(void);

    /* ---- host-side (CPU) weight preparation, bit-exact with the reference ---- */

    /* weight: fp32 [k, n] row-major. processed / unprocessed: [k, n*bits/8] bytes (unprocessed may
     * be NULL). scales: fp32 [n], the unrounded per-column scale amax * 2^-(bits-1); round it to
     * fp16 / bf16 (nearest even) for the device. */
    int w4_symmetric_quantize(int8_t* processed, int8_t* unprocessed, float* scales, const float* weight, size_t k,
        size_t n, int bits);

    /* in: [k, n*bits/8] row-major two's-complement weights (int4: even column in the low nibble). */
    int w4_preprocess_weights(int8_t* out, const int8_t* in, size_t k, size_t n, int bits);

    /* int4 weights in the layout the reference produces when the activation type is fp8 (W4A8-AWQ:
     * preprocess_weights_for_mixed_gemm with QuantType::W4_AFP8, cutlass_preprocessors.cpp:114-116,
     * 175-179: two interleaved columns, 128-row tiles, its own row permutation). in: [k, n/2] row-major
     * two's-complement nibbles; k % 128 == 0, n % 64 == 0. Same bytes as the reference. */
    int w4_preprocess_weights_w4a8(int8_t* out, const int8_t* in, size_t k, size_t n);

    /* W4A8-layout bytes (above) -> the W4A16 layout the kernels of this library consume; done once
     * when the weights are loaded. After it, a W4A8-AWQ layer (quant_algo & FP8_ALPHA,
     * weightOnlyGroupwiseQuantMatmulPlugin.cpp:206-218) is w4_gemm_launch with alpha set and the
     * float16 scales / zeros converted to the activation type; the activations stay 16-bit, as in the
     * reference's own GEMV path for W4A8 (weightOnlyBatchedGemv/utility.h:136-147). */
    int w4_relayout_w4a8_to_w4a16(int8_t* out, const int8_t* in, size_t k, size_t n);

    int w4_pack_int4(int8_t* packed, const int8_t* unpacked, size_t num_packed_bytes);
    void w4_unpack_int4(int8_t* unpacked, const int8_t* packed, size_t num_packed_bytes);

    /* ---- the same weight preparation on the GPU (device pointers, stream-ordered, no allocation) ---- */

    /* in / out: [k, n*bits/8] bytes on the device, 16-byte aligned, out != in. Same bytes as
     * w4_preprocess_weights. */
    int w4_preprocess_weights_device(void* out, const void* in, size_t k, size_t n, int bits, void* stream);

    /* w4_relayout_w4a8_to_w4a16 on device buffers: in / out [k, n/2] bytes, 16-byte aligned, out != in;
     * k % 128 == 0, n % 64 == 0. Same bytes as the host function. */
    int w4_relayout_w4a8_to_w4a16_device(void* out, const void* in, size_t k, size_t n, void* stream);

    /* weight: [k, n] row-major on the device, weight_dtype = W4_DTYPE_FP32 / FP16 / BF16 (the
     * reference's ComputeType). processed (mandatory) and unprocessed (optional) as in
     * w4_symmetric_quantize; scales: fp32 [n] (mandatory, also used as scratch for the column
     * maxima); scales_t: optional copy rounded to scales_dtype (fp16 / bf16), which is what the
     * GEMM takes. Same bytes and scale values as the host function. */
    int w4_symmetric_quantize_device(void* processed, void* unprocessed, float* scales, void* scales_t,
        int scales_dtype, const void* weight, int weight_dtype, size_t k, size_t n, int bits, void* stream);

    /* ---- row-parallel reduce over peer memory (one process per GPU, one node) ---- */

#define W4_MAX_RANKS 8
#define W4_ONESHOT_MAX_BYTES (1u << 20) /* largest message the one-shot form takes */
#define W4_ALLREDUCE_MAX_CTAS 128       /* chunks a message (one-shot) or a slice (two-shot) is cut into */
#define W4_ALLREDUCE_LL_MAX_BYTES (4u << 20) /* up to here data travels as flagged packets (no fences) */

    enum
    {
        W4_ALLREDUCE_AUTO = 0,     /* by message size, the reference's rule (allreducePlugin.cpp:258-283) */
        W4_ALLREDUCE_ONE_SHOT = 1, /* push the whole partial to every peer, reduce locally */
        W4_ALLREDUCE_TWO_SHOT = 2, /* push slices to their owners, reduce, hand the reduced slices round */
        W4_ALLREDUCE_GATHER_ONLY = 3 /* one-shot whose pushes were already made by w4_gemm_launch_push */
    };

    /*
     * out[i] = sum over ranks r = 0..world-1 (in that order, fp32) of partial_r[i]  (+ bias[i % n])
     * on every rank, bit-identical across ranks.
     *
     *   partial      THIS rank's [count] partial sums (fp16 / bf16): plain local device memory, typically
     *                the W4GemmParams.out of the row-parallel GEMM enqueued just before on the same stream.
     *   workspace[r] rank r's workspace block as mapped into THIS process: the local block for
     *                r == rank, a peer mapping (CUDA IPC / symmetric memory) otherwise. Every block is
     *                w4_allreduce_workspace_bytes(max_message_bytes, world) bytes, 256-byte aligned and
     *                ZERO before the first call (all ranks must have seen the zeroing before anyone calls).
     *                workspace_bytes is that size.
     *   mode         W4_ALLREDUCE_*; must be the same on every rank for a given call.
     *   timeout_ms   bound on every wait for the peers (0 = 2000). When it expires the kernel gives up,
     *                `out` is undefined, w4_gemm_device_status() returns W4_ERR_DEVICE_TIMEOUT and the
     *                workspace must be zeroed again on all ranks before further use.
     * count % 8 == 0, n % 8 == 0, count % n == 0; partial, out, bias 16-byte aligned; count * 2 bytes must
     * not exceed the max_message_bytes the workspace was sized for (one-shot: W4_ONESHOT_MAX_BYTES).
     * All ranks make the same sequence of calls. The call number is kept in the workspace on the device,
     * so a captured CUDA graph containing these calls can be replayed any number of times. Calls that
     * share a workspace must not overlap on the GPU (one stream). Allocates nothing.
     * Stands in for the ncclAllReduce behind the plugin in a row-parallel layer
     * (cpp/tensorrt_llm/plugins/ncclPlugin/allreducePlugin.cpp:407), in the manner of the reference's
     * custom all-reduce kernels (cpp/tensorrt_llm/kernels/customAllReduceKernels.cu:1307,1426).
     */
    typedef struct W4AllReduceParams
    {
        const void* partial;
        void* workspace[W4_MAX_RANKS];
        size_t workspace_bytes;
        const void* bias; /* optional, [n] */
        void* out;        /* local, [count] */
        size_t count;
        int n;
        int rank, world;
        int act_dtype; /* W4_DTYPE_FP16 / W4_DTYPE_BF16 */
        int mode;      /* W4_ALLREDUCE_* */
        uint32_t timeout_ms;
    } W4AllReduceParams;

    /* Bytes of one rank's workspace block for messages of up to max_message_bytes. 0 for bad arguments. */
    size_t w4_allreduce_workspace_bytes(size_t max_message_bytes, int world);

    int w4_allreduce(const W4AllReduceParams* p, void* stream);

    /*
     * The row-parallel decode GEMM with the first half of its all-reduce fused into the epilogue: the
     * kernel writes its partial sums to p->out (== r->partial) AND sends them, as the flagged packets
     * of the one-shot protocol, straight into every peer's inbox, so the reduce that follows only has
     * to gather: call w4_allreduce with mode W4_ALLREDUCE_GATHER_ONLY next on the same stream (same r
     * otherwise). Saves the reduce kernel's own pass over the partial sums and lets the data cross
     * NVLink while the GEMM is still finishing. Applies to int4 weights in the decode regime without a
     * bias (the bias belongs to the reduce: r->bias) when the message would use the one-shot packet
     * protocol; otherwise W4_ERR_UNSUPPORTED is returned and nothing has been launched.
     * The second half of f1 of the reference's road map (gemmAllReducePlugin fuses a dense GEMM with
     * its all-reduce on sm_90, cpp/tensorrt_llm/plugins/gemmAllReducePlugin; never for weight-only).
     */
    int w4_gemm_launch_push(const W4GemmParams* p, const W4AllReduceParams* r, void* stream);

    /* GEMM followed by the all-reduce of its output, in the most fused form that applies:
     *   - up to 16 rows, int4, decode regime, one-shot packet size: ONE kernel. The decode kernel's
     *     epilogue pushes its results into every rank's inbox, collects the peers' packets for the
     *     columns it owns (bounded wait, r->timeout_ms), adds them in rank order in fp32 (+ r->bias),
     *     writes r->out and advances the workspace's call number. r->partial is not written.
     *   - more rows in the decode regime: w4_gemm_launch_push, then the gather-only reduce;
     *   - otherwise: w4_gemm_launch, then w4_allreduce (r->mode).
     * p->out must be r->partial; p->bias must be NULL (the bias of a row-parallel layer is r->bias).
     * All ranks must make the same call with the same shapes, as with any collective. */
    int w4_gemm_allreduce(const W4GemmParams* p, const W4AllReduceParams* r, void* stream);

    /* The calls of all `world` ranks as ONE cooperative launch on the current GPU: ranks[r] describes
     * rank r, every workspace pointer is local memory. For machines with fewer GPUs than ranks (tests,
     * debugging): separate launches that wait for one another must never share a GPU. */
    int w4_allreduce_emulated(const W4AllReduceParams* ranks, int world, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* W4_GEMM_H */
