// torch.ops.trtllm bindings of the weight-only GEMM library (C++ side of the operator boundary).
//
// Host ops: same names, schemas, checks and return shapes as the reference's
// cpp/tensorrt_llm/thop/weightOnlyQuantOp.cpp:123-151,153-251,284-385 (CPU tensors in, CPU tensors
// out); they call the C ABI of libw4gemm.so (w4_symmetric_quantize, w4_preprocess_weights,
// w4_pack_int4, w4_unpack_int4), whose results are byte-identical to the reference's.
//
// GEMM ops: that reference version has no torch op for the weight-only GEMM (only the TensorRT
// plugins); these two follow the conventions of its other GEMM ops
// (cpp/tensorrt_llm/thop/cutlassScaledMM.cpp:121-175: TORCH_LIBRARY_FRAGMENT + TORCH_LIBRARY_IMPL for
// CUDA, CUDA-tensor checks as in thop/thUtils.h:32-49, output allocated on the input's device, the
// current stream) and take the tensors in the order the plugins do
// (plugins/weightOnlyQuantMatmulPlugin/weightOnlyQuantMatmulPlugin.cpp:287-292,
//  plugins/weightOnlyGroupwiseQuantMatmulPlugin/weightOnlyGroupwiseQuantMatmulPlugin.cpp:411-419).
// There is no CPU implementation of the GEMM ops: calling them with CPU tensors is a dispatch error.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <string>
#include <vector>

#include "../../include/w4_gemm.h"

namespace
{

using at::Tensor;

int quant_bits(at::ScalarType quant_type)
{
    TORCH_CHECK(quant_type == at::kChar || quant_type == at::kQUInt4x2, "Must be int4 or int8 quantization");
    return quant_type == at::kChar ? 8 : 4;
}

void check_cpu_contiguous(Tensor const& t, char const* name)
{
    TORCH_CHECK(t.device().is_cpu(), name, " must be a CPU tensor");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

void check_cuda_contiguous(Tensor const& t, char const* name)
{
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

void check_status(int rc, char const* where)
{
    TORCH_CHECK(rc == W4_OK, where, ": ", w4_status_string(rc), " (status ", rc, ")");
}

// ---- host ops -----------------------------------------------------------------------------------

std::vector<Tensor> symmetric_quantize_impl(Tensor const& weight, at::ScalarType quant_type, bool with_unprocessed)
{
    check_cpu_contiguous(weight, "weight");
    TORCH_CHECK(weight.numel() != 0, "weight should not be empty tensor");
    TORCH_CHECK(weight.dim() == 2 || weight.dim() == 3, "Invalid dim. The dim of weight should be 2 or 3");
    auto const st = weight.scalar_type();
    TORCH_CHECK(st == at::kFloat || st == at::kHalf || st == at::kBFloat16,
        "Invalid datatype. Weight must be FP16 or BF16");
    int const bits = quant_bits(quant_type);
    int64_t const experts = weight.dim() == 2 ? 1 : weight.size(0);
    int64_t const k = weight.size(-2), n = weight.size(-1);
    TORCH_CHECK(n * bits % 8 == 0, "The last dimension must hold whole bytes");

    std::vector<int64_t> q_shape = weight.sizes().vec();
    q_shape.back() = n * bits / 8;
    std::vector<int64_t> s_shape = weight.dim() == 2 ? std::vector<int64_t>{n} : std::vector<int64_t>{experts, n};
    Tensor processed = at::empty(q_shape, weight.options().dtype(at::kChar));
    Tensor unprocessed = at::empty(q_shape, weight.options().dtype(at::kChar));
    Tensor scales32 = at::empty(s_shape, weight.options().dtype(at::kFloat));
    Tensor const w32 = weight.to(at::kFloat).contiguous(); // exact for fp16 / bf16 inputs
    for (int64_t e = 0; e < experts; ++e)
    {
        int const rc = w4_symmetric_quantize(processed.data_ptr<int8_t>() + e * k * (n * bits / 8),
            unprocessed.data_ptr<int8_t>() + e * k * (n * bits / 8), scales32.data_ptr<float>() + e * n,
            w32.data_ptr<float>() + e * k * n, size_t(k), size_t(n), bits);
        check_status(rc, "symmetric_quantize");
    }
    // The scale tensor takes the weight's dtype (weightOnlyQuantOp.cpp:199); the cast rounds to
    // nearest even, as the reference's ComputeType(float) does.
    Tensor scales = scales32.to(st);
    if (with_unprocessed)
        return {unprocessed, processed, scales};
    return {processed, scales};
}

std::vector<Tensor> symmetric_quantize_last_axis_of_batched_matrix(Tensor weight, at::ScalarType quant_type)
{
    return symmetric_quantize_impl(weight, quant_type, false);
}

std::vector<Tensor> symmetric_quantize_last_axis_of_batched_matrix_with_unprocessed(
    Tensor weight, at::ScalarType quant_type)
{
    return symmetric_quantize_impl(weight, quant_type, true);
}

Tensor preprocess_weights_for_mixed_gemm(Tensor weight, at::ScalarType quant_type, at::ScalarType activation_type)
{
    check_cpu_contiguous(weight, "row_major_quantized_weight");
    TORCH_CHECK(weight.scalar_type() == at::kChar, "Quantized tensor must be int8 dtype");
    int const bits = quant_bits(quant_type);
    TORCH_CHECK(weight.dim() == 2 || weight.dim() == 3, "Invalid dim. The dim of weight should be 2 or 3");
    TORCH_CHECK(activation_type != at::kFloat8_e4m3fn, "W4A8 (fp8 activation) layout is not supported by this library");
    int64_t const experts = weight.dim() == 2 ? 1 : weight.size(0);
    int64_t const k = weight.size(-2), row_bytes = weight.size(-1), n = row_bytes * 8 / bits;
    Tensor out = at::zeros_like(weight);
    for (int64_t e = 0; e < experts; ++e)
    {
        int const rc = w4_preprocess_weights(out.data_ptr<int8_t>() + e * k * row_bytes,
            weight.data_ptr<int8_t>() + e * k * row_bytes, size_t(k), size_t(n), bits);
        check_status(rc, "preprocess_weights_for_mixed_gemm");
    }
    return out;
}

Tensor unpack_int4_packed_tensor_to_int8(Tensor weight)
{
    check_cpu_contiguous(weight, "weight");
    TORCH_CHECK(weight.numel() != 0, "weight should not be empty tensor");
    TORCH_CHECK(weight.scalar_type() == at::kChar, "Weight must be a packed int8 tensor");
    std::vector<int64_t> shape = weight.sizes().vec();
    shape.back() *= 2;
    Tensor out = at::zeros(shape, weight.options());
    w4_unpack_int4(out.data_ptr<int8_t>(), weight.data_ptr<int8_t>(), size_t(weight.numel()));
    return out;
}

Tensor pack_int8_tensor_to_packed_int4(Tensor weight)
{
    check_cpu_contiguous(weight, "weight");
    TORCH_CHECK(weight.numel() != 0, "weight should not be empty tensor");
    TORCH_CHECK(weight.scalar_type() == at::kChar, "Weight must be a int8 tensor");
    TORCH_CHECK(weight.size(-1) % 2 == 0, "The last dimension must be even");
    std::vector<int64_t> shape = weight.sizes().vec();
    shape.back() /= 2;
    Tensor out = at::zeros(shape, weight.options());
    int const rc = w4_pack_int4(out.data_ptr<int8_t>(), weight.data_ptr<int8_t>(), size_t(out.numel()));
    TORCH_CHECK(rc == W4_OK, "Value in unpacked tensor not in int4 range");
    return out;
}

// ---- GEMM ops (CUDA) ----------------------------------------------------------------------------

int act_dtype_of(Tensor const& act)
{
    TORCH_CHECK(act.scalar_type() == at::kHalf || act.scalar_type() == at::kBFloat16,
        "activations must be float16 or bfloat16");
    return act.scalar_type() == at::kHalf ? W4_DTYPE_FP16 : W4_DTYPE_BF16;
}

void const* opt_ptr(c10::optional<Tensor> const& t, Tensor const& act, char const* name)
{
    if (!t.has_value() || !t->defined())
        return nullptr;
    check_cuda_contiguous(*t, name);
    TORCH_CHECK(t->scalar_type() == act.scalar_type(), name, " must have the activation dtype");
    TORCH_CHECK(t->device() == act.device(), name, " must be on the activations' device");
    return t->data_ptr();
}

Tensor run_gemm(Tensor const& act, Tensor const& weight, Tensor const& scales, void const* act_scale, void const* zeros,
    void const* bias, double alpha, int bits, int group_size, bool weights_static)
{
    check_cuda_contiguous(act, "act");
    check_cuda_contiguous(weight, "weight");
    check_cuda_contiguous(scales, "scales");
    int const dt = act_dtype_of(act);
    TORCH_CHECK(scales.scalar_type() == act.scalar_type(), "scales must have the activation dtype");
    TORCH_CHECK(weight.device() == act.device() && scales.device() == act.device(), "all tensors must share a device");
    TORCH_CHECK(act.dim() >= 1, "act must have at least one dimension");
    int64_t const k = act.size(-1);
    TORCH_CHECK(weight.dim() == 2 && weight.size(0) == k, "weight must be 2-D with K rows");
    // bytes per row of the [K, N*bits/8] tensor, whatever dtype it is viewed as (the groupwise
    // plugin receives it typed as the activation dtype)
    int64_t const row_bytes = weight.size(1) * int64_t(weight.element_size());
    int64_t const n = row_bytes * 8 / bits;
    int64_t const m = k ? act.numel() / k : 0;
    std::vector<int64_t> out_shape = act.sizes().vec();
    out_shape.back() = n;
    Tensor out = at::empty(out_shape, act.options());
    if (m == 0)
        return out;

    c10::cuda::CUDAGuard guard(act.device());
    auto const stream = at::cuda::getCurrentCUDAStream(act.device().index());
    size_t const ws_bytes = w4_gemm_workspace_bytes(int(m), int(n), int(k), group_size, bits, dt, act_scale != nullptr,
        W4_REGIME_AUTO);
    Tensor ws;
    if (ws_bytes)
        ws = at::empty({int64_t(ws_bytes)}, act.options().dtype(at::kByte));

    W4GemmParams p{};
    p.act = act.data_ptr();
    p.act_scale = act_scale;
    p.weight = weight.data_ptr();
    p.scales = scales.data_ptr();
    p.zeros = zeros;
    p.bias = bias;
    p.out = out.data_ptr();
    p.alpha = float(alpha);
    p.m = int(m);
    p.n = int(n);
    p.k = int(k);
    p.group_size = group_size;
    p.weight_bits = bits;
    p.act_dtype = dt;
    p.regime = W4_REGIME_AUTO;
    p.workspace = ws_bytes ? ws.data_ptr() : nullptr;
    p.workspace_bytes = ws_bytes;
    p.flags = weights_static ? W4_GEMM_WEIGHTS_STATIC : 0u;
    check_status(w4_gemm_launch(&p, stream.stream()), "w4_gemm_launch");
    return out;
}

// Per-channel W8A16 / W4A16: act [.., K] x weight int8 [K, N*bits/8] (preprocessed), scales [N].
// weight_type_id as in the plugin: 1 = int8, 2 = int4 (weightOnlyQuantMatmulPlugin.h:38-42).
Tensor weight_only_quant_gemm(Tensor act, Tensor weight, Tensor scales, int64_t weight_type_id, bool weights_static)
{
    TORCH_CHECK(weight_type_id == 1 || weight_type_id == 2, "wTypeId=", weight_type_id, " is not supported");
    return run_gemm(act, weight, scales, nullptr, nullptr, nullptr, 1.0, weight_type_id == 1 ? 8 : 4, 0, weights_static);
}

// Groupwise (GPTQ / AWQ). quant_algo bits as in the plugin: 1 bias, 2 zero, 4 pre-quant scale,
// 8 fp8 alpha (W4A8-AWQ), 16 int8 weight
// (weightOnlyGroupwiseQuantMatmulPlugin.cpp:33-37). Optional tensors must be present exactly when
// their bit is set. With the fp8-alpha bit (int4 only): alpha multiplies the product, scales / zeros
// may be float16 whatever the activation type (cast here), the weight must already have been re-laid
// with w4_relayout_w4a8_to_w4a16, and the activations stay 16-bit.
Tensor weight_only_groupwise_quant_gemm(Tensor act, c10::optional<Tensor> pre_quant_scale, Tensor weight, Tensor scales,
    c10::optional<Tensor> zeros, c10::optional<Tensor> bias, double alpha, int64_t quant_algo, int64_t group_size,
    bool weights_static)
{
    if (quant_algo & W4_ALGO_FP8_ALPHA)
    {
        TORCH_CHECK(!(quant_algo & W4_ALGO_INT8_WEIGHT), "W4A(fp)8 requires INT4 weight");
        if (scales.scalar_type() != act.scalar_type())
            scales = scales.to(act.scalar_type());
        if (zeros.has_value() && zeros->defined() && zeros->scalar_type() != act.scalar_type())
            zeros = zeros->to(act.scalar_type());
    }
    TORCH_CHECK(group_size == 64 || group_size == 128, "group_size must be 64 or 128");
    auto present = [](c10::optional<Tensor> const& t) { return t.has_value() && t->defined(); };
    TORCH_CHECK(bool(quant_algo & W4_ALGO_PRE_QUANT_SCALE) == present(pre_quant_scale),
        "pre_quant_scale must be given exactly when its quant_algo bit is set");
    TORCH_CHECK(bool(quant_algo & W4_ALGO_ZERO) == present(zeros),
        "zeros must be given exactly when its quant_algo bit is set");
    TORCH_CHECK(bool(quant_algo & W4_ALGO_BIAS) == present(bias),
        "bias must be given exactly when its quant_algo bit is set");
    int const bits = (quant_algo & W4_ALGO_INT8_WEIGHT) ? 8 : 4;
    return run_gemm(act, weight, scales, opt_ptr(pre_quant_scale, act, "pre_quant_scale"), opt_ptr(zeros, act, "zeros"),
        opt_ptr(bias, act, "bias"), alpha, bits, int(group_size), weights_static);
}

} // namespace

TORCH_LIBRARY_FRAGMENT(trtllm, m)
{
    m.def("symmetric_quantize_last_axis_of_batched_matrix(Tensor weight, ScalarType quant_type) -> Tensor[]");
    m.def("_symmetric_quantize_last_axis_of_batched_matrix(Tensor weight, ScalarType quant_type) -> Tensor[]");
    m.def(
        "preprocess_weights_for_mixed_gemm(Tensor weight, ScalarType quant_type, ScalarType activation_type) -> Tensor");
    m.def("unpack_int4_packed_tensor_to_int8(Tensor weight) -> Tensor");
    m.def("pack_int8_tensor_to_packed_int4(Tensor weight) -> Tensor");
    m.def(
        "weight_only_quant_gemm(Tensor act, Tensor weight, Tensor scales, int weight_type_id, "
        "bool weights_static=False) -> Tensor");
    m.def(
        "weight_only_groupwise_quant_gemm(Tensor act, Tensor? pre_quant_scale, Tensor weight, Tensor scales, "
        "Tensor? zeros, Tensor? bias, float alpha, int quant_algo, int group_size, bool weights_static=False) -> Tensor");
}

TORCH_LIBRARY_IMPL(trtllm, CPU, m)
{
    m.impl("symmetric_quantize_last_axis_of_batched_matrix", &symmetric_quantize_last_axis_of_batched_matrix);
    m.impl("_symmetric_quantize_last_axis_of_batched_matrix",
        &symmetric_quantize_last_axis_of_batched_matrix_with_unprocessed);
    m.impl("preprocess_weights_for_mixed_gemm", &preprocess_weights_for_mixed_gemm);
    m.impl("unpack_int4_packed_tensor_to_int8", &unpack_int4_packed_tensor_to_int8);
    m.impl("pack_int8_tensor_to_packed_int4", &pack_int8_tensor_to_packed_int4);
}

TORCH_LIBRARY_IMPL(trtllm, CUDA, m)
{
    m.impl("weight_only_quant_gemm", &weight_only_quant_gemm);
    m.impl("weight_only_groupwise_quant_gemm", &weight_only_groupwise_quant_gemm);
}
