"""Registers the library under ``torch.ops.trtllm`` with the reference's op names.

The five host-side ops keep the schemas of cpp/tensorrt_llm/thop/weightOnlyQuantOp.cpp:358-385 of
TensorRT-LLM. The two GEMM ops are new (that reference version ships no weight-only GEMM torch op);
they follow the conventions of its other GEMM ops (cpp/tensorrt_llm/thop/cutlassScaledMM.cpp:121-175):
CUDA tensors in, output allocated on the input's device, current stream.

Importing this module is what performs the registration; importing it twice is harmless.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from . import ops, quantize

_LIB = None


def _dtype_from_int(v):
    # torch passes ScalarType arguments through unchanged when called from Python.
    return v


def register() -> None:
    global _LIB
    if _LIB is not None:
        return
    lib = torch.library.Library("trtllm", "FRAGMENT")
    lib.define("symmetric_quantize_last_axis_of_batched_matrix(Tensor weight, ScalarType quant_type) -> Tensor[]")
    lib.define("_symmetric_quantize_last_axis_of_batched_matrix(Tensor weight, ScalarType quant_type) -> Tensor[]")
    lib.define("preprocess_weights_for_mixed_gemm(Tensor weight, ScalarType quant_type, "
               "ScalarType activation_type) -> Tensor")
    lib.define("unpack_int4_packed_tensor_to_int8(Tensor weight) -> Tensor")
    lib.define("pack_int8_tensor_to_packed_int4(Tensor weight) -> Tensor")
    lib.define("weight_only_quant_gemm(Tensor act, Tensor weight, Tensor scales, int weight_type_id) -> Tensor")
    lib.define("weight_only_groupwise_quant_gemm(Tensor act, Tensor? pre_quant_scale, Tensor weight, "
               "Tensor scales, Tensor? zeros, Tensor? bias, float alpha, int quant_algo, int group_size) -> Tensor")

    lib.impl("symmetric_quantize_last_axis_of_batched_matrix",
             lambda w, qt: quantize.symmetric_quantize_last_axis_of_batched_matrix(w, qt), "CPU")
    lib.impl("_symmetric_quantize_last_axis_of_batched_matrix",
             lambda w, qt: quantize._symmetric_quantize_last_axis_of_batched_matrix(w, qt), "CPU")
    lib.impl("preprocess_weights_for_mixed_gemm",
             lambda w, qt, at: quantize.preprocess_weights_for_mixed_gemm(w, qt, at), "CPU")
    lib.impl("unpack_int4_packed_tensor_to_int8", quantize.unpack_int4_packed_tensor_to_int8, "CPU")
    lib.impl("pack_int8_tensor_to_packed_int4", quantize.pack_int8_tensor_to_packed_int4, "CPU")
    lib.impl("weight_only_quant_gemm",
             lambda a, w, s, t: ops.weight_only_quant_matmul(a, w, s, t), "CUDA")
    lib.impl("weight_only_groupwise_quant_gemm",
             lambda a, ps, w, s, z, b, alpha, algo, g: ops.weight_only_groupwise_quant_matmul(
                 a, ps, w, s, z, b, alpha, algo, g), "CUDA")
    _LIB = lib


register()
