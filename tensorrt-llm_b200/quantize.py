"""Host-side weight preparation ops with the reference's names, arguments and error behaviour
(cpp/tensorrt_llm/thop/weightOnlyQuantOp.cpp:123-353 of TensorRT-LLM). They run on CPU tensors,
as the reference's do, through the C ABI of libw4gemm.so. The two ``*_cuda`` functions at the end
are additions without a reference counterpart: the same preparation on CUDA tensors (CUDA kernels,
byte-identical results), for loaders that already hold the checkpoint on the GPU.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_QUANT_BITS = {torch.int8: 8, torch.quint4x2: 4}


def _bits(quant_type) -> int:
    if quant_type not in _QUANT_BITS:
        raise RuntimeError("Must be int4 or int8 quantization")
    return _QUANT_BITS[quant_type]


def _check_cpu_contiguous(t: torch.Tensor, name: str):
    if t.device.type != "cpu":
        raise RuntimeError(f"{name} must be a CPU tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _ptr(t: torch.Tensor):
    return ctypes.c_void_p(t.data_ptr())


def _quantize_2d(weight: torch.Tensor, bits: int):
    k, n = weight.shape
    w32 = weight.to(torch.float32).contiguous()
    processed = torch.empty((k, n * bits // 8), dtype=torch.int8)
    unprocessed = torch.empty_like(processed)
    scales = torch.empty((n,), dtype=torch.float32)
    rc = _lib.lib().w4_symmetric_quantize(_ptr(processed), _ptr(unprocessed), _ptr(scales), _ptr(w32), k, n, bits)
    _lib.check(rc, "symmetric_quantize")
    # ComputeType(float) in the reference is a round-to-nearest-even cast, as .to() is.
    return unprocessed, processed, scales.to(weight.dtype)


def _symmetric_quantize_helper(weight: torch.Tensor, quant_type, return_unprocessed: bool):
    _check_cpu_contiguous(weight, "weight")
    if weight.numel() == 0:
        raise RuntimeError("weight should not be empty tensor")
    if weight.dim() not in (2, 3):
        raise RuntimeError("Invalid dim. The dim of weight should be 2 or 3")
    if weight.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise RuntimeError("Invalid datatype. Weight must be FP16 or BF16")
    bits = _bits(quant_type)
    if weight.dim() == 2:
        u, p, s = _quantize_2d(weight, bits)
    else:
        parts = [_quantize_2d(weight[e], bits) for e in range(weight.shape[0])]
        u, p, s = (torch.stack([x[i] for x in parts]) for i in range(3))
    return [u, p, s] if return_unprocessed else [p, s]


def symmetric_quantize_last_axis_of_batched_matrix(weight: torch.Tensor, quant_type):
    """-> [processed int8 [K, N*bits/8], scales [N] in weight.dtype] (weightOnlyQuantOp.cpp:240-243)."""
    return _symmetric_quantize_helper(weight, quant_type, False)


def _symmetric_quantize_last_axis_of_batched_matrix(weight: torch.Tensor, quant_type):
    """-> [unprocessed, processed, scales] (weightOnlyQuantOp.cpp:248-251)."""
    return _symmetric_quantize_helper(weight, quant_type, True)


def preprocess_weights_for_mixed_gemm(row_major_quantized_weight: torch.Tensor, quant_type,
                                      activation_type=torch.float16) -> torch.Tensor:
    """[K, N*bits/8] int8 row-major two's-complement weights -> kernel layout
    (weightOnlyQuantOp.cpp:123-151). activation_type float8_e4m3fn selects the W4A8 layout whatever
    quant_type says, as the reference's get_ft_quant_type does (weightOnlyQuantOp.cpp:40-46); the GEMM
    kernels take that layout after relayout_w4a8_weights()."""
    t = row_major_quantized_weight
    _check_cpu_contiguous(t, "row_major_quantized_weight")
    if t.dtype != torch.int8:
        raise RuntimeError("Quantized tensor must be int8 dtype")
    bits = _bits(quant_type)
    if t.dim() not in (2, 3):
        raise RuntimeError("Invalid dim. The dim of weight should be 2 or 3")
    w4a8 = activation_type == getattr(torch, "float8_e4m3fn", None)
    if w4a8:
        bits = 4
    out = torch.zeros_like(t)
    mats = [(t, out)] if t.dim() == 2 else [(t[e], out[e]) for e in range(t.shape[0])]
    for src, dst in mats:
        k, n = src.shape[0], src.shape[1] * 8 // bits
        if w4a8:
            rc = _lib.lib().w4_preprocess_weights_w4a8(_ptr(dst), _ptr(src), k, n)
        else:
            rc = _lib.lib().w4_preprocess_weights(_ptr(dst), _ptr(src), k, n, bits)
        _lib.check(rc, "preprocess_weights_for_mixed_gemm")
    return out


def relayout_w4a8_weights(w4a8_weight: torch.Tensor) -> torch.Tensor:
    """[K, N/2] (or [E, K, N/2]) int8 bytes in the reference's W4A8 layout -> the W4A16 layout this
    library's kernels consume (w4_relayout_w4a8_to_w4a16). Done once at load time."""
    t = w4a8_weight
    _check_cpu_contiguous(t, "w4a8_weight")
    if t.dtype != torch.int8 or t.dim() not in (2, 3):
        raise RuntimeError("expected an int8 tensor [K, N/2] or [E, K, N/2]")
    out = torch.zeros_like(t)
    mats = [(t, out)] if t.dim() == 2 else [(t[e], out[e]) for e in range(t.shape[0])]
    for src, dst in mats:
        rc = _lib.lib().w4_relayout_w4a8_to_w4a16(_ptr(dst), _ptr(src), src.shape[0], src.shape[1] * 2)
        _lib.check(rc, "relayout_w4a8_weights")
    return out


def unpack_int4_packed_tensor_to_int8(weight: torch.Tensor) -> torch.Tensor:
    _check_cpu_contiguous(weight, "weight")
    if weight.numel() == 0:
        raise RuntimeError("weight should not be empty tensor")
    if weight.dtype != torch.int8:
        raise RuntimeError("Weight must be a packed int8 tensor")
    out = torch.zeros(weight.shape[:-1] + (weight.shape[-1] * 2,), dtype=torch.int8)
    _lib.lib().w4_unpack_int4(_ptr(out), _ptr(weight), weight.numel())
    return out


def pack_int8_tensor_to_packed_int4(weight: torch.Tensor) -> torch.Tensor:
    _check_cpu_contiguous(weight, "weight")
    if weight.numel() == 0:
        raise RuntimeError("weight should not be empty tensor")
    if weight.dtype != torch.int8:
        raise RuntimeError("Weight must be a int8 tensor")
    if weight.shape[-1] % 2:
        raise RuntimeError("The last dimension must be even")
    out = torch.zeros(weight.shape[:-1] + (weight.shape[-1] // 2,), dtype=torch.int8)
    rc = _lib.lib().w4_pack_int4(_ptr(out), _ptr(weight), out.numel())
    if rc != _lib.W4_OK:
        raise RuntimeError("Value in unpacked tensor not in int4 range")
    return out


# ---------------------------------------------------------------------------------------------
# GPU-side preparation (no reference counterpart: the reference prepares weights on the CPU only)
# ---------------------------------------------------------------------------------------------
_W_DTYPES = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def _check_cuda_contiguous(t: torch.Tensor, name: str):
    if t.device.type != "cuda":
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def preprocess_weights_for_mixed_gemm_cuda(row_major_quantized_weight: torch.Tensor, quant_type) -> torch.Tensor:
    """preprocess_weights_for_mixed_gemm on a CUDA int8 tensor [K, N*bits/8] (2-D); same bytes."""
    t = row_major_quantized_weight
    _check_cuda_contiguous(t, "row_major_quantized_weight")
    if t.dtype != torch.int8:
        raise RuntimeError("Quantized tensor must be int8 dtype")
    if t.dim() != 2:
        raise RuntimeError("Invalid dim. The dim of weight should be 2")
    bits = _bits(quant_type)
    out = torch.empty_like(t)
    with torch.cuda.device(t.device):
        rc = _lib.lib().w4_preprocess_weights_device(_ptr(out), _ptr(t), t.shape[0], t.shape[1] * 8 // bits, bits,
                                                     _stream(t))
    _lib.check(rc, "preprocess_weights_for_mixed_gemm_cuda")
    return out


def relayout_w4a8_weights_cuda(w4a8_weight: torch.Tensor) -> torch.Tensor:
    """relayout_w4a8_weights on a CUDA int8 tensor [K, N/2] or [E, K, N/2]; same bytes."""
    t = w4a8_weight
    _check_cuda_contiguous(t, "w4a8_weight")
    if t.dtype != torch.int8 or t.dim() not in (2, 3):
        raise RuntimeError("expected an int8 tensor [K, N/2] or [E, K, N/2]")
    out = torch.empty_like(t)
    mats = [(t, out)] if t.dim() == 2 else [(t[e], out[e]) for e in range(t.shape[0])]
    with torch.cuda.device(t.device):
        for src, dst in mats:
            rc = _lib.lib().w4_relayout_w4a8_to_w4a16_device(_ptr(dst), _ptr(src), src.shape[0], src.shape[1] * 2,
                                                             _stream(t))
            _lib.check(rc, "relayout_w4a8_weights_cuda")
    return out


def symmetric_quantize_last_axis_of_batched_matrix_cuda(weight: torch.Tensor, quant_type,
                                                         return_unprocessed: bool = False):
    """symmetric_quantize on a CUDA tensor [K, N] (fp32 / fp16 / bf16):
    -> [processed, scales] or [unprocessed, processed, scales], scales in weight.dtype."""
    _check_cuda_contiguous(weight, "weight")
    if weight.dim() != 2 or weight.numel() == 0:
        raise RuntimeError("Invalid dim. The dim of weight should be 2")
    if weight.dtype not in _W_DTYPES:
        raise RuntimeError("Invalid datatype. Weight must be FP16 or BF16")
    bits = _bits(quant_type)
    k, n = weight.shape
    processed = torch.empty((k, n * bits // 8), dtype=torch.int8, device=weight.device)
    unprocessed = torch.empty_like(processed) if return_unprocessed else None
    scales = torch.empty((n,), dtype=torch.float32, device=weight.device)
    scales_t = None if weight.dtype == torch.float32 else torch.empty((n,), dtype=weight.dtype, device=weight.device)
    with torch.cuda.device(weight.device):
        rc = _lib.lib().w4_symmetric_quantize_device(
            _ptr(processed), _ptr(unprocessed) if unprocessed is not None else None, _ptr(scales),
            _ptr(scales_t) if scales_t is not None else None, _W_DTYPES.get(weight.dtype, 0) if scales_t is not None
            else 0, _ptr(weight), _W_DTYPES[weight.dtype], k, n, bits, _stream(weight))
    _lib.check(rc, "symmetric_quantize_last_axis_of_batched_matrix_cuda")
    s = scales if scales_t is None else scales_t
    return [unprocessed, processed, s] if return_unprocessed else [processed, s]
