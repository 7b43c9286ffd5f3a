"""TEST INFRASTRUCTURE ONLY - Python face of the CPU oracle for the weight-only GEMM path.

Two halves:

* integer half: ctypes bindings of ``oracle/woq_oracle.c`` (the plain-C restatement of the
  reference's ``symmetric_quantize`` / ``preprocess_weights_for_mixed_gemm``,
  cpp/tensorrt_llm/kernels/cutlass_kernels/cutlass_preprocessors.cpp:163-762) and, when it has
  been built, of ``oracle/_ref/libwoq_ref.so`` (the reference's own code compiled from its
  sources) which pins the restatement;
* floating-point half: the reference tests' definition of the GEMM result, restated with torch
  on the CPU (tests/quantization/test_weight_only_groupwise_quant_matmul.py:223-244,
  tests/quantization/_utils.py:63-96), plus a tighter variant that mirrors the rounding of the
  reference kernels (cpp/tensorrt_llm/kernels/weightOnlyBatchedGemv/utility.h:157-162: the
  dequantised weight is ``fma(q, scale, zero)`` rounded once to the activation type).

Parity status: pinned (see the header of woq_oracle.c). Nothing in the product package imports
this module; only tests, the smoke check and the benchmark's CPU-baseline leg do.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

BIAS, ZERO, PRE_QUANT_SCALE, FP8_ALPHA, INT8_WEIGHT = 1, 2, 4, 8, 16


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def lib() -> ctypes.CDLL:
    """The C restatement, built on first use with the Makefile beside it."""
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libwoq_oracle.so")
        src = os.path.join(_HERE, "woq_oracle.c")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
            subprocess.check_call(["make", "-s", "-C", _HERE])
        _LIB = ctypes.CDLL(path)
    return _LIB


def ref_lib():
    """The reference's own integer path (oracle/_ref), or None when it was not built."""
    global _REF
    if _REF is None:
        path = os.path.join(_HERE, "_ref", "libwoq_ref.so")
        if not os.path.exists(path):
            return None
        _REF = ctypes.CDLL(path)
    return _REF


def _check(rc: int, what: str):
    if rc != 0:
        raise ValueError(f"{what}: oracle status {rc}")


def _as_u8(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    return a.view(np.uint8)


# ----------------------------------------------------------------------------- integer half

def _step(fn_name: str, q: np.ndarray, K: int, N: int, bits: int) -> np.ndarray:
    src = _as_u8(q).reshape(-1)
    assert src.size == K * N * bits // 8, (src.size, K, N, bits)
    out = np.zeros_like(src)
    rc = getattr(lib(), fn_name)(_ptr(out), _ptr(src), ctypes.c_size_t(K), ctypes.c_size_t(N), bits)
    _check(rc, fn_name)
    return out.view(np.int8).reshape(K, N * bits // 8)


def permute_rows(q, K, N, bits):
    return _step("oracle_permute_rows", q, K, N, bits)


def subbyte_transpose(q, K, N, bits):
    return _step("oracle_subbyte_transpose", q, K, N, bits)


def interleave_columns(q, K, N, bits):
    return _step("oracle_interleave_columns", q, K, N, bits)


def add_bias_and_interleave(q, bits):
    buf = _as_u8(q).reshape(-1).copy()
    _check(lib().oracle_add_bias_and_interleave(_ptr(buf), ctypes.c_size_t(buf.size * 8 // bits), bits),
           "add_bias_and_interleave")
    return buf.view(np.int8).reshape(np.asarray(q).shape)


def preprocess_weights(q, bits: int) -> np.ndarray:
    """[K, N*bits/8] int8 row-major quantised weight -> the bytes the kernels consume."""
    q = np.ascontiguousarray(q)
    K, N = q.shape[0], q.shape[1] * 8 // bits
    return _step("oracle_preprocess_weights", q, K, N, bits)


def preprocess_weights_w4a8(q) -> np.ndarray:
    """[K, N/2] int8 row-major int4 weight -> the bytes the reference produces when the activation
    type is fp8 (W4A8): a different row permutation and a 2-column, 128-row interleave."""
    q = np.ascontiguousarray(q)
    K, N = q.shape[0], q.shape[1] * 2
    src = _as_u8(q).reshape(-1)
    out = np.zeros_like(src)
    _check(lib().oracle_preprocess_weights_w4a8(_ptr(out), _ptr(src), ctypes.c_size_t(K), ctypes.c_size_t(N)),
           "preprocess_w4a8")
    return out.view(np.int8).reshape(q.shape)


def unpreprocess_to_int8(processed, K: int, N: int, bits: int) -> np.ndarray:
    """Inverse layout transform: signed integers [K, N] from preprocessed bytes."""
    src = _as_u8(processed).reshape(-1)
    out = np.zeros((K, N), dtype=np.int8)
    _check(lib().oracle_unpreprocess_to_int8(_ptr(out), _ptr(src), ctypes.c_size_t(K), ctypes.c_size_t(N), bits),
           "unpreprocess")
    return out


def unpack_int4(packed) -> np.ndarray:
    p = _as_u8(packed)
    out = np.zeros(p.shape[:-1] + (p.shape[-1] * 2,), dtype=np.int8)
    lib().oracle_unpack_int4(_ptr(out), _ptr(np.ascontiguousarray(p)), ctypes.c_size_t(p.size))
    return out


def pack_int4(unpacked) -> np.ndarray:
    u = np.ascontiguousarray(unpacked, dtype=np.int8)
    out = np.zeros(u.shape[:-1] + ((u.shape[-1] + 1) // 2,), dtype=np.int8)
    _check(lib().oracle_pack_int4(_ptr(out), _ptr(u), ctypes.c_size_t(out.size)), "pack_int4")
    return out


def symmetric_quantize(weight: torch.Tensor, bits: int):
    """Restates torch.ops.trtllm._symmetric_quantize_last_axis_of_batched_matrix for a 2-D weight
    (cpp/tensorrt_llm/thop/weightOnlyQuantOp.cpp:153-238): returns
    (unprocessed int8 [K, N*bits/8], processed int8 same shape, scales [N] in the weight's dtype)."""
    assert weight.dim() == 2 and weight.dtype in (torch.float32, torch.float16, torch.bfloat16)
    K, N = weight.shape
    w32 = np.ascontiguousarray(weight.detach().to(torch.float32).cpu().numpy())
    processed = np.zeros((K, N * bits // 8), dtype=np.int8)
    unprocessed = np.zeros_like(processed)
    scales = np.zeros((N,), dtype=np.float32)
    rc = lib().oracle_symmetric_quantize(_ptr(processed), _ptr(unprocessed), _ptr(scales), _ptr(w32),
                                         ctypes.c_size_t(K), ctypes.c_size_t(N), bits)
    _check(rc, "symmetric_quantize")
    return (torch.from_numpy(unprocessed), torch.from_numpy(processed),
            torch.from_numpy(scales).to(weight.dtype))


# --- the same entry points through the reference's own compiled code (when available)

def ref_preprocess_weights(q, bits: int, sm=(10, 0)) -> np.ndarray:
    r = ref_lib()
    assert r is not None, "oracle/_ref was not built"
    q = np.ascontiguousarray(q)
    K, N = q.shape[0], q.shape[1] * 8 // bits
    src = _as_u8(q).reshape(-1)
    out = np.zeros_like(src)
    r.ref_set_sm(sm[0], sm[1])
    _check(r.ref_preprocess_weights_for_mixed_gemm(_ptr(out), _ptr(src), ctypes.c_size_t(K), ctypes.c_size_t(N), bits),
           "ref_preprocess")
    return out.view(np.int8).reshape(q.shape)


def ref_preprocess_weights_w4a8(q, sm=(10, 0)) -> np.ndarray:
    r = ref_lib()
    assert r is not None, "oracle/_ref was not built"
    q = np.ascontiguousarray(q)
    K, N = q.shape[0], q.shape[1] * 2
    src = _as_u8(q).reshape(-1)
    out = np.zeros_like(src)
    r.ref_set_sm(sm[0], sm[1])
    _check(r.ref_preprocess_weights_w4a8(_ptr(out), _ptr(src), ctypes.c_size_t(K), ctypes.c_size_t(N)), "ref_w4a8")
    return out.view(np.int8).reshape(q.shape)


def ref_step(name: str, q, K, N, bits) -> np.ndarray:
    r = ref_lib()
    assert r is not None, "oracle/_ref was not built"
    src = _as_u8(q).reshape(-1)
    out = np.zeros_like(src)
    _check(getattr(r, name)(_ptr(out), _ptr(src), ctypes.c_size_t(K), ctypes.c_size_t(N), bits), name)
    return out.view(np.int8).reshape(K, N * bits // 8)


def ref_add_bias_and_interleave(q, bits):
    r = ref_lib()
    assert r is not None
    buf = _as_u8(q).reshape(-1).copy()
    _check(r.ref_add_bias_and_interleave_inplace(_ptr(buf), ctypes.c_size_t(buf.size * 8 // bits), bits), "ref_bias")
    return buf.view(np.int8).reshape(np.asarray(q).shape)


def ref_symmetric_quantize(weight: torch.Tensor, bits: int):
    """Same contract as symmetric_quantize() above, through the reference's own code."""
    r = ref_lib()
    assert r is not None, "oracle/_ref was not built"
    K, N = weight.shape
    processed = np.zeros((K, N * bits // 8), dtype=np.int8)
    unprocessed = np.zeros_like(processed)
    r.ref_set_sm(10, 0)
    if weight.dtype == torch.float32:
        # thop uses symmetric_quantize<float, float>; the 7-argument form is not instantiated for it,
        # so take the unprocessed tensor from the <half, float> instantiation (same integers).
        w = np.ascontiguousarray(weight.numpy())
        scales = np.zeros((N,), dtype=np.float32)
        _check(r.ref_symmetric_quantize_f32(_ptr(processed), None, _ptr(scales), _ptr(w), ctypes.c_size_t(K),
                                            ctypes.c_size_t(N), bits, 0), "ref_sq_f32")
        tmp_p = np.zeros_like(processed)
        tmp_s = np.zeros((N,), dtype=np.float16)
        _check(r.ref_symmetric_quantize_f32(_ptr(tmp_p), _ptr(unprocessed), _ptr(tmp_s), _ptr(w), ctypes.c_size_t(K),
                                            ctypes.c_size_t(N), bits, 1), "ref_sq_f32h")
        st = torch.from_numpy(scales)
    elif weight.dtype == torch.float16:
        w = np.ascontiguousarray(weight.view(torch.int16).numpy())
        scales = np.zeros((N,), dtype=np.int16)
        _check(r.ref_symmetric_quantize_f16(_ptr(processed), _ptr(unprocessed), _ptr(scales), _ptr(w),
                                            ctypes.c_size_t(K), ctypes.c_size_t(N), bits), "ref_sq_f16")
        st = torch.from_numpy(scales).view(torch.float16)
    else:
        w = np.ascontiguousarray(weight.view(torch.int16).numpy())
        scales = np.zeros((N,), dtype=np.int16)
        _check(r.ref_symmetric_quantize_bf16(_ptr(processed), _ptr(unprocessed), _ptr(scales), _ptr(w),
                                             ctypes.c_size_t(K), ctypes.c_size_t(N), bits), "ref_sq_bf16")
        st = torch.from_numpy(scales).view(torch.bfloat16)
    return torch.from_numpy(unprocessed), torch.from_numpy(processed), st


# ----------------------------------------------------------------------------- floating-point half

def signed_weights(processed, K: int, N: int, bits: int) -> torch.Tensor:
    """int8 [K, N] signed integer weights recovered from preprocessed bytes."""
    p = processed.detach().cpu().contiguous().view(torch.int8).numpy() if isinstance(processed, torch.Tensor) \
        else processed
    return torch.from_numpy(unpreprocess_to_int8(p, K, N, bits))


def _expand_groups(t: torch.Tensor, K: int, group_size: int) -> torch.Tensor:
    return t.repeat_interleave(group_size, dim=0)[:K, :]


def groupwise_matmul_test_ref(act, q_int8, scales, zeros=None, bias=None, pre_quant_scale=None,
                              group_size=128, alpha=1.0):
    """The reference test's ground truth, op for op in the activation dtype
    (tests/quantization/test_weight_only_groupwise_quant_matmul.py:223-244 and
    tests/quantization/_utils.py:63-67): every torch op rounds to that dtype."""
    T = act.dtype
    K = act.shape[-1]
    w = q_int8.to(T) * _expand_groups(scales.to(T), K, group_size)
    if zeros is not None:
        w = w + _expand_groups(zeros.to(T), K, group_size)
    a = act
    if alpha != 1.0:
        a = a * alpha
    if pre_quant_scale is not None:
        a = torch.mul(a, pre_quant_scale.reshape(1, K).to(T))
    ref = torch.matmul(a, w.to(T))
    if bias is not None:
        ref = ref + bias.reshape(1, -1).to(T)
    return ref


def per_channel_matmul_test_ref(act, q_int8, scales):
    """tests/quantization/_utils.py:70-96: fp32 matmul of activations with the raw integers,
    scaled per output column, cast to the activation dtype."""
    ref = torch.matmul(act.to(torch.float32), q_int8.to(torch.float32))
    ref = ref * scales.to(torch.float32).reshape(1, -1)
    return ref.to(act.dtype)


def kernel_rounding_ref(act, q_int8, scales, zeros=None, bias=None, pre_quant_scale=None,
                        group_size=0, alpha=1.0):
    """Tight oracle: the dequantised weight is fma(q, s, z) rounded once to the activation dtype
    (weightOnlyBatchedGemv/utility.h:157-162; cutlass_extensions/gemm/warp/
    mma_tensorop_dequantizer.h:247-262), the pre-quant scale product is rounded to that dtype
    (utility.h:116), the dot product is accumulated in float64 here, and alpha*acc + bias is
    rounded once at the end (utility.h:256-266). group_size 0 = one scale per column."""
    T = act.dtype
    K = act.shape[-1]
    s = scales.to(torch.float64)
    if group_size == 0:
        s = s.reshape(1, -1).expand(K, -1)
    else:
        s = _expand_groups(s, K, group_size)
    w = q_int8.to(torch.float64) * s
    if zeros is not None:
        z = zeros.to(torch.float64)
        z = z.reshape(1, -1).expand(K, -1) if group_size == 0 else _expand_groups(z, K, group_size)
        w = w + z
    w = w.to(T).to(torch.float64)
    a = act
    if pre_quant_scale is not None:
        a = (a.to(torch.float64) * pre_quant_scale.reshape(1, K).to(torch.float64)).to(T)
    out = torch.matmul(a.to(torch.float64), w) * float(alpha)
    if bias is not None:
        out = out + bias.reshape(1, -1).to(torch.float64)
    return out.to(T)


def tolerance(ref: torch.Tensor) -> float:
    """Allowed max|out - ref|: 1e-2 of max|ref| (the bound this path is held to)."""
    return 1e-2 * float(ref.to(torch.float32).abs().max())
