"""ctypes binding of libw4gemm.so (the C ABI in include/w4_gemm.h).

The library is built in-tree by csrc/build.sh. There is no CPU or PyTorch fallback: if the shared
object is missing the import of any GPU entry point raises.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libw4gemm.so")

W4_OK = 0
W4_LOG_TRACE, W4_LOG_DEBUG, W4_LOG_INFO, W4_LOG_WARNING, W4_LOG_ERROR = 0, 10, 20, 30, 40
W4_ERR_NULL_POINTER, W4_ERR_BAD_SHAPE, W4_ERR_BAD_GROUP, W4_ERR_BAD_DTYPE, W4_ERR_MISALIGNED = -1, -2, -3, -4, -5
W4_ERR_UNSUPPORTED, W4_ERR_WORKSPACE, W4_ERR_CUDA, W4_ERR_BAD_REGIME = -6, -7, -8, -9
W4_DTYPE_FP16, W4_DTYPE_BF16 = 0, 1
W4_REGIME_AUTO, W4_REGIME_GEMV, W4_REGIME_GEMM = 0, 1, 2
# quant_algo bits of the groupwise plugin
BIAS, ZERO, PRE_QUANT_SCALE, FP8_ALPHA, INT8_WEIGHT = 1, 2, 4, 8, 16

EXPORTS = (
    "w4_gemm_version", "w4_status_string", "w4_gemm_validate", "w4_gemm_launch", "w4_gemm_workspace_bytes",
    "w4_gemm_select_regime", "w4_gemm_device_status", "w4_symmetric_quantize", "w4_preprocess_weights",
    "w4_pack_int4", "w4_unpack_int4", "w4_gemm_launch_static_scratch", "w4_gemm_static_scratch_bytes",
    "w4_preprocess_weights_device", "w4_symmetric_quantize_device", "w4_allreduce", "w4_allreduce_emulated",
    "w4_allreduce_workspace_bytes",
    "w4_gemm_workspace_bytes_max", "w4_gemm_run_host", "w4_gemm_launch_experts",
    "w4_preprocess_weights_w4a8", "w4_relayout_w4a8_to_w4a16", "w4_gemm_launch_push", "w4_gemm_allreduce",
    "w4_relayout_w4a8_to_w4a16_device", "w4_set_log_level", "w4_get_log_level",
    "w4_gemm_select_regime_typed",
)


class W4GemmParams(ctypes.Structure):
    _fields_ = [
        ("act", ctypes.c_void_p), ("act_scale", ctypes.c_void_p), ("weight", ctypes.c_void_p),
        ("scales", ctypes.c_void_p), ("zeros", ctypes.c_void_p), ("bias", ctypes.c_void_p),
        ("out", ctypes.c_void_p), ("alpha", ctypes.c_float), ("m", ctypes.c_int), ("n", ctypes.c_int),
        ("k", ctypes.c_int), ("group_size", ctypes.c_int), ("weight_bits", ctypes.c_int),
        ("act_dtype", ctypes.c_int), ("regime", ctypes.c_int), ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t), ("flags", ctypes.c_uint),
    ]


# W4GemmParams.flags
W4_GEMM_WEIGHTS_STATIC = 1

W4_MAX_RANKS = 8
W4_ONESHOT_MAX_BYTES = 1 << 20
W4_ALLREDUCE_MAX_CTAS = 128
W4_ALLREDUCE_LL_MAX_BYTES = 4 << 20
W4_ERR_DEVICE_TIMEOUT = -10
W4_ALLREDUCE_AUTO, W4_ALLREDUCE_ONE_SHOT, W4_ALLREDUCE_TWO_SHOT, W4_ALLREDUCE_GATHER_ONLY = 0, 1, 2, 3


class W4AllReduceParams(ctypes.Structure):
    _fields_ = [
        ("partial", ctypes.c_void_p), ("workspace", ctypes.c_void_p * W4_MAX_RANKS),
        ("workspace_bytes", ctypes.c_size_t), ("bias", ctypes.c_void_p), ("out", ctypes.c_void_p),
        ("count", ctypes.c_size_t), ("n", ctypes.c_int), ("rank", ctypes.c_int), ("world", ctypes.c_int),
        ("act_dtype", ctypes.c_int), ("mode", ctypes.c_int), ("timeout_ms", ctypes.c_uint32),
    ]


class W4Error(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: {status_string(status)} (status {status})")


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with tensorrt-llm_b200/csrc/build.sh "
                "(there is no fallback path)")
        l = ctypes.CDLL(LIB_PATH)
        l.w4_status_string.restype = ctypes.c_char_p
        l.w4_status_string.argtypes = [ctypes.c_int]
        l.w4_gemm_validate.argtypes = [ctypes.POINTER(W4GemmParams)]
        l.w4_gemm_launch.argtypes = [ctypes.POINTER(W4GemmParams), ctypes.c_void_p]
        l.w4_gemm_launch_static_scratch.argtypes = [ctypes.POINTER(W4GemmParams), ctypes.c_void_p]
        l.w4_gemm_launch_experts.argtypes = [ctypes.POINTER(W4GemmParams), ctypes.c_int, ctypes.POINTER(ctypes.c_int),
                                             ctypes.c_void_p]
        l.w4_gemm_run_host.argtypes = [ctypes.POINTER(W4GemmParams), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        l.w4_gemm_static_scratch_bytes.restype = ctypes.c_size_t
        l.w4_gemm_workspace_bytes.restype = ctypes.c_size_t
        l.w4_gemm_workspace_bytes.argtypes = [ctypes.c_int] * 8
        l.w4_gemm_workspace_bytes_max.restype = ctypes.c_size_t
        l.w4_gemm_workspace_bytes_max.argtypes = [ctypes.c_int] * 7
        l.w4_gemm_select_regime.argtypes = [ctypes.c_int] * 5
        l.w4_gemm_select_regime_typed.argtypes = [ctypes.c_int] * 6
        l.w4_symmetric_quantize.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                            ctypes.c_size_t, ctypes.c_size_t, ctypes.c_int]
        l.w4_preprocess_weights.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t,
                                            ctypes.c_int]
        l.w4_preprocess_weights_w4a8.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t]
        l.w4_relayout_w4a8_to_w4a16.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t]
        l.w4_relayout_w4a8_to_w4a16_device.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t,
                                                       ctypes.c_size_t, ctypes.c_void_p]
        l.w4_preprocess_weights_device.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t,
                                                   ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
        l.w4_symmetric_quantize_device.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                   ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                                   ctypes.c_size_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
        l.w4_allreduce.argtypes = [ctypes.POINTER(W4AllReduceParams), ctypes.c_void_p]
        l.w4_gemm_launch_push.argtypes = [ctypes.POINTER(W4GemmParams), ctypes.POINTER(W4AllReduceParams), ctypes.c_void_p]
        l.w4_gemm_allreduce.argtypes = [ctypes.POINTER(W4GemmParams), ctypes.POINTER(W4AllReduceParams), ctypes.c_void_p]
        l.w4_allreduce_emulated.argtypes = [ctypes.POINTER(W4AllReduceParams), ctypes.c_int, ctypes.c_void_p]
        l.w4_allreduce_workspace_bytes.restype = ctypes.c_size_t
        l.w4_allreduce_workspace_bytes.argtypes = [ctypes.c_size_t, ctypes.c_int]
        l.w4_pack_int4.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
        l.w4_unpack_int4.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
        l.w4_unpack_int4.restype = None
        l.w4_set_log_level.argtypes = [ctypes.c_int]
        l.w4_set_log_level.restype = None
        _lib = l
    return _lib


def status_string(status: int) -> str:
    return lib().w4_status_string(int(status)).decode()


def check(status: int, where: str):
    if status != W4_OK:
        raise W4Error(status, where)
