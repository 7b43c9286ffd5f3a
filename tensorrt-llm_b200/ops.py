"""GPU entry points of the weight-only GEMM, mirroring the reference's operator boundary.

* ``weight_only_quant_matmul`` / ``weight_only_groupwise_quant_matmul``: functional form with the
  argument order of the reference's graph emitters
  (tensorrt_llm/quantization/functional.py:216-256 and :259-347 of TensorRT-LLM).
* ``WeightOnlyQuantMatmulPlugin`` / ``WeightOnlyGroupwiseQuantMatmulPlugin``: the same fields,
  tensor order, workspace contract and ``enqueue`` behaviour as the TensorRT plugins
  (cpp/tensorrt_llm/plugins/weightOnlyQuantMatmulPlugin/weightOnlyQuantMatmulPlugin.cpp:283-339,
  cpp/tensorrt_llm/plugins/weightOnlyGroupwiseQuantMatmulPlugin/weightOnlyGroupwiseQuantMatmulPlugin.cpp:189-201,407-495).

Everything funnels into ``w4_gemm_launch`` of libw4gemm.so on the tensors' CUDA stream. torch is
used for device memory and streams only; there is no torch/CPU compute fallback.
"""
from __future__ import annotations

import ctypes
import struct
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import (BIAS, FP8_ALPHA, INT8_WEIGHT, PRE_QUANT_SCALE, W4_DTYPE_BF16, W4_DTYPE_FP16, W4_REGIME_AUTO,
                   W4_REGIME_GEMM, W4_REGIME_GEMV, ZERO, W4GemmParams)

# nvinfer1::DataType values used by the plugins' type_id field
TRT_HALF, TRT_BF16 = 1, 7
# WeightTypeId of the per-channel plugin (weightOnlyQuantMatmulPlugin.h:38-42)
WEIGHT_TYPE_INT8, WEIGHT_TYPE_INT4 = 1, 2

_DTYPES = {torch.float16: W4_DTYPE_FP16, torch.bfloat16: W4_DTYPE_BF16}
_TRT_TO_TORCH = {TRT_HALF: torch.float16, TRT_BF16: torch.bfloat16}


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _require_cuda(t: torch.Tensor, name: str):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def select_regime(m: int, n: int, k: int, group_size: int, weight_bits: int, dtype: torch.dtype = torch.float16) -> int:
    """The kernel an automatic launch takes for this problem (activation type included)."""
    return _lib.lib().w4_gemm_select_regime_typed(m, n, k, group_size, weight_bits, _DTYPES[dtype])


def workspace_bytes(m: int, n: int, k: int, group_size: int, weight_bits: int, dtype: torch.dtype,
                    has_act_scale: bool, regime: int = W4_REGIME_AUTO) -> int:
    return int(_lib.lib().w4_gemm_workspace_bytes(m, n, k, group_size, weight_bits, _DTYPES[dtype],
                                                  int(has_act_scale), regime))


def workspace_bytes_max(max_m: int, n: int, k: int, group_size: int, weight_bits: int, dtype: torch.dtype,
                        has_act_scale: bool) -> int:
    """Largest workspace over m = 1..max_m: what a plugin reserves at configure time."""
    return int(_lib.lib().w4_gemm_workspace_bytes_max(max_m, n, k, group_size, weight_bits, _DTYPES[dtype],
                                                      int(has_act_scale)))


def gemm_raw(act, weight, scales, out, *, n: int, k: int, weight_bits: int, group_size: int, zeros=None,
             bias=None, act_scale=None, alpha: float = 1.0, regime: int = W4_REGIME_AUTO, workspace=None,
             stream: Optional[int] = None, weights_static: bool = False) -> None:
    """Thin wrapper of w4_gemm_launch: borrows every pointer, allocates nothing, returns at once.
    ``weights_static`` sets W4_GEMM_WEIGHTS_STATIC: weight / scales / zeros / act_scale were written
    before the kernel preceding this call on the stream was launched (inference weights)."""
    m = act.numel() // k if k else 0
    params = W4GemmParams(
        act=_p(act), act_scale=_p(act_scale), weight=_p(weight), scales=_p(scales), zeros=_p(zeros),
        bias=_p(bias), out=_p(out), alpha=float(alpha), m=m, n=n, k=k, group_size=group_size,
        weight_bits=weight_bits, act_dtype=_DTYPES[act.dtype], regime=regime, workspace=_p(workspace),
        workspace_bytes=workspace.numel() * workspace.element_size() if workspace is not None else 0,
        flags=_lib.W4_GEMM_WEIGHTS_STATIC if weights_static else 0)
    if stream is None:
        stream = torch.cuda.current_stream(act.device).cuda_stream
    with torch.cuda.device(act.device):
        rc = _lib.lib().w4_gemm_launch(ctypes.byref(params), ctypes.c_void_p(stream))
    _lib.check(rc, "w4_gemm_launch")


def moe_gemm(act, weight, scales, expert_first_row: Sequence[int], *, weight_bits: int, group_size: int, zeros=None,
             bias=None, act_scale=None, alpha: float = 1.0, out=None, weights_static: bool = False):
    """w4_gemm_launch_experts: ``weight`` [E, K, N*bits/8] (laid out per expert), ``scales`` / ``zeros``
    [E, K/G, N] or [E, N], ``bias`` [E, N]; rows of ``act`` sorted by expert, expert e owning rows
    expert_first_row[e] .. expert_first_row[e+1]-1. Returns [M, N]."""
    for name, t in (("act", act), ("weight", weight), ("scales", scales)):
        _require_cuda(t, name)
    if weight.dim() != 3:
        raise RuntimeError("weight must be [experts, K, N*bits/8]")
    e, k = weight.shape[0], weight.shape[1]
    n = weight.shape[2] * weight.element_size() * 8 // weight_bits
    m = act.numel() // k
    first = [int(x) for x in expert_first_row]
    if len(first) != e + 1 or first[0] != 0 or first[-1] != m:
        raise RuntimeError("expert_first_row must hold experts + 1 offsets from 0 to M")
    if out is None:
        out = torch.empty((m, n), dtype=act.dtype, device=act.device)
    if m == 0:
        return out
    biggest = max(b - a for a, b in zip(first[:-1], first[1:]))
    nws = workspace_bytes_max(biggest, n, k, group_size, weight_bits, act.dtype, act_scale is not None)
    ws = torch.empty(max(nws, 16), dtype=torch.uint8, device=act.device)
    params = W4GemmParams(
        act=_p(act), act_scale=_p(act_scale), weight=_p(weight), scales=_p(scales), zeros=_p(zeros), bias=_p(bias),
        out=_p(out), alpha=float(alpha), m=m, n=n, k=k, group_size=group_size, weight_bits=weight_bits,
        act_dtype=_DTYPES[act.dtype], regime=W4_REGIME_AUTO, workspace=_p(ws), workspace_bytes=ws.numel(),
        flags=_lib.W4_GEMM_WEIGHTS_STATIC if weights_static else 0)
    offsets = (ctypes.c_int * (e + 1))(*first)
    with torch.cuda.device(act.device):
        rc = _lib.lib().w4_gemm_launch_experts(ctypes.byref(params), e, offsets,
                                               ctypes.c_void_p(torch.cuda.current_stream(act.device).cuda_stream))
    _lib.check(rc, "w4_gemm_launch_experts")
    return out


class PreparedGemm:
    """One GEMM whose buffers do not move between calls (a decode step: same weights, same staging
    buffers every token): the parameter block is built once, a call costs one C-ABI call.

    ``launch`` enqueues w4_gemm_launch; ``run_host`` is w4_gemm_run_host: activations come from and the
    result goes to pinned host tensors, ``act`` / ``out`` are the device staging buffers, and the call
    returns when the result has landed."""

    def __init__(self, act, weight, scales, out, *, n: int, k: int, weight_bits: int, group_size: int, zeros=None,
                 bias=None, act_scale=None, alpha: float = 1.0, regime: int = W4_REGIME_AUTO, workspace=None,
                 weights_static: bool = False):
        for name, t in (("act", act), ("weight", weight), ("scales", scales), ("out", out)):
            _require_cuda(t, name)
        self._keep = (act, weight, scales, out, zeros, bias, act_scale, workspace)
        self.device = act.device
        self.m = act.numel() // k if k else 0
        self.n, self.k = n, k
        self.params = W4GemmParams(
            act=_p(act), act_scale=_p(act_scale), weight=_p(weight), scales=_p(scales), zeros=_p(zeros),
            bias=_p(bias), out=_p(out), alpha=float(alpha), m=self.m, n=n, k=k, group_size=group_size,
            weight_bits=weight_bits, act_dtype=_DTYPES[act.dtype], regime=regime, workspace=_p(workspace),
            workspace_bytes=workspace.numel() * workspace.element_size() if workspace is not None else 0,
            flags=_lib.W4_GEMM_WEIGHTS_STATIC if weights_static else 0)
        _lib.check(_lib.lib().w4_gemm_validate(ctypes.byref(self.params)), "w4_gemm_validate")
        self._ref = ctypes.byref(self.params)
        self._launch = _lib.lib().w4_gemm_launch
        self._run_host = _lib.lib().w4_gemm_run_host

    def launch(self, stream: int) -> None:
        """Enqueue on the CUDA stream handle ``stream`` (the caller has made the device current)."""
        rc = self._launch(self._ref, stream)
        if rc:
            _lib.check(rc, "w4_gemm_launch")

    def run_host(self, host_act, host_out, stream: int) -> None:
        if host_act.is_cuda or host_out.is_cuda:
            raise RuntimeError("run_host takes host tensors")
        if host_act.numel() != self.m * self.k or host_out.numel() != self.m * self.n \
                or not host_act.is_contiguous() or not host_out.is_contiguous():
            raise RuntimeError("host tensors must be contiguous [M, K] and [M, N]")
        rc = self._run_host(self._ref, host_act.data_ptr(), host_out.data_ptr(), stream)
        if rc:
            _lib.check(rc, "w4_gemm_run_host")


def _run(act, weight, scales, zeros, bias, act_scale, alpha, weight_bits, group_size, regime, out=None,
         weights_static=False):
    for name, t in (("act", act), ("weight", weight), ("scales", scales)):
        _require_cuda(t, name)
    if act.dtype not in _DTYPES:
        raise RuntimeError("activations must be float16 or bfloat16")
    for name, t in (("scales", scales), ("zeros", zeros), ("bias", bias), ("pre_quant_scale", act_scale)):
        if t is not None:
            _require_cuda(t, name)
            if t.dtype != act.dtype:
                raise RuntimeError(f"{name} must have the activation dtype")
    k = act.shape[-1]
    # weight bytes per row of the [K, N*bits/8] tensor, whatever dtype it is viewed as
    row_bytes = weight.shape[-1] * weight.element_size()
    if weight.dim() != 2 or weight.shape[0] != k:
        raise RuntimeError("weight must be 2-D with K rows")
    n = row_bytes * 8 // weight_bits
    m = act.numel() // k
    if out is None:
        out = torch.empty(act.shape[:-1] + (n,), dtype=act.dtype, device=act.device)
    elif out.dtype != act.dtype or out.numel() != m * n or not out.is_contiguous() or out.device != act.device:
        raise RuntimeError("out must be a contiguous [.., N] tensor of the activation dtype on the same device")
    if m == 0:
        return out
    ws_bytes = workspace_bytes(m, n, k, group_size, weight_bits, act.dtype, act_scale is not None, regime)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=act.device) if ws_bytes else None
    gemm_raw(act, weight, scales, out, n=n, k=k, weight_bits=weight_bits, group_size=group_size, zeros=zeros,
             bias=bias, act_scale=act_scale, alpha=alpha, regime=regime, workspace=ws,
             weights_static=weights_static)
    return out


def weight_only_quant_matmul(act: torch.Tensor, weight: torch.Tensor, scales: torch.Tensor,
                             weight_type_id: int, regime: int = W4_REGIME_AUTO,
                             weights_static: bool = False) -> torch.Tensor:
    """Per-channel W8A16 / W4A16: act [.., K] x weight int8 [K, N*bits/8] (preprocessed) with
    scales [N]. weight_type_id: 1 = int8, 2 = int4. ``weights_static``: see ``gemm_raw``."""
    if weight_type_id not in (WEIGHT_TYPE_INT8, WEIGHT_TYPE_INT4):
        raise RuntimeError(f"wTypeId={weight_type_id} is not supported")
    bits = 8 if weight_type_id == WEIGHT_TYPE_INT8 else 4
    return _run(act, weight, scales, None, None, None, 1.0, bits, 0, regime, weights_static=weights_static)


def weight_only_groupwise_quant_matmul(act, pre_quant_scale, weight, scales, zeros, bias, alpha: float,
                                       quant_algo: int, group_size: int,
                                       regime: int = W4_REGIME_AUTO, out=None,
                                       weights_static: bool = False) -> torch.Tensor:
    """Groupwise W4A16 / W8A16 (GPTQ / AWQ). quant_algo bits: 1 bias, 2 zero, 4 pre-quant scale,
    8 fp8 alpha (W4A8-AWQ), 16 int8 weight. Optional tensors must be present exactly when their bit is
    set. The weight may be viewed as the activation dtype, as the plugin takes it.

    With the fp8-alpha bit (int4 only) the layer is a W4A8-AWQ one: ``alpha`` multiplies the product and
    scales / zeros may arrive as float16 whatever the activation type (they are cast). The weight must
    already be in this library's layout (``prepare_w4a8_layer``). Activations stay 16-bit: nothing is
    rounded to e4m3, which keeps the result inside the reference test's tolerance of its own ground
    truth (tests/quantization/test_weight_only_groupwise_quant_matmul.py:233-245) with room to spare."""
    if quant_algo & FP8_ALPHA:
        if quant_algo & INT8_WEIGHT:
            raise RuntimeError("W4A(fp)8 requires INT4 weight")
        scales = scales if scales.dtype == act.dtype else scales.to(act.dtype)
        if zeros is not None and zeros.dtype != act.dtype:
            zeros = zeros.to(act.dtype)
    if group_size not in (64, 128):
        raise RuntimeError("group_size must be 64 or 128")
    for bit, t, name in ((PRE_QUANT_SCALE, pre_quant_scale, "pre_quant_scale"), (ZERO, zeros, "zeros"),
                         (BIAS, bias, "bias")):
        if bool(quant_algo & bit) != (t is not None):
            raise RuntimeError(f"{name} must be given exactly when its quant_algo bit is set")
    bits = 8 if quant_algo & INT8_WEIGHT else 4
    return _run(act, weight, scales, zeros, bias, pre_quant_scale, alpha, bits, group_size, regime, out,
                weights_static=weights_static)


def prepare_w4a8_layer(weight_w4a8, scales, zeros, act_dtype, device):
    """What a W4A8-AWQ layer's constants need once, at load time: the weight, laid out by the reference
    for fp8 activations (preprocess_weights_for_mixed_gemm with activation type float8_e4m3fn), is
    re-laid into the layout the kernels consume, and the float16 scales / zeros are cast to the
    activation type. Returns (weight, scales, zeros) on ``device``. A weight that already sits on a
    GPU is re-laid there (no round trip through the host)."""
    from . import quantize
    w = weight_w4a8.detach().contiguous().view(torch.int8)
    if w.device.type == "cuda":
        w = quantize.relayout_w4a8_weights_cuda(w).to(device)
    else:
        w = quantize.relayout_w4a8_weights(w).to(device)
    s = scales.to(device=device, dtype=act_dtype)
    z = None if zeros is None else zeros.to(device=device, dtype=act_dtype)
    return w, s, z


class _PluginBase:
    """What both TensorRT plugins share: the activation type, one output, borrowed pointers."""

    plugin_namespace = "tensorrt_llm"
    plugin_version = "1"

    def __init__(self, type_id: int):
        if type_id not in _TRT_TO_TORCH:
            raise RuntimeError("Unsupported data type")
        self.type_id = type_id
        self.dtype = _TRT_TO_TORCH[type_id]
        self.dims = None  # (minM, maxM, n, k) once configured
        # TensorRT-LLM feeds these plugins engine constants (weights, scales, zeros, pre-quant
        # scale are network parameters), so the decode kernel may fetch them ahead of the
        # preceding layer's kernel. Clear it when a layer computes the weights on the fly.
        self.weights_static = True

    def get_nb_outputs(self) -> int:
        return 1

    def get_output_data_type(self, index: int = 0):
        assert index == 0
        return self.dtype

    def supports_format_combination(self, pos: int, dtypes: Sequence[torch.dtype]) -> bool:
        raise NotImplementedError


class WeightOnlyQuantMatmulPlugin(_PluginBase):
    """Mirror of plugin "WeightOnlyQuantMatmul" v1: fields type_id, weight_type_id; inputs
    [act T[.., K], weight int8 [K, N*bits/8], scales T[N]]; output T[.., N]."""

    plugin_type = "WeightOnlyQuantMatmul"

    def __init__(self, type_id: int, weight_type_id: int):
        super().__init__(type_id)
        if weight_type_id not in (WEIGHT_TYPE_INT8, WEIGHT_TYPE_INT4):
            raise RuntimeError("Unsupported weight type")
        self.weight_type_id = weight_type_id
        self.bits = 8 if weight_type_id == WEIGHT_TYPE_INT8 else 4

    def supports_format_combination(self, pos, dtypes):
        # input 1 (weight) is int8; everything else has the plugin's type (.cpp:229-253)
        return dtypes[pos] == (torch.int8 if pos == 1 else self.dtype)

    def get_output_dimensions(self, act_shape, weight_shape):
        return tuple(act_shape[:-1]) + (weight_shape[1] * (2 if self.bits == 4 else 1),)

    def configure_plugin(self, min_m, max_m, n, k):
        self.dims = (min_m, max_m, n, k)

    def get_workspace_size(self, max_m=None) -> int:
        if self.dims is None:
            return 0
        _, mm, n, k = self.dims
        return workspace_bytes_max(max_m or mm, n, k, 0, self.bits, self.dtype, False)

    def enqueue(self, inputs, outputs, workspace=None, stream=None, regime=W4_REGIME_AUTO) -> int:
        """Returns 0 on success and a non-zero status instead of raising, as the noexcept
        reference enqueue does."""
        try:
            act, weight, scales = inputs
            k = act.shape[-1]
            n = weight.shape[1] * (2 if self.bits == 4 else 1)
            if act.numel() == 0:
                return 0
            gemm_raw(act, weight, scales, outputs[0], n=n, k=k, weight_bits=self.bits, group_size=0,
                     regime=regime, workspace=workspace, stream=stream, weights_static=self.weights_static)
            return 0
        except _lib.W4Error as e:
            return e.status

    def serialize(self) -> bytes:
        d = self.dims or (0, 0, 0, 0)
        # type, weightTypeId, GemmDims{minM, maxM, n, k}, then an empty tactic map (count = 0)
        return struct.pack("<ii4qi", self.type_id, self.weight_type_id, *d, 0)

    @classmethod
    def deserialize(cls, blob: bytes):
        t, w, a, b, c, d, _ = struct.unpack("<ii4qi", blob[:struct.calcsize("<ii4qi")])
        self = cls(t, w)
        self.dims = (a, b, c, d)
        return self


class WeightOnlyGroupwiseQuantMatmulPlugin(_PluginBase):
    """Mirror of plugin "WeightOnlyGroupwiseQuantMatmul" v1: fields type_id, quant_algo, group_size,
    alpha; inputs [act, (pre_quant_scale), weight (viewed as T), scales, (zeros), (bias)]."""

    plugin_type = "WeightOnlyGroupwiseQuantMatmul"

    def __init__(self, type_id: int, quant_algo: int, group_size: int, alpha: float = 1.0):
        super().__init__(type_id)
        if (quant_algo & FP8_ALPHA) and (quant_algo & INT8_WEIGHT):
            raise RuntimeError("W4A(fp)8 kernel requires INT4 weight!")  # the reference's assert (.cpp:213)
        self._w4a8_cache = {}  # W4A8: constants prepared on first use, keyed by the weight's address
        if group_size not in (64, 128):
            raise RuntimeError("group_size must be 64 or 128")
        self.quant_algo, self.group_size, self.alpha = quant_algo, group_size, float(alpha)
        # input index math of the reference's init() (.cpp:197-201)
        self.pre_quant_scale_idx = 1 if quant_algo & PRE_QUANT_SCALE else 0
        self.weight_idx = self.pre_quant_scale_idx + 1
        self.scales_idx = self.weight_idx + 1
        self.zeros_idx = self.scales_idx + 1 if quant_algo & ZERO else self.scales_idx
        self.bias_idx = self.zeros_idx + 1 if quant_algo & BIAS else self.zeros_idx
        self.bits = 8 if quant_algo & INT8_WEIGHT else 4

    @property
    def nb_inputs(self) -> int:
        return self.bias_idx + 1

    def supports_format_combination(self, pos, dtypes):
        return dtypes[pos] == self.dtype  # every tensor, weight included, carries the plugin type

    def _real_n(self, weight) -> int:
        return weight.shape[1] * weight.element_size() * 8 // self.bits

    def get_output_dimensions(self, act_shape, weight):
        return tuple(act_shape[:-1]) + (self._real_n(weight),)

    def configure_plugin(self, min_m, max_m, n, k):
        self.dims = (min_m, max_m, n, k)

    def get_workspace_size(self, max_m=None) -> int:
        if self.dims is None:
            return 0
        _, mm, n, k = self.dims
        return workspace_bytes_max(max_m or mm, n, k, self.group_size, self.bits, self.dtype,
                                   bool(self.quant_algo & PRE_QUANT_SCALE))

    def enqueue(self, inputs, outputs, workspace=None, stream=None, regime=W4_REGIME_AUTO) -> int:
        try:
            if len(inputs) != self.nb_inputs:
                return _lib.lib().w4_gemm_validate(None)
            act = inputs[0]
            weight = inputs[self.weight_idx]
            if act.numel() == 0:
                return 0
            scales = inputs[self.scales_idx]
            zeros = inputs[self.zeros_idx] if self.quant_algo & ZERO else None
            if self.quant_algo & FP8_ALPHA:
                # the engine's constants are in the reference's W4A8 form: prepare them once
                key = weight.data_ptr()
                if key not in self._w4a8_cache:
                    self._w4a8_cache[key] = prepare_w4a8_layer(weight, scales, zeros, act.dtype, act.device)
                weight, scales, zeros = self._w4a8_cache[key]
            gemm_raw(act, weight, scales, outputs[0], n=self._real_n(weight), k=act.shape[-1],
                     weight_bits=self.bits, group_size=self.group_size,
                     zeros=zeros,
                     bias=inputs[self.bias_idx] if self.quant_algo & BIAS else None,
                     act_scale=inputs[self.pre_quant_scale_idx] if self.quant_algo & PRE_QUANT_SCALE else None,
                     alpha=self.alpha, regime=regime, workspace=workspace, stream=stream,
                     weights_static=self.weights_static)
            return 0
        except _lib.W4Error as e:
            return e.status

    def serialize(self) -> bytes:
        d = self.dims or (0, 0, 0, 0)
        return struct.pack("<iiif4qi", self.type_id, self.quant_algo, self.group_size, self.alpha, *d, 0)

    @classmethod
    def deserialize(cls, blob: bytes):
        fmt = "<iiif4qi"
        t, q, g, al, a, b, c, d, _ = struct.unpack(fmt, blob[:struct.calcsize(fmt)])
        self = cls(t, q, g, al)
        self.dims = (a, b, c, d)
        return self


def allreduce_workspace_bytes(max_message_bytes: int, world: int) -> int:
    """Size of one rank's peer-mapped workspace block for messages of up to ``max_message_bytes``."""
    return int(_lib.lib().w4_allreduce_workspace_bytes(int(max_message_bytes), int(world)))


def _allreduce_params(partial, workspace_ptrs, workspace_bytes, out, n, rank, bias, mode, timeout_ms):
    world = len(workspace_ptrs)
    if not 1 <= world <= _lib.W4_MAX_RANKS:
        raise RuntimeError("allreduce: need 1..8 ranks")
    p = _lib.W4AllReduceParams()
    p.partial = partial.data_ptr()
    for r in range(world):
        p.workspace[r] = int(workspace_ptrs[r])
    p.workspace_bytes = int(workspace_bytes)
    p.bias = bias.data_ptr() if bias is not None else None
    p.out = out.data_ptr()
    p.count, p.n, p.rank, p.world = out.numel(), n, rank, world
    p.act_dtype, p.mode, p.timeout_ms = _DTYPES[out.dtype], mode, timeout_ms
    return p


def allreduce(partial: torch.Tensor, workspace_ptrs, workspace_bytes: int, out: torch.Tensor, n: int, rank: int,
              bias=None, mode: int = _lib.W4_ALLREDUCE_AUTO, timeout_ms: int = 0, stream=None) -> None:
    """out = sum over ranks (rank order, fp32) of every rank's ``partial`` (+ bias), through peer memory.
    ``workspace_ptrs[r]``: device address of rank r's workspace block as mapped into this process (see
    ``tp.PeerAllReduce``). Mirrors the custom all-reduce the reference uses behind dense row-parallel
    layers (kernels/customAllReduceKernels.cu:1307,1426)."""
    p = _allreduce_params(partial, workspace_ptrs, workspace_bytes, out, n, rank, bias, mode, timeout_ms)
    s = stream if stream is not None else torch.cuda.current_stream(out.device)
    with torch.cuda.device(out.device):
        rc = _lib.lib().w4_allreduce(ctypes.byref(p), ctypes.c_void_p(s.cuda_stream))
    _lib.check(rc, "allreduce")


def gemm_push(act, weight, scales, partial, workspace_ptrs, workspace_bytes: int, rank: int, *, n: int, k: int,
              group_size: int, zeros=None, act_scale=None, alpha: float = 1.0, weights_static: bool = False,
              regime: int = W4_REGIME_GEMV, stream=None) -> bool:
    """w4_gemm_launch_push: the int4 decode GEMM writes ``partial`` and sends it, as the packets of the
    one-shot all-reduce, into every peer's inbox. Follow it with ``allreduce(partial, ..., mode=
    W4_ALLREDUCE_GATHER_ONLY)``. Returns False, having launched nothing, when the fused form does not
    apply to this problem (the caller then runs ``gemm_raw`` and an ordinary ``allreduce``). ``regime``
    defaults to the decode kernel, the only one with a pushing epilogue; W4_REGIME_AUTO lets the cost
    model refuse row counts it would give to the tensor-core kernel."""
    m = act.numel() // k if k else 0
    g = W4GemmParams(
        act=_p(act), act_scale=_p(act_scale), weight=_p(weight), scales=_p(scales), zeros=_p(zeros), bias=None,
        out=_p(partial), alpha=float(alpha), m=m, n=n, k=k, group_size=group_size, weight_bits=4,
        act_dtype=_DTYPES[act.dtype], regime=regime, workspace=None, workspace_bytes=0,
        flags=_lib.W4_GEMM_WEIGHTS_STATIC if weights_static else 0)
    r = _allreduce_params(partial, workspace_ptrs, workspace_bytes, partial, n, rank, None, _lib.W4_ALLREDUCE_AUTO, 0)
    s = stream if stream is not None else torch.cuda.current_stream(act.device)
    with torch.cuda.device(act.device):
        rc = _lib.lib().w4_gemm_launch_push(ctypes.byref(g), ctypes.byref(r), ctypes.c_void_p(s.cuda_stream))
    if rc == _lib.W4_ERR_UNSUPPORTED:
        return False
    _lib.check(rc, "w4_gemm_launch_push")
    return True


def gemm_allreduce(act, weight, scales, partial, out, workspace_ptrs, workspace_bytes: int, rank: int, *, n: int,
                   k: int, weight_bits: int, group_size: int, zeros=None, act_scale=None, bias=None, alpha: float = 1.0,
                   weights_static: bool = False, regime: int = W4_REGIME_AUTO, timeout_ms: int = 0,
                   stream=None) -> None:
    """w4_gemm_allreduce: the row-parallel GEMM and the all-reduce of its output in the most fused form
    that applies (one kernel up to 16 rows on int4 weights; GEMM with pushing epilogue + gather; or two
    ordinary launches). ``partial`` [M, N] is scratch for the forms that need it, ``out`` receives the
    reduced result (+ ``bias``) on every rank."""
    m = act.numel() // k if k else 0
    nws = workspace_bytes_max(max(m, 1), n, k, group_size, weight_bits, act.dtype, act_scale is not None)
    ws = torch.empty(max(nws, 16), dtype=torch.uint8, device=act.device)
    g = W4GemmParams(
        act=_p(act), act_scale=_p(act_scale), weight=_p(weight), scales=_p(scales), zeros=_p(zeros), bias=None,
        out=_p(partial), alpha=float(alpha), m=m, n=n, k=k, group_size=group_size, weight_bits=weight_bits,
        act_dtype=_DTYPES[act.dtype], regime=regime, workspace=_p(ws), workspace_bytes=ws.numel(),
        flags=_lib.W4_GEMM_WEIGHTS_STATIC if weights_static else 0)
    r = _allreduce_params(partial, workspace_ptrs, workspace_bytes, out, n, rank, bias, _lib.W4_ALLREDUCE_AUTO,
                          timeout_ms)
    s = stream if stream is not None else torch.cuda.current_stream(act.device)
    with torch.cuda.device(act.device):
        rc = _lib.lib().w4_gemm_allreduce(ctypes.byref(g), ctypes.byref(r), ctypes.c_void_p(s.cuda_stream))
    _lib.check(rc, "w4_gemm_allreduce")


def allreduce_emulated(partials, workspaces, outs, n: int, biases=None, mode: int = _lib.W4_ALLREDUCE_AUTO,
                       timeout_ms: int = 0, stream=None) -> None:
    """All ranks of an all-reduce as one cooperative launch on the current GPU (every buffer local):
    ``partials[r]``, ``workspaces[r]`` (uint8 tensors), ``outs[r]`` belong to rank r."""
    world = len(partials)
    arr = (_lib.W4AllReduceParams * world)()
    ptrs = [w.data_ptr() for w in workspaces]
    for r in range(world):
        arr[r] = _allreduce_params(partials[r], ptrs, workspaces[r].numel(), outs[r], n, r,
                                   None if biases is None else biases[r], mode, timeout_ms)
    s = stream if stream is not None else torch.cuda.current_stream(outs[0].device)
    with torch.cuda.device(outs[0].device):
        rc = _lib.lib().w4_allreduce_emulated(arr, world, ctypes.c_void_p(s.cuda_stream))
    _lib.check(rc, "allreduce_emulated")
