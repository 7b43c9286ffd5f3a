"""The C++ TensorRT plugin shim (include/w4_trt_plugin.h) driven through a small ctypes harness
compiled against a stand-in for TensorRT's header (tests/cpp/mock_trt): creator fields, output
dimensions, format checks, workspace, serialise / deserialise / clone on the CPU; enqueue of every
quant_algo input layout on the GPU against the CPU oracle."""
import ctypes
import itertools
import os
import struct
import subprocess

import pytest
import torch

import tensorrt_llm_b200 as pkg
from tensorrt_llm_b200 import ops
from oracle import woq_oracle as oracle
from _cases import make_problem, max_err, oracle_out

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SRC = os.path.join(HERE, "cpp", "plugin_harness.cpp")
HDR = os.path.join(ROOT, "include", "w4_trt_plugin.h")
LIB = os.path.join(HERE, "cpp", "libplugin_harness.so")


@pytest.fixture(scope="module")
def harness():
    pkg._lib.lib()  # libw4gemm.so must exist (no fallback)
    stale = (not os.path.exists(LIB)) or os.path.getmtime(LIB) < max(os.path.getmtime(SRC), os.path.getmtime(HDR))
    if stale:
        subprocess.check_call(["g++", "-std=c++17", "-O1", "-fPIC", "-shared", "-Wall", "-Werror",
                               "-I" + os.path.join(HERE, "cpp", "mock_trt"), SRC, "-o", LIB,
                               "-L" + os.path.join(ROOT, "tensorrt-llm_b200"), "-lw4gemm",
                               "-Wl,-rpath," + os.path.join(ROOT, "tensorrt-llm_b200")])
    h = ctypes.CDLL(LIB)
    h.harness_run.argtypes = [ctypes.c_int] * 4 + [ctypes.c_float] + [ctypes.c_int] * 4 + [
        ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong,
        ctypes.c_void_p, ctypes.POINTER(ctypes.c_longlong)]
    h.harness_serialize_groupwise.argtypes = [ctypes.c_int] * 3 + [ctypes.c_float] + [ctypes.c_longlong] * 4 + [
        ctypes.c_char_p, ctypes.c_int]
    return h


def test_header_compiles_without_tensorrt():
    """Without TensorRT headers only the TensorRT-independent layer is compiled; it must stand alone."""
    subprocess.check_call(["g++", "-std=c++17", "-fsyntax-only", "-Wall", "-Werror", "-x", "c++", HDR])


@pytest.mark.parametrize("algo", range(32))
def test_groupwise_input_indices_match_python_mirror(harness, algo):
    idx = (ctypes.c_int * 5)()
    nb = harness.harness_groupwise_indices(algo, idx)
    if (algo & pkg.FP8_ALPHA) and (algo & pkg.INT8_WEIGHT):
        return  # W4A8 exists for int4 weights only: refused by both layers
    m = pkg.WeightOnlyGroupwiseQuantMatmulPlugin(ops.TRT_HALF, algo, 128)
    assert list(idx) == [m.pre_quant_scale_idx, m.weight_idx, m.scales_idx, m.zeros_idx, m.bias_idx]
    assert nb == m.nb_inputs


def test_serialisation_layout(harness):
    buf = ctypes.create_string_buffer(64)
    n = harness.harness_serialize_groupwise(ops.TRT_BF16, 6, 128, 0.5, 1, 256, 14336, 4096, buf, 64)
    blob = buf.raw[:n]
    # type, quant_algo, group_size, alpha, GemmDims{minM, maxM, n, k}, empty tactic map
    assert struct.unpack("<iiif4qi", blob) == (ops.TRT_BF16, 6, 128, 0.5, 1, 256, 14336, 4096, 0)
    mirror = pkg.WeightOnlyGroupwiseQuantMatmulPlugin(ops.TRT_BF16, 6, 128, 0.5)
    mirror.configure_plugin(1, 256, 14336, 4096)
    assert mirror.serialize() == blob


def test_creators_refuse_what_the_library_cannot_run(harness):
    assert harness.harness_create_fails(1, ops.TRT_BF16, pkg.FP8_ALPHA, 128) == 1   # W4A8 with bf16: fp16 scales
    assert harness.harness_create_fails(1, ops.TRT_HALF, pkg.FP8_ALPHA | pkg.INT8_WEIGHT, 128) == 1
    assert harness.harness_create_fails(1, ops.TRT_HALF, pkg.FP8_ALPHA | pkg.PRE_QUANT_SCALE, 128) == 0
    assert harness.harness_create_fails(1, ops.TRT_HALF, 0, 32) == 1                # group size
    assert harness.harness_create_fails(1, 0, 0, 128) == 1                          # fp32 activations
    assert harness.harness_create_fails(0, ops.TRT_HALF, 3, 0) == 1                 # weight type
    assert harness.harness_create_fails(1, ops.TRT_BF16, 7, 64) == 0
    assert harness.harness_create_fails(0, ops.TRT_BF16, 2, 0) == 0


@pytest.mark.parametrize("groupwise,algo", [(1, 0), (1, 7), (1, 16 + 2), (0, 1), (0, 2)])
def test_interface_walk_without_device(harness, groupwise, algo):
    """Creator -> plugin -> dimensions / formats / configure / serialise / deserialise / clone."""
    want = ctypes.c_longlong(-1)
    nb = pkg.WeightOnlyGroupwiseQuantMatmulPlugin(ops.TRT_HALF, algo, 128).nb_inputs if groupwise else 3
    rc = harness.harness_run(groupwise, ops.TRT_HALF, algo, 128, 1.0, 64, 8, 1024, 512, None, nb, None, None, 0, None,
                             ctypes.byref(want))
    assert rc == 0
    bits = (8 if algo & 16 else 4) if groupwise else (8 if algo == 1 else 4)
    assert want.value == ops.workspace_bytes_max(64, 1024, 512, 128 if groupwise else 0, bits, torch.float16,
                                                 bool(groupwise and algo & 4))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [1, 8, 48])
@pytest.mark.parametrize("bias,zero,prequant,int8", list(itertools.product([False, True], repeat=4)))
def test_groupwise_enqueue_every_input_layout(harness, dtype, m, bias, zero, prequant, int8):
    """All 16 quant_algo combinations: the plugin picks every tensor from the right input slot."""
    n, k, group = 512, 1024, 128
    p = make_problem(m, n, k, 8 if int8 else 4, group, dtype, zero=zero, bias=bias, prequant=prequant, seed=m + 17)
    algo = (pkg.BIAS if bias else 0) | (pkg.ZERO if zero else 0) | (pkg.PRE_QUANT_SCALE if prequant else 0) \
        | (pkg.INT8_WEIGHT if int8 else 0)
    dev = "cuda"
    tensors = [p["act"].to(dev)]
    if prequant:
        tensors.append(p["ps"].to(dev))
    tensors += [p["processed"].to(dev), p["scales"].to(dev)]
    if zero:
        tensors.append(p["zeros"].to(dev))
    if bias:
        tensors.append(p["bias"].to(dev))
    out = torch.empty((m, n), dtype=dtype, device=dev)
    ws = torch.empty(ops.workspace_bytes_max(64, n, k, group, 8 if int8 else 4, dtype, prequant) + 16,
                     dtype=torch.uint8, device=dev)
    ptrs = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    type_id = ops.TRT_HALF if dtype == torch.float16 else ops.TRT_BF16
    rc = harness.harness_run(1, type_id, algo, group, 1.0, 64, m, n, k, ptrs, len(tensors), out.data_ptr(),
                             ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream, None)
    assert rc == 0
    torch.cuda.synchronize()
    ref = oracle_out(p)
    assert max_err(out.cpu(), ref) <= oracle.tolerance(ref)  # 1e-2 * max|ref|
    assert pkg._lib.lib().w4_gemm_device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("m", [2, 40])
def test_groupwise_enqueue_w4a8_float16(harness, m):
    """W4A8-AWQ through the C++ plugin: float16 activations, alpha, weights re-laid by the emitter."""
    from tensorrt_llm_b200 import quantize
    n, k, group, alpha = 512, 1024, 128, 0.41
    p = make_problem(m, n, k, 4, group, torch.float16, zero=True, bias=False, prequant=True, seed=m + 3)
    w4a8 = quantize.preprocess_weights_for_mixed_gemm(p["packed"].contiguous(), torch.quint4x2, torch.float8_e4m3fn)
    relaid = quantize.relayout_w4a8_weights(w4a8)
    algo = pkg.FP8_ALPHA | pkg.ZERO | pkg.PRE_QUANT_SCALE
    dev = "cuda"
    tensors = [p["act"].to(dev), p["ps"].to(dev), relaid.to(dev), p["scales"].to(dev), p["zeros"].to(dev)]
    out = torch.empty((m, n), dtype=torch.float16, device=dev)
    ws = torch.empty(ops.workspace_bytes_max(64, n, k, group, 4, torch.float16, True) + 16, dtype=torch.uint8, device=dev)
    ptrs = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    rc = harness.harness_run(1, ops.TRT_HALF, algo, group, alpha, 64, m, n, k, ptrs, len(tensors), out.data_ptr(),
                             ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream, None)
    assert rc == 0
    torch.cuda.synchronize()
    ref = oracle_out(p, alpha=alpha)
    assert max_err(out.cpu(), ref) <= oracle.tolerance(ref)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("wtype,m", [(1, 1), (1, 16), (2, 4), (2, 40)])
def test_per_channel_enqueue(harness, dtype, wtype, m):
    n, k = 1024, 512
    p = make_problem(m, n, k, 8 if wtype == 1 else 4, 0, dtype, seed=5, scale_lo=0.0005, scale_hi=0.002)
    dev = "cuda"
    tensors = [p["act"].to(dev), p["processed"].to(dev), p["scales"].to(dev)]
    out = torch.empty((m, n), dtype=dtype, device=dev)
    ws = torch.empty(ops.workspace_bytes_max(64, n, k, 0, 8 if wtype == 1 else 4, dtype, False) + 16,
                     dtype=torch.uint8, device=dev)
    ptrs = (ctypes.c_void_p * 3)(*[t.data_ptr() for t in tensors])
    type_id = ops.TRT_HALF if dtype == torch.float16 else ops.TRT_BF16
    rc = harness.harness_run(0, type_id, wtype, 0, 1.0, 64, m, n, k, ptrs, 3, out.data_ptr(), ws.data_ptr(), ws.numel(),
                             torch.cuda.current_stream().cuda_stream, None)
    assert rc == 0
    torch.cuda.synchronize()
    ref = oracle_out(p)
    assert max_err(out.cpu(), ref) <= oracle.tolerance(ref)
