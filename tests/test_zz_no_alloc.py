"""GPU: the allocation-free entry point (w4_gemm_launch_static_scratch) against the ordinary one.

Some users of this library cannot hand a workspace to w4_gemm_launch: they run where device
allocation is closed (an allocation-free region of a serving loop, a plugin host that granted no
workspace, a process whose allocator belongs to somebody else). For them the library keeps the
one scratch buffer the prefill kernel needs - the activations times the AWQ pre-quant scale -
in an 8 MiB array inside its own image. This test calls that entry point through the C ABI twice
in a row, with different problems so that the second call finds the first call's data in the
shared array, and requires the same output as w4_gemm_launch with a caller-owned workspace
(bit for bit: both run the same kernels). It is collected last on purpose.
"""
import ctypes

import pytest
import torch

import tensorrt_llm_b200 as pkg
from tensorrt_llm_b200._lib import W4GemmParams
from _cases import make_problem

pytestmark = pytest.mark.gpu


def _params(p, dev, out, workspace):
    t = {k: (None if p[k] is None else p[k].to(dev)) for k in ("act", "ps", "processed", "scales", "zeros", "bias")}
    ptr = lambda x: None if x is None else ctypes.c_void_p(x.data_ptr())
    params = W4GemmParams(
        act=ptr(t["act"]), act_scale=ptr(t["ps"]), weight=ptr(t["processed"]), scales=ptr(t["scales"]),
        zeros=ptr(t["zeros"]), bias=ptr(t["bias"]), out=ptr(out), alpha=1.0, m=p["m"], n=p["n"], k=p["k"],
        group_size=p["group"], weight_bits=p["bits"], act_dtype=1 if p["dtype"] == torch.bfloat16 else 0,
        regime=pkg.W4_REGIME_GEMM, workspace=ptr(workspace),
        workspace_bytes=0 if workspace is None else workspace.numel())
    return params, t  # keep the device tensors alive with the struct


def test_static_scratch_matches_workspace_path_twice():
    lib = pkg._lib.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    assert lib.w4_gemm_static_scratch_bytes() == 8 * 1024 * 1024
    problems = [
        make_problem(384, 256, 1024, 4, 128, torch.bfloat16, zero=True, bias=True, prequant=True, seed=31),
        make_problem(100, 512, 512, 8, 64, torch.float16, zero=True, bias=False, prequant=True, seed=32),
        # few output tiles: the kernel also parks the fp32 partial tiles of its split-k in the array,
        # behind the scaled activations (1 MiB + 4.4 MiB here); run twice in a row
        make_problem(64, 1280, 8192, 4, 128, torch.bfloat16, zero=True, bias=True, prequant=True, seed=33),
        make_problem(64, 1280, 8192, 4, 128, torch.bfloat16, zero=True, bias=True, prequant=True, seed=34),
    ]
    for p in problems:
        need = lib.w4_gemm_workspace_bytes(p["m"], p["n"], p["k"], p["group"], p["bits"],
                                           1 if p["dtype"] == torch.bfloat16 else 0, 1, pkg.W4_REGIME_GEMM)
        assert 0 < need <= 8 * 1024 * 1024
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        ref_out = torch.zeros((p["m"], p["n"]), dtype=p["dtype"], device=dev)
        params, keep = _params(p, dev, ref_out, ws)
        assert lib.w4_gemm_launch(ctypes.byref(params), stream) == 0

        out = torch.zeros_like(ref_out)
        params2, keep2 = _params(p, dev, out, None)  # no workspace at all
        # a first call resolves the array's address and loads the kernels; the device's free memory
        # (driver view: catches a cudaMalloc inside the library, which torch's own counter would not)
        # must not move across the second
        assert lib.w4_gemm_launch_static_scratch(ctypes.byref(params2), stream) == 0
        torch.cuda.synchronize()
        out.zero_()
        free_before, _ = torch.cuda.mem_get_info(dev)
        before = torch.cuda.memory_allocated(dev)
        assert lib.w4_gemm_launch_static_scratch(ctypes.byref(params2), stream) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(dev) == before
        assert torch.cuda.mem_get_info(dev)[0] >= free_before  # nothing was taken from the device
        assert lib.w4_gemm_device_status() == 0
        assert torch.equal(out, ref_out), float((out.float() - ref_out.float()).abs().max())
        assert float(out.float().abs().max()) > 0


def test_static_scratch_rejects_oversized_problem():
    lib = pkg._lib.lib()
    big = W4GemmParams(act=16, act_scale=16, weight=16, scales=16, out=16, alpha=1.0, m=4096, n=4096, k=4096,
                       group_size=128, weight_bits=4, act_dtype=1, regime=0)
    rc = lib.w4_gemm_launch_static_scratch(ctypes.byref(big), None)  # rejected before any pointer is used
    assert rc == -11 and "scratch" in pkg._lib.status_string(rc)
