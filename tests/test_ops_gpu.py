"""The operator boundary on the GPU (needs a B200): the C++ torch.ops.trtllm GEMM ops and both
plugin mirrors' enqueue, every quant_algo input layout, against the CPU oracle."""
import itertools

import pytest
import torch

import tensorrt_llm_b200 as pkg
import tensorrt_llm_b200.torch_ops  # noqa: F401  (loads the C++ registrations)
from tensorrt_llm_b200 import ops
from oracle import woq_oracle as oracle
from _cases import make_problem, max_err, oracle_out

pytestmark = pytest.mark.gpu


def _d(t):
    return None if t is None else t.to("cuda")


def _assert_close(out, p, alpha=1.0):
    ref = oracle_out(p, alpha=alpha)
    assert out.shape == ref.shape and out.dtype == ref.dtype
    assert max_err(out.cpu(), ref) <= oracle.tolerance(ref)  # 1e-2 * max|ref|
    assert pkg._lib.lib().w4_gemm_device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("m", [1, 16, 300])
def test_torch_op_per_channel(dtype, bits, m):
    p = make_problem(m, 1024, 512, bits, 0, dtype, seed=m, scale_lo=0.0005, scale_hi=0.002)
    out = torch.ops.trtllm.weight_only_quant_gemm(_d(p["act"]), _d(p["processed"]), _d(p["scales"]),
                                                  1 if bits == 8 else 2)
    _assert_close(out, p)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [1, 12, 256])
@pytest.mark.parametrize("bias,zero,prequant,int8", list(itertools.product([False, True], repeat=4)))
def test_torch_op_groupwise_every_algo(dtype, m, bias, zero, prequant, int8):
    p = make_problem(m, 512, 1024, 8 if int8 else 4, 128, dtype, zero=zero, bias=bias, prequant=prequant, seed=3 + m)
    algo = (pkg.BIAS if bias else 0) | (pkg.ZERO if zero else 0) | (pkg.PRE_QUANT_SCALE if prequant else 0) \
        | (pkg.INT8_WEIGHT if int8 else 0)
    out = torch.ops.trtllm.weight_only_groupwise_quant_gemm(
        _d(p["act"]), _d(p["ps"]), _d(p["processed"]), _d(p["scales"]), _d(p["zeros"]), _d(p["bias"]), 0.75, algo, 128,
        weights_static=True)
    _assert_close(out, p, alpha=0.75)


def test_torch_op_leading_dims_and_weight_viewed_as_activation_type():
    """[B, S, K] activations; the weight viewed as fp16 as the groupwise plugin receives it."""
    p = make_problem(6, 512, 256, 4, 64, torch.float16, zero=True, seed=2)
    act = _d(p["act"]).reshape(2, 3, 256)
    w = _d(p["processed"]).view(torch.float16)
    out = torch.ops.trtllm.weight_only_groupwise_quant_gemm(act, None, w, _d(p["scales"]), _d(p["zeros"]), None, 1.0,
                                                            pkg.ZERO, 64)
    assert out.shape == (2, 3, 512)
    _assert_close(out.reshape(6, 512), p)


def test_torch_op_errors():
    p = make_problem(2, 256, 256, 4, 128, torch.float16, zero=True, seed=1)
    a, w, s, z = _d(p["act"]), _d(p["processed"]), _d(p["scales"]), _d(p["zeros"])
    with pytest.raises(RuntimeError, match="zeros must be given exactly"):
        torch.ops.trtllm.weight_only_groupwise_quant_gemm(a, None, w, s, None, None, 1.0, pkg.ZERO, 128)
    with pytest.raises(RuntimeError, match="INT4"):  # W4A8 exists for int4 weights only
        torch.ops.trtllm.weight_only_groupwise_quant_gemm(a, None, w, s, z, None, 1.0,
                                                          pkg.ZERO | pkg.FP8_ALPHA | pkg.INT8_WEIGHT, 128)
    with pytest.raises(RuntimeError, match="group_size"):
        torch.ops.trtllm.weight_only_groupwise_quant_gemm(a, None, w, s, z, None, 1.0, pkg.ZERO, 32)
    with pytest.raises(RuntimeError, match="wTypeId"):
        torch.ops.trtllm.weight_only_quant_gemm(a, w, s[0].contiguous(), 3)
    with pytest.raises(RuntimeError):  # no CPU implementation of the GEMM: a dispatch error, not a fallback
        torch.ops.trtllm.weight_only_quant_gemm(p["act"], p["processed"], p["scales"][0].contiguous(), 2)
    empty = torch.ops.trtllm.weight_only_groupwise_quant_gemm(a[:0], None, w, s, z, None, 1.0, pkg.ZERO, 128)
    assert empty.shape == (0, 256)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [1, 9, 200])
@pytest.mark.parametrize("bias,zero,prequant,int8", list(itertools.product([False, True], repeat=4)))
def test_groupwise_plugin_mirror_enqueue(dtype, m, bias, zero, prequant, int8):
    """Inputs in the plugin's order [act, (pre_quant_scale), weight, scales, (zeros), (bias)],
    caller-owned output and workspace, status code instead of an exception."""
    n, k = 512, 1024
    p = make_problem(m, n, k, 8 if int8 else 4, 128, dtype, zero=zero, bias=bias, prequant=prequant, seed=11 + m)
    algo = (pkg.BIAS if bias else 0) | (pkg.ZERO if zero else 0) | (pkg.PRE_QUANT_SCALE if prequant else 0) \
        | (pkg.INT8_WEIGHT if int8 else 0)
    plugin = pkg.WeightOnlyGroupwiseQuantMatmulPlugin(ops.TRT_HALF if dtype == torch.float16 else ops.TRT_BF16, algo, 128)
    plugin.configure_plugin(1, 256, n, k)
    inputs = [_d(p["act"])] + ([_d(p["ps"])] if prequant else []) + [_d(p["processed"]).view(dtype), _d(p["scales"])] \
        + ([_d(p["zeros"])] if zero else []) + ([_d(p["bias"])] if bias else [])
    assert len(inputs) == plugin.nb_inputs
    out = torch.empty((m, n), dtype=dtype, device="cuda")
    nws = plugin.get_workspace_size()
    ws = torch.empty(max(nws, 1), dtype=torch.uint8, device="cuda")
    assert plugin.enqueue(inputs, [out], ws if nws else None) == 0
    _assert_close(out, p)
    # a missing input is a status code, not an exception
    assert plugin.enqueue(inputs[:-1], [out], ws if nws else None) != 0
    # serialise -> deserialise keeps the behaviour
    twin = pkg.WeightOnlyGroupwiseQuantMatmulPlugin.deserialize(plugin.serialize())
    out2 = torch.empty_like(out)
    assert twin.enqueue(inputs, [out2], ws if nws else None) == 0
    assert torch.equal(out, out2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("wtype,m", [(1, 1), (1, 4), (1, 33), (2, 2), (2, 16), (2, 130)])
def test_per_channel_plugin_mirror_enqueue(dtype, wtype, m):
    n, k = 1024, 512
    p = make_problem(m, n, k, 8 if wtype == 1 else 4, 0, dtype, seed=7, scale_lo=0.0005, scale_hi=0.002)
    plugin = pkg.WeightOnlyQuantMatmulPlugin(ops.TRT_HALF if dtype == torch.float16 else ops.TRT_BF16, wtype)
    plugin.configure_plugin(1, 256, n, k)
    out = torch.empty((m, n), dtype=dtype, device="cuda")
    nws = plugin.get_workspace_size()
    ws = torch.empty(max(nws, 1), dtype=torch.uint8, device="cuda")
    assert plugin.enqueue([_d(p["act"]), _d(p["processed"]), _d(p["scales"])], [out], ws if nws else None) == 0
    _assert_close(out, p)
    assert plugin.enqueue([_d(p["act"])[:0], _d(p["processed"]), _d(p["scales"])], [out[:0]], None) == 0  # m == 0


@pytest.mark.parametrize("m,regime", [(1, pkg.W4_REGIME_GEMV), (5, pkg.W4_REGIME_AUTO), (200, pkg.W4_REGIME_GEMM)])
def test_host_entry_point(m, regime):
    """w4_gemm_run_host: pinned host activations in, pinned host result out, valid on return; twice
    with different activations through the same prepared parameter block."""
    p = make_problem(m, 1024, 512, 4, 128, torch.bfloat16, zero=True, bias=True, prequant=True, seed=40 + m)
    d_act = torch.empty_like(_d(p["act"]))
    d_out = torch.empty((m, 1024), dtype=torch.bfloat16, device="cuda")
    nb = ops.workspace_bytes(m, 1024, 512, 128, 4, torch.bfloat16, True, regime)
    ws = torch.empty(max(nb, 16), dtype=torch.uint8, device="cuda")
    g = ops.PreparedGemm(d_act, _d(p["processed"]), _d(p["scales"]), d_out, n=1024, k=512, weight_bits=4,
                         group_size=128, zeros=_d(p["zeros"]), bias=_d(p["bias"]), act_scale=_d(p["ps"]),
                         regime=regime, workspace=ws)
    h_out = torch.zeros((m, 1024), dtype=torch.bfloat16).pin_memory()
    stream = torch.cuda.current_stream().cuda_stream
    for scale in (1.0, -2.0):
        q = dict(p)
        q["act"] = (p["act"].float() * scale).to(torch.bfloat16)
        g.run_host(q["act"].contiguous().pin_memory(), h_out, stream)
        _assert_close(h_out, q)  # no synchronize here: the call returns with the result in place
    # pageable host memory takes the copy path
    pageable_out = torch.zeros((m, 1024), dtype=torch.bfloat16)
    g.run_host(p["act"].contiguous(), pageable_out, stream)
    _assert_close(pageable_out, p)
    with pytest.raises(RuntimeError):
        g.run_host(d_act, h_out, stream)
    with pytest.raises(RuntimeError):
        g.run_host(p["act"][:, :256].contiguous(), h_out, stream)


@pytest.mark.parametrize("bits,group", [(4, 128), (8, 0)])
def test_experts_over_3d_weights(bits, group):
    """w4_gemm_launch_experts: 3-D weights laid out per expert by the (3-D capable) layout op, rows
    sorted by expert, one expert without rows, row counts on both sides of the regime switch."""
    from tensorrt_llm_b200 import quantize
    dtype, k, n = torch.float16, 512, 384
    rows = [3, 0, 40, 1, 9]
    first = [0]
    for r in rows:
        first.append(first[-1] + r)
    probs = [make_problem(max(r, 1), n, k, bits, group, dtype, zero=group != 0, bias=group != 0, seed=70 + e)
             for e, r in enumerate(rows)]
    # the layout op on the stacked tensor must equal the per-expert layout (what the kernels consume)
    stacked = torch.stack([p["packed"] for p in probs]).contiguous()
    qt = torch.quint4x2 if bits == 4 else torch.int8
    w3 = quantize.preprocess_weights_for_mixed_gemm(stacked, qt, torch.float16)
    for e, p in enumerate(probs):
        assert torch.equal(w3[e], p["processed"])
    act = torch.cat([p["act"][:r] for p, r in zip(probs, rows)])
    stack = lambda key: None if probs[0][key] is None else torch.stack([p[key] for p in probs]).cuda()
    out = ops.moe_gemm(act.cuda(), w3.cuda(), stack("scales"), first, weight_bits=bits, group_size=group,
                       zeros=stack("zeros"), bias=stack("bias")).cpu()
    assert out.shape == (sum(rows), n)
    for e, (p, r) in enumerate(zip(probs, rows)):
        if r == 0:
            continue
        q = dict(p)
        q["act"] = p["act"][:r]
        ref = oracle_out(q)
        got = out[first[e]:first[e + 1]]
        assert max_err(got, ref) <= oracle.tolerance(ref), e
    assert pkg._lib.lib().w4_gemm_device_status() == 0
    with pytest.raises(RuntimeError):
        ops.moe_gemm(act.cuda(), w3.cuda(), stack("scales"), first[:-1], weight_bits=bits, group_size=group)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [1, 12, 300])
def test_w4a8_awq_layer(dtype, m):
    """A W4A8-AWQ layer as the reference's test builds it (tests/quantization/
    test_weight_only_groupwise_quant_matmul.py:150-245): int4 weights laid out for fp8 activations,
    float16 scales and zeros whatever the activation type, a pre-quant scale and an fp8 alpha. The
    constants are prepared once; result against the reference test's ground truth
    (act * alpha * pre_quant_scale) @ (q * s + z) + bias through the three public routes."""
    from tensorrt_llm_b200 import quantize
    k, n, group, alpha = 512, 384, 128, 0.37
    p = make_problem(m, n, k, 4, group, dtype, zero=True, bias=True, prequant=True, seed=90 + m)
    s16, z16 = p["scales"].to(torch.float16), p["zeros"].to(torch.float16)
    p["scales"], p["zeros"] = s16.to(dtype), z16.to(dtype)  # what the kernels see after the cast
    w4a8 = quantize.preprocess_weights_for_mixed_gemm(p["packed"].contiguous(), torch.quint4x2, torch.float8_e4m3fn)
    assert not torch.equal(w4a8, p["processed"])
    algo = pkg.FP8_ALPHA | pkg.ZERO | pkg.BIAS | pkg.PRE_QUANT_SCALE
    ref = oracle_out(p, alpha=alpha)
    w, s, z = ops.prepare_w4a8_layer(w4a8, s16, z16, dtype, "cuda")
    assert torch.equal(w.cpu(), p["processed"])
    out = ops.weight_only_groupwise_quant_matmul(_d(p["act"]), _d(p["ps"]), w, _d(s16), _d(z16), _d(p["bias"]), alpha,
                                                 algo, group)
    assert max_err(out.cpu(), ref) <= oracle.tolerance(ref)
    out2 = torch.ops.trtllm.weight_only_groupwise_quant_gemm(_d(p["act"]), _d(p["ps"]), w, _d(s16), _d(z16),
                                                             _d(p["bias"]), alpha, algo, group)
    assert torch.equal(out2, out)
    # the plugin mirror takes the engine's constants as the reference would hand them over
    plug = pkg.WeightOnlyGroupwiseQuantMatmulPlugin(ops.TRT_HALF if dtype == torch.float16 else ops.TRT_BF16, algo,
                                                    group, alpha)
    plug.configure_plugin(1, 512, n, k)
    ws = torch.empty(max(plug.get_workspace_size(), 16), dtype=torch.uint8, device="cuda")
    out3 = torch.empty((m, n), dtype=dtype, device="cuda")
    inputs = [_d(p["act"]), _d(p["ps"]), _d(w4a8), _d(s16), _d(z16), _d(p["bias"])]
    for _ in range(2):  # the second call uses the cached constants
        assert plug.enqueue(inputs, [out3], ws) == 0
        torch.cuda.synchronize()
        assert torch.equal(out3, out)


def test_debug_log_names_the_kernel_taken(capfd):
    """At DEBUG the library prints one line per launch: the shape and which kernel ran."""
    lib = pkg._lib.lib()
    small = make_problem(2, 256, 512, 4, 128, torch.float16, zero=True, seed=1)
    large = make_problem(300, 256, 512, 4, 128, torch.float16, zero=True, seed=2)
    try:
        lib.w4_set_log_level(pkg._lib.W4_LOG_DEBUG)
        capfd.readouterr()
        for p in (small, large):
            out = ops.weight_only_groupwise_quant_matmul(_d(p["act"]), None, _d(p["processed"]), _d(p["scales"]),
                                                         _d(p["zeros"]), None, 1.0, pkg.ZERO, 128)
            _assert_close(out, p)
        lines = [l for l in capfd.readouterr().err.splitlines() if l.startswith("[w4_gemm][DEBUG] w4_gemm_launch")]
        assert len(lines) == 2
        assert "m=2 n=256 k=512 bits=4 group=128" in lines[0] and "decode kernel (chosen)" in lines[0]
        assert "m=300" in lines[1] and "tensor-core kernel (chosen)" in lines[1]
    finally:
        lib.w4_set_log_level(-1)
