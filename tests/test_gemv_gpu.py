"""Parity of the decode kernel with the CPU oracle, through the C ABI (needs a B200)."""
import pytest
import torch

import tensorrt_llm_b200 as pkg
from oracle import woq_oracle as oracle
from _cases import make_problem, max_err, oracle_out, run_gpu

pytestmark = pytest.mark.gpu

GEMV = pkg.W4_REGIME_GEMV


def _check(p, alpha=1.0, regime=GEMV):
    out = run_gpu(p, regime=regime, alpha=alpha)
    ref = oracle_out(p, alpha=alpha)
    assert out.shape == ref.shape and out.dtype == ref.dtype
    assert torch.isfinite(out.float()).all()
    # Bound this path is held to: max abs error <= 1e-2 of max|ref|.
    tol = oracle.tolerance(ref)
    err = max_err(out, ref)
    assert err <= tol, f"max err {err} > {tol}"
    assert pkg._lib.lib().w4_gemm_device_status() == 0
    return err / max(tol * 100, 1e-30)  # error as a fraction of max|ref|


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("group", [64, 128])
@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 9, 16])
def test_groupwise_all_options(dtype, bits, group, m):
    p = make_problem(m, 256, 512, bits, group, dtype, zero=True, bias=True, prequant=True, seed=m)
    _check(p, alpha=1.0)


@pytest.mark.parametrize("zero,bias,prequant", [(False, False, False), (True, False, False), (False, True, False),
                                                (False, False, True), (True, True, False)])
@pytest.mark.parametrize("bits", [4, 8])
def test_groupwise_option_subsets(zero, bias, prequant, bits):
    p = make_problem(4, 512, 1024, bits, 128, torch.bfloat16, zero=zero, bias=bias, prequant=prequant, seed=7)
    _check(p)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("m,n,k", [(1, 1024, 4096), (16, 4096, 4096), (4, 64, 64), (7, 192, 320), (2, 6144, 2048)])
def test_per_channel(dtype, bits, m, n, k):
    p = make_problem(m, n, k, bits, 0, dtype, seed=3, scale_lo=0.0005, scale_hi=0.002)
    _check(p)


# The reference's own test shapes for the groupwise plugin
# (tests/quantization/test_weight_only_groupwise_quant_matmul.py:248-407), decode-sized rows.
@pytest.mark.parametrize("m,n,k,group", [(1, 1024, 64, 64), (16, 1024, 256, 64), (2, 1024, 128, 128),
                                         (8, 1024, 256, 128), (3, 2048, 384, 64), (4, 2048, 1024, 128)])
@pytest.mark.parametrize("bits", [4, 8])
def test_reference_test_shapes(m, n, k, group, bits):
    p = make_problem(m, n, k, bits, group, torch.float16, zero=True, bias=True, prequant=True, seed=11)
    _check(p)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("m,n,k,group", [(3, 1024, 8192, 128), (8, 2048, 12288, 128), (12, 512, 6144, 64),
                                         (1, 14336, 8192, 128), (16, 4096, 14336, 128)])
def test_several_k_panels(m, n, k, group, bits):
    """K larger than one shared-memory panel: column groups are walked in sub-batches that share
    the activation fragments."""
    p = make_problem(m, n, k, bits, group, torch.bfloat16, zero=True, bias=True, prequant=True, seed=k // 64 + m)
    _check(p)


def test_alpha_scaling():
    p = make_problem(2, 256, 256, 4, 128, torch.bfloat16, zero=True, seed=5)
    _check(p, alpha=0.5)


def test_larger_m_runs_in_passes():
    p = make_problem(40, 512, 512, 4, 128, torch.bfloat16, zero=True, bias=True, seed=9)
    _check(p)


def test_matches_reference_test_ground_truth():
    """Against the reference test's own ground truth (every torch op rounded to the activation
    type), same 1e-2 * max|ref| bound."""
    p = make_problem(8, 1024, 2048, 4, 128, torch.bfloat16, zero=True, bias=True, prequant=True, seed=13)
    out = run_gpu(p, regime=GEMV)
    ref = oracle.groupwise_matmul_test_ref(p["act"], p["q"], p["scales"], p["zeros"], p["bias"], p["ps"], 128)
    assert max_err(out, ref) <= oracle.tolerance(ref)


def test_identity_activation_recovers_layout():
    """The reference's layout round trip (tests/quantization/test_weight_only_quant_matmul.py:147-164):
    multiplying the preprocessed weight by an identity activation returns the dequantised weight,
    so every column/row permutation of the layout is exercised. Exact: each output is one product."""
    k = n = 256
    for bits in (4, 8):
        p = make_problem(16, n, k, bits, 0, torch.float16, seed=17)
        scales = torch.ones(n, dtype=torch.float16)
        got = []
        for r0 in range(0, k, 16):
            act = torch.zeros(16, k, dtype=torch.float16)
            act[torch.arange(16), r0 + torch.arange(16)] = 1.0
            q = dict(p, act=act, scales=scales)
            got.append(run_gpu(q, regime=GEMV))
        w = torch.cat(got, 0)
        assert torch.equal(w.to(torch.int32), p["q"].to(torch.int32))


def test_c2_decode_shape_all_m():
    """BASELINE config 2 at full size: int4 g128 AWQ (zeros + pre-quant scale), bf16, K=4096, N=14336."""
    g = torch.Generator().manual_seed(1)
    p = make_problem(16, 14336, 4096, 4, 128, torch.bfloat16, zero=True, prequant=True, seed=1)
    p["ps"] = torch.ones(4096, dtype=torch.bfloat16)
    full = oracle_out(p)
    for m in (1, 2, 4, 8, 16):
        q = dict(p, act=p["act"][:m].contiguous(), m=m)
        out = run_gpu(q, regime=GEMV)
        assert max_err(out, full[:m]) <= oracle.tolerance(full[:m])


def test_c1_w8a16_per_channel():
    """BASELINE config 1: W8A16 per-channel, fp16, M=16, K=N=4096, weights ~N(0, 0.02) quantised by
    symmetric_quantize_last_axis_of_batched_matrix."""
    torch.manual_seed(0)
    act = torch.randn(16, 4096).to(torch.float16)
    w = torch.randn(4096, 4096) * 0.02
    u, processed, scales = pkg.quantize._symmetric_quantize_last_axis_of_batched_matrix(w, torch.int8)
    scales = scales.to(torch.float16)
    out = pkg.ops.weight_only_quant_matmul(act.cuda(), processed.cuda(), scales.cuda(), 1, regime=GEMV).cpu()
    ref = oracle.per_channel_matmul_test_ref(act, u, scales)
    assert max_err(out, ref) <= oracle.tolerance(ref)
    # and it approximates the unquantised product as well as int8 allows
    dense = (act.float() @ w).to(torch.float16)
    assert max_err(out, dense) <= 2e-2 * float(dense.float().abs().max())
