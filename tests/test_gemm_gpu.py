"""Parity of the tcgen05 tensor-core kernel with the CPU oracle, through the C ABI (needs a B200)."""
import pytest
import torch

import tensorrt_llm_b200 as pkg
from oracle import woq_oracle as oracle
from _cases import make_problem, max_err, oracle_out, run_gpu

pytestmark = pytest.mark.gpu
GEMM = pkg.W4_REGIME_GEMM


def _check(p, alpha=1.0, regime=GEMM):
    out = run_gpu(p, regime=regime, alpha=alpha)
    ref = oracle_out(p, alpha=alpha)
    assert out.shape == ref.shape and out.dtype == ref.dtype
    assert torch.isfinite(out.float()).all()
    tol = oracle.tolerance(ref)  # 1e-2 of max|ref|
    err = max_err(out, ref)
    assert err <= tol, f"max err {err} > {tol}"
    assert pkg._lib.lib().w4_gemm_device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("group", [64, 128])
@pytest.mark.parametrize("m", [17, 64, 100, 128, 200, 256, 300, 513])
def test_groupwise_all_options(dtype, bits, group, m):
    p = make_problem(m, 256, 512, bits, group, dtype, zero=True, bias=True, prequant=True, seed=m)
    _check(p)


@pytest.mark.parametrize("zero,bias,prequant", [(False, False, False), (True, False, False), (False, True, False),
                                                (False, False, True)])
@pytest.mark.parametrize("bits", [4, 8])
def test_groupwise_option_subsets(zero, bias, prequant, bits):
    p = make_problem(384, 512, 1024, bits, 128, torch.bfloat16, zero=zero, bias=bias, prequant=prequant, seed=7)
    _check(p)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("m,n,k", [(128, 6144, 1024), (64, 1024, 4096), (256, 192, 320), (1000, 64, 64)])
def test_per_channel(dtype, bits, m, n, k):
    p = make_problem(m, n, k, bits, 0, dtype, seed=3, scale_lo=0.0005, scale_hi=0.002)
    _check(p)


# Prefill-sized rows of the reference's groupwise test list
# (tests/quantization/test_weight_only_groupwise_quant_matmul.py:248-407).
@pytest.mark.parametrize("m,n,k,group", [(32, 2048, 384, 64), (64, 2048, 1024, 64), (48, 2048, 384, 128),
                                         (96, 2048, 1024, 128), (192, 1024, 256, 128), (512, 2048, 1024, 128)])
@pytest.mark.parametrize("bits", [4, 8])
def test_reference_test_shapes(m, n, k, group, bits):
    p = make_problem(m, n, k, bits, group, torch.float16, zero=True, bias=True, prequant=True, seed=11)
    _check(p)


def test_alpha_and_many_tiles_per_cta():
    # more tiles than SMs: every CTA runs several tiles back to back through the same TMEM
    p = make_problem(1024, 4096, 256, 4, 128, torch.bfloat16, zero=True, bias=True, seed=5)
    _check(p, alpha=0.25)


def test_agrees_with_decode_kernel():
    """Both regimes on the same problem: they may differ only by rounding."""
    p = make_problem(16, 512, 1024, 4, 128, torch.bfloat16, zero=True, bias=True, seed=21)
    a = run_gpu(p, regime=pkg.W4_REGIME_GEMV)
    b = run_gpu(p, regime=GEMM)
    ref = oracle_out(p)
    assert max_err(a, b) <= oracle.tolerance(ref)


def test_matches_reference_test_ground_truth():
    p = make_problem(256, 1024, 2048, 4, 128, torch.bfloat16, zero=True, bias=True, prequant=True, seed=13)
    out = run_gpu(p, regime=GEMM)
    ref = oracle.groupwise_matmul_test_ref(p["act"], p["q"], p["scales"], p["zeros"], p["bias"], p["ps"], 128)
    assert max_err(out, ref) <= oracle.tolerance(ref)


def test_linearity_at_full_size():
    """BASELINE config 3 shape (M=4096, K=14336, N=4096): too large for the CPU oracle on every row,
    so check a size-independent property on all outputs - f(a1 + a2) = f(a1) + f(a2) up to
    rounding - and the oracle on a sample of rows."""
    m, n, k = 4096, 4096, 14336
    p = make_problem(m, n, k, 4, 128, torch.bfloat16, zero=True, seed=2)
    g = torch.Generator().manual_seed(99)
    a2 = torch.randn((m, k), generator=g).to(torch.bfloat16)
    y1 = run_gpu(p, regime=GEMM).float()
    y2 = run_gpu(dict(p, act=a2), regime=GEMM).float()
    s = (p["act"].float() + a2.float()).to(torch.bfloat16)
    resid = (s.float() - p["act"].float() - a2.float())  # rounding of the sum, accounted for below
    y12 = run_gpu(dict(p, act=s), regime=GEMM).float()
    scale = float(y12.abs().max())
    assert float((y12 - y1 - y2).abs().max()) <= 2e-2 * scale + float(resid.abs().max()) * k * 0.1
    # rows at the boundaries of every candidate row tile (128 / 192 / 256, the ragged last tile
    # included: 4096 = 21 * 192 + 64) and a few random ones
    from _cases import sample_rows
    rows = torch.tensor(sample_rows(m, seed=4))
    ref = oracle_out(dict(p, act=p["act"][rows].contiguous(), m=len(rows)))
    assert max_err(y1[rows].to(torch.bfloat16), ref) <= oracle.tolerance(ref)


@pytest.mark.parametrize("m,n,k,bits", [(1024, 4096, 4096, 4), (2048, 4096, 2048, 4), (176, 2048, 4096, 8),
                                        (192, 2048, 4096, 8), (192, 32768, 2048, 8), (384, 16384, 1152, 8)])
def test_odd_stage_counts_over_a_long_ring(m, n, k, bits):
    """Row tiles whose shared-memory ring has three stages (int4 with 256 rows; int8 with 192 rows,
    which the cost model picks when the column tiles fill several waves), with 9 to 32 k steps, one
    case with an odd number of steps per tile: each conversion group meets a stage in every second
    pass of the ring only, and with an odd step count the stages it meets change from tile to tile."""
    p = make_problem(m, n, k, bits, 128, torch.bfloat16, zero=True, seed=m + bits)
    rows = list(range(0, m, 37)) + [m - 1]
    out = run_gpu(p, regime=GEMM)
    ref = oracle_out(dict(p, act=p["act"][rows].contiguous(), m=len(rows)))
    assert max_err(out[rows], ref) <= oracle.tolerance(ref)


@pytest.mark.parametrize("m,n,k,bits,group,dtype", [
    (64, 1280, 8192, 4, 128, torch.bfloat16),   # 10 tiles: 14-way split
    (100, 512, 4096, 8, 64, torch.bfloat16),
    (200, 1024, 2048, 8, 0, torch.float16),     # per-channel scales, splits start mid-matrix
    (17, 256, 4160, 4, 64, torch.float16),      # k = 65 * 64: the last step of the last split is half empty
    (256, 4096, 14336, 4, 128, torch.bfloat16),
])
def test_split_k(m, n, k, bits, group, dtype):
    """Few output tiles: the k range is split over SMs (fp32 partial tiles in the workspace, added
    in split order by a second kernel). Same oracle, same tolerance; and the same problem with only
    the mandatory part of the workspace (no split) agrees to rounding."""
    full = group != 0
    p = make_problem(m, n, k, bits, group, dtype, zero=full, bias=full, prequant=full, seed=m + k)
    lib = pkg._lib.lib()
    dt = pkg._lib.W4_DTYPE_FP16 if dtype == torch.float16 else pkg._lib.W4_DTYPE_BF16
    need = lib.w4_gemm_workspace_bytes(m, n, k, group, bits, dt, int(full), GEMM)
    assert need > (m * k * 2 if full else 0), "this shape is expected to use split-k"
    alpha = 0.5 if full else 1.0
    _check(p, alpha=alpha)
    # unsplit run of the same problem through the raw entry point with the minimal workspace
    d = lambda t: None if t is None else t.cuda()
    out = torch.empty(m, n, dtype=dtype, device="cuda")
    ws = torch.empty(max(m * k * 2, 16), dtype=torch.uint8, device="cuda") if full else None
    pkg.ops.gemm_raw(d(p["act"]), d(p["processed"]), d(p["scales"]), out, n=n, k=k, weight_bits=bits, group_size=group,
                     zeros=d(p["zeros"]), bias=d(p["bias"]), act_scale=d(p["ps"]), alpha=alpha, regime=GEMM,
                     workspace=ws)
    ref = oracle_out(p, alpha=alpha)
    assert max_err(out.cpu(), ref) <= oracle.tolerance(ref)
