"""Parity on the real layer shapes the path is benchmarked on (needs a B200), AUTO regime, through
the C ABI: the tensor-parallel Llama-3-70B shard shapes (per-rank K / N at tp = 1, 2, 4, 8) and the
seven Llama-3-8B shapes in every weight format and activation type. Large problems are checked on a
sample of rows and columns (row-tile boundaries included) against the float64 oracle."""
import pytest
import torch

import tensorrt_llm_b200 as pkg
from oracle import woq_oracle as oracle
from _cases import make_problem, max_err, oracle_subset, sample_cols, sample_rows

pytestmark = pytest.mark.gpu

# (name, K, N, split): column-parallel layers split N, row-parallel layers split K
# (tensorrt_llm/layers/linear.py:340-343, 466-468 of the reference).
LLAMA70B = [("qkv", 8192, 10240, "n"), ("gate_up", 8192, 57344, "n"), ("o_proj", 8192, 8192, "k"),
            ("down", 28672, 8192, "k")]
# distinct (K, N) of the Llama-3-8B linears: q / o, k / v, gate / up, down
LLAMA8B = [(4096, 4096), (4096, 1024), (4096, 14336), (14336, 4096)]
FORMATS = [("w8_pc", 8, 0), ("w4_g64", 4, 64), ("w4_g128", 4, 128)]


def _run_rows(p, dev_tensors, m, regime=0):
    act = p["act"][:m].contiguous().to("cuda")
    w, s, z, b, ps = dev_tensors
    if p["group"] == 0:
        return pkg.ops.weight_only_quant_matmul(act, w, s, 1 if p["bits"] == 8 else 2, regime=regime)
    algo = (pkg.INT8_WEIGHT if p["bits"] == 8 else 0) | (pkg.ZERO if z is not None else 0) \
        | (pkg.BIAS if b is not None else 0) | (pkg.PRE_QUANT_SCALE if ps is not None else 0)
    return pkg.ops.weight_only_groupwise_quant_matmul(act, ps, w, s, z, b, 1.0, algo, p["group"], regime=regime)


def _check_m_values(p, ms, seed):
    d = lambda t: None if t is None else t.to("cuda")
    dev = (d(p["processed"]), d(p["scales"]), d(p["zeros"]), d(p["bias"]), d(p["ps"]))
    cols = sample_cols(p["n"], seed=seed)
    for m in ms:
        out = _run_rows(p, dev, m).cpu()
        rows = sample_rows(m, seed=seed + m)
        q = dict(p, act=p["act"][:m])
        ref = oracle_subset(q, rows, cols)
        got = out[rows][:, cols]
        assert torch.isfinite(got.float()).all()
        err, tol = max_err(got, ref), oracle.tolerance(ref)  # 1e-2 * max|ref|
        assert err <= tol, f"m={m}: max err {err} > {tol}"
    assert pkg._lib.lib().w4_gemm_device_status() == 0


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
@pytest.mark.parametrize("name,k,n,split", LLAMA70B)
def test_llama70b_shard_shapes(name, k, n, split, tp):
    """W4A16 group 128 bf16 with zeros (and a bias on the column-parallel layers), M = 1, 64, 2048."""
    kk, nn = (k // tp, n) if split == "k" else (k, n // tp)
    p = make_problem(2048, nn, kk, 4, 128, torch.bfloat16, zero=True, bias=(split == "n"), seed=tp * 10 + len(name))
    _check_m_values(p, (1, 64, 2048), seed=tp)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("fmt,bits,group", FORMATS)
@pytest.mark.parametrize("k,n", LLAMA8B)
def test_llama8b_shapes_every_format(k, n, fmt, bits, group, dtype):
    """M = 1, 8, 16, 32, 128, 512 on each shape: both sides of the regime switch."""
    if group == 0:
        p = make_problem(512, n, k, bits, 0, dtype, seed=k // 1024 + n // 1024, scale_lo=0.0005, scale_hi=0.002)
    else:
        p = make_problem(512, n, k, bits, group, dtype, zero=True, bias=True, prequant=True, seed=k // 512 + bits)
    _check_m_values(p, (1, 8, 16, 32, 128, 512), seed=bits + group)


@pytest.mark.parametrize("m", [7, 8, 9, 15, 16, 17, 24, 33])
def test_agreement_across_the_regime_switch(m):
    """The decode kernel folds scale and zero into the group sums, the tensor-core kernel rounds
    every dequantised weight first: their results for the same rows must stay within twice the
    bound either is held to."""
    p = make_problem(m, 4096, 4096, 4, 128, torch.bfloat16, zero=True, prequant=True, seed=m)
    d = lambda t: None if t is None else t.to("cuda")
    dev = (d(p["processed"]), d(p["scales"]), d(p["zeros"]), d(p["bias"]), d(p["ps"]))
    a = _run_rows(p, dev, m, regime=pkg.W4_REGIME_GEMV).cpu()
    b = _run_rows(p, dev, m, regime=pkg.W4_REGIME_GEMM).cpu()
    assert max_err(a, b) <= 2 * oracle.tolerance(b)
