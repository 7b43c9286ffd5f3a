"""GPU: bounds evidence for the kernels without a memory checker.

(1) Canary bands: the output and the workspace sit inside larger buffers whose margins hold a known
pattern; after a launch the margins must be untouched and the output must still match the oracle.
Covers the decode kernel (all row counts of a pass, ragged column ranges per CTA), the tensor-core
kernel (every row tile, ragged last tile), split-k (fp32 partial tiles in the workspace) and the
pre-quant-scale pre-pass (scaled activations in the workspace).
(2) Small-shape grid: every M from 1 to 17 on the smallest shapes the format rules allow, both
regimes, int4/int8, every group size that divides K - the shapes where an index that runs one tile
too far has nowhere to hide.
"""

import pytest
import torch

import tensorrt_llm_b200 as pkg
from tensorrt_llm_b200 import ops
from oracle import woq_oracle as oracle
from _cases import make_problem, max_err, oracle_out

pytestmark = pytest.mark.gpu

GUARD = 8192  # bytes on either side
PATTERN = 0xA5


def _guarded(nbytes, device):
    """(whole buffer, view of the payload) with GUARD bytes of PATTERN before and after; the payload
    starts on a 256-byte boundary."""
    whole = torch.full((GUARD + nbytes + GUARD,), PATTERN, dtype=torch.uint8, device=device)
    return whole, whole[GUARD:GUARD + nbytes]


def _intact(whole, nbytes):
    return bool((whole[:GUARD] == PATTERN).all()) and bool((whole[GUARD + nbytes:] == PATTERN).all())


def _run_guarded(p, regime):
    dev = torch.device("cuda")
    m, n, k = p["m"], p["n"], p["k"]
    d = lambda t: None if t is None else t.to(dev)
    out_whole, out_bytes = _guarded(m * n * 2, dev)
    out = out_bytes.view(p["dtype"]).view(m, n)
    nws = ops.workspace_bytes(m, n, k, p["group"], p["bits"], p["dtype"], p["ps"] is not None, regime)
    ws_whole, ws = _guarded(max(nws, 256), dev)
    ops.gemm_raw(d(p["act"]), d(p["processed"]), d(p["scales"]), out, n=n, k=k, weight_bits=p["bits"],
                 group_size=p["group"], zeros=d(p["zeros"]), bias=d(p["bias"]), act_scale=d(p["ps"]), regime=regime,
                 workspace=ws if nws else None)
    torch.cuda.synchronize()
    assert pkg._lib.lib().w4_gemm_device_status() == 0
    assert _intact(out_whole, m * n * 2), "output margins were written"
    assert _intact(ws_whole, max(nws, 256)), "workspace margins were written"
    return out.cpu()


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("n,k,bits,group", [(2368, 512, 4, 128), (1216, 4224, 4, 64), (608, 576, 8, 64), (1504, 256, 8, 0)])
def test_canaries_decode(m, n, k, bits, group):
    # n chosen so that the 148 CTAs get ragged, unequal ranges of interleaved rows
    p = make_problem(m, n, k, bits, group, torch.bfloat16, zero=group != 0, bias=group != 0, prequant=group != 0,
                     seed=m + n)
    out = _run_guarded(p, pkg.W4_REGIME_GEMV)
    ref = oracle_out(p)
    assert max_err(out, ref) <= oracle.tolerance(ref)


@pytest.mark.parametrize("m", [17, 64, 129, 200, 257, 520])
@pytest.mark.parametrize("n,k,bits,group,prequant", [(384, 512, 4, 128, True), (1280, 8192, 4, 128, True),
                                                     (320, 1088, 8, 64, False), (256, 320, 8, 0, False)])
def test_canaries_tensor_core_and_split_k(m, n, k, bits, group, prequant):
    # (1280, 8192) at m <= 256 runs split-k: fp32 partial tiles fill the workspace behind the scaled activations
    p = make_problem(m, n, k, bits, group, torch.float16, zero=group != 0, bias=group != 0, prequant=prequant,
                     seed=m + k)
    out = _run_guarded(p, pkg.W4_REGIME_GEMM)
    ref = oracle_out(p)
    assert max_err(out, ref) <= oracle.tolerance(ref)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("bits", [4, 8])
def test_small_shape_grid(dtype, bits):
    dev = torch.device("cuda")
    d = lambda t: None if t is None else t.to(dev)
    n_min = 64 if bits == 4 else 32
    checked = 0
    for k in (64, 128, 256, 320):
        for n in (n_min, 3 * n_min, 5 * n_min):
            for group in (0, 64, 128):
                if group and k % group:
                    continue
                base = make_problem(17, n, k, bits, group, dtype, zero=group != 0, bias=group != 0,
                                    prequant=group != 0, seed=k + n + group)
                ref_all = oracle_out(base)
                w, s, z, b, ps = (d(base[x]) for x in ("processed", "scales", "zeros", "bias", "ps"))
                for m in range(1, 18):
                    act = d(base["act"][:m].contiguous())
                    for regime in (pkg.W4_REGIME_GEMV, pkg.W4_REGIME_GEMM):
                        out = torch.zeros((m, n), dtype=dtype, device=dev)
                        nws = ops.workspace_bytes(m, n, k, group, bits, dtype, ps is not None, regime)
                        ws = torch.empty(nws, dtype=torch.uint8, device=dev) if nws else None
                        ops.gemm_raw(act, w, s, out, n=n, k=k, weight_bits=bits, group_size=group, zeros=z, bias=b,
                                     act_scale=ps, regime=regime, workspace=ws)
                        ref = ref_all[:m]
                        err = max_err(out.cpu(), ref)
                        assert err <= oracle.tolerance(ref), (m, n, k, group, regime, err)
                        checked += 1
    assert checked >= 17 * 2 * 4 * 3 * 2
    assert pkg._lib.lib().w4_gemm_device_status() == 0
