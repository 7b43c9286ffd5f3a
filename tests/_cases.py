"""Seeded synthetic problems shared by the CPU and GPU tests (test infrastructure)."""
from __future__ import annotations

import torch

import tensorrt_llm_b200 as pkg
from tensorrt_llm_b200 import quantize
from oracle import woq_oracle as oracle


def make_problem(m, n, k, bits, group, dtype, zero=False, bias=False, prequant=False, seed=0,
                 act_scale=1.0, scale_lo=0.001, scale_hi=0.02):
    """Random integer weights in the full int range, scales ~U(scale_lo, scale_hi), zeros
    ~U(-0.1, 0.1), activations ~N(0, 1)*act_scale. group 0 = one scale per column."""
    g = torch.Generator().manual_seed(seed)
    lo, hi = (-8, 8) if bits == 4 else (-128, 128)
    q = torch.randint(lo, hi, (k, n), dtype=torch.int8, generator=g)
    packed = quantize.pack_int8_tensor_to_packed_int4(q) if bits == 4 else q
    qt = torch.quint4x2 if bits == 4 else torch.int8
    processed = quantize.preprocess_weights_for_mixed_gemm(packed.contiguous(), qt, torch.float16)
    rows = 1 if group == 0 else k // group
    shape = (n,) if group == 0 else (rows, n)
    scales = (torch.rand(shape, generator=g) * (scale_hi - scale_lo) + scale_lo).to(dtype)
    zeros = ((torch.rand(shape, generator=g) * 0.2 - 0.1).to(dtype)) if zero else None
    b = torch.randn((n,), generator=g).to(dtype) if bias else None
    ps = (torch.rand((k,), generator=g) + 0.5).to(dtype) if prequant else None
    act = (torch.randn((m, k), generator=g) * act_scale).to(dtype)
    return dict(m=m, n=n, k=k, bits=bits, group=group, dtype=dtype, q=q, packed=packed, processed=processed,
                scales=scales, zeros=zeros, bias=b, ps=ps, act=act)


def oracle_out(p, alpha=1.0):
    return oracle.kernel_rounding_ref(p["act"], p["q"], p["scales"], zeros=p["zeros"], bias=p["bias"],
                                      pre_quant_scale=p["ps"], group_size=p["group"], alpha=alpha)


def run_gpu(p, regime=0, alpha=1.0, device="cuda"):
    """Through the public op (and so through the C ABI)."""
    d = lambda t: None if t is None else t.to(device)
    if p["group"] == 0:
        assert p["zeros"] is None and p["bias"] is None and p["ps"] is None and alpha == 1.0
        return pkg.ops.weight_only_quant_matmul(d(p["act"]), d(p["processed"]), d(p["scales"]),
                                                1 if p["bits"] == 8 else 2, regime=regime).cpu()
    algo = (pkg.INT8_WEIGHT if p["bits"] == 8 else 0) | (pkg.ZERO if p["zeros"] is not None else 0) \
        | (pkg.BIAS if p["bias"] is not None else 0) | (pkg.PRE_QUANT_SCALE if p["ps"] is not None else 0)
    return pkg.ops.weight_only_groupwise_quant_matmul(
        d(p["act"]), d(p["ps"]), d(p["processed"]), d(p["scales"]), d(p["zeros"]), d(p["bias"]), alpha, algo,
        p["group"], regime=regime).cpu()


def max_err(out, ref):
    return float((out.to(torch.float64) - ref.to(torch.float64)).abs().max())


def oracle_subset(p, rows, cols, alpha=1.0):
    """The tight oracle on a sample of activation rows and output columns (large shapes: the
    float64 reference of the whole problem would take minutes on the host)."""
    rows = torch.as_tensor(rows, dtype=torch.long)
    cols = torch.as_tensor(cols, dtype=torch.long)
    pick = (lambda t: None if t is None else t[..., cols])
    return oracle.kernel_rounding_ref(p["act"][rows], p["q"][:, cols], pick(p["scales"]), zeros=pick(p["zeros"]),
                                      bias=pick(p["bias"]), pre_quant_scale=p["ps"], group_size=p["group"], alpha=alpha)


def sample_rows(m, tile=192, extra=8, seed=0):
    """Row sample that hits the first and last row of every `tile`-row block (the prefill kernel's
    largest row tile is 256, its usual one 192; both boundaries are included), the ragged last block
    and a few random rows."""
    if m <= 64:
        return list(range(m))
    rows = {0, m - 1}
    for t in (128, 192, 256):
        for b in range(0, m, t):
            rows.update((b, min(m - 1, b + t - 1)))
    g = torch.Generator().manual_seed(seed)
    rows.update(int(x) for x in torch.randint(0, m, (extra,), generator=g))
    rows = sorted(rows)
    if len(rows) > 96:  # keep the oracle cheap: boundaries of a spread of blocks
        step = len(rows) / 96.0
        rows = sorted({rows[int(i * step)] for i in range(96)} | {0, m - 1})
    return rows


def sample_cols(n, count=384, seed=0):
    """First and last 128-column tile plus random columns."""
    cols = set(range(min(n, 128))) | set(range(max(0, n - 128), n))
    g = torch.Generator().manual_seed(seed + 1)
    cols.update(int(x) for x in torch.randint(0, n, (count,), generator=g))
    return sorted(cols)


def boundary_weights(bits, dtype, amax, k=128, n=64):
    """[k, n] weights whose quotient w / scale sits on or next to a rounding boundary (m + 0.5): exact
    ties where the scale is a power of two, values one unit in the last place either side, and the
    same for scales that are not powers of two. Row 0 pins every column's maximum, hence the scale."""
    half_range = 1 << (bits - 1)
    scale = amax / half_range
    g = torch.Generator().manual_seed(bits + int(amax * 1000))
    m = torch.randint(-half_range, half_range, (k, n), generator=g).double()
    sign = torch.where(m < 0, -1.0, 1.0)
    w = ((m + 0.5 * sign) * scale).to(dtype)                      # quotient ~ m +- 0.5
    nudge = torch.randint(-1, 2, (k, n), generator=g)             # -1, 0, +1 units in the last place
    if dtype == torch.float32:
        w = torch.where(nudge > 0, torch.nextafter(w, torch.full_like(w, 1e9)),
                        torch.where(nudge < 0, torch.nextafter(w, torch.full_like(w, -1e9)), w))
    else:
        w = (w.view(torch.int16) + nudge.to(torch.int16)).view(dtype)
    w = torch.where(torch.isfinite(w.float()), w.float(), torch.zeros(())).to(dtype)
    w[0, :] = amax
    w.clamp_(-amax, amax)
    return w
