"""CPU: the oracle against the committed golden vectors (made from the reference's own compiled
code by tests/golden/make_golden.py) and, where oracle/_ref is present, against that code live."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import woq_oracle as o

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "quant_*.npz")))
_DT = {"torch.float32": torch.float32, "torch.float16": torch.float16, "torch.bfloat16": torch.bfloat16}


def test_golden_files_present():
    assert len(GOLDEN) >= 4


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_oracle_matches_golden(path):
    g = np.load(path)
    dt = _DT[str(g["dtype"])]
    w = torch.from_numpy(g["weight_f32"]).to(dt)
    for bits in (8, 4):
        u, p, s = o.symmetric_quantize(w, bits)
        assert np.array_equal(u.numpy(), g[f"unprocessed_int{bits}"])
        assert np.array_equal(p.numpy(), g[f"processed_int{bits}"])
        assert np.array_equal(s.to(torch.float32).numpy(), g[f"scales_int{bits}_f32"])
        assert np.array_equal(o.preprocess_weights(g[f"raw_int{bits}"], bits), g[f"raw_processed_int{bits}"])


def test_w4a8_layout_matches_golden_and_reference():
    """int4 weights laid out for fp8 activations: the oracle against vectors made by the reference's
    own code, and against that code live when it is built."""
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "layout_w4a8.npz"))
    for key in g.files:
        if key.startswith("raw_"):
            shape = key[4:]
            assert np.array_equal(o.preprocess_weights_w4a8(g[key]), g[f"w4a8_{shape}"])
            assert not np.array_equal(o.preprocess_weights(g[key], 4), g[f"w4a8_{shape}"])  # a different layout
    if o.ref_lib() is not None:
        q = np.random.default_rng(3).integers(-128, 128, size=(384, 64), dtype=np.int8)
        assert np.array_equal(o.preprocess_weights_w4a8(q), o.ref_preprocess_weights_w4a8(q))
    with pytest.raises(ValueError):
        o.preprocess_weights_w4a8(np.zeros((64, 32), dtype=np.int8))  # K must be a multiple of 128


@pytest.mark.parametrize("bits", [4, 8])
def test_layout_round_trip(bits):
    rng = np.random.default_rng(5)
    K, N = 192, 128
    q = rng.integers(-128, 128, size=(K, N * bits // 8), dtype=np.int8)
    back = o.unpreprocess_to_int8(o.preprocess_weights(q, bits), K, N, bits)
    assert np.array_equal(back, o.unpack_int4(q) if bits == 4 else q)


def test_quantize_properties():
    """Known answers that follow from the algorithm: scale = amax / 2^(bits-1); the column maximum
    maps to the positive clamp; zero columns give q = 0 and scale 0; rounding is half away from zero."""
    w = torch.zeros(64, 64)
    w[:, 0] = torch.linspace(-1, 1, 64)
    w[0, 1], w[1, 1] = 0.5, -0.25
    u, _, s = o.symmetric_quantize(w, 8)
    assert float(s[0]) == 1.0 / 128 and float(s[2]) == 0.0
    assert int(u[-1, 0]) == 127 and int(u[0, 0]) == -128 and int(u[:, 2].abs().max()) == 0
    assert int(u[0, 1]) == 127 and int(u[1, 1]) == -64
    w2 = torch.zeros(64, 64)
    w2[0, 0], w2[1, 0], w2[2, 0] = 8.0, 2.5, -2.5  # scale 1 -> 2.5 rounds to 3, -2.5 to -3
    u4, _, s4 = o.symmetric_quantize(w2, 4)
    q = o.unpack_int4(u4.numpy())
    assert float(s4[0]) == 1.0 and q[0, 0] == 7 and q[1, 0] == 3 and q[2, 0] == -3


def test_pack_unpack():
    x = np.arange(-8, 8, dtype=np.int8).reshape(2, 8)
    assert np.array_equal(o.unpack_int4(o.pack_int4(x)), x)
    with pytest.raises(ValueError):
        o.pack_int4(np.array([[9, 0]], dtype=np.int8))


def test_bad_shapes_rejected():
    q = np.zeros((48, 64), dtype=np.int8)  # K not a multiple of 64
    with pytest.raises(ValueError):
        o.preprocess_weights(q, 8)


@pytest.mark.skipif(o.ref_lib() is None, reason="oracle/_ref not built (reference tree absent)")
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("K,N", [(64, 64), (128, 192), (320, 256), (64, 1024)])
def test_oracle_matches_reference_live(bits, K, N):
    rng = np.random.default_rng(K + N + bits)
    q = rng.integers(-128, 128, size=(K, N * bits // 8), dtype=np.int8)
    assert np.array_equal(o.preprocess_weights(q, bits), o.ref_preprocess_weights(q, bits))
    assert np.array_equal(o.permute_rows(q, K, N, bits), o.ref_step("ref_permute_B_rows", q, K, N, bits))
    assert np.array_equal(o.subbyte_transpose(q, K, N, bits), o.ref_step("ref_subbyte_transpose", q, K, N, bits))
    assert np.array_equal(o.add_bias_and_interleave(q, bits), o.ref_add_bias_and_interleave(q, bits))
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        w = (torch.randn(K, N, generator=torch.Generator().manual_seed(K)) * 0.02).to(dt)
        a, b = o.symmetric_quantize(w, bits), o.ref_symmetric_quantize(w, bits)
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
        assert torch.equal(a[2].to(torch.float32), b[2].to(torch.float32))


def test_floating_point_oracles_agree():
    """The reference test's ground truth and the kernel-rounding oracle differ only by rounding."""
    from _cases import make_problem, oracle_out
    p = make_problem(4, 128, 256, 4, 128, torch.bfloat16, zero=True, bias=True, prequant=True, seed=1)
    tight = oracle_out(p)
    loose = o.groupwise_matmul_test_ref(p["act"], p["q"], p["scales"], p["zeros"], p["bias"], p["ps"], 128)
    assert float((tight.float() - loose.float()).abs().max()) <= o.tolerance(tight)


@pytest.mark.skipif(o.ref_lib() is None, reason="oracle/_ref not built (reference tree absent)")
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_oracle_matches_reference_live_at_rounding_boundaries(bits, dtype):
    """The quantiser's rounding (division, round half away from zero) on weights that sit on and next
    to the boundaries m + 0.5: the oracle against the reference's own compiled code."""
    from _cases import boundary_weights
    for amax in (1.0, 1.3, 0.0371):
        w = boundary_weights(bits, dtype, amax)
        a, b = o.symmetric_quantize(w, bits), o.ref_symmetric_quantize(w, bits)
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
        assert torch.equal(a[2].to(torch.float32), b[2].to(torch.float32))
