"""CPU: the product's host-side code (C ABI of libw4gemm.so + the Python mirror of the reference's
ops) against the oracle and the golden vectors; no kernel is launched here."""
import ctypes
import glob
import os

import numpy as np
import pytest
import torch

import tensorrt_llm_b200 as pkg
from oracle import woq_oracle as o
from tensorrt_llm_b200 import quantize
from tensorrt_llm_b200._lib import W4GemmParams

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "quant_*.npz")))
_DT = {"torch.float32": torch.float32, "torch.float16": torch.float16, "torch.bfloat16": torch.bfloat16}
_QT = {8: torch.int8, 4: torch.quint4x2}


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(os.path.dirname(__file__), "..", "include", "w4_gemm.h")).read()
    import re
    declared = set(re.findall(r"\b(w4_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/w4_gemm.h but not exported"
    assert set(pkg._lib.EXPORTS) <= declared
    assert lib.w4_gemm_version() >= 112
    assert pkg._lib.status_string(0) == "ok" and "null" in pkg._lib.status_string(-1)


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_host_ops_match_golden(path):
    g = np.load(path)
    w = torch.from_numpy(g["weight_f32"]).to(_DT[str(g["dtype"])])
    for bits in (8, 4):
        u, p, s = quantize._symmetric_quantize_last_axis_of_batched_matrix(w, _QT[bits])
        assert np.array_equal(u.numpy(), g[f"unprocessed_int{bits}"])
        assert np.array_equal(p.numpy(), g[f"processed_int{bits}"])
        assert s.dtype == w.dtype and np.array_equal(s.to(torch.float32).numpy(), g[f"scales_int{bits}_f32"])
        raw = torch.from_numpy(g[f"raw_int{bits}"])
        got = quantize.preprocess_weights_for_mixed_gemm(raw, _QT[bits], torch.float16)
        assert np.array_equal(got.numpy(), g[f"raw_processed_int{bits}"])


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("K,N", [(64, 64), (128, 448), (1024, 1024)])
def test_host_ops_match_oracle(bits, K, N):
    w = torch.randn(K, N, generator=torch.Generator().manual_seed(K + N)) * 0.02
    got = quantize._symmetric_quantize_last_axis_of_batched_matrix(w, _QT[bits])
    exp = o.symmetric_quantize(w, bits)
    for a, b in zip(got, exp):
        assert torch.equal(a, b)
    p2, s2 = quantize.symmetric_quantize_last_axis_of_batched_matrix(w, _QT[bits])
    assert torch.equal(p2, exp[1]) and torch.equal(s2, exp[2])


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("amax", [1.0, 1.3, 0.0371])
def test_host_quantize_at_rounding_boundaries(bits, dtype, amax):
    """The host quantiser multiplies with the reciprocal of the scale and lets the division decide
    near a rounding boundary: on weights that sit on and next to the boundaries the result is still
    the reference's round(w / scale), bit for bit (oracle: division and C round())."""
    from _cases import boundary_weights
    w = boundary_weights(bits, dtype, amax)
    got = quantize._symmetric_quantize_last_axis_of_batched_matrix(w, _QT[bits])
    exp = o.symmetric_quantize(w, bits)
    for a, b in zip(got, exp):
        assert torch.equal(a, b)


def test_w4a8_layout_and_relayout():
    """preprocess_weights_for_mixed_gemm with an fp8 activation type gives the reference's W4A8 bytes
    (golden vectors made by the reference's code); relayout_w4a8_weights turns them into the layout
    the kernels consume, i.e. what the same integers give through the W4A16 transform."""
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "layout_w4a8.npz"))
    for key in g.files:
        if not key.startswith("raw_"):
            continue
        raw = torch.from_numpy(g[key])
        a8 = quantize.preprocess_weights_for_mixed_gemm(raw, torch.quint4x2, torch.float8_e4m3fn)
        assert np.array_equal(a8.numpy(), g["w4a8_" + key[4:]])
        a16 = quantize.relayout_w4a8_weights(a8)
        assert torch.equal(a16, quantize.preprocess_weights_for_mixed_gemm(raw, torch.quint4x2, torch.float16))
    rng = np.random.default_rng(9)
    q = torch.from_numpy(rng.integers(-128, 128, size=(2, 256, 64), dtype=np.int8))  # 3-D: per expert
    a8 = quantize.preprocess_weights_for_mixed_gemm(q, torch.quint4x2, torch.float8_e4m3fn)
    for e in range(2):
        assert np.array_equal(a8[e].numpy(), o.preprocess_weights_w4a8(q[e].numpy()))
    assert torch.equal(quantize.relayout_w4a8_weights(a8),
                       quantize.preprocess_weights_for_mixed_gemm(q, torch.quint4x2, torch.float16))
    with pytest.raises(pkg.W4Error):
        quantize.preprocess_weights_for_mixed_gemm(torch.zeros(64, 32, dtype=torch.int8), torch.quint4x2,
                                                   torch.float8_e4m3fn)


def test_batched_weights():
    w = torch.randn(3, 64, 64, generator=torch.Generator().manual_seed(0))
    p, s = quantize.symmetric_quantize_last_axis_of_batched_matrix(w, torch.int8)
    assert p.shape == (3, 64, 64) and s.shape == (3, 64)
    for e in range(3):
        assert torch.equal(p[e], o.symmetric_quantize(w[e], 8)[1])


def test_torch_ops_registered():
    import tensorrt_llm_b200.torch_ops  # noqa: F401
    w = torch.randn(64, 64)
    a = torch.ops.trtllm.symmetric_quantize_last_axis_of_batched_matrix(w, torch.quint4x2)
    b = quantize.symmetric_quantize_last_axis_of_batched_matrix(w, torch.quint4x2)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    x = torch.randint(-8, 8, (4, 16), dtype=torch.int8)
    packed = torch.ops.trtllm.pack_int8_tensor_to_packed_int4(x)
    assert torch.equal(torch.ops.trtllm.unpack_int4_packed_tensor_to_int8(packed), x)
    assert hasattr(torch.ops.trtllm, "weight_only_groupwise_quant_gemm")


def test_error_behaviour_of_host_ops():
    with pytest.raises(RuntimeError):
        quantize.symmetric_quantize_last_axis_of_batched_matrix(torch.zeros(0, 64), torch.int8)
    with pytest.raises(RuntimeError):
        quantize.symmetric_quantize_last_axis_of_batched_matrix(torch.zeros(64, 64, dtype=torch.float64), torch.int8)
    with pytest.raises(RuntimeError):
        quantize.symmetric_quantize_last_axis_of_batched_matrix(torch.zeros(64, 64), torch.int32)
    with pytest.raises(RuntimeError):
        quantize.preprocess_weights_for_mixed_gemm(torch.zeros(64, 64), torch.int8)
    with pytest.raises(RuntimeError):
        quantize.pack_int8_tensor_to_packed_int4(torch.full((2, 2), 9, dtype=torch.int8))
    with pytest.raises(pkg.W4Error):
        quantize.preprocess_weights_for_mixed_gemm(torch.zeros(48, 64, dtype=torch.int8), torch.int8)


def _params(**kw):
    base = dict(act=16, weight=16, scales=16, out=16, alpha=1.0, m=1, n=128, k=128, group_size=128, weight_bits=4,
                act_dtype=1, regime=1)
    base.update(kw)
    return W4GemmParams(**base)


def test_launch_argument_validation(lib):
    """w4_gemm_validate runs the launcher's checks without touching a device."""
    v = lambda **kw: lib.w4_gemm_validate(ctypes.byref(_params(**kw)))
    assert v() == 0
    assert lib.w4_gemm_validate(None) == -1
    assert v(act=0) == -1 and v(out=0) == -1
    assert v(k=100) == -2 and v(n=100) == -2 and v(n=96, weight_bits=8) == 0 and v(n=96) == -2
    assert v(group_size=32) == -3 and v(k=192, group_size=128) == -3 and v(k=192, group_size=64) == 0
    assert v(act_dtype=5) == -4 and v(weight_bits=2) == -4
    assert v(act=8) == -5 and v(zeros=4) == -5
    assert v(regime=7) == -9
    assert v(m=0, act=0, out=0) == 0  # empty batch: nothing to do, as the plugins return early
    # tensor-core regime with a pre-quant scale needs the caller's workspace
    need = lib.w4_gemm_workspace_bytes(512, 128, 128, 128, 4, 1, 1, 2)
    assert need == 512 * 128 * 2
    assert v(m=512, regime=2, act_scale=16) == -7
    assert v(m=512, regime=2, act_scale=16, workspace=16, workspace_bytes=need) == 0
    assert lib.w4_gemm_workspace_bytes(8, 128, 128, 128, 4, 1, 1, 1) == 0


def test_regime_heuristic(lib):
    for m in (1, 2, 4, 8):
        assert lib.w4_gemm_select_regime(m, 14336, 4096, 128, 4) == pkg.W4_REGIME_GEMV
    # above 8 rows the cost model decides: decode passes (16 rows at a time, then up to 8) against the
    # (split-k) tensor-core kernel. One 16-row pass wins on this shape (17.2 vs 25.7 us); two passes lose.
    assert lib.w4_gemm_select_regime(16, 14336, 4096, 128, 4) == pkg.W4_REGIME_GEMV
    assert lib.w4_gemm_select_regime(24, 14336, 4096, 128, 4) == pkg.W4_REGIME_GEMM
    assert lib.w4_gemm_select_regime(32, 4096, 14336, 128, 4) == pkg.W4_REGIME_GEMM
    # a tiny weight: streaming it twice is cheaper than the tensor-core kernel's fixed cost
    assert lib.w4_gemm_select_regime(16, 256, 512, 128, 4) == pkg.W4_REGIME_GEMV
    # workspace: the split-k partial tiles are on top of the mandatory part
    assert lib.w4_gemm_workspace_bytes(64, 1280, 8192, 128, 4, 1, 0, pkg.W4_REGIME_GEMM) >= 2 * 64 * 1280 * 4
    assert lib.w4_gemm_workspace_bytes(4096, 4096, 14336, 128, 4, 1, 0, pkg.W4_REGIME_GEMM) == 0
    # a plugin sizes its workspace once, for every m up to the profile's maximum
    big = lib.w4_gemm_workspace_bytes_max(4096, 1280, 8192, 128, 4, 1, 0)
    assert big >= max(lib.w4_gemm_workspace_bytes(m, 1280, 8192, 128, 4, 1, 0, 0) for m in (1, 16, 64, 200, 256, 4096))
    assert lib.w4_gemm_workspace_bytes_max(4096, 1280, 8192, 128, 4, 1, 1) >= 4096 * 8192 * 2
    for m in (256, 4096, 8192):
        assert lib.w4_gemm_select_regime(m, 4096, 14336, 128, 4) == pkg.W4_REGIME_GEMM


def test_regime_heuristic_knows_the_activation_type(lib):
    """int8 weights with bf16 activations: a decode pass costs more (two nibble planes), so two
    16-row passes over a small matrix lose to the tensor-core kernel where float16 still takes them
    (measured 12.5 against 9.7 us); int4 does not depend on the type; the untyped function answers
    for float16; workspace sizes follow the typed answer."""
    FP16, BF16 = pkg._lib.W4_DTYPE_FP16, pkg._lib.W4_DTYPE_BF16
    typed = lib.w4_gemm_select_regime_typed
    assert typed(32, 1024, 4096, 0, 8, FP16) == pkg.W4_REGIME_GEMV
    assert typed(32, 1024, 4096, 0, 8, BF16) == pkg.W4_REGIME_GEMM
    assert pkg.ops.select_regime(32, 1024, 4096, 0, 8, torch.bfloat16) == pkg.W4_REGIME_GEMM
    for m in (1, 8, 16, 24, 32, 64, 300):
        for n, k in ((1024, 4096), (4096, 4096), (14336, 4096)):
            assert typed(m, n, k, 128, 4, FP16) == typed(m, n, k, 128, 4, BF16)
            assert typed(m, n, k, 0, 8, FP16) == lib.w4_gemm_select_regime(m, n, k, 0, 8)
            for dt in (FP16, BF16):
                auto = lib.w4_gemm_workspace_bytes(m, n, k, 0, 8, dt, 1, pkg.W4_REGIME_AUTO)
                assert auto == lib.w4_gemm_workspace_bytes(m, n, k, 0, 8, dt, 1, typed(m, n, k, 0, 8, dt))


def test_plugin_mirror_fields_and_serialisation():
    g = pkg.WeightOnlyGroupwiseQuantMatmulPlugin(pkg.ops.TRT_BF16, pkg.ZERO | pkg.PRE_QUANT_SCALE | pkg.BIAS, 128, 1.0)
    assert (g.pre_quant_scale_idx, g.weight_idx, g.scales_idx, g.zeros_idx, g.bias_idx, g.nb_inputs) == (1, 2, 3, 4, 5, 6)
    g2 = pkg.WeightOnlyGroupwiseQuantMatmulPlugin(pkg.ops.TRT_HALF, pkg.INT8_WEIGHT, 64)
    assert (g2.weight_idx, g2.scales_idx, g2.zeros_idx, g2.bias_idx, g2.bits) == (1, 2, 2, 2, 8)
    g.configure_plugin(1, 4096, 4096, 14336)
    r = pkg.WeightOnlyGroupwiseQuantMatmulPlugin.deserialize(g.serialize())
    assert (r.type_id, r.quant_algo, r.group_size, r.alpha, r.dims) == (g.type_id, g.quant_algo, 128, 1.0, g.dims)
    assert g.get_workspace_size() == 4096 * 14336 * 2  # smoothed activations, as the reference sizes it
    p = pkg.WeightOnlyQuantMatmulPlugin(pkg.ops.TRT_HALF, pkg.ops.WEIGHT_TYPE_INT4)
    assert p.get_output_dimensions((2, 3, 64), (64, 32)) == (2, 3, 64)
    assert p.supports_format_combination(1, [torch.float16, torch.int8, torch.float16, torch.float16])
    w4a8 = pkg.WeightOnlyGroupwiseQuantMatmulPlugin(pkg.ops.TRT_HALF, pkg.FP8_ALPHA | pkg.PRE_QUANT_SCALE, 128, 0.5)
    assert (w4a8.bits, w4a8.alpha, w4a8.weight_idx) == (4, 0.5, 2)
    with pytest.raises(RuntimeError):  # W4A8 exists for int4 weights only (the reference asserts the same)
        pkg.WeightOnlyGroupwiseQuantMatmulPlugin(pkg.ops.TRT_HALF, pkg.FP8_ALPHA | pkg.INT8_WEIGHT, 128)
    with pytest.raises(RuntimeError):
        pkg.WeightOnlyQuantMatmulPlugin(0, 1)


def test_logger_levels_and_refusal_line(lib, capfd):
    """The logger takes the reference logger's level numbers; a refused launch prints one WARNING line
    when the level allows it and nothing at the default level (no device is touched: validation fails
    first)."""
    p = W4GemmParams()
    p.m, p.n, p.k, p.weight_bits, p.group_size, p.act_dtype = 4, 64, 100, 4, 0, pkg._lib.W4_DTYPE_FP16
    try:
        lib.w4_set_log_level(pkg._lib.W4_LOG_ERROR)
        assert lib.w4_get_log_level() == 40
        assert lib.w4_gemm_launch(ctypes.byref(p), None) == pkg._lib.W4_ERR_BAD_SHAPE
        assert capfd.readouterr().err == ""
        lib.w4_set_log_level(pkg._lib.W4_LOG_WARNING)
        assert lib.w4_gemm_launch(ctypes.byref(p), None) == pkg._lib.W4_ERR_BAD_SHAPE
        err = capfd.readouterr().err
        assert err.startswith("[w4_gemm][WARNING] w4_gemm_launch refused:") and "k=100" in err
        assert err.count("\n") == 1
    finally:
        lib.w4_set_log_level(-1)  # back to the environment's setting


@pytest.mark.parametrize("env,expect", [({"W4_LOG_LEVEL": "DEBUG"}, 10), ({"TLLM_LOG_LEVEL": "VERBOSE"}, 10),
                                        ({"TLLM_LOG_LEVEL": "INFO", "W4_LOG_LEVEL": "TRACE"}, 0),
                                        ({"W4_LOG_LEVEL": "nonsense"}, 40), ({}, 40)])
def test_log_level_from_environment(env, expect):
    import subprocess
    import sys
    root = os.path.join(os.path.dirname(__file__), "..")
    child_env = {k: v for k, v in os.environ.items() if k not in ("W4_LOG_LEVEL", "TLLM_LOG_LEVEL")}
    child_env.update(env)
    out = subprocess.check_output([sys.executable, "-c",
                                   "import tensorrt_llm_b200 as p; print(p._lib.lib().w4_get_log_level())"],
                                  cwd=root, env=child_env, text=True)
    assert int(out.strip().splitlines()[-1]) == expect


@pytest.mark.parametrize("force", ["gemv", "gemm", "other", None])
def test_forced_regime_governs_workspace_sizes(lib, force):
    """W4_FORCE_REGIME overrides the cost model wherever the library resolves the regime itself: seen
    here through the workspace size of an automatic launch (0 for the decode kernel); the cost model's
    own answer (w4_gemm_select_regime) is unchanged."""
    import subprocess
    import sys
    root = os.path.join(os.path.dirname(__file__), "..")
    child_env = {k: v for k, v in os.environ.items() if k != "W4_FORCE_REGIME"}
    if force is not None:
        child_env["W4_FORCE_REGIME"] = force
    code = ("import tensorrt_llm_b200 as p; l = p._lib.lib(); "
            "print(l.w4_gemm_workspace_bytes(1, 1280, 8192, 128, 4, 1, 1, 0), "
            "l.w4_gemm_workspace_bytes(4096, 4096, 4096, 128, 4, 1, 1, 0), "
            "l.w4_gemm_select_regime(1, 1280, 8192, 128, 4), l.w4_gemm_select_regime(4096, 4096, 4096, 128, 4))")
    out = subprocess.check_output([sys.executable, "-c", code], cwd=root, env=child_env, text=True)
    small, large, r_small, r_large = (int(x) for x in out.strip().splitlines()[-1].split())
    assert (r_small, r_large) == (pkg.W4_REGIME_GEMV, pkg.W4_REGIME_GEMM)
    gemm_small = lib.w4_gemm_workspace_bytes(1, 1280, 8192, 128, 4, 1, 1, pkg.W4_REGIME_GEMM)
    gemm_large = lib.w4_gemm_workspace_bytes(4096, 4096, 4096, 128, 4, 1, 1, pkg.W4_REGIME_GEMM)
    assert gemm_small > 0 and gemm_large > 0
    if force == "gemv":
        assert (small, large) == (0, 0)
    elif force == "gemm":
        assert (small, large) == (gemm_small, gemm_large)
    else:
        assert (small, large) == (0, gemm_large)
