"""GPU: device-side quantise / layout kernels (w4_preprocess_weights_device,
w4_symmetric_quantize_device, w4_relayout_w4a8_to_w4a16_device) through the C ABI, byte for byte against the oracle, the committed
golden vectors made from the reference's own code, and the host functions of the library."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import woq_oracle as o
import tensorrt_llm_b200 as pkg
from tensorrt_llm_b200 import quantize as Q

pytestmark = pytest.mark.gpu

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "quant_*.npz")))
_DT = {"torch.float32": torch.float32, "torch.float16": torch.float16, "torch.bfloat16": torch.bfloat16}
_QT = {8: torch.int8, 4: torch.quint4x2}


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_golden_vectors(path):
    g = np.load(path)
    dt = _DT[str(g["dtype"])]
    w = torch.from_numpy(g["weight_f32"]).to(dt).cuda()
    for bits in (8, 4):
        u, p, s = Q.symmetric_quantize_last_axis_of_batched_matrix_cuda(w, _QT[bits], return_unprocessed=True)
        assert np.array_equal(u.cpu().numpy(), g[f"unprocessed_int{bits}"])
        assert np.array_equal(p.cpu().numpy(), g[f"processed_int{bits}"])
        assert s.dtype == dt
        assert np.array_equal(s.float().cpu().numpy(), g[f"scales_int{bits}_f32"])
        raw = torch.from_numpy(g[f"raw_int{bits}"]).cuda()
        out = Q.preprocess_weights_for_mixed_gemm_cuda(raw, _QT[bits])
        assert np.array_equal(out.cpu().numpy(), g[f"raw_processed_int{bits}"])


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("k,n", [(64, 64), (64, 576), (192, 1088), (4096, 14336), (8192, 4096)])
def test_preprocess_matches_oracle(bits, k, n):
    rng = np.random.default_rng(k + n + bits)
    q = rng.integers(-128, 128, size=(k, n * bits // 8), dtype=np.int8)
    out = Q.preprocess_weights_for_mixed_gemm_cuda(torch.from_numpy(q).cuda(), _QT[bits])
    assert np.array_equal(out.cpu().numpy(), o.preprocess_weights(q, bits))


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("k,n", [(64, 64), (320, 704), (4096, 4096)])
def test_quantize_matches_oracle(bits, dtype, k, n):
    torch.manual_seed(k * 7 + n + bits)
    w = (torch.randn(k, n) * 0.02).to(dtype)
    w[:, 3] = 0  # a zero column: scale 0, q = 0
    w[5, 7] = w[:, 7].abs().max() * 2  # a clear column maximum
    u_ref, p_ref, s_ref = o.symmetric_quantize(w, bits)
    u, p, s = Q.symmetric_quantize_last_axis_of_batched_matrix_cuda(w.cuda(), _QT[bits], return_unprocessed=True)
    assert torch.equal(u.cpu(), u_ref)
    assert torch.equal(p.cpu(), p_ref)
    assert torch.equal(s.cpu().float(), s_ref.float())
    # and the library's own host path (what a CPU caller gets)
    p_host, s_host = Q.symmetric_quantize_last_axis_of_batched_matrix(w, _QT[bits])
    assert torch.equal(p.cpu(), p_host) and torch.equal(s.cpu(), s_host)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("amax", [1.0, 1.3, 0.0371])
def test_quantize_at_rounding_boundaries(bits, dtype, amax):
    """Weights whose quotient w / scale sits on or next to a rounding boundary (m + 0.5): exact ties
    (power-of-two scale), values one unit in the last place either side, and the same for scales that
    are not powers of two. The kernel multiplies with the reciprocal and falls back to the division
    near a boundary; the result must still be the reference's division, bit for bit."""
    from _cases import boundary_weights
    w = boundary_weights(bits, dtype, amax)
    u_ref, p_ref, s_ref = o.symmetric_quantize(w, bits)
    u, p, s = Q.symmetric_quantize_last_axis_of_batched_matrix_cuda(w.cuda(), _QT[bits], return_unprocessed=True)
    assert torch.equal(s.cpu().float(), s_ref.float())
    assert torch.equal(u.cpu(), u_ref)
    assert torch.equal(p.cpu(), p_ref)


@pytest.mark.parametrize("k,n", [(128, 64), (256, 192), (4096, 14336), (8192, 1024)])
def test_w4a8_relayout_matches_host_and_oracle(k, n):
    """W4A8-layout bytes -> the kernels' layout on the device: the bytes the host function gives,
    which are the oracle's plain int4 layout of the same weights."""
    rng = np.random.default_rng(k + n)
    q = rng.integers(-128, 128, size=(k, n // 2), dtype=np.int8)
    w4a8 = Q.preprocess_weights_for_mixed_gemm(torch.from_numpy(q), torch.quint4x2, torch.float8_e4m3fn)
    out = Q.relayout_w4a8_weights_cuda(w4a8.cuda())
    assert np.array_equal(out.cpu().numpy(), o.preprocess_weights(q, 4))
    assert torch.equal(out.cpu(), Q.relayout_w4a8_weights(w4a8))


def test_w4a8_relayout_experts_and_error_codes():
    rng = np.random.default_rng(5)
    q = rng.integers(-128, 128, size=(3, 256, 64), dtype=np.int8)
    w4a8 = Q.preprocess_weights_for_mixed_gemm(torch.from_numpy(q), torch.quint4x2, torch.float8_e4m3fn)
    out = Q.relayout_w4a8_weights_cuda(w4a8.cuda())
    for e in range(3):
        assert np.array_equal(out[e].cpu().numpy(), o.preprocess_weights(q[e], 4))
    lib = pkg._lib.lib()
    a = torch.zeros(128, 32, dtype=torch.int8, device="cuda")
    b = torch.zeros_like(a)
    assert lib.w4_relayout_w4a8_to_w4a16_device(None, a.data_ptr(), 128, 64, None) == pkg._lib.W4_ERR_NULL_POINTER
    assert lib.w4_relayout_w4a8_to_w4a16_device(b.data_ptr(), a.data_ptr(), 64, 64, None) == pkg._lib.W4_ERR_BAD_SHAPE
    assert lib.w4_relayout_w4a8_to_w4a16_device(b.data_ptr(), a.data_ptr(), 128, 32, None) == pkg._lib.W4_ERR_BAD_SHAPE
    assert lib.w4_relayout_w4a8_to_w4a16_device(a.data_ptr(), a.data_ptr(), 128, 64, None) == pkg._lib.W4_ERR_UNSUPPORTED
    assert lib.w4_relayout_w4a8_to_w4a16_device(b.data_ptr() + 4, a.data_ptr(), 128, 64, None) \
        == pkg._lib.W4_ERR_MISALIGNED


def test_round_trip_through_gemm():
    """Weights prepared on the GPU feed the GEMM and give the oracle's result."""
    from _cases import max_err
    torch.manual_seed(11)
    k, n, m = 4096, 4096, 4
    w = (torch.randn(k, n) * 0.02).to(torch.float16)
    p, s = Q.symmetric_quantize_last_axis_of_batched_matrix_cuda(w.cuda(), torch.int8)
    act = torch.randn(m, k, dtype=torch.float16, device="cuda")
    out = pkg.ops.weight_only_quant_matmul(act, p, s, 1)
    u_ref, _, s_ref = o.symmetric_quantize(w, 8)
    ref = act.float().cpu() @ (u_ref.float() * s_ref.float()[None, :])
    assert max_err(out.float().cpu(), ref) <= 1e-2 * ref.abs().max()


def test_error_codes():
    lib = pkg._lib.lib()
    a = torch.zeros(64, 32, dtype=torch.int8, device="cuda")
    b = torch.zeros_like(a)
    assert lib.w4_preprocess_weights_device(None, a.data_ptr(), 64, 64, 4, None) == pkg._lib.W4_ERR_NULL_POINTER
    assert lib.w4_preprocess_weights_device(b.data_ptr(), a.data_ptr(), 64, 64, 5, None) == pkg._lib.W4_ERR_BAD_DTYPE
    assert lib.w4_preprocess_weights_device(b.data_ptr(), a.data_ptr(), 48, 64, 4, None) == pkg._lib.W4_ERR_BAD_SHAPE
    assert lib.w4_preprocess_weights_device(a.data_ptr(), a.data_ptr(), 64, 64, 4, None) == pkg._lib.W4_ERR_UNSUPPORTED


@pytest.mark.parametrize("bits,m", [(4, 1), (8, 4)])
def test_gemm_right_behind_weight_preparation_on_one_stream(bits, m):
    """The decode kernel is a programmatic dependent launch that may fetch weights before the
    kernel in front of it has finished - but only when the caller declares them static. Here the
    kernel in front WRITES the weights: quantise (fresh values each round, same buffers) -> GEMM,
    200 times back to back on one stream without the static flag. Every output must equal the one
    the same weights give when the GEMM runs alone."""
    lib = pkg._lib.lib()
    import ctypes
    torch.manual_seed(5)
    k, n = 2048, 2048
    dev = "cuda"
    variants = [(torch.randn(k, n, device=dev) * (0.01 * (i + 1))).to(torch.bfloat16) for i in range(4)]
    act = torch.randn(m, k, device=dev).to(torch.bfloat16)
    processed = torch.empty((k, n * bits // 8), dtype=torch.int8, device=dev)
    s32 = torch.empty((n,), dtype=torch.float32, device=dev)
    scales = torch.empty((n,), dtype=torch.bfloat16, device=dev)
    stream = torch.cuda.current_stream()
    sp = ctypes.c_void_p(stream.cuda_stream)

    def quantise(w):
        rc = lib.w4_symmetric_quantize_device(processed.data_ptr(), None, s32.data_ptr(), scales.data_ptr(), 1,
                                              w.data_ptr(), 1, k, n, bits, sp)
        assert rc == 0

    def gemm(out):
        pkg.ops.gemm_raw(act, processed, scales, out, n=n, k=k, weight_bits=bits, group_size=0,
                         regime=pkg.W4_REGIME_GEMV, weights_static=False)

    alone = []
    for w in variants:
        quantise(w)
        torch.cuda.synchronize()
        out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
        gemm(out)
        torch.cuda.synchronize()
        alone.append(out)
    assert not torch.equal(alone[0], alone[1])
    rounds = 200
    outs = torch.empty((rounds, m, n), dtype=torch.bfloat16, device=dev)
    for i in range(rounds):
        quantise(variants[i % 4])
        gemm(outs[i])
    torch.cuda.synchronize()
    for i in range(rounds):
        assert torch.equal(outs[i], alone[i % 4]), f"round {i}: the GEMM saw weights of another round"
    assert lib.w4_gemm_device_status() == 0
