"""Checkpoint conversion (GPTQ / AutoAWQ -> the library's tensors): CPU checks of the unpacking and
of the zero-point folding against the formats' own dequantisation formulas, the TensorRT-LLM
parameter names, and (GPU) a forward pass through the kernels against the float reference."""
import numpy as np
import pytest
import torch

import tensorrt_llm_b200 as pkg
from tensorrt_llm_b200 import checkpoint as ck
from tensorrt_llm_b200 import quantize
from tensorrt_llm_b200.mapping import Mapping

AWQ_ORDER = [0, 4, 1, 5, 2, 6, 3, 7]  # position in the word of logical nibble i (AutoAWQ's packing order)


def _pack_words(u, order=None):
    """uint nibbles [R, 8C] -> int32 [R, C], nibble i of every group of eight at 4 * pos(i)."""
    r, c8 = u.shape
    g = u.reshape(r, c8 // 8, 8).astype(np.uint32)
    w = np.zeros((r, c8 // 8), dtype=np.uint32)
    for i in range(8):
        pos = i if order is None else order[i]
        w |= g[:, :, i] << np.uint32(4 * pos)
    return torch.from_numpy(w.view(np.int32))


def _make(k=256, n=128, group=128, seed=0):
    rng = np.random.default_rng(seed)
    u = rng.integers(0, 16, size=(k, n))
    uz = rng.integers(0, 16, size=(k // group, n))
    s = torch.from_numpy(rng.uniform(0.001, 0.02, size=(k // group, n)).astype(np.float32)).half()
    return u, uz, s


def test_unpack_orders():
    u = np.arange(16).reshape(1, 16) % 16
    assert ck.unpack_int32_into_int8(_pack_words(u)).tolist() == u.tolist()
    assert ck.unpack_int32_into_int8(_pack_words(u, AWQ_ORDER), True).tolist() == u.tolist()


@pytest.mark.parametrize("fmt", ["gptq", "awq"])
def test_conversion_matches_format_formula(fmt):
    k, n, group = 256, 128, 128
    u, uz, s = _make(k, n, group)
    if fmt == "gptq":  # packed along K; stored zero is z - 1; w = (u - (stored + 1)) * s
        qweight = _pack_words(u.T.copy()).T.contiguous()
        qzeros = _pack_words(uz)
        q, sc, zero = ck.gptq_to_signed(qweight, qzeros, s)
        w_ref = (torch.from_numpy(u - (np.repeat(uz, group, 0) + 1)).float() * s.float().repeat_interleave(group, 0))
    else:  # packed along N in AutoAWQ order; w = (u - z) * s
        qweight = _pack_words(u, AWQ_ORDER)
        qzeros = _pack_words(uz, AWQ_ORDER)
        q, sc, zero = ck.hf_awq_to_signed(qweight, qzeros, s)
        w_ref = (torch.from_numpy(u - np.repeat(uz, group, 0)).float() * s.float().repeat_interleave(group, 0))
    assert q.dtype == torch.int8 and int(q.min()) >= -8 and int(q.max()) <= 7
    assert torch.equal(q, torch.from_numpy(u - 8).to(torch.int8))
    w = q.float() * sc.float().repeat_interleave(group, 0) + zero.float().repeat_interleave(group, 0)
    # zero is rounded to fp16 once, as the reference does: a few fp16 ulps of |z * s|
    assert float((w - w_ref).abs().max()) <= 2 ** -10 * float((zero.float().abs()).max()) + 1e-7


def test_tllm_tensor_names_and_bytes():
    u, uz, s = _make()
    q, sc, zero = ck.hf_awq_to_signed(_pack_words(u, AWQ_ORDER), _pack_words(uz, AWQ_ORDER), s)
    t = ck.to_tllm_tensors("transformer.layers.0.mlp.fc", q, sc, zero, torch.float16,
                           prequant_scale=torch.ones(256), bias=torch.zeros(128))
    p = "transformer.layers.0.mlp.fc"
    assert set(t) == {f"{p}.weight", f"{p}.weights_scaling_factor", f"{p}.zero", f"{p}.prequant_scaling_factor",
                      f"{p}.bias"}
    assert t[f"{p}.weight"].dtype == torch.float16 and tuple(t[f"{p}.weight"].shape) == (256, 128 // 4)
    assert tuple(t[f"{p}.prequant_scaling_factor"].shape) == (1, 256)
    packed = quantize.pack_int8_tensor_to_packed_int4(q)
    expect = quantize.preprocess_weights_for_mixed_gemm(packed, torch.quint4x2, torch.float16)
    assert torch.equal(t[f"{p}.weight"].view(torch.int8), expect)


def test_bad_inputs():
    u, uz, s = _make()
    with pytest.raises(ValueError):
        ck.gptq_to_signed(_pack_words(u.T.copy()).T.contiguous(), _pack_words(uz), s[:, :64])
    with pytest.raises(ValueError):
        ck.sharded_linear_from_checkpoint("ggml", None, None, None, mapping=Mapping(), parallel="column")


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["gptq", "awq"])
def test_forward_from_checkpoint(fmt):
    k, n, group, m = 1024, 512, 128, 5
    u, uz, s = _make(k, n, group, seed=3)
    if fmt == "gptq":
        qweight, qzeros = _pack_words(u.T.copy()).T.contiguous(), _pack_words(uz)
        q, sc, zero = ck.gptq_to_signed(qweight, qzeros, s)
        w_ref = torch.from_numpy(u - (np.repeat(uz, group, 0) + 1)).float() * s.float().repeat_interleave(group, 0)
    else:
        qweight, qzeros = _pack_words(u, AWQ_ORDER), _pack_words(uz, AWQ_ORDER)
        q, sc, zero = ck.hf_awq_to_signed(qweight, qzeros, s)
        w_ref = torch.from_numpy(u - np.repeat(uz, group, 0)).float() * s.float().repeat_interleave(group, 0)
    layer = ck.WeightOnlyGroupwiseQuantLinear(ck.to_tllm_tensors("l", q, sc, zero), "l", group)
    torch.manual_seed(1)
    x = torch.randn(m, k).half()
    y = layer(x.cuda()).float().cpu()
    ref = x.float() @ w_ref
    assert float((y - ref).abs().max()) <= 1e-2 * float(ref.abs().max())
    # and the sharded form on a one-rank mapping goes through the same tensors
    col = ck.sharded_linear_from_checkpoint(fmt, qweight, qzeros, s, mapping=Mapping(), parallel="column")
    assert float((col(x.cuda()).float().cpu() - ref).abs().max()) <= 1e-2 * float(ref.abs().max())
