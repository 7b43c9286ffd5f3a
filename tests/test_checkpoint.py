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


def test_modelopt_awq_unpacking():
    """ModelOpt INT4-AWQ: bytes [N/2, K] of two's-complement nibble pairs of adjacent output features,
    scales [N, K/G], a pre-quant scale; no zeros."""
    rng = np.random.default_rng(5)
    k, n, group = 256, 64, 128
    q = rng.integers(-8, 8, size=(k, n)).astype(np.int8)
    u = (q.astype(np.int16) & 15).astype(np.uint8)          # two's-complement nibbles
    weight = torch.from_numpy((u[:, 0::2] | (u[:, 1::2] << 4)).T.copy())  # [N/2, K]
    wscale = torch.from_numpy(rng.uniform(0.001, 0.02, size=(n, k // group)).astype(np.float32))
    ps = torch.from_numpy(rng.uniform(0.5, 1.5, size=(k,)).astype(np.float32))
    q2, s2, z2, ps2 = ck.modelopt_awq_to_signed(weight, wscale, ps)
    assert z2 is None and torch.equal(q2, torch.from_numpy(q))
    assert tuple(s2.shape) == (k // group, n) and torch.equal(s2, wscale.half().T.contiguous())
    assert torch.equal(ps2, ps.half())
    with pytest.raises(ValueError):
        ck.modelopt_awq_to_signed(weight.to(torch.int32), wscale, ps)


@pytest.mark.parametrize("fmt", ["gptq", "awq", "modelopt_awq"])
@pytest.mark.parametrize("tp_size", [1, 2])
def test_llama_layer_key_mapping_and_sharding(fmt, tp_size):
    """One Hugging Face Llama decoder layer -> TensorRT-LLM names, q/k/v fused, sharded per rank; the
    dequantised shards reassemble to the dequantised full matrices."""
    rng = np.random.default_rng(11)
    hidden, inter, kv, group = 256, 512, 256, 128
    dims = {"self_attn.q_proj": (hidden, hidden), "self_attn.k_proj": (hidden, kv), "self_attn.v_proj": (hidden, kv),
            "self_attn.o_proj": (hidden, hidden), "mlp.gate_proj": (hidden, inter), "mlp.up_proj": (hidden, inter),
            "mlp.down_proj": (inter, hidden)}
    state, dense = {}, {}
    for name, (k, n) in dims.items():
        u = rng.integers(0, 16, size=(k, n))
        uz = rng.integers(0, 16, size=(k // group, n))
        s = rng.uniform(0.001, 0.02, size=(k // group, n)).astype(np.float32)
        pre = f"model.layers.3.{name}"
        if fmt == "gptq":
            state[f"{pre}.qweight"], state[f"{pre}.qzeros"] = _pack_words(u.T.copy()).T.contiguous(), _pack_words(uz)
            state[f"{pre}.scales"] = torch.from_numpy(s).half()
            w = (u - (np.repeat(uz, group, 0) + 1)) * np.repeat(torch.from_numpy(s).half().float().numpy(), group, 0)
        elif fmt == "awq":
            state[f"{pre}.qweight"], state[f"{pre}.qzeros"] = _pack_words(u, AWQ_ORDER), _pack_words(uz, AWQ_ORDER)
            state[f"{pre}.scales"] = torch.from_numpy(s).half()
            w = (u - np.repeat(uz, group, 0)) * np.repeat(torch.from_numpy(s).half().float().numpy(), group, 0)
        else:
            q = (u - 8).astype(np.int8)
            nib = (q.astype(np.int16) & 15).astype(np.uint8)
            state[f"{pre}.weight"] = torch.from_numpy((nib[:, 0::2] | (nib[:, 1::2] << 4)).T.copy())
            state[f"{pre}.weight_scale"] = torch.from_numpy(s.T.copy())
            state[f"{pre}.input_quantizer._pre_quant_scale"] = torch.ones(k)
            w = q * np.repeat(torch.from_numpy(s).half().float().numpy(), group, 0)
        dense[name] = w

    from oracle import woq_oracle as oracle

    def dequant(t, prefix):
        wq = oracle.signed_weights(t[f"{prefix}.weight"].view(torch.int8), t[f"{prefix}.weight"].shape[0],
                                   t[f"{prefix}.weight"].shape[1] * 4, 4).float()
        s_ = t[f"{prefix}.weights_scaling_factor"].float().repeat_interleave(group, 0)
        z_ = t.get(f"{prefix}.zero")
        return wq * s_ + (0 if z_ is None else z_.float().repeat_interleave(group, 0))

    shards = [ck.convert_llama_layer(fmt, state, 3, mapping=Mapping(tp_size, r, tp_size=tp_size), group_size=group)
              for r in range(tp_size)]
    p = "transformer.layers.3"
    expect_keys = {f"{p}.{m}.{t}" for m in ("attention.qkv", "attention.dense", "mlp.fc", "mlp.gate", "mlp.proj")
                   for t in (("weight", "weights_scaling_factor") + (("zero",) if fmt != "modelopt_awq" else
                                                                     ("prequant_scaling_factor",)))}
    assert set(shards[0]) == expect_keys
    tol = 2 ** -9 * 0.4  # zero-point products are rounded to fp16 once
    # row-parallel: K chunks stack; column-parallel: N chunks concatenate
    for tllm, hf, dim in (("attention.dense", "self_attn.o_proj", 0), ("mlp.proj", "mlp.down_proj", 0),
                          ("mlp.fc", "mlp.gate_proj", 1), ("mlp.gate", "mlp.up_proj", 1)):
        whole = torch.cat([dequant(sh, f"{p}.{tllm}") for sh in shards], dim=dim)
        assert float((whole - torch.from_numpy(dense[hf]).float()).abs().max()) <= tol
    # fused qkv: every rank holds [q chunk | k chunk | v chunk]
    for r, sh in enumerate(shards):
        w = dequant(sh, f"{p}.attention.qkv")
        parts = [torch.from_numpy(dense[f"self_attn.{x}_proj"]).float().chunk(tp_size, dim=1)[r] for x in "qkv"]
        assert float((w - torch.cat(parts, dim=1)).abs().max()) <= tol


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
