"""Checkpoint tensors -> what the weight-only groupwise GEMM consumes.

Restates, for one linear layer, what TensorRT-LLM does when it loads a 4-bit GPTQ or AutoAWQ
(Hugging Face AWQ) checkpoint into a ``WeightOnlyGroupwiseQuant{Column,Row}Linear``
(``tensorrt_llm/quantization/functional.py:835-846`` unpacking, ``:901-1037``
``postprocess_weight_only_groupwise``; parameter names ``weight`` / ``weights_scaling_factor`` /
``zero`` / ``prequant_scaling_factor`` / ``bias`` from ``tensorrt_llm/quantization/layers.py:1030-1037``):

* GPTQ:    ``qweight`` int32 [K/8, N] (eight nibbles per word along K), ``qzeros`` int32 [K/G, N/8],
           ``scales`` [K/G, N];  w = (u - (z + 1)) * s
* HF-AWQ:  ``qweight`` int32 [K, N/8] (eight nibbles per word along N in AutoAWQ's order
           0,4,1,5,2,6,3,7), ``qzeros`` int32 [K/G, N/8] in the same order, ``scales`` [K/G, N];
           w = (u - z) * s

* ModelOpt-AWQ (TensorRT-LLM unified checkpoints): ``weight`` uint8 [N/2, K] holding two's-complement
           int4 pairs of adjacent output features (low nibble first), ``weight_scale`` [N, K/G],
           ``input_quantizer._pre_quant_scale`` [K]; no zeros;  w = q * s on activations x * pre_quant_scale

GPTQ and HF-AWQ become signed int4 weights q = u - 8 with ``zero = (8 - z [- 1 for GPTQ]) * s`` already
multiplied by the scale, which is the form the kernels (and the reference's plugin) take. Host-side
tensor code only; the layout transform and the GEMM run through the library.

``convert_llama_layer`` applies this to the seven linears of one Hugging Face Llama decoder layer and
emits the TensorRT-LLM parameter names (q/k/v fused into ``attention.qkv``, ``o_proj`` ->
``attention.dense``, ``gate_proj`` -> ``mlp.fc``, ``up_proj`` -> ``mlp.gate``, ``down_proj`` ->
``mlp.proj``; tensorrt_llm/models/model_weights_loader.py:56-62 of the reference), sharded for one
tensor-parallel rank.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from . import _lib, ops, quantize, tp
from .mapping import Mapping

_AWQ_ORDER = (0, 4, 1, 5, 2, 6, 3, 7)


def unpack_int32_into_int8(w_packed: torch.Tensor, autoawq_reorder: bool = False) -> torch.Tensor:
    """int32 (or any 4-byte type) [R, C] -> int8 [R, 8C] of unsigned nibbles, low nibble first;
    ``autoawq_reorder`` undoes AutoAWQ's order inside every group of eight."""
    b = w_packed.contiguous().view(torch.uint8)
    out = torch.empty((b.shape[0], b.shape[1] * 2), dtype=torch.int8)
    out[:, 0::2] = (b & 0xF).to(torch.int8)
    out[:, 1::2] = (b >> 4).to(torch.int8)
    if autoawq_reorder:
        out = out.view(-1, 8)[:, list(_AWQ_ORDER)].reshape(out.shape)
    return out.contiguous()


def _finish(u: torch.Tensor, uz: torch.Tensor, scales: torch.Tensor, dtype: torch.dtype, gptq: bool):
    if u.shape[1] != scales.shape[1] or uz.shape != scales.shape:
        raise ValueError(f"shape mismatch: weights {tuple(u.shape)}, zeros {tuple(uz.shape)}, scales {tuple(scales.shape)}")
    if u.shape[0] % scales.shape[0]:
        raise ValueError("K is not a multiple of the number of scale groups")
    q = (u - 8).to(torch.int8)  # signed int4 in [-8, 7]
    s = scales.to(dtype)
    zero = ((-uz.to(torch.int32) + 8 - (1 if gptq else 0)).to(s.dtype) * s).to(dtype)  # as functional.py:1010-1014
    return q, s, zero


def gptq_to_signed(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, dtype=torch.float16):
    """-> (q int8 [K, N] in [-8, 7], scales [K/G, N] dtype, zero [K/G, N] dtype = (7 - z) * s)."""
    u = unpack_int32_into_int8(qweight.T).T.contiguous()
    uz = unpack_int32_into_int8(qzeros)
    return _finish(u, uz, scales, dtype, gptq=True)


def hf_awq_to_signed(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, dtype=torch.float16):
    """-> (q int8 [K, N] in [-8, 7], scales [K/G, N] dtype, zero [K/G, N] dtype = (8 - z) * s)."""
    u = unpack_int32_into_int8(qweight, True)
    uz = unpack_int32_into_int8(qzeros, True)
    return _finish(u, uz, scales, dtype, gptq=False)


def modelopt_awq_to_signed(weight: torch.Tensor, weight_scale: torch.Tensor, pre_quant_scale: torch.Tensor,
                           dtype=torch.float16):
    """ModelOpt INT4-AWQ tensors of one layer -> (q int8 [K, N] in [-8, 7], scales [K/G, N] dtype, None,
    pre_quant_scale [K] dtype) (functional.py:962-968, 919-937, 1023-1031 of the reference)."""
    if weight.dtype not in (torch.uint8, torch.int8):
        raise ValueError("ModelOpt-AWQ weight must be a byte tensor [N/2, K]")
    u = unpack_int32_into_int8(weight.T)            # [K, N], nibbles as 0..15
    q = torch.where(u >= 8, u - 16, u).to(torch.int8)  # two's-complement int4
    k, n = q.shape
    if weight_scale.numel() % n:
        raise ValueError("weight_scale does not hold whole groups for every output feature")
    scales = weight_scale.to(dtype).reshape(n, -1).T.contiguous()
    if k % scales.shape[0]:
        raise ValueError("K is not a multiple of the number of scale groups")
    return q, scales, None, pre_quant_scale.to(dtype).reshape(-1)


# Hugging Face Llama module -> TensorRT-LLM module, and how each is sharded
LLAMA_LINEARS = (
    ("attention.qkv", ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"), "column"),
    ("attention.dense", ("self_attn.o_proj",), "row"),
    ("mlp.fc", ("mlp.gate_proj",), "column"),
    ("mlp.gate", ("mlp.up_proj",), "column"),
    ("mlp.proj", ("mlp.down_proj",), "row"),
)


def _layer_to_signed(fmt: str, state: Dict[str, torch.Tensor], name: str, dtype):
    """(q, scales, zero, pre_quant_scale) of one Hugging Face linear in checkpoint format ``fmt``."""
    if fmt == "gptq":
        return gptq_to_signed(state[f"{name}.qweight"], state[f"{name}.qzeros"], state[f"{name}.scales"], dtype) + (None,)
    if fmt == "awq":
        return hf_awq_to_signed(state[f"{name}.qweight"], state[f"{name}.qzeros"], state[f"{name}.scales"], dtype) + (None,)
    if fmt == "modelopt_awq":
        return modelopt_awq_to_signed(state[f"{name}.weight"], state[f"{name}.weight_scale"],
                                      state[f"{name}.input_quantizer._pre_quant_scale"], dtype)
    raise ValueError("fmt must be 'gptq', 'awq' or 'modelopt_awq'")


def convert_llama_layer(fmt: str, state: Dict[str, torch.Tensor], layer: int, *, mapping: Optional[Mapping] = None,
                        group_size: int = 128, dtype=torch.float16, hf_prefix: str = "model.layers",
                        tllm_prefix: str = "transformer.layers") -> Dict[str, torch.Tensor]:
    """The TensorRT-LLM tensors of decoder layer ``layer`` for one tensor-parallel rank, from a Hugging
    Face Llama state dict in GPTQ, AutoAWQ or ModelOpt-AWQ format. Column-parallel linears keep this
    rank's chunk of the output features (q, k and v are chunked separately, then fused), row-parallel
    ones this rank's chunk of the input features; features are padded to whole tiles / groups per rank
    first, as the reference's layers do."""
    mapping = mapping or Mapping(world_size=1, rank=0, tp_size=1)
    tp_size, r = mapping.tp_size, mapping.tp_rank
    out: Dict[str, torch.Tensor] = {}
    for tllm_name, hf_names, kind in LLAMA_LINEARS:
        shards = []
        for hf in hf_names:
            q, s, z, ps = _layer_to_signed(fmt, state, f"{hf_prefix}.{layer}.{hf}", dtype)
            bias = state.get(f"{hf_prefix}.{layer}.{hf}.bias")
            q, s, z, bias, ps, _, _ = tp.pad_quantized_for_tp(q, s, z, bias, ps, group_size, tp_size)
            if kind == "column":
                last = lambda t: None if t is None else tp.split(t, tp_size, r, dim=t.dim() - 1)  # noqa: E731
                shards.append((tp.split(q, tp_size, r, dim=1), last(s), last(z), last(bias), ps))
            else:
                rows = lambda t: None if t is None else tp.split(t, tp_size, r, dim=0)  # noqa: E731
                shards.append((tp.split(q, tp_size, r, dim=0), rows(s), rows(z), bias, rows(ps)))
        cat = lambda i: None if shards[0][i] is None else torch.cat([x[i] for x in shards], dim=-1)  # noqa: E731
        q, s, z, bias = cat(0), cat(1), cat(2), cat(3)
        out.update(to_tllm_tensors(f"{tllm_prefix}.{layer}.{tllm_name}", q, s, z, dtype,
                                   prequant_scale=shards[0][4], bias=bias))
    return out


def to_tllm_tensors(prefix: str, q: torch.Tensor, scales: torch.Tensor, zero: Optional[torch.Tensor],
                    dtype=torch.float16, prequant_scale: Optional[torch.Tensor] = None,
                    bias: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
    """The parameter dict of one TensorRT-LLM groupwise layer: ``weight`` holds the preprocessed
    bytes viewed as ``dtype`` ([K, N/4]), as the reference stores them."""
    packed = quantize.pack_int8_tensor_to_packed_int4(q.contiguous())
    w = quantize.preprocess_weights_for_mixed_gemm(packed.contiguous(), torch.quint4x2, torch.float16)
    out = {f"{prefix}.weight": w.view(dtype), f"{prefix}.weights_scaling_factor": scales.to(dtype)}
    if zero is not None:
        out[f"{prefix}.zero"] = zero.to(dtype)
    if prequant_scale is not None:
        out[f"{prefix}.prequant_scaling_factor"] = prequant_scale.to(dtype).reshape(1, -1)
    if bias is not None:
        out[f"{prefix}.bias"] = bias.to(dtype)
    return out


class WeightOnlyGroupwiseQuantLinear:
    """y = x @ dequant(W) (+ bias) for one unsharded layer, from TensorRT-LLM-named tensors
    (the single-GPU counterpart of ``tp.WeightOnly{Column,Row}Linear``)."""

    def __init__(self, tensors: Dict[str, torch.Tensor], prefix: str, group_size: int = 128, device="cuda"):
        g = lambda k: tensors.get(f"{prefix}.{k}")  # noqa: E731
        if g("weight") is None or g("weights_scaling_factor") is None:
            raise KeyError(f"{prefix}.weight / {prefix}.weights_scaling_factor missing")
        mv = lambda t: None if t is None else t.contiguous().to(device)  # noqa: E731
        self.weight, self.scales, self.zero = mv(g("weight")), mv(g("weights_scaling_factor")), mv(g("zero"))
        ps = g("prequant_scaling_factor")
        self.prequant_scale = None if ps is None else mv(ps.reshape(-1))
        self.bias, self.group_size = mv(g("bias")), group_size
        self.quant_algo = (_lib.ZERO if self.zero is not None else 0) | (_lib.BIAS if self.bias is not None else 0) \
            | (_lib.PRE_QUANT_SCALE if self.prequant_scale is not None else 0)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return ops.weight_only_groupwise_quant_matmul(x, self.prequant_scale, self.weight, self.scales, self.zero,
                                                      self.bias, 1.0, self.quant_algo, self.group_size)


def sharded_linear_from_checkpoint(fmt: str, qweight, qzeros, scales, *, mapping: Mapping, parallel: str,
                                   group_size: int = 128, dtype=torch.float16, device="cuda", bias=None, group=None):
    """GPTQ (``fmt="gptq"``) or AutoAWQ (``fmt="awq"``) tensors of one layer -> this rank's
    tensor-parallel layer (column: split N; row: split K, all-reduce after)."""
    if fmt not in ("gptq", "awq", "modelopt_awq"):
        raise ValueError("fmt must be 'gptq', 'awq' or 'modelopt_awq'")
    ps = None
    if fmt == "modelopt_awq":  # (weight, pre_quant_scale, weight_scale) in place of (qweight, qzeros, scales)
        q, s, z, ps = modelopt_awq_to_signed(qweight, scales, qzeros, dtype)
    else:
        q, s, z = (gptq_to_signed if fmt == "gptq" else hf_awq_to_signed)(qweight, qzeros, scales, dtype)
    if parallel == "column":
        return tp.WeightOnlyColumnLinear.from_quantized(mapping, q, s, z, bias, ps, bits=4, group_size=group_size,
                                                        dtype=dtype, device=device)
    if parallel == "row":
        return tp.WeightOnlyRowLinear.from_quantized(mapping, q, s, z, bias, ps, bits=4, group_size=group_size,
                                                     dtype=dtype, device=device, group=group)
    raise ValueError("parallel must be 'column' or 'row'")
