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

Both become signed int4 weights q = u - 8 with ``zero = (8 - z [- 1 for GPTQ]) * s`` already
multiplied by the scale, which is the form the kernels (and the reference's plugin) take. Host-side
tensor code only; the layout transform and the GEMM run through the library.
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
    if fmt not in ("gptq", "awq"):
        raise ValueError("fmt must be 'gptq' or 'awq'")
    q, s, z = (gptq_to_signed if fmt == "gptq" else hf_awq_to_signed)(qweight, qzeros, scales, dtype)
    if parallel == "column":
        return tp.WeightOnlyColumnLinear.from_quantized(mapping, q, s, z, bias, bits=4, group_size=group_size,
                                                        dtype=dtype, device=device)
    if parallel == "row":
        return tp.WeightOnlyRowLinear.from_quantized(mapping, q, s, z, bias, bits=4, group_size=group_size,
                                                     dtype=dtype, device=device, group=group)
    raise ValueError("parallel must be 'column' or 'row'")
