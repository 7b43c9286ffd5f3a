"""Tensor-parallel weight-only linear layers, sharded the way the reference does it.

* Column-parallel (QKV, gate/up): the output features N are split into ``tp_size`` contiguous
  chunks (tensorrt_llm/layers/linear.py:340-343, tensorrt_llm/models/convert_utils.py:37-43 of
  TensorRT-LLM); scales and zeros are split on N; activations are replicated; no communication
  when the output is not gathered (tensorrt_llm/quantization/layers.py:1056-1058).
* Row-parallel (o_proj, down): the input features K are split (layers/linear.py:466-468); scale
  and zero *rows* are split with K; every rank produces a full [M, N] partial result and one
  all-reduce (sum) over the TP group finishes it (quantization/layers.py:1185-1186,
  cpp/tensorrt_llm/plugins/ncclPlugin/allreducePlugin.cpp:407). The bias of a row-parallel layer
  is added once, after the reduction.
* Shards are cut BEFORE quantisation / the layout transform (convert_utils.py:70-88,
  quantization/functional.py:881-889): per-channel scales of a K shard come from that shard's own
  maximum and the interleaved layout is built per shard.

One process per GPU; the collective is ``torch.distributed.all_reduce`` (NCCL over NVLink on GPUs,
gloo in the CPU tests) on the tensor the GEMM wrote. ``matmul`` is the hook through which a caller
substitutes the local product (the CPU tests do, to exercise the sharding logic without a GPU).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from . import _lib, ops, quantize
from .mapping import Mapping


def split(v: torch.Tensor, tp_size: int, idx: int, dim: int = 0) -> torch.Tensor:
    """Contiguous chunk ``idx`` of ``tp_size`` along ``dim`` (convert_utils.py:37-43)."""
    if tp_size == 1:
        return v
    if v.shape[dim] % tp_size:
        raise ValueError(f"dimension {dim} of size {v.shape[dim]} is not divisible by tp_size {tp_size}")
    return torch.chunk(v, tp_size, dim=dim)[idx].contiguous()


def padded_features(features: int, group_size: int, tp_size: int) -> int:
    """Feature count the reference's quantised linears round in/out features up to before sharding:
    a multiple of max(64, group_size) * tp_size (tensorrt_llm/quantization/layers.py:719-726 for
    per-channel, :965-972 and :1091-1098 for groupwise layers), so that every shard keeps whole
    64-wide tiles and whole scale groups."""
    multiple = max(64, group_size) * tp_size
    return -(-features // multiple) * multiple


def pad_like(t: Optional[torch.Tensor], shape, value=0) -> Optional[torch.Tensor]:
    """Pads ``t`` at the end of every dimension up to ``shape`` (functional.py:861-872 of the reference)."""
    if t is None or tuple(t.shape) == tuple(shape):
        return t
    pad = []
    for dim in range(len(shape)):
        d = -1 - dim
        pad += [0, max(0, shape[d] - t.shape[d])]
    return torch.nn.functional.pad(t, pad, value=value)


def pad_quantized_for_tp(q, scales, zeros, bias, pre_quant_scale, group_size: int, tp_size: int):
    """Pads a whole (unsharded) layer's tensors to ``padded_features`` in both dimensions: integer
    weights and zeros with 0, scales with 1, bias and pre-quant scale with 0. Padded input features
    meet zero activations and padded output features are cut off by the caller, so the fill values
    never reach a result (the reference fills with the same neutral values,
    tensorrt_llm/quantization/functional.py:983-1009). Returns the padded tensors and (k, n) padded."""
    k, n = q.shape
    kp, np_ = padded_features(k, group_size, tp_size), padded_features(n, group_size, tp_size)
    if (kp, np_) == (k, n):
        return q, scales, zeros, bias, pre_quant_scale, k, n
    q = pad_like(q, (kp, np_), 0)
    if group_size == 0:
        scales, zeros = pad_like(scales, (np_,), 1), pad_like(zeros, (np_,), 0)
    else:
        scales = pad_like(scales, (kp // group_size, np_), 1)
        zeros = pad_like(zeros, (kp // group_size, np_), 0)
    bias = pad_like(bias, (np_,), 0)
    if pre_quant_scale is not None:
        pre_quant_scale = pad_like(pre_quant_scale.reshape(-1), (kp,), 0)
    return q, scales, zeros, bias, pre_quant_scale, kp, np_


def _check_shard(k: int, n: int, bits: int, group_size: int):
    if k % 64 or (n * bits // 8) % 32:
        raise ValueError(f"shard [{k}, {n}] violates the layout's divisibility rules (k % 64, n*bits/8 % 32)")
    if group_size and k % group_size:
        raise ValueError(f"shard k={k} is not a multiple of the group size {group_size}")


class _ShardedLinear:
    """State shared by the two layer kinds: one rank's preprocessed weight, scales, zeros."""

    def __init__(self, mapping: Mapping, bits: int, group_size: int, dtype: torch.dtype, device):
        self.mapping, self.bits, self.group_size, self.dtype, self.device = mapping, bits, group_size, dtype, device
        self.weight = self.scales = self.zeros = self.bias = self.pre_quant_scale = None
        self.matmul: Optional[Callable] = None  # test hook; None = the CUDA op

    def _load(self, q_shard, scales, zeros, bias, pre_quant_scale):
        """q_shard: signed int8 [k_local, n_local] integers of this rank."""
        k, n = q_shard.shape
        _check_shard(k, n, self.bits, self.group_size)
        packed = quantize.pack_int8_tensor_to_packed_int4(q_shard.contiguous()) if self.bits == 4 else q_shard
        qt = torch.quint4x2 if self.bits == 4 else torch.int8
        self.q = q_shard  # kept for the test hook only
        self.weight = quantize.preprocess_weights_for_mixed_gemm(packed.contiguous(), qt, torch.float16).to(self.device)
        mv = lambda t: None if t is None else t.to(self.dtype).contiguous().to(self.device)
        self.scales, self.zeros, self.bias, self.pre_quant_scale = mv(scales), mv(zeros), mv(bias), mv(pre_quant_scale)
        self.k_local, self.n_local = k, n

    def _gemm(self, x: torch.Tensor, with_bias: bool) -> torch.Tensor:
        bias = self.bias if with_bias else None
        if self.matmul is not None:
            return self.matmul(self, x, bias)
        if self.group_size == 0:
            return ops.weight_only_quant_matmul(x, self.weight, self.scales, 1 if self.bits == 8 else 2)
        algo = (_lib.INT8_WEIGHT if self.bits == 8 else 0) | (_lib.ZERO if self.zeros is not None else 0) \
            | (_lib.BIAS if bias is not None else 0) | (_lib.PRE_QUANT_SCALE if self.pre_quant_scale is not None else 0)
        return ops.weight_only_groupwise_quant_matmul(x, self.pre_quant_scale, self.weight, self.scales, self.zeros,
                                                      bias, 1.0, algo, self.group_size)


class WeightOnlyColumnLinear(_ShardedLinear):
    """y_local[.., N/tp] = x[.., K] @ W[:, chunk]; no communication (gather_output = False)."""

    @classmethod
    def from_quantized(cls, mapping, q, scales, zeros=None, bias=None, pre_quant_scale=None, *, bits=4,
                       group_size=128, dtype=torch.bfloat16, device="cpu"):
        """q: signed int8 [K, N]; scales/zeros: [K/G, N] (or [N] for group_size 0); bias [N]. Features
        that do not divide into whole tiles / groups per rank are padded first, as the reference does;
        ``in_features`` / ``out_features`` keep the padded sizes, ``n_valid`` the real output width."""
        self = cls(mapping, bits, group_size, dtype, device)
        tp, r = mapping.tp_size, mapping.tp_rank
        self.n_valid = q.shape[1]
        q, scales, zeros, bias, pre_quant_scale, self.in_features, self.out_features = pad_quantized_for_tp(
            q, scales, zeros, bias, pre_quant_scale, group_size, tp)
        last = lambda t: None if t is None else split(t, tp, r, dim=t.dim() - 1)
        self._load(split(q, tp, r, dim=1), last(scales), last(zeros), last(bias), pre_quant_scale)
        return self

    @classmethod
    def from_float(cls, mapping, weight, *, bits=8, dtype=torch.float16, device="cpu"):
        """Per-channel: weight fp [K, N]; the N chunk is cut first, then quantised with its own scales."""
        self = cls(mapping, bits, 0, dtype, device)
        shard = split(weight, mapping.tp_size, mapping.tp_rank, dim=1)
        qt = torch.quint4x2 if bits == 4 else torch.int8
        u, _, s = quantize._symmetric_quantize_last_axis_of_batched_matrix(shard.contiguous(), qt)
        self._load(quantize.unpack_int4_packed_tensor_to_int8(u) if bits == 4 else u, s, None, None, None)
        return self

    def forward(self, x):
        return self._gemm(x, with_bias=True)

    __call__ = forward


class WeightOnlyRowLinear(_ShardedLinear):
    """y[.., N] = all_reduce_sum_over_tp( x_local[.., K/tp] @ W[chunk, :] ) (+ bias once)."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.group = None  # torch.distributed process group of mapping.tp_group

    @classmethod
    def from_quantized(cls, mapping, q, scales, zeros=None, bias=None, pre_quant_scale=None, *, bits=4,
                       group_size=128, dtype=torch.bfloat16, device="cpu", group=None):
        """As the column-parallel form; a padded K means this rank expects ``in_features / tp`` input
        features per row (zeros in the padded tail, as the padded layer in front of it produces)."""
        self = cls(mapping, bits, group_size, dtype, device)
        tp, r = mapping.tp_size, mapping.tp_rank
        self.n_valid = q.shape[1]
        q, scales, zeros, bias, pre_quant_scale, self.in_features, self.out_features = pad_quantized_for_tp(
            q, scales, zeros, bias, pre_quant_scale, group_size, tp)
        rows = lambda t: None if t is None else (t if group_size == 0 else split(t, tp, r, dim=0))
        ps = None if pre_quant_scale is None else split(pre_quant_scale.reshape(-1), tp, r, dim=0)
        self._load(split(q, tp, r, dim=0), rows(scales), rows(zeros), bias, ps)
        self.group = group
        return self

    @classmethod
    def from_float(cls, mapping, weight, *, bits=8, dtype=torch.float16, device="cpu", group=None):
        self = cls(mapping, bits, 0, dtype, device)
        shard = split(weight, mapping.tp_size, mapping.tp_rank, dim=0)
        qt = torch.quint4x2 if bits == 4 else torch.int8
        u, _, s = quantize._symmetric_quantize_last_axis_of_batched_matrix(shard.contiguous(), qt)
        self._load(quantize.unpack_int4_packed_tensor_to_int8(u) if bits == 4 else u, s, None, None, None)
        self.group = group
        return self

    def forward(self, x_local, all_reduce: bool = True, peer: "PeerAllReduce | None" = None):
        """``peer``: finish with the library's peer-memory all-reduce when the message fits its
        workspace (the GEMM then writes straight into its partial buffer); otherwise NCCL."""
        m = x_local.numel() // x_local.shape[-1]
        nbytes = m * self.n_local * x_local.element_size()
        if (peer is not None and all_reduce and self.mapping.tp_size > 1 and peer.fits(nbytes)
                and self.matmul is None and self.group_size != 0):
            part = peer.partial(m, self.n_local)
            y = torch.empty(x_local.shape[:-1] + (self.n_local,), dtype=x_local.dtype, device=x_local.device)
            # decode sizes on int4 weights: one kernel computes, pushes its results to the peers,
            # collects theirs and writes the reduced output
            if self.bits == 4 and m <= 16:
                return peer.gemm_allreduce(x_local, self, part, y)
            algo = (_lib.INT8_WEIGHT if self.bits == 8 else 0) | (_lib.ZERO if self.zeros is not None else 0) \
                | (_lib.PRE_QUANT_SCALE if self.pre_quant_scale is not None else 0)
            ops.weight_only_groupwise_quant_matmul(x_local, self.pre_quant_scale, self.weight, self.scales, self.zeros,
                                                   None, 1.0, algo, self.group_size, out=part)
            return peer.reduce(y, bias=self.bias)
        y = self._gemm(x_local, with_bias=False)
        if all_reduce and self.mapping.tp_size > 1:
            import torch.distributed as dist
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        if self.bias is not None:
            y = y + self.bias
        return y

    __call__ = forward


class PeerAllReduce:
    """Peer-memory all-reduce for the [M, N] partial sums of row-parallel layers.

    Owns one workspace block per rank in symmetric memory (``torch.distributed._symmetric_memory``
    maps every rank's block into every process of the group: plumbing) and one private buffer for
    the local partial sums. ``partial(m, n)`` returns the buffer the next GEMM must write;
    ``reduce(out)`` launches the library's kernel behind it on the current stream: one-shot (push to
    all peers, reduce locally) for latency-bound sizes, two-shot (reduce-scatter, then gather) above.
    The call number lives in the workspace on the device, so a captured graph of GEMM + reduce steps
    can be replayed. All ranks must make the same sequence of calls, as with any collective. Plain
    peer loads and stores only (no multicast)."""

    def __init__(self, group, device, dtype=torch.bfloat16, max_bytes: int = 32 << 20):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if self.world > _lib.W4_MAX_RANKS:
            raise RuntimeError(f"PeerAllReduce supports at most {_lib.W4_MAX_RANKS} ranks")
        self.dtype, self.max_bytes = dtype, int(max_bytes)
        self.ws_bytes = ops.allreduce_workspace_bytes(self.max_bytes, self.world)
        self.buf = symm_mem.empty(self.ws_bytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        torch.cuda.synchronize(device)
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        dist.barrier(self.group)  # every rank's workspace is zero before anyone makes call 1
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self._partial = torch.empty(self.max_bytes, dtype=torch.uint8, device=device)
        self.calls = 0  # host-side count, for information only

    def fits(self, nbytes: int) -> bool:
        return nbytes <= self.max_bytes and nbytes % 16 == 0

    def partial(self, m: int, n: int) -> torch.Tensor:
        """Local buffer for the partial sums of the next call to ``reduce``."""
        nbytes = m * n * torch.empty(0, dtype=self.dtype).element_size()
        if nbytes > self.max_bytes:
            raise RuntimeError("message too large for this PeerAllReduce")
        return self._partial[:nbytes].view(self.dtype).view(m, n)

    def gemm_push(self, x_local, layer, part, weights_static: bool = True) -> bool:
        """The layer's int4 decode GEMM into ``part`` with its results pushed to the peers (see
        ``ops.gemm_push``); False when the fused form does not apply and nothing was launched."""
        return ops.gemm_push(x_local, layer.weight, layer.scales, part, self.ptrs, self.ws_bytes, self.rank,
                             n=layer.n_local, k=x_local.shape[-1], group_size=layer.group_size, zeros=layer.zeros,
                             act_scale=layer.pre_quant_scale, weights_static=weights_static)

    def gemm_allreduce(self, x_local, layer, part, out, weights_static: bool = True):
        """The layer's GEMM and the all-reduce of its output, fused as far as the sizes allow
        (``ops.gemm_allreduce``). Counts as one call of the collective."""
        self.calls += 1
        ops.gemm_allreduce(x_local, layer.weight, layer.scales, part, out, self.ptrs, self.ws_bytes, self.rank,
                           n=layer.n_local, k=x_local.shape[-1], weight_bits=layer.bits, group_size=layer.group_size,
                           zeros=layer.zeros, act_scale=layer.pre_quant_scale, bias=layer.bias,
                           weights_static=weights_static)
        return out

    def reduce(self, out: torch.Tensor, bias=None, mode: int = _lib.W4_ALLREDUCE_AUTO, timeout_ms: int = 0,
               partial: Optional[torch.Tensor] = None) -> torch.Tensor:
        src = partial if partial is not None else self._partial[:out.numel() * out.element_size()].view(self.dtype)
        self.calls += 1
        ops.allreduce(src, self.ptrs, self.ws_bytes, out, out.shape[-1], self.rank, bias=bias, mode=mode,
                      timeout_ms=timeout_ms)
        return out


LLAMA70B_LAYERS = (  # name, K, N, parallel kind (BASELINE config 4)
    ("qkv", 8192, 10240, "column"),
    ("gate_up", 8192, 57344, "column"),
    ("o_proj", 8192, 8192, "row"),
    ("down", 28672, 8192, "row"),
)
