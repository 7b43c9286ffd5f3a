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
gloo in the CPU tests) on the tensor the GEMM wrote. ``matmul`` can be replaced (the CPU tests pass
the oracle) so that the sharding logic is testable without a GPU.
"""
from __future__ import annotations

import time
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
        """q: signed int8 [K, N]; scales/zeros: [K/G, N] (or [N] for group_size 0); bias [N]."""
        self = cls(mapping, bits, group_size, dtype, device)
        tp, r = mapping.tp_size, mapping.tp_rank
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
        self = cls(mapping, bits, group_size, dtype, device)
        tp, r = mapping.tp_size, mapping.tp_rank
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

    def forward(self, x_local, all_reduce: bool = True, oneshot: "OneShotAllReduce | None" = None):
        """``oneshot``: use the peer-memory all-reduce for this call when the message fits it (the
        GEMM then writes straight into the shared partial buffer); otherwise NCCL."""
        m = x_local.numel() // x_local.shape[-1]
        nbytes = m * self.n_local * x_local.element_size()
        if (oneshot is not None and all_reduce and self.mapping.tp_size > 1 and oneshot.preferred(nbytes)
                and self.matmul is None and self.group_size != 0):
            part = oneshot.partial(m, self.n_local)
            algo = (_lib.INT8_WEIGHT if self.bits == 8 else 0) | (_lib.ZERO if self.zeros is not None else 0) \
                | (_lib.PRE_QUANT_SCALE if self.pre_quant_scale is not None else 0)
            ops.weight_only_groupwise_quant_matmul(x_local, self.pre_quant_scale, self.weight, self.scales, self.zeros,
                                                   None, 1.0, algo, self.group_size, out=part)
            y = torch.empty(x_local.shape[:-1] + (self.n_local,), dtype=x_local.dtype, device=x_local.device)
            return oneshot.reduce(y, bias=self.bias)
        y = self._gemm(x_local, with_bias=False)
        if all_reduce and self.mapping.tp_size > 1:
            import torch.distributed as dist
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        if self.bias is not None:
            y = y + self.bias
        return y

    __call__ = forward


class OneShotAllReduce:
    """Peer-memory all-reduce for the small [M, N] partial sums of row-parallel layers (decode).

    Owns one symmetric-memory allocation per rank (``torch.distributed._symmetric_memory``: every
    rank's block is mapped into every process of the group): 256 bytes of flag words, then two
    partial buffers used alternately. ``partial(m, n)`` returns the local buffer the next GEMM must
    write; ``reduce(out)`` launches the library's one-shot kernel behind it on the current stream.
    All ranks must make the same sequence of calls, as with any collective. Plain peer loads and
    stores only (no multicast). Messages above ``W4_ONESHOT_MAX_BYTES`` belong to NCCL."""

    FLAG_BYTES = 256

    def __init__(self, group, device, dtype=torch.bfloat16, max_bytes: int = _lib.W4_ONESHOT_MAX_BYTES):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if self.world > _lib.W4_MAX_RANKS:
            raise RuntimeError(f"OneShotAllReduce supports at most {_lib.W4_MAX_RANKS} ranks")
        self.dtype, self.max_bytes = dtype, int(max_bytes)
        self.buf = symm_mem.empty(self.FLAG_BYTES + 2 * self.max_bytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        torch.cuda.synchronize(device)
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        dist.barrier(self.group)  # every rank's flags are zero before anyone announces call 1
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.epoch = 0

    def preferred(self, nbytes: int) -> bool:
        """The reference's choice between its one-shot kernel and NCCL
        (plugins/ncclPlugin/allreducePlugin.cpp:258-283): always up to 2 ranks, below 1 MB up to 4,
        below 500 kB beyond; and never above this buffer's capacity."""
        if nbytes > self.max_bytes or nbytes % 16:
            return False
        if self.world <= 2:
            return True
        return nbytes < (1_000_000 if self.world <= 4 else 500_000)

    def _offset(self, epoch: int) -> int:
        return self.FLAG_BYTES + (epoch & 1) * self.max_bytes

    def partial(self, m: int, n: int) -> torch.Tensor:
        """Local buffer for the partial sums of the next call to ``reduce``."""
        nbytes = m * n * self.buf.new_empty(0, dtype=self.dtype).element_size()
        if nbytes > self.max_bytes:
            raise RuntimeError("message too large for the one-shot all-reduce")
        off = self._offset(self.epoch + 1)
        return self.buf[off:off + nbytes].view(self.dtype).view(m, n)

    def reduce(self, out: torch.Tensor, bias=None, timeout_ms: int = 0) -> torch.Tensor:
        self.epoch += 1
        off = self._offset(self.epoch)
        ops.allreduce_oneshot([p + off for p in self.ptrs], self.ptrs, out, out.shape[-1], self.rank, self.epoch,
                              bias=bias, timeout_ms=timeout_ms)
        return out


# ------------------------------------------------------------------------------------------------
# Measurement helper: the Llama-3-70B linear set under tensor parallelism
# ------------------------------------------------------------------------------------------------
LLAMA70B_LAYERS = (  # name, K, N, parallel kind
    ("qkv", 8192, 10240, "column"),
    ("gate_up", 8192, 57344, "column"),
    ("o_proj", 8192, 8192, "row"),
    ("down", 28672, 8192, "row"),
)


def bench_llama70b_layer_set(device, rank, world, barrier, max_over_ranks, ms=(1, 64, 2048), reps=20,
                             group_size=128):
    """Times every linear of one Llama-3-70B layer at tp = world size: W4A16 group-128 with zeros,
    bf16, seeded random shard contents (random bytes are what the layout of random int4 weights
    is). Column-parallel layers: the local GEMM only. Row-parallel layers: local GEMM, then the
    NCCL all-reduce of the [M, 8192] partial sums, each timed with CUDA events (max over ranks).
    Between repetitions a buffer larger than the L2 is written so that weights stream from HBM."""
    import torch.distributed as dist

    g = torch.Generator(device=device).manual_seed(3 + rank)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)
    out = {}
    one, one_err = None, None
    if world > 1:
        try:
            one = OneShotAllReduce(None, device, torch.bfloat16)
        except Exception as e:  # symmetric memory not available on this box: NCCL only, and say so
            one_err = f"{type(e).__name__}: {e}"[:200]
    for name, K, N, kind in LLAMA70B_LAYERS:
        k_loc, n_loc = (K, N // world) if kind == "column" else (K // world, N)
        _check_shard(k_loc, n_loc, 4, group_size)
        w = torch.randint(0, 256, (k_loc, n_loc // 2), dtype=torch.uint8, device=device, generator=g).view(torch.int8)
        s = (torch.rand((k_loc // group_size, n_loc), device=device, generator=g) * 0.019 + 0.001).to(torch.bfloat16)
        z = (torch.rand((k_loc // group_size, n_loc), device=device, generator=g) * 0.2 - 0.1).to(torch.bfloat16)
        for m in ms:
            x = torch.randn((m, k_loc), device=device, generator=g).to(torch.bfloat16)
            y = torch.empty((m, n_loc), dtype=torch.bfloat16, device=device)
            ws_bytes = ops.workspace_bytes(m, n_loc, k_loc, group_size, 4, torch.bfloat16, False)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device) if ws_bytes else None

            def gemm():
                ops.gemm_raw(x, w, s, y, n=n_loc, k=k_loc, weight_bits=4, group_size=group_size, zeros=z,
                             workspace=ws)

            try:
                gemm()
            except _lib.W4Error as e:
                out[f"{name}_m{m}"] = {"unavailable": str(e)}
                continue
            t_gemm, t_ar = [], []
            for _ in range(reps):
                flush.zero_()
                barrier()
                e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
                e0.record()
                gemm()
                e1.record()
                if kind == "row" and world > 1:
                    dist.all_reduce(y, op=dist.ReduceOp.SUM)
                e2.record()
                torch.cuda.synchronize()
                t_gemm.append(e0.elapsed_time(e1))
                t_ar.append(e1.elapsed_time(e2))
            # Row-parallel decode step as it runs in a serving loop: GEMM + reduce, back to back, no
            # host in between (one CUDA graph of `reps` steps, replayed once: the one-shot kernel's
            # call numbers are baked into the launches). Weights stay L2-warm here; the comparison
            # of interest is the reduce. NCCL and the peer-memory kernel see the same GEMM.
            use_one = kind == "row" and world > 1 and one is not None and one.preferred(m * n_loc * 2)
            step_us = {}
            if kind == "row" and world > 1:
                y2 = torch.empty_like(y)

                def step_nccl():
                    gemm()
                    dist.all_reduce(y, op=dist.ReduceOp.SUM)

                def step_one():
                    part = one.partial(m, n_loc)
                    ops.gemm_raw(x, w, s, part, n=n_loc, k=k_loc, weight_bits=4, group_size=group_size, zeros=z,
                                 workspace=ws)
                    one.reduce(y2)

                for label, fn in (("gemm", gemm), ("nccl", step_nccl)) + ((("oneshot", step_one),) if use_one else ()):
                    try:
                        st = torch.cuda.Stream(device=device)
                        with torch.cuda.stream(st):
                            for _ in range(3):
                                fn()
                            st.synchronize()
                            barrier()
                            greps = reps * (5 if m <= 64 else 1)  # long enough to hide the one-off graph upload
                            graph = torch.cuda.CUDAGraph()
                            with torch.cuda.graph(graph, stream=st):
                                for _ in range(greps):
                                    fn()
                            e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(2))
                            st.synchronize()
                            barrier()  # capture takes a different time on every rank: start together
                            e1.record(st)
                            graph.replay()
                            e2.record(st)
                            st.synchronize()
                        step_us[label] = max_over_ranks(e1.elapsed_time(e2) * 1e3 / greps)
                        del graph
                    except Exception as e:  # capture not possible on this box: say so, keep going
                        step_us[label] = f"unavailable: {type(e).__name__}: {e}"[:160]
                        max_over_ranks(0.0)
            t_gemm.sort()
            t_ar.sort()
            gemm_us = max_over_ranks(t_gemm[len(t_gemm) // 2] * 1e3)
            ar_us = max_over_ranks(t_ar[len(t_ar) // 2] * 1e3) if kind == "row" and world > 1 else 0.0
            nbytes = k_loc * n_loc // 2 + 2 * (k_loc // group_size) * n_loc * 2 + m * k_loc * 2 + m * n_loc * 2
            flops = 2.0 * m * n_loc * k_loc
            out[f"{name}_m{m}"] = {
                "kind": kind, "k_local": k_loc, "n_local": n_loc, "gemm_us": gemm_us, "allreduce_us": ar_us,
                "allreduce_bytes": m * n_loc * 2 if kind == "row" and world > 1 else 0,
                "per_gpu_GB/s": nbytes / gemm_us / 1e3, "per_gpu_TFLOP/s": flops / gemm_us / 1e6,
                "regime": "gemv" if ops.select_regime(m, n_loc, k_loc, group_size, 4) == _lib.W4_REGIME_GEMV else "gemm",
            }
            if kind == "row" and world > 1:
                out[f"{name}_m{m}"]["graph_step_us_gemm_only"] = step_us.get("gemm")
                out[f"{name}_m{m}"]["graph_step_us_gemm_plus_nccl"] = step_us.get("nccl")
                out[f"{name}_m{m}"]["graph_step_us_gemm_plus_oneshot"] = step_us.get("oneshot") if use_one else (
                    one_err or "message above the one-shot threshold for this world size: NCCL")
    del flush
    return out
