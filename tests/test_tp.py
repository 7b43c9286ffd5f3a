"""CPU: tensor-parallel sharding logic. Rank math against the reference's expectations
(tests/test_mapping.py:22-50 of TensorRT-LLM) and the column/row-parallel layers run as two gloo
ranks, with the CPU oracle standing in for the GPU kernel."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import woq_oracle as oracle
from tensorrt_llm_b200 import tp
from tensorrt_llm_b200.mapping import Mapping


def test_mapping_groups_tp2_pp2_cp2():
    m = Mapping(world_size=8, rank=0, tp_size=2, pp_size=2, cp_size=2)
    assert m.tp_groups == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert m.pp_groups == [[0, 4], [1, 5], [2, 6], [3, 7]]
    assert m.cp_groups == [[0, 2], [1, 3], [4, 6], [5, 7]]
    m = Mapping(world_size=8, rank=6, tp_size=2, pp_size=2, cp_size=2)
    assert (m.tp_rank, m.cp_rank, m.pp_rank) == (0, 1, 1)
    assert m.tp_group == [6, 7] and m.pp_group == [2, 6] and m.cp_group == [4, 6]


def test_mapping_tp8_and_errors():
    for r in range(8):
        m = Mapping(world_size=8, rank=r, tp_size=8)
        assert m.tp_rank == r and m.tp_group == list(range(8)) and m.pp_group == [r]
    m = Mapping(world_size=8, rank=5, tp_size=4, pp_size=2)
    assert m.tp_group == [4, 5, 6, 7] and m.pp_group == [1, 5] and m.pp_rank == 1 and m.is_last_pp_rank()
    with pytest.raises(ValueError):
        Mapping(world_size=8, rank=0, tp_size=3)
    with pytest.raises(ValueError):
        Mapping(world_size=4, rank=4, tp_size=4)


def test_split_and_shard_rules():
    x = torch.arange(24).reshape(4, 6)
    assert torch.equal(tp.split(x, 2, 1, dim=0), x[2:]) and torch.equal(tp.split(x, 3, 0, dim=1), x[:, :2])
    with pytest.raises(ValueError):
        tp.split(x, 4, 0, dim=1)


def test_feature_padding_like_the_reference():
    """Features that do not split into whole 64-wide tiles / scale groups per rank are rounded up to a
    multiple of max(64, group) * tp first (quantization/layers.py:719-726, 965-972 of the reference);
    the padded layer gives the same result on zero-extended activations."""
    assert tp.padded_features(192, 64, 2) == 256 and tp.padded_features(4096, 128, 8) == 4096
    assert tp.padded_features(11008, 128, 8) == 11264 and tp.padded_features(100, 0, 4) == 256
    g = torch.Generator().manual_seed(4)
    K, N, G, M, world = 192, 160, 64, 3, 2
    q = torch.randint(-8, 8, (K, N), dtype=torch.int8, generator=g)
    scales = (torch.rand(K // G, N, generator=g) * 0.02 + 0.001).half()
    zeros = (torch.rand(K // G, N, generator=g) * 0.2 - 0.1).half()
    bias = torch.randn(N, generator=g).half()
    x = torch.randn(M, K, generator=g).half()
    full = oracle.kernel_rounding_ref(x, q, scales, zeros=zeros, bias=bias, group_size=G)
    xp = torch.nn.functional.pad(x, (0, 256 - K))
    # row-parallel: K 192 -> 256, 128 per rank; partial sums add up to the unpadded result
    acc = torch.zeros(M, 256, dtype=torch.float32)
    for r in range(world):
        layer = tp.WeightOnlyRowLinear.from_quantized(Mapping(world, r, tp_size=world), q, scales, zeros, bias, bits=4,
                                                      group_size=G, dtype=torch.float16)
        assert (layer.in_features, layer.out_features, layer.k_local, layer.n_local, layer.n_valid) == (256, 256, 128, 256, N)
        layer.matmul = _oracle_matmul
        acc += layer(tp.split(xp, world, r, dim=1), all_reduce=False).float() - (bias_pad := torch.nn.functional.pad(
            bias, (0, 256 - N))).float()
    got = (acc + bias_pad.float())[:, :N]
    assert float((got - full.float()).abs().max()) <= 2e-3 * float(full.float().abs().max())
    # column-parallel: N 160 -> 256, 128 per rank; the valid columns of the gathered output match
    outs = []
    for r in range(world):
        layer = tp.WeightOnlyColumnLinear.from_quantized(Mapping(world, r, tp_size=world), q, scales, zeros, bias, bits=4,
                                                         group_size=G, dtype=torch.float16)
        layer.matmul = _oracle_matmul
        outs.append(layer(xp))
    got = torch.cat(outs, dim=1)[:, :N]
    assert float((got.float() - full.float()).abs().max()) <= 2e-3 * float(full.float().abs().max())


def _oracle_matmul(layer, x, bias):
    return oracle.kernel_rounding_ref(x, layer.q, layer.scales.cpu(), zeros=None if layer.zeros is None else
                                      layer.zeros.cpu(), bias=bias, pre_quant_scale=layer.pre_quant_scale,
                                      group_size=layer.group_size)


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mapping = Mapping(world_size=world, rank=rank, tp_size=world)
        g = torch.Generator().manual_seed(0)  # same full problem on every rank
        K, N, M, G = 256, 256, 3, 64
        q = torch.randint(-8, 8, (K, N), dtype=torch.int8, generator=g)
        scales = (torch.rand(K // G, N, generator=g) * 0.02 + 0.001).to(torch.bfloat16)
        zeros = (torch.rand(K // G, N, generator=g) * 0.2 - 0.1).to(torch.bfloat16)
        bias = torch.randn(N, generator=g).to(torch.bfloat16)
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        full = oracle.kernel_rounding_ref(x, q, scales, zeros=zeros, bias=bias, group_size=G)

        col = tp.WeightOnlyColumnLinear.from_quantized(mapping, q, scales, zeros, bias, bits=4, group_size=G)
        col.matmul = _oracle_matmul
        y_col = col(x)
        assert y_col.shape == (M, N // world)
        exp_col = full[:, rank * (N // world):(rank + 1) * (N // world)]
        assert torch.equal(y_col, exp_col), "column-parallel shard differs from the matching slice"

        row = tp.WeightOnlyRowLinear.from_quantized(mapping, q, scales, zeros, bias, bits=4, group_size=G)
        row.matmul = _oracle_matmul
        x_local = tp.split(x, world, rank, dim=1)
        y_row = row(x_local)
        err = float((y_row.float() - full.float()).abs().max())
        assert err <= oracle.tolerance(full), f"row-parallel result off by {err}"
        # every rank holds the same reduced tensor
        gathered = [torch.empty_like(y_row) for _ in range(world)]
        dist.all_gather(gathered, y_row)
        assert all(torch.equal(gathered[0], t) for t in gathered)

        # per-channel: a K shard is quantised with its own scales
        w = torch.randn(K, N, generator=g) * 0.02
        rowf = tp.WeightOnlyRowLinear.from_float(mapping, w, bits=8, dtype=torch.float16)
        u_ref, _, s_ref = oracle.symmetric_quantize(tp.split(w, world, rank, dim=0).contiguous(), 8)
        assert torch.equal(rowf.q, u_ref) and torch.equal(rowf.scales, s_ref.to(torch.float16))
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_column_and_row_parallel_two_ranks():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29500 + (os.getpid() % 500)
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: "ok", 1: "ok"}


def test_rank_that_never_joins_times_out():
    """Failure on the host side: a rendezvous that a rank never joins ends with an error after the
    timeout instead of hanging."""
    from datetime import timedelta
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(29400 + (os.getpid() % 90))
    with pytest.raises(Exception):
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=timedelta(seconds=2))
    if dist.is_initialized():
        dist.destroy_process_group()


def test_peer_allreduce_workspace_sizing():
    """Host logic of the peer-memory all-reduce (no GPU): the workspace grows monotonically with the
    largest message, holds a whole one-shot message per sender or a slice of a two-shot one, and the
    helper refuses messages beyond it."""
    from tensorrt_llm_b200 import tp, ops, _lib

    header = 256 + 2 * (2 * _lib.W4_MAX_RANKS * _lib.W4_ALLREDUCE_MAX_CTAS * 4)
    prev = 0
    for world in (1, 2, 4, 8):
        for mb in (16384, 1 << 20, (1 << 20) + 16, 8 << 20, 32 << 20):
            nbytes = ops.allreduce_workspace_bytes(mb, world)
            assert nbytes % 256 == 0 and nbytes > header
            one = min(mb, _lib.W4_ONESHOT_MAX_BYTES)
            # two copies of: world sender slots (a one-shot message or a slice) + the reduced slice
            assert nbytes >= header + 2 * world * max(one, -(-mb // world)) + 2 * -(-mb // world)
            if mb > 16384:
                assert nbytes >= prev
            prev = nbytes
        prev = 0
    assert ops.allreduce_workspace_bytes(1 << 20, 0) == 0 and ops.allreduce_workspace_bytes(1 << 20, 9) == 0
    h = object.__new__(tp.PeerAllReduce)
    h.max_bytes = 1 << 20
    assert h.fits(1 << 20) and h.fits(16384) and not h.fits((1 << 20) + 16) and not h.fits(16380)
