"""GPU: the peer-memory all-reduce behind row-parallel layers (w4_allreduce).

On one GPU the ranks are emulated by ONE cooperative launch over all ranks' buffers
(w4_allreduce_emulated): every "peer" block is local memory and the CTAs of all ranks are
co-resident, so no kernel ever waits for another kernel. The call number lives in the workspace on the
device: the same launch is repeated (and replayed from a CUDA graph) without any host-side counter.
The bounded wait is exercised with a single-rank launch whose peer never pushes and a short limit:
the kernel must give up and report the timeout through the device status word. With two or more
GPUs the real thing runs as child processes against NCCL."""
import os
import subprocess
import sys

import pytest
import torch

import tensorrt_llm_b200 as pkg
from tensorrt_llm_b200 import ops

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
L = pkg._lib


def _setup(world, m, n, dtype, max_bytes, seed, bias=False):
    torch.manual_seed(seed)
    dev = "cuda"
    parts = [torch.randn(m, n, device=dev).to(dtype) for _ in range(world)]
    nws = ops.allreduce_workspace_bytes(max_bytes, world)
    wss = [torch.zeros(nws, dtype=torch.uint8, device=dev) for _ in range(world)]
    outs = [torch.zeros(m, n, dtype=dtype, device=dev) for _ in range(world)]
    b = torch.randn(n, device=dev).to(dtype) if bias else None
    return parts, wss, outs, b


def _expected(parts, b):
    acc = torch.zeros_like(parts[0], dtype=torch.float32)
    for p in parts:  # rank order, fp32: the kernel's order
        acc += p.float()
    if b is not None:
        acc += b.float()
    return acc.to(parts[0].dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("world", [1, 2, 3, 4, 5, 7, 8])
@pytest.mark.parametrize("mode", [L.W4_ALLREDUCE_ONE_SHOT, L.W4_ALLREDUCE_TWO_SHOT])
@pytest.mark.parametrize("m,n", [(1, 8192), (3, 1024), (64, 8192), (7, 4104)])
def test_emulated_ranks_bit_exact(dtype, world, mode, m, n):
    parts, wss, outs, b = _setup(world, m, n, dtype, max(m * n * 2, 1 << 16), world * 100 + m, bias=(m == 3))
    biases = None if b is None else [b] * world
    for call in range(3):  # consecutive calls use alternate copies of the inbox and the flags
        for p in parts:
            p.add_(1.0)
        ops.allreduce_emulated(parts, wss, outs, n, biases=biases, mode=mode)
        torch.cuda.synchronize()
        ref = _expected(parts, b)
        for r in range(world):
            assert torch.equal(outs[r], ref), f"call {call}, rank {r}"
        # the device-side call number of every rank
        assert [int(w[:4].view(torch.int32)[0]) for w in wss] == [call + 1] * world
    assert L.lib().w4_gemm_device_status() == 0


@pytest.mark.parametrize("mode,m", [(L.W4_ALLREDUCE_AUTO, 1), (L.W4_ALLREDUCE_AUTO, 64), (L.W4_ALLREDUCE_TWO_SHOT, 512)])
def test_large_and_auto_modes(mode, m):
    """AUTO picks by size (16 KB one-shot, 1 MB two-shot at 8 ranks); 8 MB through the two-shot path."""
    world, n = 8, 8192
    parts, wss, outs, _ = _setup(world, m, n, torch.bfloat16, 8 << 20, m)
    ops.allreduce_emulated(parts, wss, outs, n, mode=mode)
    torch.cuda.synchronize()
    ref = _expected(parts, None)
    for r in range(world):
        assert torch.equal(outs[r], ref)


@pytest.mark.parametrize("world", [3, 6])
def test_flag_protocol_with_ragged_slices(world):
    """Above 4 MiB the plain-data protocol with arrival flags runs; 271 625 vectors do not divide by the
    rank count, so the slices and their chunks are ragged. Twice, for both copies of the buffers."""
    m, n = 265, 8200
    assert m * n * 2 > L.W4_ALLREDUCE_LL_MAX_BYTES
    parts, wss, outs, b = _setup(world, m, n, torch.bfloat16, m * n * 2, world, bias=True)
    for call in range(2):
        for p in parts:
            p.mul_(-0.75)
        ops.allreduce_emulated(parts, wss, outs, n, biases=[b] * world)
        torch.cuda.synchronize()
        ref = _expected(parts, b)
        for r in range(world):
            assert torch.equal(outs[r], ref), f"call {call}, rank {r}"
    assert L.lib().w4_gemm_device_status() == 0


def test_graph_replay_needs_no_host_counter():
    """A captured launch replayed many times: every replay is a new call (fresh inputs each time)."""
    world, m, n = 4, 2, 4096
    parts, wss, outs, _ = _setup(world, m, n, torch.bfloat16, 1 << 20, 3)
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        ops.allreduce_emulated(parts, wss, outs, n, stream=st)  # warm-up outside the capture
        st.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            ops.allreduce_emulated(parts, wss, outs, n, stream=st)
        for it in range(7):
            for p in parts:
                p.mul_(-0.5).add_(float(it))
            g.replay()
            st.synchronize()
            ref = _expected(parts, None)
            assert all(torch.equal(o, ref) for o in outs), f"replay {it}"
    assert int(wss[0][:4].view(torch.int32)[0]) == 8  # 1 warm-up + 7 replays (the capture itself runs nothing)


def test_peer_that_never_arrives_times_out():
    """Rank 0 of a 2-rank group launched alone: rank 1 never pushes. The wait must run out (20 ms)."""
    n = 1024
    parts, wss, outs, _ = _setup(2, 1, n, torch.bfloat16, 1 << 16, 9)
    ops.allreduce(parts[0], [w.data_ptr() for w in wss], wss[0].numel(), outs[0], n, 0, timeout_ms=20)
    torch.cuda.synchronize()
    assert L.lib().w4_gemm_device_status() == L.W4_ERR_DEVICE_TIMEOUT
    assert L.lib().w4_gemm_device_status() == 0  # reading clears it
    # rank 0 did push its partial into rank 1's inbox before waiting (inbox copy of call 1 is copy 1)
    # the context is still usable, and a cleared workspace works again
    for w in wss:
        w.zero_()
    ops.allreduce_emulated(parts, wss, outs, n)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], _expected(parts, None)) and torch.equal(outs[1], outs[0])


def test_argument_errors():
    dev = "cuda"
    a = torch.zeros(1, 1024, dtype=torch.bfloat16, device=dev)
    ws = torch.zeros(ops.allreduce_workspace_bytes(1 << 16, 1), dtype=torch.uint8, device=dev)
    with pytest.raises(L.W4Error):  # count not a multiple of 8
        ops.allreduce(a[:, :1020].contiguous(), [ws.data_ptr()], ws.numel(), a[:, :1020].contiguous(), 1020, 0)
    big = torch.zeros(64, 1024, dtype=torch.bfloat16, device=dev)  # 128 KiB > the 64 KiB the workspace was sized for
    with pytest.raises(L.W4Error):
        ops.allreduce(big, [ws.data_ptr()], ws.numel(), big, 1024, 0)
    with pytest.raises(RuntimeError):
        ops.allreduce(a, [ws.data_ptr()] * 9, ws.numel(), a, 1024, 0)
    with pytest.raises(L.W4Error):  # one-shot forced above its limit
        huge = torch.zeros(1024, 1024, dtype=torch.bfloat16, device=dev)
        ws2 = torch.zeros(ops.allreduce_workspace_bytes(4 << 20, 2), dtype=torch.uint8, device=dev)
        ops.allreduce(huge, [ws2.data_ptr()] * 2, ws2.numel(), huge, 1024, 0, mode=L.W4_ALLREDUCE_ONE_SHOT)
    assert ops.allreduce_workspace_bytes(0, 2) == 0 and ops.allreduce_workspace_bytes(1024, 9) == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_real_gpus_against_nccl():
    """Row-parallel layer on all visible GPUs (2..8): GEMM + peer-memory reduce vs GEMM + NCCL, several
    sizes through both forms, and a replayed CUDA graph of GEMM + reduce steps."""
    n = min(torch.cuda.device_count(), 8)
    n = 8 if n >= 8 else (4 if n >= 4 else 2)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr",
           "127.0.0.1", "--master-port", "29541", os.path.join(ROOT, "tests", "_peer_allreduce_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "PEER_ALLREDUCE_OK" in r.stdout


@pytest.mark.parametrize("world,m", [(2, 1), (4, 5), (8, 1), (8, 12), (8, 20)])
def test_gemm_epilogue_push_then_gather(world, m):
    """The fused form of a row-parallel decode step on emulated ranks: every rank's int4 decode GEMM
    writes its partial sums locally and pushes them as flagged packets into all inboxes
    (w4_gemm_launch_push; the ranks' GEMMs are separate launches, they wait for nobody), then one
    cooperative launch gathers on all ranks (W4_ALLREDUCE_GATHER_ONLY). Two rounds with fresh
    activations (both copies of the inbox); 20 rows take a 16-row and a 4-row pass."""
    from _cases import make_problem, oracle_out, max_err
    from oracle import woq_oracle as oracle
    n, k_local, group = 1024, 512, 128
    dev = "cuda"
    probs = [make_problem(m, n, k_local, 4, group, torch.bfloat16, zero=True, prequant=True, seed=300 + 10 * world + r)
             for r in range(world)]
    nws = ops.allreduce_workspace_bytes(1 << 20, world)
    wss = [torch.zeros(nws, dtype=torch.uint8, device=dev) for _ in range(world)]
    ptrs = [w.data_ptr() for w in wss]
    partials = [torch.zeros(m, n, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    outs = [torch.zeros(m, n, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    bias = torch.randn(n, device=dev).to(torch.bfloat16)
    d = lambda t: t.to(dev)
    dev_t = [{key: d(p[key]) for key in ("processed", "scales", "zeros", "ps")} for p in probs]
    for rnd in range(2):
        acts = [d((p["act"].float() * (1.0 - 1.5 * rnd)).to(torch.bfloat16)) for p in probs]
        for r in range(world):
            t = dev_t[r]
            pushed = ops.gemm_push(acts[r], t["processed"], t["scales"], partials[r], ptrs, nws, r, n=n, k=k_local,
                                   group_size=group, zeros=t["zeros"], act_scale=t["ps"])
            assert pushed
        ops.allreduce_emulated(partials, wss, outs, n, biases=[bias] * world, mode=L.W4_ALLREDUCE_GATHER_ONLY)
        torch.cuda.synchronize()
        for r in range(world):  # every rank's GEMM against the oracle
            ref = oracle_out(dict(probs[r], act=acts[r].cpu()))
            assert max_err(partials[r].cpu(), ref) <= oracle.tolerance(ref)
        ref = _expected(partials, bias)
        for r in range(world):
            assert torch.equal(outs[r], ref), f"round {rnd}, rank {r}"
    assert [int(w[:4].view(torch.int32)[0]) for w in wss] == [2] * world
    assert L.lib().w4_gemm_device_status() == 0
    # an ordinary call afterwards continues the same sequence of call numbers
    ops.allreduce_emulated(partials, wss, outs, n)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], _expected(partials, None))


def pkg_regime_auto():
    import tensorrt_llm_b200 as pkg
    return pkg.W4_REGIME_AUTO


def test_push_is_refused_where_it_does_not_apply():
    from _cases import make_problem
    dev = "cuda"
    d = lambda t: t.to(dev)
    nws = ops.allreduce_workspace_bytes(1 << 20, 2)
    ws = torch.zeros(nws, dtype=torch.uint8, device=dev)
    p8 = make_problem(1, 1024, 512, 8, 128, torch.bfloat16, zero=True, seed=1)  # int8: no pushing epilogue
    out = torch.zeros(1, 1024, dtype=torch.bfloat16, device=dev)
    from tensorrt_llm_b200._lib import W4GemmParams
    import ctypes
    par = W4GemmParams(act=d(p8["act"]).data_ptr(), weight=d(p8["processed"]).data_ptr(), scales=d(p8["scales"]).data_ptr(),
                       zeros=d(p8["zeros"]).data_ptr(), out=out.data_ptr(), alpha=1.0, m=1, n=1024, k=512, group_size=128,
                       weight_bits=8, act_dtype=1, regime=0)
    r = ops._allreduce_params(out, [ws.data_ptr()] * 2, nws, out, 1024, 0, None, L.W4_ALLREDUCE_AUTO, 0)
    rc = L.lib().w4_gemm_launch_push(ctypes.byref(par), ctypes.byref(r), None)
    assert rc == L.W4_ERR_UNSUPPORTED
    p4 = make_problem(64, 1024, 512, 4, 128, torch.bfloat16, zero=True, seed=2)  # 64 rows: tensor-core regime
    big = torch.zeros(64, 1024, dtype=torch.bfloat16, device=dev)
    assert not ops.gemm_push(d(p4["act"]), d(p4["processed"]), d(p4["scales"]), big, [ws.data_ptr()] * 2, nws, 0, n=1024,
                             k=512, group_size=128, zeros=d(p4["zeros"]), regime=pkg_regime_auto())


@pytest.mark.parametrize("m", [1, 7, 16])
def test_single_kernel_gemm_allreduce_one_rank(m):
    """w4_gemm_allreduce with a group of one rank: the decode kernel pushes into its own inbox slot,
    collects it again, adds the bias, writes the output and advances the call number - the whole
    single-kernel path without a peer to wait for (with peers it runs in the multi-GPU worker test).
    Three calls in a row (both buffer copies), then an ordinary all-reduce continues the numbering."""
    from _cases import make_problem, oracle_out, max_err
    from oracle import woq_oracle as oracle
    n, k, group = 1024, 512, 128
    dev = "cuda"
    p = make_problem(m, n, k, 4, group, torch.bfloat16, zero=True, prequant=True, seed=500 + m)
    d = lambda t: t.to(dev)
    nws = ops.allreduce_workspace_bytes(1 << 20, 1)
    ws = torch.zeros(nws, dtype=torch.uint8, device=dev)
    part = torch.zeros(m, n, dtype=torch.bfloat16, device=dev)
    out = torch.zeros(m, n, dtype=torch.bfloat16, device=dev)
    bias = torch.randn(n, device=dev).to(torch.bfloat16)
    w, s, z, ps = d(p["processed"]), d(p["scales"]), d(p["zeros"]), d(p["ps"])
    for call in range(3):
        act = d((p["act"].float() * (1.0 + call)).to(torch.bfloat16))
        out.zero_()
        ops.gemm_allreduce(act, w, s, part, out, [ws.data_ptr()], nws, 0, n=n, k=k, weight_bits=4, group_size=group,
                           zeros=z, act_scale=ps, bias=bias, timeout_ms=50)
        torch.cuda.synchronize()
        assert L.lib().w4_gemm_device_status() == 0
        ref_part = oracle.kernel_rounding_ref(act.cpu(), p["q"], p["scales"], zeros=p["zeros"], pre_quant_scale=p["ps"],
                                              group_size=group)
        ref = (ref_part.float() + bias.cpu().float()).to(torch.bfloat16)
        assert max_err(out.cpu(), ref) <= oracle.tolerance(ref)
        assert int(ws[:4].view(torch.int32)[0]) == call + 1 and int(ws[4:8].view(torch.int32)[0]) == 0
    ops.allreduce(out, [ws.data_ptr()], nws, part, n, 0)
    torch.cuda.synchronize()
    assert torch.equal(part, out) and int(ws[:4].view(torch.int32)[0]) == 4
