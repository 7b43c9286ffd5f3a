"""GPU: the one-shot peer-memory all-reduce behind row-parallel layers (w4_allreduce_oneshot).

On one GPU the ranks are emulated by one launch over all ranks' data: every "peer" buffer is local
and the flag words of the other ranks are set from the host before the launch, so no kernel ever
waits for another kernel. The bounded wait is exercised with a flag that nothing sets and a short
limit: the kernel must give up, leave the output alone and report the timeout through the device
status word. With two or more GPUs the real thing runs as child processes against NCCL."""
import os
import subprocess
import sys

import pytest
import torch

import tensorrt_llm_b200 as pkg
from tensorrt_llm_b200 import ops

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _emulated(world, m, n, dtype, rank, epoch, bias):
    torch.manual_seed(world * 100 + m + epoch)
    dev = "cuda"
    parts = [torch.randn(m, n, device=dev).to(dtype) for _ in range(world)]
    flags = [torch.zeros(8, dtype=torch.int32, device=dev) for _ in range(world)]
    # every rank has "announced" (word `rank` is also written by the kernel); int32 view of the uint32 call number
    flags[rank][:world] = epoch - (1 << 32) if epoch >= (1 << 31) else epoch
    out = torch.zeros(m, n, dtype=dtype, device=dev)
    b = torch.randn(n, device=dev).to(dtype) if bias else None
    ops.allreduce_oneshot([p.data_ptr() for p in parts], [f.data_ptr() for f in flags], out, n, rank, epoch, bias=b)
    torch.cuda.synchronize()
    acc = torch.zeros(m, n, dtype=torch.float32, device=dev)
    for p in parts:  # rank order, fp32: the kernel's order
        acc += p.float()
    if bias:
        acc += b.float()
    # what the kernel told the "peers": word `rank` of every rank's flags
    announced = [int(f[rank]) & 0xFFFFFFFF for f in flags]
    return out, acc.to(dtype), announced


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("m,n", [(1, 8192), (3, 1024), (64, 8192)])
def test_emulated_ranks_bit_exact(dtype, world, m, n):
    rank, epoch = world - 1, 5
    out, ref, announced = _emulated(world, m, n, dtype, rank, epoch, bias=(m == 3))
    assert torch.equal(out, ref)
    assert announced == [epoch] * world
    assert pkg._lib.lib().w4_gemm_device_status() == 0


def test_epoch_wraps():
    out, ref, _ = _emulated(2, 1, 1024, torch.bfloat16, 0, 0xFFFFFFFF, bias=False)
    assert torch.equal(out, ref)


def test_peer_that_never_arrives_times_out():
    dev = "cuda"
    n = 1024
    parts = [torch.ones(1, n, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    flags = [torch.zeros(8, dtype=torch.int32, device=dev) for _ in range(2)]  # rank 1 never announces
    out = torch.full((1, n), 7.0, dtype=torch.bfloat16, device=dev)
    ops.allreduce_oneshot([p.data_ptr() for p in parts], [f.data_ptr() for f in flags], out, n, 0, 1, timeout_ms=20)
    torch.cuda.synchronize()
    assert pkg._lib.lib().w4_gemm_device_status() == pkg._lib.W4_ERR_DEVICE_TIMEOUT
    assert pkg._lib.lib().w4_gemm_device_status() == 0  # reading clears it
    assert bool((out == 7.0).all())  # untouched
    # the context is still usable
    out2, ref2, _ = _emulated(2, 1, n, torch.bfloat16, 0, 2, bias=False)
    assert torch.equal(out2, ref2)


def test_argument_errors():
    dev = "cuda"
    a = torch.zeros(1, 1024, dtype=torch.bfloat16, device=dev)
    f = torch.zeros(8, dtype=torch.int32, device=dev)
    with pytest.raises(pkg._lib.W4Error):  # count not a multiple of 8
        ops.allreduce_oneshot([a.data_ptr()], [f.data_ptr()], a[:, :1020].contiguous(), 1020, 0, 1)
    big = torch.zeros(1024, 1024, dtype=torch.bfloat16, device=dev)  # 2 MiB > one-shot limit
    with pytest.raises(pkg._lib.W4Error):
        ops.allreduce_oneshot([big.data_ptr()], [f.data_ptr()], big, 1024, 0, 1)
    with pytest.raises(RuntimeError):
        ops.allreduce_oneshot([a.data_ptr()] * 9, [f.data_ptr()] * 9, a, 1024, 0, 1)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_against_nccl():
    """Row-parallel layer on 2 GPUs: GEMM into the shared buffer + one-shot reduce vs GEMM + NCCL."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29541", os.path.join(ROOT, "tests", "_oneshot_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "ONESHOT_OK" in r.stdout
