"""Child process of tests/test_allreduce_gpu.py (one per GPU, started by torch.distributed.run):
a row-parallel W4A16 layer whose partial sums are reduced by the library's peer-memory kernel,
compared with the same layer reduced by NCCL over several calls and sizes (one-shot and two-shot
forms; up to 16 rows through the fused form, whose GEMM pushes its results itself), then CUDA graphs
of GEMM + reduce steps, unfused and fused, replayed several times. Plain peer loads and
stores only; NVLS is off in the parent's environment."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import tensorrt_llm_b200 as pkg  # noqa: E402
from tensorrt_llm_b200 import tp  # noqa: E402
from tensorrt_llm_b200.mapping import Mapping  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    mapping = Mapping(world_size=world, rank=rank, tp_size=world)
    k, n, g = 1024 * world, 4096, 128
    gen = torch.Generator().manual_seed(1234)  # same full tensors on every rank
    q = torch.randint(-8, 8, (k, n), dtype=torch.int8, generator=gen)
    scales = (torch.rand(k // g, n, generator=gen) * 0.019 + 0.001).to(torch.bfloat16)
    zeros = (torch.rand(k // g, n, generator=gen) * 0.2 - 0.1).to(torch.bfloat16)
    bias = torch.randn(n, generator=gen).to(torch.bfloat16)
    layer = tp.WeightOnlyRowLinear.from_quantized(mapping, q, scales, zeros, bias, bits=4, group_size=g,
                                                  dtype=torch.bfloat16, device=dev, group=None)
    peer = tp.PeerAllReduce(None, dev, torch.bfloat16, max_bytes=8 << 20)
    worst = 0.0
    for call, m in enumerate((1, 4, 1, 16, 8, 1, 64, 512, 1024, 3)):  # 8 KB .. 8 MB: both forms
        x = torch.randn(m, k, generator=gen).to(torch.bfloat16)
        x_loc = tp.split(x, world, rank, dim=1).contiguous().to(dev)
        y_nccl = layer(x_loc)
        y_peer = layer(x_loc, peer=peer)
        torch.cuda.synchronize()
        assert pkg._lib.lib().w4_gemm_device_status() == 0
        # NCCL adds bf16 partials in its own order; the peer kernel adds them in fp32: compare with a
        # tolerance of a few bf16 ulps of the largest value, and across ranks bit for bit.
        err = float((y_peer.float() - y_nccl.float()).abs().max())
        tol = 4 * 2.0 ** -8 * float(y_nccl.float().abs().max())
        assert err <= tol, (call, m, err, tol)
        worst = max(worst, err / tol)
        gathered = [torch.empty_like(y_peer) for _ in range(world)]
        dist.all_gather(gathered, y_peer)
        for other in gathered:
            assert torch.equal(other, gathered[0]), "ranks disagree"

    # A decode step (GEMM into the partial buffer, then the reduce) captured once, replayed 5 times
    # with new activations each time: the call number lives on the device.
    m = 2
    x_loc = torch.zeros(m, k // world, dtype=torch.bfloat16, device=dev)
    y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    st = torch.cuda.Stream(device=dev)

    def step():
        part = peer.partial(m, n)
        pkg.ops.weight_only_groupwise_quant_matmul(x_loc, None, layer.weight, layer.scales, layer.zeros, None, 1.0,
                                                   pkg.ZERO, g, out=part)
        peer.reduce(y, bias=layer.bias)

    with torch.cuda.stream(st):
        step()
        st.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            step()
            step()
            step()  # an odd number of calls per replay: buffer parity cannot be baked into the graph
        for it in range(5):
            x = torch.randn(m, k, generator=gen).to(torch.bfloat16)
            x_loc.copy_(tp.split(x, world, rank, dim=1))
            graph.replay()
            st.synchronize()
            ref = layer(x_loc)  # NCCL
            torch.cuda.synchronize()
            err = float((y.float() - ref.float()).abs().max())
            assert err <= 4 * 2.0 ** -8 * float(ref.float().abs().max()), (it, err)
    # The same with the fused form: the GEMM's epilogue pushes its results to the peers, the reduce only
    # gathers (what layer(x, peer=peer) does by itself for up to 16 rows).
    def fused_step():
        assert peer.gemm_push(x_loc, layer, peer.partial(m, n))
        peer.reduce(y, bias=layer.bias, mode=pkg._lib.W4_ALLREDUCE_GATHER_ONLY)

    with torch.cuda.stream(st):
        fused_step()
        st.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            fused_step()
            fused_step()
            fused_step()
        for it in range(5):
            x = torch.randn(m, k, generator=gen).to(torch.bfloat16)
            x_loc.copy_(tp.split(x, world, rank, dim=1))
            graph.replay()
            st.synchronize()
            ref = layer(x_loc)  # NCCL
            torch.cuda.synchronize()
            err = float((y.float() - ref.float()).abs().max())
            assert err <= 4 * 2.0 ** -8 * float(ref.float().abs().max()), ("fused", it, err)
    # And as ONE kernel per step (w4_gemm_allreduce: compute, push, collect, add, write).
    def one_kernel_step():
        peer.gemm_allreduce(x_loc, layer, peer.partial(m, n), y)

    with torch.cuda.stream(st):
        one_kernel_step()
        st.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            one_kernel_step()
            one_kernel_step()
            one_kernel_step()
        for it in range(5):
            x = torch.randn(m, k, generator=gen).to(torch.bfloat16)
            x_loc.copy_(tp.split(x, world, rank, dim=1))
            graph.replay()
            st.synchronize()
            ref = layer(x_loc)  # NCCL
            torch.cuda.synchronize()
            err = float((y.float() - ref.float()).abs().max())
            assert err <= 4 * 2.0 ** -8 * float(ref.float().abs().max()), ("one kernel", it, err)
            gathered = [torch.empty_like(y) for _ in range(world)]
            dist.all_gather(gathered, y)
            for other in gathered:
                assert torch.equal(other, gathered[0]), "ranks disagree"
    assert pkg._lib.lib().w4_gemm_device_status() == 0
    dist.barrier()
    if rank == 0:
        print(f"PEER_ALLREDUCE_OK world {world} worst err/tol {worst:.3f}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
