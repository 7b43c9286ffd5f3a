#!/usr/bin/env python
"""Benchmark of the weight-only quantised GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-sweep]

One "step" is one pass of the hot path over one batch: the W4A16 group-128 AWQ decode GEMM of
BASELINE config 2 (bf16 activations [M=1, K=4096], int4 weights [4096, 14336] with bf16 scales and
zeros per 128 rows, pre-quant scale; the Llama-3-8B gate/up projection). The headline metric is the
HBM bandwidth the step sustains: algorithmic bytes / time. Inputs are synthetic and seeded. Each
step reads a different copy of the weights (a ring of copies larger than twice the L2) so that
every step streams from HBM.

With N > 1 (launched under torchrun) every rank runs the same step on its own GPU (independent
replicas, no collective on the data path: "weak" scaling) and the value is the sum over ranks;
the tensor-parallel Llama-3-70B layer set (column-parallel without communication, row-parallel
with an all-reduce: NCCL and the library's peer-memory kernel) is timed and parity-checked in the
same run and reported under "tp_llama70b".

The JSON line also carries: "e2e" (same metric through torch.ops.trtllm with host buffers: the
activations are copied from pinned host memory and the result read back inside the timed region;
weights stay resident in HBM as they do in serving), "roofline" (achieved / measured HBM copy
bandwidth), "cpu_baseline" (the CPU definition of the path timed on the host cores), "points"
(every M of config 2, config 1, the prefill GEMM of config 3 with and without a pre-quant scale,
weight preparation, split-k) and "sweep" (config 5: the Llama-3-8B shapes x weight formats x
activation types x M = 1..8192 with the regime chosen, the roofline fraction against the bound that
applies and a parity flag per point), and "clocks" (NVML samples taken during the timed region).

--impl reference times the reference's CPU definition of the path (dequantise then matmul with
torch on all host cores) on a bounded column sample of the same workload. Only that arm and the
parity checks / cpu_baseline of this file use anything under oracle/.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

L2_BYTES = 126 * 1024 * 1024
METRIC = "W4A16 g128 AWQ decode GEMM (M=1, K=4096, N=14336, bf16): HBM GB/s"
WORKLOAD = ("BASELINE config 2: W4A16 g128 AWQ decode GEMM (zeros + pre-quant scale), M=1, K=4096, N=14336, bf16; "
            "one GEMM per step")
C2 = dict(n=14336, k=4096, group=128, bits=4)
C3 = dict(m=4096, n=4096, k=14336, group=128, bits=4)
REF_SAMPLE_COLS = 512  # columns of config 2 one step of the CPU arm computes
# config 5: distinct (K, N) of the seven Llama-3-8B linears, weight formats, M values
SWEEP_SHAPES = [("q/o", 4096, 4096), ("k/v", 4096, 1024), ("gate/up", 4096, 14336), ("down", 14336, 4096)]
SWEEP_FORMATS = [("w8_pc", 8, 0), ("w4_g64", 4, 64), ("w4_g128", 4, 128)]
SWEEP_MS = [1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192]
LLAMA70B_LAYERS = (("qkv", 8192, 10240, "column"), ("gate_up", 8192, 57344, "column"),
                   ("o_proj", 8192, 8192, "row"), ("down", 28672, 8192, "row"))


def algorithmic_bytes(m, n, k, bits, group, zeros, prequant, bias=False):
    """K*N*bits/8 + n_sz*(K/G)*N*2 + M*K*2 + [ps]*K*2 + [bias]*N*2 + M*N*2 (G = K for per-channel)."""
    groups = 1 if group == 0 else k // group
    n_sz = 2 if zeros else 1
    return (k * n * bits // 8 + n_sz * groups * n * 2 + m * k * 2 + (k * 2 if prequant else 0)
            + (n * 2 if bias else 0) + m * n * 2)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def captured_traffic(key):
    """DRAM bytes per launch from the committed ncu summary (profiles/traffic.json), or None."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        return json.load(f).get(key)


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while a region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _once(self):
        try:
            self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
            mask = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            for bit, name in self.REASONS.items():
                if mask & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            self._once()
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        if self._thread is not None:
            self._once()
            self._stop.set()
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------ problems

class Problem:
    """One seeded synthetic GEMM problem resident on the device: signed integer weights generated
    on the GPU, packed and laid out by the library's device-side preparation (byte-identical to the
    host path), scales ~U(0.001, 0.02), zeros ~U(-0.1, 0.1), activations ~N(0, 1). Extra weight /
    scale / zero sets (random bytes: what the layout of random integers is) let consecutive launches
    stream different memory."""

    def __init__(self, device, m, n, k, bits, group, dtype, zeros, prequant, seed, copies=1, ps_ones=False):
        from tensorrt_llm_b200 import quantize
        g = torch.Generator(device=device).manual_seed(seed)
        self.m, self.n, self.k, self.bits, self.group, self.dtype = m, n, k, bits, group, dtype
        lo, hi = (-8, 8) if bits == 4 else (-128, 128)
        self.q = torch.randint(lo, hi, (k, n), dtype=torch.int8, device=device, generator=g)
        if bits == 4:
            packed = ((self.q[:, 0::2] & 15) | (self.q[:, 1::2] << 4)).contiguous()
            qt = torch.quint4x2
        else:
            packed, qt = self.q, torch.int8
        w0 = quantize.preprocess_weights_for_mixed_gemm_cuda(packed, qt)
        shape = (n,) if group == 0 else (k // group, n)
        slo, shi = (0.0005, 0.002) if group == 0 else (0.001, 0.02)

        def new_scales():
            s = (torch.rand(shape, device=device, generator=g) * (shi - slo) + slo).to(dtype)
            z = (torch.rand(shape, device=device, generator=g) * 0.2 - 0.1).to(dtype) if zeros else None
            return s, z

        self.sets = [(w0,) + new_scales()]
        for _ in range(copies - 1):
            w = torch.randint(0, 256, w0.shape, dtype=torch.uint8, device=device, generator=g).view(torch.int8)
            self.sets.append((w,) + new_scales())
        self.act = torch.randn((m, k), device=device, generator=g).to(dtype)
        self.ps = None
        if prequant:
            self.ps = (torch.ones(k, device=device) if ps_ones
                       else torch.rand(k, device=device, generator=g) + 0.5).to(dtype)

    def launcher(self, m, regime=0, weights_static=True):
        """fn(i): one GEMM of the first m rows on weight set i; returns (fn, out)."""
        from tensorrt_llm_b200 import ops
        act = self.act[:m].contiguous()
        out = torch.empty((m, self.n), dtype=self.dtype, device=act.device)
        nb = ops.workspace_bytes(m, self.n, self.k, self.group, self.bits, self.dtype, self.ps is not None, regime)
        ws = torch.empty(nb, dtype=torch.uint8, device=act.device) if nb else None

        def fn(i):
            w, s, z = self.sets[i % len(self.sets)]
            ops.gemm_raw(act, w, s, out, n=self.n, k=self.k, weight_bits=self.bits, group_size=self.group, zeros=z,
                         act_scale=self.ps, regime=regime, workspace=ws, weights_static=weights_static)

        return fn, out

    def parity(self, out, m, seed=0):
        """max|out - ref| / max|ref| on a sample of rows and columns of weight set 0 against the
        float64 CPU oracle (the checker; bound: 1e-2)."""
        from oracle import woq_oracle as oracle
        gen = torch.Generator().manual_seed(seed)
        rows = sorted(set([0, m - 1] + [int(x) for x in torch.randint(0, m, (14,), generator=gen)]))
        if m > 256:  # row-tile boundaries of the tensor-core kernel
            rows = sorted(set(rows + [b for t in (128, 192, 256) for b in (t - 1, t, m - m % t - 1, m - m % t)
                                      if 0 <= b < m]))
        cols = sorted(set(list(range(64)) + list(range(self.n - 64, self.n))
                          + [int(x) for x in torch.randint(0, self.n, (128,), generator=gen)]))
        ri, ci = torch.tensor(rows), torch.tensor(cols)
        _, s, z = self.sets[0]
        pick = lambda t: None if t is None else t.cpu()[..., ci]
        ref = oracle.kernel_rounding_ref(self.act[:m].cpu()[ri], self.q.cpu()[:, ci], pick(s), zeros=pick(z),
                                         pre_quant_scale=None if self.ps is None else self.ps.cpu(),
                                         group_size=self.group)
        got = out.cpu()[ri][:, ci]
        scale = float(ref.double().abs().max())
        return float((got.double() - ref.double()).abs().max()) / (scale if scale > 0 else 1.0)


def copies_for(nbytes):
    """Weight sets needed for consecutive launches to stream more than twice the L2."""
    return max(2, min(160, (2 * L2_BYTES + nbytes - 1) // nbytes + 1))


def time_graph(fn, reps, stream, replays=2):
    """Microseconds per launch of `reps` consecutive launches captured in one CUDA graph (the decode
    kernel lasts a few microseconds: launching it from Python one call at a time would measure the
    interpreter, not the GPU). Best of `replays` timed replays after one untimed replay."""
    with torch.cuda.stream(stream):
        for i in range(3):
            fn(i)
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for i in range(reps):
                fn(i)
        g.replay()
        stream.synchronize()
        best = float("inf")
        for _ in range(replays):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            g.replay()
            e1.record(stream)
            stream.synchronize()
            best = min(best, e0.elapsed_time(e1) * 1e3 / reps)
    return best


def time_steps(fn, steps, warmup, sync, barrier):
    """W untimed steps, then exactly `steps` timed ones between a barrier + synchronize on both
    sides, timed with CUDA events on the launching stream. Returns milliseconds for all steps."""
    for i in range(warmup):
        fn(i)
    sync()
    barrier()
    sync()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        fn(warmup + i)
    stop.record()
    sync()
    barrier()
    sync()
    return start.elapsed_time(stop)


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


# ------------------------------------------------------------------------------------------ CPU arm

def cpu_problem(ncols, seed=1):
    """Config 2 cut into slices of `ncols` output columns, built with torch only (the CPU arm must not
    touch the product library): signed int4 weights, bf16 scales / zeros, pre-quant scale 1. All
    14336 columns exist, so that consecutive steps read different weights, as the GPU arm's do."""
    g = torch.Generator().manual_seed(seed)
    k = C2["k"]
    slices = []
    for _ in range(C2["n"] // ncols):
        q = torch.randint(-8, 8, (k, ncols), dtype=torch.int8, generator=g)
        s = (torch.rand((k // 128, ncols), generator=g) * 0.019 + 0.001).to(torch.bfloat16)
        z = (torch.rand((k // 128, ncols), generator=g) * 0.2 - 0.1).to(torch.bfloat16)
        slices.append((q, s, z))
    act = torch.randn((1, k), generator=g).to(torch.bfloat16)
    ps = torch.ones(k, dtype=torch.bfloat16)
    return slices, act, ps


def cpu_step_fn(ncols):
    """One step of the reference's CPU definition of the path (its tests' ground truth,
    tests/quantization/test_weight_only_groupwise_quant_matmul.py:223-244 of the reference): dequantise
    the signed integers with the group scales and zeros in bf16, apply the pre-quant scale, matmul.
    The weights arrive as signed integers, as they do in the reference's test (the layout transform is
    an offline step and is not part of the timed region)."""
    from oracle import woq_oracle as oracle
    slices, act, ps = cpu_problem(ncols)
    torch.set_num_threads(os.cpu_count() or 1)
    counter = [0]

    def step():
        q, s, z = slices[counter[0] % len(slices)]
        counter[0] += 1
        return oracle.groupwise_matmul_test_ref(act, q, s, z, None, ps, 128)

    return step, algorithmic_bytes(1, ncols, C2["k"], 4, 128, True, True)


def run_reference(args):
    """The reference's CPU definition of the path on the host cores (rank 0 only; other ranks exit)."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    step, nbytes = cpu_step_fn(REF_SAMPLE_COLS)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    sec = (time.perf_counter() - t0) / args.steps
    gbs = nbytes / sec / 1e9
    cores = torch.get_num_threads()
    sample = (f"{REF_SAMPLE_COLS} of the 14336 output columns per step, a different slice every step (dequantise + "
              f"matmul with torch on {cores} host threads); GB/s = algorithmic bytes of the slice / time")
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit_line(line)


# ------------------------------------------------------------------------------------------ GPU arm

def run_ours(args):
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    import tensorrt_llm_b200 as pkg
    import tensorrt_llm_b200.torch_ops  # noqa: F401  (C++ torch.ops.trtllm registrations)

    use_dist = world > 1
    if use_dist:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if use_dist:
            dist.barrier()

    def max_over_ranks(x):
        if not use_dist:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sync = torch.cuda.synchronize
    peaks = measured_peaks()
    m = 1
    set_bytes = algorithmic_bytes(m, C2["n"], C2["k"], 4, 128, True, True)
    copies = copies_for(set_bytes)
    prob = Problem(device, 16, C2["n"], C2["k"], 4, 128, torch.bfloat16, zeros=True, prequant=True, seed=1,
                   copies=copies, ps_ones=True)
    parity = {}
    for mm in (1, 16):
        fn, out = prob.launcher(mm)
        fn(0)
        sync()
        parity[f"m{mm}"] = prob.parity(out, mm)
        if parity[f"m{mm}"] > 1e-2:
            raise SystemExit(f"parity FAILED for decode M={mm}: {parity[f'm{mm}']} of max|ref| > 1e-2")

    # ---- device-resident metric: exactly K steps in one graph replay
    stream = torch.cuda.Stream(device)
    fn, out = prob.launcher(m)
    with torch.cuda.stream(stream):
        for i in range(max(args.warmup, 3)):
            fn(i)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(args.steps):
                fn(i)
        graph.replay()  # one untimed replay
        stream.synchronize()
        barrier()
        sync()
        clocks = ClockSampler(local)
        with clocks:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            graph.replay()
            e1.record(stream)
            stream.synchronize()
        barrier()
        sync()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_step = ms_total / args.steps
    gbs_rank = set_bytes / (ms_step * 1e-3) / 1e9
    del graph

    # ---- end to end with host buffers: every step takes the activations from pinned host memory and
    # leaves the result in pinned host memory, synchronised. Through the C ABI's host entry point
    # (w4_gemm_run_host: copy in, GEMM, copy out, synchronise in one call) and, for comparison, through
    # the torch op with the copies made by torch around it.
    h_act = prob.act[:m].cpu().contiguous().pin_memory()
    h_out = torch.empty((m, C2["n"]), dtype=torch.bfloat16).pin_memory()
    d_act = torch.empty((m, C2["k"]), dtype=torch.bfloat16, device=device)
    d_out = torch.empty((m, C2["n"]), dtype=torch.bfloat16, device=device)
    algo = pkg.ZERO | pkg.PRE_QUANT_SCALE
    op = torch.ops.trtllm.weight_only_groupwise_quant_gemm
    cur = torch.cuda.current_stream()
    prepared = [pkg.ops.PreparedGemm(d_act, w, s, d_out, n=C2["n"], k=C2["k"], weight_bits=4, group_size=128, zeros=z,
                                     act_scale=prob.ps, regime=pkg.W4_REGIME_GEMV, weights_static=True)
                for (w, s, z) in prob.sets]
    cur_handle = cur.cuda_stream

    def e2e_step(i):
        prepared[i % len(prepared)].run_host(h_act, h_out, cur_handle)

    def e2e_torch_step(i):
        w, s, z = prob.sets[i % len(prob.sets)]
        d_act.copy_(h_act, non_blocking=True)
        y = op(d_act, prob.ps, w, s, z, None, 1.0, algo, 128, True)
        h_out.copy_(y, non_blocking=True)
        cur.synchronize()

    e2e_steps = min(args.steps, 2000)
    h_out.zero_()
    e2e_step(0)
    parity["e2e_host_m1"] = prob.parity(h_out, m)
    if parity["e2e_host_m1"] > 1e-2:
        raise SystemExit(f"parity FAILED for the host entry point: {parity['e2e_host_m1']} of max|ref| > 1e-2")
    e2e_ms = max_over_ranks(time_steps(e2e_step, e2e_steps, max(args.warmup, 3), sync, barrier)) / e2e_steps
    e2e_gbs = set_bytes / (e2e_ms * 1e-3) / 1e9
    e2e_torch_ms = max_over_ranks(time_steps(e2e_torch_step, e2e_steps, max(args.warmup, 3), sync, barrier)) / e2e_steps

    line = {
        "metric": METRIC, "value": gbs_rank * world, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "replicas": "one replica per GPU, no collective on the data path",
                   "l2": f"each step reads a different one of {copies} weight sets "
                         f"({copies * set_bytes / 2**20:.0f} MiB > 2 x 126 MiB L2)",
                   "timing": "K steps captured in one CUDA graph, CUDA events on its stream, max over ranks",
                   "weights_static": "W4_GEMM_WEIGHTS_STATIC set (inference weights: written once at load time)",
                   "algorithmic_bytes_per_step": set_bytes},
        "e2e": {"value": e2e_gbs * world, "unit": "GB/s", "h2d_bytes_per_step": m * C2["k"] * 2,
                "d2h_bytes_per_step": m * C2["n"] * 2, "ms_per_step": e2e_ms, "steps": e2e_steps,
                "api": "w4_gemm_run_host (C ABI: pinned host activations in, pinned host result out, synchronised)",
                "torch_op_ms_per_step": e2e_torch_ms,
                "torch_op_api": "torch.ops.trtllm.weight_only_groupwise_quant_gemm (C++ registration) with "
                                "torch copies from / to pinned host memory around it"},
        "gpu_launches": args.steps,
        "roofline": {"bound": "hbm", "achieved": gbs_rank, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs_rank / peaks["hbm_gbs"], "frac_of_8TBs": gbs_rank / 8000.0,
                     "peak_source": peaks["source"], "kernel": "w4::gemv::gemv_kernel<bf16, int4, MB=1, zero, act_scale, folded>",
                     "traffic": captured_traffic("gemv_c2_m1")},
        "clocks": clocks.summary(),
        "parity_err_frac_of_max": parity,
    }

    if rank == 0 and world == 1:
        line["points"] = extra_points(pkg, prob, device, peaks, stream)
        if not args.no_sweep:
            line["sweep"] = sweep(pkg, device, peaks, stream)
        step, nbytes = cpu_step_fn(REF_SAMPLE_COLS)
        for _ in range(3):
            step()
        t0, n_cpu = time.perf_counter(), 0
        while time.perf_counter() - t0 < 10.0:
            step()
            n_cpu += 1
        total = time.perf_counter() - t0
        sec = total / n_cpu
        line["cpu_baseline"] = {"value": nbytes / sec / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(),
                                "kind": "port", "ms": sec * 1e3,
                                "sample": f"{REF_SAMPLE_COLS} of the 14336 output columns of config 2 at M=1 per pass, a "
                                          f"different slice every pass (dequantise + matmul with torch), mean of "
                                          f"{n_cpu} passes ({total:.0f} s of CPU work)"}
    if world > 1:
        line["tp_llama70b"] = tp_layer_set(pkg, device, rank, world, barrier, max_over_ranks)
    if rank == 0:
        emit_line(line)
    if use_dist:
        dist.destroy_process_group()


def roofline_of(us, nbytes, flops, peaks):
    """Fraction of the bound that applies: the larger of the time at the measured HBM copy rate and
    the time at the measured burst bf16 tensor rate, over the measured time."""
    t_hbm = nbytes / (peaks["hbm_gbs"] * 1e3)        # us
    t_tc = flops / (peaks["bf16_tflops"] * 1e6)      # us
    bound = "hbm" if t_hbm >= t_tc else "tensor"
    return bound, max(t_hbm, t_tc) / us


def extra_points(pkg, prob, device, peaks, stream):
    """Per-M decode points of config 2, config 1, the prefill GEMM of config 3 (single GPU)."""
    points = {}
    for mm in (1, 2, 4, 8, 16):
        fn, _ = prob.launcher(mm)
        us = time_graph(fn, 300, stream)
        nbytes = algorithmic_bytes(mm, C2["n"], C2["k"], 4, 128, True, True)
        gbs = nbytes / us / 1e3
        points[f"c2_m{mm}"] = {"us": us, "GB/s": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                               "frac_of_8TBs": gbs / 8000.0,
                               "regime": "gemv" if pkg.ops.select_regime(mm, C2["n"], C2["k"], 128, 4) == 1 else "gemm"}
    # the same step with the early weight fetch fenced (flag off): what a caller pays who cannot
    # promise static weights
    fn, _ = prob.launcher(1, weights_static=False)
    points["c2_m1_weights_not_static"] = {"us": time_graph(fn, 300, stream)}
    points["c1_w8a16_m16"] = c1_point(pkg, device, peaks, stream)
    points["c3_m4096"] = prefill_point(pkg, device, peaks, prequant=False)
    points["c3_m4096_prequant"] = prefill_point(pkg, device, peaks, prequant=True)
    points["prep_c2"] = prep_point(pkg, device, peaks)
    points["splitk_m64_k8192_n1280"] = splitk_point(pkg, device)
    return points


def c1_point(pkg, device, peaks, stream):
    """BASELINE config 1: W8A16 per-channel, fp16, M=16, K=4096, N=4096: weights ~N(0, 0.02)
    quantised by the library's device-side symmetric quantiser (byte-identical to the host op)."""
    from oracle import woq_oracle as oracle
    from tensorrt_llm_b200 import ops, quantize
    m, k, n = 16, 4096, 4096
    g = torch.Generator(device=device).manual_seed(0)
    nbytes = algorithmic_bytes(m, n, k, 8, 0, False, False)
    sets = []
    for _ in range(copies_for(nbytes)):
        w = (torch.randn((k, n), device=device, generator=g) * 0.02).to(torch.float16)
        sets.append(quantize.symmetric_quantize_last_axis_of_batched_matrix_cuda(w, torch.int8,
                                                                                return_unprocessed=len(sets) == 0))
    unprocessed, p0, s0 = sets[0]
    sets[0] = [p0, s0]
    act = torch.randn((m, k), device=device, generator=g).to(torch.float16)
    out = torch.empty((m, n), dtype=torch.float16, device=device)
    nb = ops.workspace_bytes(m, n, k, 0, 8, torch.float16, False)
    ws = torch.empty(nb, dtype=torch.uint8, device=device) if nb else None

    def fn(i):
        p, s = sets[i % len(sets)]
        ops.gemm_raw(act, p, s, out, n=n, k=k, weight_bits=8, group_size=0, workspace=ws, weights_static=True)

    fn(0)
    torch.cuda.synchronize()
    ref = oracle.kernel_rounding_ref(act.cpu(), unprocessed.cpu(), s0.cpu(), group_size=0)
    err = float((out.cpu().double() - ref.double()).abs().max()) / float(ref.double().abs().max())
    if err > 1e-2:
        raise SystemExit(f"parity FAILED for config 1: {err}")
    us = time_graph(fn, 200, stream)
    gbs = nbytes / us / 1e3
    return {"us": us, "GB/s": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "frac_of_8TBs": gbs / 8000.0,
            "regime": "gemv" if ops.select_regime(m, n, k, 0, 8) == 1 else "gemm", "parity_err_frac_of_max": err}


def sweep(pkg, device, peaks, stream):
    """BASELINE config 5: every distinct Llama-3-8B linear shape x {W8 per-channel, W4 g64, W4 g128} x
    {fp16, bf16} x M = 1 .. 8192, AUTO regime, graph-timed, weights rotated over sets larger than twice
    the L2. Groupwise formats carry zeros and a pre-quant scale (the AWQ layout), per-channel has
    neither. Around the regime switch (M = 16 .. 256) the other regime is timed too; points where AUTO
    was not the faster one are listed under "auto_not_fastest"."""
    cols = ["shape", "K", "N", "format", "dtype", "M", "regime", "us", "GB/s", "TFLOP/s", "bound", "frac", "parity_ok"]
    rows, slower = [], []
    t_start = time.perf_counter()
    for name, k, n in SWEEP_SHAPES:
        for fmt, bits, group in SWEEP_FORMATS:
            for dtype in (torch.float16, torch.bfloat16):
                grouped = group != 0
                wbytes = k * n * bits // 8
                prob = Problem(device, max(SWEEP_MS), n, k, bits, group, dtype, zeros=grouped, prequant=grouped,
                               seed=k // 512 + n // 512 + bits + group, copies=copies_for(wbytes))
                for m in SWEEP_MS:
                    regime = pkg.ops.select_regime(m, n, k, group, bits, dtype)
                    fn, out = prob.launcher(m)
                    fn(0)
                    torch.cuda.synchronize()
                    ok = prob.parity(out, m, seed=m) <= 1e-2
                    nbytes = algorithmic_bytes(m, n, k, bits, group, grouped, grouped)
                    flops = 2.0 * m * n * k
                    est_us = max(nbytes / 3e6, flops / 1e9)  # rough: 3 TB/s, 1 PFLOP/s
                    reps = int(max(4, min(60, 3000 / max(est_us, 1))))
                    us = time_graph(fn, reps, stream)
                    bound, frac = roofline_of(us, nbytes, flops, peaks)
                    rows.append([name, k, n, fmt, str(dtype)[6:], m, "gemv" if regime == 1 else "gemm", round(us, 2),
                                 round(nbytes / us / 1e3, 1), round(flops / us / 1e6, 2), bound, round(frac, 3), ok])
                    if 16 <= m <= 256:
                        other = 2 if regime == 1 else 1
                        fn2, _ = prob.launcher(m, regime=other)
                        us2 = time_graph(fn2, reps, stream)
                        if us2 < 0.97 * us:
                            slower.append({"shape": name, "format": fmt, "dtype": str(dtype)[6:], "M": m,
                                           "auto": "gemv" if regime == 1 else "gemm", "auto_us": round(us, 2),
                                           "other_us": round(us2, 2)})
                del prob
                torch.cuda.empty_cache()
    return {"columns": cols, "rows": rows, "auto_not_fastest": slower,
            "parity_all_ok": all(r[-1] for r in rows), "seconds": round(time.perf_counter() - t_start, 1),
            "note": "frac = time at the measured peak of the bound that applies (HBM copy rate or burst bf16 tensor "
                    "rate, whichever gives the longer time) / measured time"}


def prep_point(pkg, device, peaks):
    """GPU-side weight preparation of a config-2 matrix (K=4096, N=14336): layout only (int4) and
    quantise + layout from bf16, checked byte for byte against the host path, timed beside it."""
    from tensorrt_llm_b200 import quantize as Q
    k, n = C2["k"], C2["n"]
    g = torch.Generator().manual_seed(7)
    raw = torch.randint(-128, 128, (k, n // 2), dtype=torch.int8, generator=g)
    t0 = time.perf_counter()
    ref = Q.preprocess_weights_for_mixed_gemm(raw, torch.quint4x2)
    cpu_ms = (time.perf_counter() - t0) * 1e3
    raw_d = raw.to(device)
    out = Q.preprocess_weights_for_mixed_gemm_cuda(raw_d, torch.quint4x2)
    if not torch.equal(out.cpu(), ref):
        raise SystemExit("parity FAILED for the GPU layout kernel")
    w = (torch.randn(k, n, generator=g) * 0.02).to(torch.bfloat16)
    t0 = time.perf_counter()
    p_ref, s_ref = Q.symmetric_quantize_last_axis_of_batched_matrix(w, torch.quint4x2)
    cpu_q_ms = (time.perf_counter() - t0) * 1e3
    w_d = w.to(device)
    p_gpu, s_gpu = Q.symmetric_quantize_last_axis_of_batched_matrix_cuda(w_d, torch.quint4x2)
    if not (torch.equal(p_gpu.cpu(), p_ref) and torch.equal(s_gpu.cpu(), s_ref)):
        raise SystemExit("parity FAILED for the GPU quantise kernel")

    def timed(fn, reps=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    us_l = timed(lambda: Q.preprocess_weights_for_mixed_gemm_cuda(raw_d, torch.quint4x2))
    us_q = timed(lambda: Q.symmetric_quantize_last_axis_of_batched_matrix_cuda(w_d, torch.quint4x2))
    bytes_l = 2 * k * n // 2                      # read + write the packed matrix
    bytes_q = 2 * k * n * 2 + k * n // 2          # two passes over the bf16 matrix (amax, quantise) + write
    return {"layout_us": us_l, "layout_GB/s": bytes_l / us_l / 1e3,
            "layout_frac_of_measured_hbm": bytes_l / us_l / 1e3 / peaks["hbm_gbs"],
            "layout_cpu_ms_host_threads": cpu_ms,
            "quantize_us": us_q, "quantize_GB/s": bytes_q / us_q / 1e3,
            "quantize_frac_of_measured_hbm": bytes_q / us_q / 1e3 / peaks["hbm_gbs"],
            "quantize_cpu_ms_host_threads": cpu_q_ms, "includes": "output allocation by the torch wrapper"}


def splitk_point(pkg, device):
    """A few-tile tensor-core shape (Llama-3-70B qkv shard at tp=8, M=64) with and without the
    optional split-k workspace, graph-timed."""
    from tensorrt_llm_b200 import ops
    m, n, k = 64, 1280, 8192
    w = torch.randint(0, 256, (k, n // 2), dtype=torch.uint8, device=device).view(torch.int8)
    s = (torch.rand(k // 128, n, device=device) * 0.019 + 0.001).to(torch.bfloat16)
    act = torch.randn(m, k, device=device).to(torch.bfloat16)
    out = torch.empty(m, n, dtype=torch.bfloat16, device=device)
    res = {}
    for label, nb in (("unsplit_us", 0), ("split_us", ops.workspace_bytes(m, n, k, 128, 4, torch.bfloat16, False,
                                                                           pkg.W4_REGIME_GEMM))):
        ws = torch.empty(nb, dtype=torch.uint8, device=device) if nb else None
        st = torch.cuda.Stream(device=device)
        fn = lambda _i=0: ops.gemm_raw(act, w, s, out, n=n, k=k, weight_bits=4, group_size=128,  # noqa: E731
                                       regime=pkg.W4_REGIME_GEMM, workspace=ws)
        res[label] = time_graph(fn, 50, st, replays=1)
    res["workspace_bytes"] = int(nb)
    return res


def prefill_point(pkg, device, peaks, prequant):
    """BASELINE config 3: M=4096, K=14336, N=4096, int4 g128 with zeros, bf16 (tensor-core regime);
    optionally with an AWQ pre-quant scale, which the tensor-core path applies in a separate pass."""
    if pkg.ops.select_regime(C3["m"], C3["n"], C3["k"], 128, 4) != pkg.W4_REGIME_GEMM:
        return None
    prob = Problem(device, C3["m"], C3["n"], C3["k"], 4, 128, torch.bfloat16, zeros=True, prequant=prequant, seed=2)
    fn, out = prob.launcher(C3["m"], regime=pkg.W4_REGIME_GEMM)
    try:
        fn(0)
    except pkg.W4Error as e:
        return {"unavailable": str(e)}
    torch.cuda.synchronize()
    err = prob.parity(out, C3["m"], seed=3)  # sampled rows (tile boundaries included) and columns
    if err > 1e-2:
        raise SystemExit(f"parity FAILED for prefill config 3: {err}")
    for _ in range(3):
        fn(0)
    torch.cuda.synchronize()
    reps = 20
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn(0)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    tflops = 2.0 * C3["m"] * C3["n"] * C3["k"] / (ms * 1e-3) / 1e12
    return {"ms": ms, "TFLOP/s": tflops, "frac_of_measured_bf16_sustained": tflops / peaks["bf16_tflops_sustained"],
            "frac_of_measured_bf16_burst": tflops / peaks["bf16_tflops"], "frac_of_2250_dense_spec": tflops / 2250.0,
            "parity_err_frac_of_max": err}


# ------------------------------------------------------------------------------------------ tensor parallel

def tp_layer_set(pkg, device, rank, world, barrier, max_over_ranks, ms=(1, 64, 2048), reps=20, group_size=128):
    """Every linear of one Llama-3-70B layer (BASELINE config 4) at tp = world size: W4A16 group-128
    with zeros, bf16, each rank's shard generated from its own seed. Column-parallel layers: the local
    GEMM only (checked against the oracle on sampled rows / columns). Row-parallel layers: local GEMM,
    then the all-reduce of the [M, 8192] partial sums - NCCL and the library's peer-memory kernel - both
    CHECKED before timing against the fp32 sum, in rank order, of the gathered partials (bit-exact for
    the peer kernel, a few bf16 ulps for NCCL). Timings: CUDA events with an L2 flush between
    repetitions (max over ranks), and the GEMM + reduce step as one CUDA graph of back-to-back steps."""
    import torch.distributed as dist
    from tensorrt_llm_b200 import ops, tp

    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)
    out = {}
    peer, peer_err = None, None
    try:
        peer = tp.PeerAllReduce(None, device, torch.bfloat16, max_bytes=max(ms) * 8192 * 2)
    except Exception as e:  # symmetric memory not available on this box: NCCL only, and say so
        peer_err = f"{type(e).__name__}: {e}"[:200]
    for name, K, N, kind in LLAMA70B_LAYERS:
        k_loc, n_loc = (K, N // world) if kind == "column" else (K // world, N)
        prob = Problem(device, max(ms), n_loc, k_loc, 4, group_size, torch.bfloat16, zeros=True, prequant=False,
                       seed=3 + rank + 17 * len(name))
        w, s, z = prob.sets[0]
        for m in ms:
            x = prob.act[:m].contiguous()
            y = torch.empty((m, n_loc), dtype=torch.bfloat16, device=device)
            ws_bytes = ops.workspace_bytes(m, n_loc, k_loc, group_size, 4, torch.bfloat16, False)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device) if ws_bytes else None

            def gemm(dst=y):
                ops.gemm_raw(x, w, s, dst, n=n_loc, k=k_loc, weight_bits=4, group_size=group_size, zeros=z,
                             workspace=ws, weights_static=True)

            entry = {"kind": kind, "k_local": k_loc, "n_local": n_loc,
                     "regime": "gemv" if ops.select_regime(m, n_loc, k_loc, group_size, 4) == 1 else "gemm"}
            # ---- parity first
            gemm()
            torch.cuda.synchronize()
            entry["parity_gemm_err_frac_of_max"] = max_over_ranks(prob.parity(y, m, seed=m))
            use_peer = kind == "row" and peer is not None and peer.fits(m * n_loc * 2)
            if kind == "row":
                parts = [torch.empty_like(y) for _ in range(world)]
                dist.all_gather(parts, y)
                acc = torch.zeros_like(y, dtype=torch.float32)
                for p_ in parts:
                    acc += p_.float()
                expect = acc.to(torch.bfloat16)
                del parts, acc
                y_nccl = y.clone()
                dist.all_reduce(y_nccl, op=dist.ReduceOp.SUM)
                scale = float(expect.float().abs().max())
                entry["parity_nccl_err_frac_of_max"] = max_over_ranks(
                    float((y_nccl.float() - expect.float()).abs().max()) / scale)
                if use_peer:
                    y_peer = torch.empty_like(y)
                    gemm(peer.partial(m, n_loc))
                    peer.reduce(y_peer)
                    torch.cuda.synchronize()
                    entry["parity_peer_bit_exact"] = bool(max_over_ranks(0.0 if torch.equal(y_peer, expect) else 1.0) == 0.0)
                    # the fused form (decode sizes): the GEMM's epilogue pushes, the reduce only gathers
                    y_peer.zero_()
                    fused = ops.gemm_push(x, w, s, peer.partial(m, n_loc), peer.ptrs, peer.ws_bytes, peer.rank,
                                          n=n_loc, k=k_loc, group_size=group_size, zeros=z, weights_static=True,
                                          regime=pkg.W4_REGIME_AUTO)
                    if fused:
                        peer.reduce(y_peer, mode=pkg._lib.W4_ALLREDUCE_GATHER_ONLY)
                        torch.cuda.synchronize()
                        entry["parity_fused_bit_exact"] = bool(
                            max_over_ranks(0.0 if torch.equal(y_peer, expect) else 1.0) == 0.0)
                    entry["fused_applies"] = bool(fused)
                    if fused and m <= 16:
                        # the whole step as ONE kernel (GEMM, push, collect, add, write)
                        y_peer.zero_()
                        ops.gemm_allreduce(x, w, s, peer.partial(m, n_loc), y_peer, peer.ptrs, peer.ws_bytes, peer.rank,
                                           n=n_loc, k=k_loc, weight_bits=4, group_size=group_size, zeros=z,
                                           weights_static=True)
                        torch.cuda.synchronize()
                        entry["parity_one_kernel_bit_exact"] = bool(
                            max_over_ranks(0.0 if torch.equal(y_peer, expect) else 1.0) == 0.0)
                    del y_peer
                del y_nccl, expect
            entry["parity_ok"] = bool(entry["parity_gemm_err_frac_of_max"] <= 1e-2
                                      and entry.get("parity_nccl_err_frac_of_max", 0.0) <= 2e-2
                                      and entry.get("parity_peer_bit_exact", True)
                                      and entry.get("parity_fused_bit_exact", True)
                                      and entry.get("parity_one_kernel_bit_exact", True))
            # ---- eager timings with an L2 flush between repetitions
            t_gemm, t_ar = [], []
            for _ in range(reps):
                flush.zero_()
                barrier()
                e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
                e0.record()
                gemm()
                e1.record()
                if kind == "row":
                    dist.all_reduce(y, op=dist.ReduceOp.SUM)
                e2.record()
                torch.cuda.synchronize()
                t_gemm.append(e0.elapsed_time(e1))
                t_ar.append(e1.elapsed_time(e2))
            t_gemm.sort()
            t_ar.sort()
            gemm_us = max_over_ranks(t_gemm[len(t_gemm) // 2] * 1e3)
            nbytes = algorithmic_bytes(m, n_loc, k_loc, 4, group_size, True, False)
            flops = 2.0 * m * n_loc * k_loc
            entry.update({"gemm_us": gemm_us, "per_gpu_GB/s": nbytes / gemm_us / 1e3,
                          "per_gpu_TFLOP/s": flops / gemm_us / 1e6})
            # ---- the row-parallel step as a serving loop runs it: GEMM + reduce back to back in one
            # CUDA graph (weights L2-warm; the comparison of interest is the reduce)
            if kind == "row":
                entry["allreduce_bytes"] = m * n_loc * 2
                entry["nccl_allreduce_us"] = max_over_ranks(t_ar[len(t_ar) // 2] * 1e3)
                y2 = torch.empty_like(y)

                def step_nccl():
                    gemm()
                    dist.all_reduce(y, op=dist.ReduceOp.SUM)

                def step_peer():
                    gemm(peer.partial(m, n_loc))
                    peer.reduce(y2)

                def step_fused():
                    ops.gemm_push(x, w, s, peer.partial(m, n_loc), peer.ptrs, peer.ws_bytes, peer.rank, n=n_loc, k=k_loc,
                                  group_size=group_size, zeros=z, weights_static=True)
                    peer.reduce(y2, mode=pkg._lib.W4_ALLREDUCE_GATHER_ONLY)

                def step_one_kernel():
                    ops.gemm_allreduce(x, w, s, peer.partial(m, n_loc), y2, peer.ptrs, peer.ws_bytes, peer.rank, n=n_loc,
                                       k=k_loc, weight_bits=4, group_size=group_size, zeros=z, weights_static=True)

                steps = (("gemm_only", gemm), ("gemm_plus_nccl", step_nccl)) + (
                    (("gemm_plus_peer", step_peer),) if use_peer else ()) + (
                    (("gemm_plus_peer_fused", step_fused),) if use_peer and entry.get("fused_applies") else ()) + (
                    (("gemm_allreduce_one_kernel", step_one_kernel),)
                    if use_peer and "parity_one_kernel_bit_exact" in entry else ())
                for label, fn in steps:
                    try:
                        st = torch.cuda.Stream(device=device)
                        with torch.cuda.stream(st):
                            for _ in range(3):
                                fn()
                            st.synchronize()
                            barrier()
                            greps = reps * (5 if m <= 64 else 1)
                            graph = torch.cuda.CUDAGraph()
                            with torch.cuda.graph(graph, stream=st):
                                for _ in range(greps):
                                    fn()
                            graph.replay()
                            st.synchronize()
                            barrier()  # capture takes a different time on every rank: start together
                            e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(2))
                            e1.record(st)
                            graph.replay()
                            e2.record(st)
                            st.synchronize()
                        entry[f"graph_step_us_{label}"] = max_over_ranks(e1.elapsed_time(e2) * 1e3 / greps)
                        del graph
                    except Exception as e:  # capture not possible on this box: say so, keep going
                        entry[f"graph_step_us_{label}"] = f"unavailable: {type(e).__name__}: {e}"[:160]
                        max_over_ranks(0.0)
                if not use_peer:
                    entry["graph_step_us_gemm_plus_peer"] = peer_err or "message larger than the peer workspace"
            out[f"{name}_m{m}"] = entry
        del prob
        torch.cuda.empty_cache()
    del flush
    return out


_REAL_STDOUT = None


def emit_line(line):
    data = (json.dumps(line) + "\n").encode()
    if _REAL_STDOUT is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_REAL_STDOUT, data)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-sweep", action="store_true", help="skip the config-5 sweep (about half a minute)")
    args = ap.parse_args()
    args.steps = max(1, min(args.steps, 20000))
    args.warmup = max(0, args.warmup)
    # Libraries print on stdout (NCCL its version line, for one): everything but the one JSON line goes
    # to stderr. emit_line() writes to the real stdout.
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
