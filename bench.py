#!/usr/bin/env python
"""Benchmark of the weight-only quantised GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the hot path over one batch: the W4A16 group-128 AWQ decode GEMM of
BASELINE config 2 (bf16 activations [M=1, K=4096], int4 weights [4096, 14336] with bf16 scales and
zeros per 128 rows, pre-quant scale; the Llama-3-8B gate/up projection). The headline metric is the
HBM bandwidth the step sustains: algorithmic bytes / time. Inputs are synthetic and seeded. Each
step reads a different copy of the weights (a ring of copies larger than twice the L2) so that
every step streams from HBM.

With N > 1 (launched under torchrun) every rank runs the same step on its own GPU (independent
replicas, no collective on the data path: "weak" scaling) and the value is the sum over ranks;
the tensor-parallel Llama-3-70B layer set (column-parallel without communication, row-parallel
with an NCCL all-reduce) is timed in the same run and reported under "tp_llama70b".

The JSON line also carries: "e2e" (same metric through the public op with host buffers: the
activations are copied from pinned host memory and the result read back inside the timed region;
weights stay resident in HBM as they do in serving), "roofline" (achieved / measured HBM copy
bandwidth), "cpu_baseline" (the CPU oracle timed on the host cores), "points" (every M of config 2
and the prefill GEMM of config 3) and "clocks" (NVML samples taken during the timed region).

--impl reference times the reference's CPU definition of the path (dequantise then matmul with
torch on all host cores) on the same workload.
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
sys.path.insert(0, os.path.join(ROOT, "tests"))

import torch  # noqa: E402

L2_BYTES = 126 * 1024 * 1024
METRIC = "W4A16 g128 AWQ decode GEMM (M=1, K=4096, N=14336, bf16): HBM GB/s"
C2 = dict(n=14336, k=4096, group=128, bits=4)
C3 = dict(m=4096, n=4096, k=14336, group=128, bits=4)


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


# ------------------------------------------------------------------------------------------ workloads

def make_decode_sets(device, m, copies, seed):
    """`copies` independent weight/scale/zero sets of config 2 on the device, plus activations.
    Set 0 goes through the real host path (pack + layout transform) so it can be checked against
    the oracle; the others are random bytes, which is what the layout of random nibbles is."""
    from _cases import make_problem

    p = make_problem(m, C2["n"], C2["k"], 4, 128, torch.bfloat16, zero=True, prequant=True, seed=seed)
    p["ps"] = torch.ones(C2["k"], dtype=torch.bfloat16)  # config 2: pre-quant scale 1
    g = torch.Generator(device=device).manual_seed(seed + 100)
    sets = []
    for c in range(copies):
        if c == 0:
            w, s, z = p["processed"].to(device), p["scales"].to(device), p["zeros"].to(device)
        else:
            w = torch.randint(0, 256, p["processed"].shape, dtype=torch.uint8, device=device,
                              generator=g).view(torch.int8)
            s = (torch.rand(p["scales"].shape, device=device, generator=g) * 0.019 + 0.001).to(torch.bfloat16)
            z = (torch.rand(p["zeros"].shape, device=device, generator=g) * 0.2 - 0.1).to(torch.bfloat16)
        sets.append((w, s, z))
    return p, sets


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


def decode_runner(pkg, p, sets, m, device):
    """Returns fn(i) launching one decode GEMM on weight set i % len(sets), and the output buffer."""
    from tensorrt_llm_b200 import ops

    act = p["act"][:m].contiguous().to(device)
    ps = p["ps"].to(device)
    out = torch.empty((m, C2["n"]), dtype=torch.bfloat16, device=device)
    # the regime is chosen by the library; the tensor-core kernel wants scratch for the pre-quant scale
    ws_bytes = ops.workspace_bytes(m, C2["n"], C2["k"], 128, 4, torch.bfloat16, True)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device) if ws_bytes else None

    def fn(i):
        w, s, z = sets[i % len(sets)]
        ops.gemm_raw(act, w, s, out, n=C2["n"], k=C2["k"], weight_bits=4, group_size=128, zeros=z, act_scale=ps,
                     regime=pkg.W4_REGIME_AUTO, workspace=ws)

    return fn, out, act, ps


def check_decode_parity(pkg, p, sets, m, device):
    from _cases import max_err, oracle_out
    from oracle import woq_oracle as oracle

    fn, out, _, _ = decode_runner(pkg, p, sets, m, device)
    fn(0)
    torch.cuda.synchronize()
    q = dict(p, act=p["act"][:m].contiguous(), m=m)
    ref = oracle_out(q)
    err, tol = max_err(out.cpu(), ref), oracle.tolerance(ref)
    if err > tol:
        raise SystemExit(f"parity FAILED for decode M={m}: {err} > {tol}")
    return err / (tol * 100)


def cpu_oracle_decode(p, m, repeats):
    """The CPU definition of the path (dequantise to bf16, apply the pre-quant scale, matmul) with
    torch on all host cores; best of `repeats`. Returns (seconds, cores)."""
    from oracle import woq_oracle as oracle

    torch.set_num_threads(os.cpu_count() or 1)
    act = p["act"][:m].contiguous()
    best = float("inf")
    for _ in range(repeats + 1):  # first pass is a warm-up
        t0 = time.perf_counter()
        q = oracle.signed_weights(p["processed"], C2["k"], C2["n"], 4)
        oracle.groupwise_matmul_test_ref(act, q, p["scales"], p["zeros"], None, p["ps"], 128)
        best = min(best, time.perf_counter() - t0)
    return best, torch.get_num_threads()


def graph_of(fn, count, stream):
    """CUDA graph with `count` consecutive steps (the decode kernel lasts a few microseconds, so
    launching it from Python one call at a time would measure the interpreter, not the GPU)."""
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        for i in range(count):
            fn(i)
    return g


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def run_reference(args):
    """The reference's CPU definition of the path on the host cores (rank 0 only)."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from _cases import make_problem

    p = make_problem(1, C2["n"], C2["k"], 4, 128, torch.bfloat16, zero=True, prequant=True, seed=1)
    p["ps"] = torch.ones(C2["k"], dtype=torch.bfloat16)
    nbytes = algorithmic_bytes(1, C2["n"], C2["k"], 4, 128, True, True)
    from oracle import woq_oracle as oracle

    torch.set_num_threads(os.cpu_count() or 1)
    act = p["act"]

    def step():
        q = oracle.signed_weights(p["processed"], C2["k"], C2["n"], 4)
        return oracle.groupwise_matmul_test_ref(act, q, p["scales"], p["zeros"], None, p["ps"], 128)

    steps = max(1, min(args.steps, 5))  # bounded: each step is the whole config-2 problem on the CPU
    for _ in range(max(1, min(args.warmup, 2))):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    sec = (time.perf_counter() - t0) / steps
    gbs = nbytes / sec / 1e9
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": max(1, min(args.warmup, 2)), "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "BASELINE config 2: W4A16 g128 AWQ decode GEMM, M=1, K=4096, N=14336, bf16",
                   "note": "reference's CPU definition (unpack, dequantise, matmul with torch) on host cores; "
                           "steps capped at 5 because one step is the whole problem"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"full config-2 M=1 problem, mean of {steps} steps"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    import tensorrt_llm_b200 as pkg
    from tensorrt_llm_b200 import ops

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
    copies = max(2, (2 * L2_BYTES + set_bytes - 1) // set_bytes + 1)
    p, sets = make_decode_sets(device, 16, copies, seed=1)
    parity = {f"m{mm}": check_decode_parity(pkg, p, sets, mm, device) for mm in (1, 16)}

    # ---- device-resident metric: exactly K steps in one graph replay
    stream = torch.cuda.Stream(device)
    fn, out, act, ps = decode_runner(pkg, p, sets, m, device)
    with torch.cuda.stream(stream):
        for i in range(max(args.warmup, 3)):
            fn(i)
        stream.synchronize()
        graph = graph_of(fn, args.steps, stream)
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

    # ---- end to end through the public op: pinned host activations in, result out, every step
    h_act = p["act"][:m].contiguous().pin_memory()
    h_out = torch.empty((m, C2["n"]), dtype=torch.bfloat16).pin_memory()
    d_ps = ps
    algo = pkg.ZERO | pkg.PRE_QUANT_SCALE

    # End to end through the plugin-facing call (the mirror of the TensorRT plugin's enqueue:
    # caller-owned device inputs / outputs / workspace, as the TensorRT runtime hands them over):
    # every step copies the activations from pinned host memory, enqueues, reads the result back.
    plugin = pkg.WeightOnlyGroupwiseQuantMatmulPlugin(ops.TRT_BF16, algo, 128, 1.0)
    d_act = torch.empty((m, C2["k"]), dtype=torch.bfloat16, device=device)
    d_out = torch.empty((m, C2["n"]), dtype=torch.bfloat16, device=device)
    ws_n = ops.workspace_bytes(m, C2["n"], C2["k"], 128, 4, torch.bfloat16, True)
    d_ws = torch.empty(ws_n, dtype=torch.uint8, device=device) if ws_n else None

    def e2e_step(i):
        w, s, z = sets[i % len(sets)]
        d_act.copy_(h_act, non_blocking=True)
        rc = plugin.enqueue([d_act, d_ps, w, s, z], [d_out], d_ws)
        if rc != 0:
            raise SystemExit(f"plugin enqueue failed with status {rc}")
        h_out.copy_(d_out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_steps = min(args.steps, 2000)
    e2e_ms = max_over_ranks(time_steps(e2e_step, e2e_steps, max(args.warmup, 3), sync, barrier)) / e2e_steps
    e2e_gbs = set_bytes / (e2e_ms * 1e-3) / 1e9

    line = {
        "metric": METRIC, "value": gbs_rank * world, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "BASELINE config 2: W4A16 g128 AWQ decode GEMM (zeros + pre-quant scale), M=1, "
                               "K=4096, N=14336, bf16; one GEMM per step, one replica per GPU",
                   "l2": f"each step reads a different one of {copies} weight sets "
                         f"({copies * set_bytes / 2**20:.0f} MiB > 2 x 126 MiB L2)",
                   "timing": "K steps captured in one CUDA graph, CUDA events on its stream, max over ranks",
                   "algorithmic_bytes_per_step": set_bytes},
        "e2e": {"value": e2e_gbs * world, "unit": "GB/s", "h2d_bytes_per_step": m * C2["k"] * 2,
                "d2h_bytes_per_step": m * C2["n"] * 2, "ms_per_step": e2e_ms, "steps": e2e_steps},
        "gpu_launches": args.steps,
        "roofline": {"bound": "hbm", "achieved": gbs_rank, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs_rank / peaks["hbm_gbs"], "frac_of_8TBs": gbs_rank / 8000.0,
                     "peak_source": peaks["source"], "kernel": "w4::gemv::gemv_kernel<bf16,4,1,zero,act_scale>",
                     "traffic": captured_traffic("gemv_c2_m1")},
        "clocks": clocks.summary(),
        "parity_err_frac_of_max": parity,
    }

    if rank == 0 and world == 1:
        line["points"] = extra_points(pkg, p, sets, device, peaks, stream)
        sec, cores = cpu_oracle_decode(p, m, repeats=2)
        line["cpu_baseline"] = {"value": set_bytes / sec / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
                                "sample": "full config-2 M=1 problem (unpack, dequantise, matmul with torch), "
                                          "best of 2 after a warm-up", "ms": sec * 1e3}
    if world > 1:
        line["tp_llama70b"] = tp_layer_set(pkg, device, rank, world, barrier, max_over_ranks)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if use_dist:
        dist.destroy_process_group()


def extra_points(pkg, p, sets, device, peaks, stream):
    """Per-M decode points of config 2 and the prefill GEMM of config 3 (single GPU)."""
    points = {}
    with torch.cuda.stream(stream):
        for mm in (1, 2, 4, 8, 16):
            fn, _, _, _ = decode_runner(pkg, p, sets, mm, device)
            for i in range(3):
                fn(i)
            stream.synchronize()
            reps = 300
            g = graph_of(fn, reps, stream)
            g.replay()
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            g.replay()
            e1.record(stream)
            stream.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / reps
            nbytes = algorithmic_bytes(mm, C2["n"], C2["k"], 4, 128, True, True)
            gbs = nbytes / us / 1e3
            points[f"c2_m{mm}"] = {"us": us, "GB/s": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                                   "frac_of_8TBs": gbs / 8000.0}
    points["c3_m4096"] = prefill_point(pkg, device, peaks)
    points["prep_c2"] = prep_point(pkg, device, peaks)
    points["splitk_m64_k8192_n1280"] = splitk_point(pkg, device)
    return points


def prep_point(pkg, device, peaks):
    """GPU-side weight preparation of a config-2 matrix (K=4096, N=14336): layout only (int4) and
    quantise + layout from bf16, checked byte for byte against the host path, timed beside it."""
    import time

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
        with torch.cuda.stream(st):
            fn = lambda _i=0: ops.gemm_raw(act, w, s, out, n=n, k=k, weight_bits=4, group_size=128,  # noqa: E731
                                           regime=pkg.W4_REGIME_GEMM, workspace=ws)
            for _ in range(3):
                fn()
            st.synchronize()
            g = graph_of(fn, 50, st)
            g.replay()
            st.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            g.replay()
            e1.record(st)
            st.synchronize()
        res[label] = e0.elapsed_time(e1) * 1e3 / 50
    res["workspace_bytes"] = int(nb)
    return res


def prefill_point(pkg, device, peaks):
    """BASELINE config 3: M=4096, K=14336, N=4096, int4 g128 with zeros, bf16 (tensor-core regime)."""
    from _cases import make_problem, max_err, oracle_out
    from oracle import woq_oracle as oracle
    from tensorrt_llm_b200 import ops

    if pkg.ops.select_regime(C3["m"], C3["n"], C3["k"], 128, 4) != pkg.W4_REGIME_GEMM:
        return None
    p = make_problem(C3["m"], C3["n"], C3["k"], 4, 128, torch.bfloat16, zero=True, seed=2)
    act, w, s, z = (p[x].to(device) for x in ("act", "processed", "scales", "zeros"))
    out = torch.empty((C3["m"], C3["n"]), dtype=torch.bfloat16, device=device)

    def fn():
        ops.gemm_raw(act, w, s, out, n=C3["n"], k=C3["k"], weight_bits=4, group_size=128, zeros=z,
                     regime=pkg.W4_REGIME_GEMM)

    try:
        fn()
    except pkg.W4Error as e:
        return {"unavailable": str(e)}
    torch.cuda.synchronize()
    # parity on a sample of rows (the float64 oracle for all 4096 rows would take minutes on the host)
    rows = torch.arange(0, C3["m"], 61)
    q = dict(p, act=p["act"][rows].contiguous(), m=len(rows))
    ref = oracle_out(q)
    err, tol = max_err(out.cpu()[rows], ref), oracle.tolerance(ref)
    if err > tol:
        raise SystemExit(f"parity FAILED for prefill config 3: {err} > {tol}")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    reps = 20
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    tflops = 2.0 * C3["m"] * C3["n"] * C3["k"] / (ms * 1e-3) / 1e12
    return {"ms": ms, "TFLOP/s": tflops, "frac_of_measured_bf16_sustained": tflops / peaks["bf16_tflops_sustained"],
            "frac_of_measured_bf16_burst": tflops / peaks["bf16_tflops"], "frac_of_2250_dense_spec": tflops / 2250.0,
            "parity_err_frac_of_max": err / (tol * 100)}


def tp_layer_set(pkg, device, rank, world, barrier, max_over_ranks):
    """Tensor-parallel Llama-3-70B linear set (BASELINE config 4) at tp = world size."""
    try:
        from tensorrt_llm_b200 import tp
    except ImportError:
        return None
    return tp.bench_llama70b_layer_set(device, rank, world, barrier, max_over_ranks)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    args.steps = max(1, min(args.steps, 20000))
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
