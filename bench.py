#!/usr/bin/env python
"""Benchmark of the fused transformer-inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (N=1): the isolated fused-attention op of the baseline's second config —
fp16 Q/K/V [8, 12, 512, 64] ~ N(0,1), non-causal, per-sequence random padding mask (valid length
uniform in [64, 512]), sm_scale = 1/8. One "step" = one attention forward over that batch.
Metric: fused attention TFLOP/s with the algorithmic flop count 4·B·H·M·N·D (padding is additive
data and is not discounted).

Timing: K back-to-back steps bracketed by one CUDA-event pair on the launching stream. The steps
cycle through 10 independent input sets (252 MB in total, twice the 126 MB L2), so every step finds
its Q/K/V cold without a flush inside the timed region, and they are enqueued as CUDA-graph replays
(the reference's own production mode) so that host launch latency is not part of the number.
ms_per_step = elapsed / K; with N GPUs each rank runs the same per-GPU batch (independent replicas,
no collective in the data path), the ranks are bracketed by barrier + synchronize, and the slowest
rank's time is used.

Extra objects on the JSON line: `roofline` (tensor-pipe bound of the attention kernel, against the
measured cuBLAS bf16 peak), `cpu_baseline` (the CPU oracle — a restatement of the reference's eager
attention — timed on this box's host cores), `e2e` (the same op through the public Python API with
pinned host buffers: H2D of q/k/v/mask + kernel + D2H of the output inside the timed region),
`ops` (fused linear and norm kernels against their own rooflines) and `clocks`.

`--impl reference` times the reference's CPU implementation of the same op (its eager
`attention_reference`, restated by the oracle) on the host cores with all threads.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = {"B": 8, "H": 12, "S": 512, "D": 64}
WORKLOAD_NAME = ("attention fwd [batch 8, heads 12, seq 512, head_dim 64], per-sequence padding mask, "
                 "non-causal, sm_scale 1/8 (baseline config 2)")
TRAFFIC_PROFILE = os.path.join("profiles", "attention_persist_d64_config2_padmask.md")
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            p = json.load(open(path))
            return {k: float(p[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def make_inputs(seed=0):
    """Seeded CPU fp32 inputs of the headline workload, so the CPU baseline and the GPU see the
    same values."""
    import torch

    B, H, S, D = (WORKLOAD[k] for k in "BHSD")
    g = torch.Generator().manual_seed(seed)
    q = torch.randn((B, H, S, D), generator=g)
    k = torch.randn((B, H, S, D), generator=g)
    v = torch.randn((B, H, S, D), generator=g)
    valid = torch.randint(64, S + 1, (B,), generator=g)
    mask = torch.where(valid[:, None] > torch.arange(S)[None, :], 0.0, float("-inf")).reshape(B, 1, 1, S)
    return q, k, v, mask


def attention_flops():
    B, H, S, D = (WORKLOAD[k] for k in "BHSD")
    return 4.0 * B * H * S * S * D


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = [s for (t, s) in self.samples if t0 - 0.05 <= t <= t1 + 0.15] or [s for (_, s) in self.samples]
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            parts = [x.strip() for x in r.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(mhz)}


def time_cpu_attention(steps, warmup):
    """The reference's eager attention (restated by the oracle) on the host cores, fp32."""
    import torch
    from oracle import kernl_oracle as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    q, k, v, mask = make_inputs()
    for _ in range(warmup):
        O.attention(q, k, v, 0.125, False, mask)
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        O.attention(q, k, v, 0.125, False, mask)
        ts.append(time.perf_counter() - t0)
    return statistics.mean(ts), cores


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = args.steps, max(args.warmup, 1)
    sec, cores = time_cpu_attention(steps, warmup)
    tflops = attention_flops() / sec / 1e12
    line = {
        "impl": "reference",
        "metric": "fused attention TFLOP/s", "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD_NAME,
                   "note": "reference's eager attention_reference restated in fp32 PyTorch on the host CPU; "
                           "its Triton path needs an Ampere+ GPU and Triton 2.0 and cannot run here"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"{steps} full steps of the workload"},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def event_time(fn, steps, warmup, flush):
    """Per-step CUDA-event durations (ms) with an L2 flush before each step, outside the events."""
    import torch

    for _ in range(warmup):
        flush.zero_()
        fn()
    torch.cuda.synchronize()
    pairs = []
    for _ in range(steps):
        flush.zero_()
        s = torch.cuda.Event(enable_timing=True)
        e = torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        pairs.append((s, e))
    torch.cuda.synchronize()
    return [s.elapsed_time(e) for s, e in pairs]


def graph_time(step_for_set, n_sets, steps, warmup, min_total_ms=0.0, repeats=1):
    """Device time per step (ms) of `steps` back-to-back steps that cycle through `n_sets`
    independent input sets whose total size exceeds L2, so every step finds its inputs cold
    without any flush inside the timed region. The steps are enqueued as replays of one CUDA graph
    holding one step per input set (the way the reference runs its kernels in production:
    src/kernl/optimizer/cuda_graph.py), so host launch latency is not part of the number; one
    CUDA-event pair on the launching stream brackets all of them. `repeats` > 1 (sweeps and the
    side measurements, never the headline) takes the best of several such measurements: the replays
    are enqueued from Python, and a host stall while the GPU waits for the next replay (seen as one
    case in fifty reading 40x slow) is not device time."""
    import torch

    for i in range(max(warmup, n_sets)):
        step_for_set(i % n_sets)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for i in range(n_sets):
            step_for_set(i)
    torch.cuda.current_stream().wait_stream(side)
    # untimed replays for at least 30 ms, so that the SM clocks are up (input generation on the
    # host leaves the GPU idle for seconds) before anything is timed
    t_warm = time.perf_counter()
    while time.perf_counter() - t_warm < 0.03:
        for _ in range(10):
            graph.replay()
        torch.cuda.synchronize()
    while True:
        replays, rest = divmod(steps, n_sets)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(replays):
            graph.replay()
        for i in range(rest):
            step_for_set(i)
        e.record()
        torch.cuda.synchronize()
        total = s.elapsed_time(e)
        if total >= min_total_ms or steps >= 20000:
            best = total
            for _ in range(repeats - 1):
                s.record()
                for _ in range(replays):
                    graph.replay()
                for i in range(rest):
                    step_for_set(i)
                e.record()
                torch.cuda.synchronize()
                best = min(best, s.elapsed_time(e))
            return best / steps
        # microsecond kernels: a handful of steps is dominated by the latency of the first
        # launch, so repeat with enough steps (whole replays only) to fill min_total_ms
        steps = n_sets * max(replays + 1, int(1.5 * min_total_ms / max(total, 1e-3) * max(replays, 1)) + 1)


def headline_traffic_bytes():
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the headline workload, as the
    committed ncu summary of the kernel that ships records it (a line `dram_bytes_per_launch: N`);
    None when the summary carries no such line."""
    import re

    try:
        text = open(os.path.join(ROOT, TRAFFIC_PROFILE)).read()
    except OSError:
        return None
    m = re.search(r"^dram_bytes_per_launch:\s*([0-9]+)", text, flags=re.M)
    return int(m.group(1)) if m else None



def bind_to_gpu_numa_node(local_rank):
    """Run this process on the CPUs next to its GPU, so that the pinned host buffers allocated
    afterwards (first touch) and the copy threads sit on the GPU's own NUMA node. Returns what it
    found: {"nodes": NUMA nodes of the host, "gpu_node": the GPU's node or -1, "bound": whether the
    affinity was changed}. A host with one node (or without the sysfs entries) is left alone."""
    info = {"nodes": 1, "gpu_node": -1, "bound": False}
    try:
        nodes = [d for d in os.listdir("/sys/devices/system/node") if d.startswith("node") and d[4:].isdigit()]
        info["nodes"] = max(1, len(nodes))
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        bus = pynvml.nvmlDeviceGetPciInfo(handle).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        dev_dir = os.path.join("/sys/bus/pci/devices", bus[-12:].lower())  # 0000:1b:00.0
        node = int(open(os.path.join(dev_dir, "numa_node")).read().strip())
        info["gpu_node"] = node
        if info["nodes"] > 1 and node >= 0:
            cpus = set()
            for part in open(os.path.join(dev_dir, "local_cpulist")).read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
            allowed = cpus & os.sched_getaffinity(0)
            if allowed:
                os.sched_setaffinity(0, allowed)
                info["bound"] = True
    except Exception:
        pass
    return info


def run_ours(args):
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (sm_100a); there is no CPU fallback")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        # The tensor-parallel prefill overlaps its all-reduces with the other half-batch's GEMMs,
        # which leave 24 SMs free for them (LlamaTP.overlap_reserved_sms): the collective is told to
        # stay within that many CTAs (from four ranks on; two ranks measured better uncapped). Has to be
        # set before the communicator exists.
        if world >= 4:
            os.environ.setdefault("NCCL_MAX_CTAS", "24")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from kernl_b200 import _lib, build
    from kernl_b200.implementations.attention import attention_forward
    from kernl_b200.implementations.layer_norm import layer_norm
    from kernl_b200.implementations.linear_layer import linear_layer

    build.build()
    _lib.load()
    peaks, peak_kind = load_peaks()
    steps, warmup = args.steps, max(args.warmup, 3)
    dev = torch.device("cuda", local_rank)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.int8, device=dev)

    q32, k32, v32, mask32 = make_inputs()
    # 10 independent input sets of 25.2 MB each (252 MB > 126 MB of L2): set 0 holds the seeded
    # workload, the others the same distribution under other seeds
    n_sets = 10
    sets = []
    for i in range(n_sets):
        qi, ki, vi, mi = (q32, k32, v32, mask32) if i == 0 else make_inputs(seed=i)
        qd, kd, vd, md = (t.half().to(dev) for t in (qi, ki, vi, mi))
        sets.append((qd, kd, vd, md, torch.empty_like(qd)))
    q, k, v, mask, out = sets[0]

    def step_for_set(i):
        qd, kd, vd, md, od = sets[i]
        attention_forward(qd, kd, vd, od, 0.125, False, md)

    # ---------------- timed region: K steps, device-timed, bracketed by barrier + synchronize
    step_for_set(0)
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    t_wall0 = time.time()
    ms_local = graph_time(step_for_set, n_sets, steps, warmup)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    t_wall1 = time.time()
    clocks = sampler.stop(t_wall0, t_wall1)
    _lib.device_status()
    ms = ms_local
    if dist is not None:
        t = torch.tensor([ms_local], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    flops = attention_flops()
    value = world * flops / (ms * 1e-3) / 1e12
    # key blocks (64 keys) that are padding for a whole sequence are not visited by the kernel; the
    # metric counts the dense FLOPs of the shape, this is what was actually multiplied
    visited = 0.0
    for (_, _, _, md, _) in sets:
        live = (md.float().reshape(md.shape[0], -1) > -30000.0)
        blocks = live.reshape(live.shape[0], -1, 64).any(-1).sum(-1).float()
        visited += float(blocks.sum().item()) * 64
    executed_fraction = visited / (len(sets) * WORKLOAD["B"] * WORKLOAD["S"])

    # ---------------- end to end through the public API with host buffers
    numa = bind_to_gpu_numa_node(local_rank)
    hq, hk, hv, hm = (t.half().pin_memory() for t in (q32, k32, v32, mask32))
    hout = torch.empty(q.shape, dtype=torch.float16).pin_memory()
    dq, dk, dv, dm, do = (torch.empty_like(t, device=dev) for t in (hq, hk, hv, hm, hq))

    def serial_step():
        dq.copy_(hq, non_blocking=True)
        dk.copy_(hk, non_blocking=True)
        dv.copy_(hv, non_blocking=True)
        dm.copy_(hm, non_blocking=True)
        attention_forward(dq, dk, dv, do, 0.125, False, dm)
        hout.copy_(do, non_blocking=True)

    # latency of one call on one stream (copy in, kernel, copy out, nothing overlapped)
    for _ in range(3):
        serial_step()
    torch.cuda.synchronize()
    lat_t0 = time.perf_counter()
    for _ in range(steps):
        serial_step()
        torch.cuda.synchronize()
    e2e_latency_ms = (time.perf_counter() - lat_t0) * 1e3 / steps

    # throughput: the package's host pipeline — every step still copies its operands in and its
    # result out, but the result of step i travels while the operands of step i + 1 arrive
    from kernl_b200.host_pipeline import HostAttentionPipeline

    pipe = HostAttentionPipeline(hq.shape, hk.shape, hm.shape, torch.float16, dev)
    for _ in range(3):
        pipe.submit(hq, hk, hv, hm, hout, 0.125)
    pipe.synchronize()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    e2e_t0 = time.perf_counter()
    for _ in range(steps):
        pipe.submit(hq, hk, hv, hm, hout, 0.125)
    pipe.synchronize()
    e2e_ms_local = (time.perf_counter() - e2e_t0) * 1e3 / steps
    e2e_ms = e2e_ms_local
    if dist is not None:
        t = torch.tensor([e2e_ms_local], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hm))
    d2h = hout.numel() * hout.element_size()

    # ---------------- N > 1: the ranks of this job as ONE tensor-parallel group (baseline config 5)
    tp = None
    if world > 1 and not args.no_tp:
        del sets, pipe, flush
        torch.cuda.empty_cache()
        tp = {"workload": "Llama-2-7B-shaped decoder, 32 layers, bf16, prefill batch 8 x 2048 causal + 128 greedy decode steps, "
                          f"tensor parallel over {world} GPUs (strong scaling; baseline config 5)"}
        for kind in ("peer", "nccl"):
            try:
                par = llama_tp_parity(world, rank, dev, dist, kind)
                r = measure_llama(world, rank, dev, dist, kind, layers=32, decode_steps=128, prefill_reps=2)
                tp[kind] = {"prefill_ms": round(r["prefill_ms"], 3), "decode_ms_per_step": round(r["decode_ms_per_step"], 4),
                            "logits_vs_one_rank_2_layers": par}
            except Exception as exc:  # the headline line must still be printed
                tp[kind] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        tp["all_reduce"] = {"peer": "fused peer-memory all-reduce + residual + RMSNorm kernel for decode messages, NCCL for prefill",
                            "nccl": "NCCL all-reduce for every message"}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---------------- rank 0 only: other hot-path kernels against their rooflines, CPU baseline
    ops = {}
    g = torch.Generator().manual_seed(0)
    M, K, N = 8192, 4096, 11008
    x = torch.randn((M, K), generator=g).half().to(dev)
    w = (torch.randn((N, K), generator=g) * 0.02).half().to(dev)
    b = (torch.randn((N,), generator=g) * 0.02).half().to(dev)
    # same method as the headline: CUDA-graph replays cycling through input sets larger than L2
    w = (torch.randn((N, K), generator=g) * 0.02).half().to(dev)
    b = (torch.randn((N,), generator=g) * 0.02).half().to(dev)
    xs = [torch.randn((M, K), generator=g).half().to(dev) for _ in range(4)]  # 4 x (67 MB in + 180 MB out)
    ys = [torch.empty((M, N), dtype=torch.float16, device=dev) for _ in range(4)]
    for act in ("", "gelu"):
        t_ms = graph_time(lambda i: linear_layer(xs[i], w, b, act, out=ys[i]), 4, 12, 3, min_total_ms=3.0, repeats=3)
        tf = 2.0 * M * N * K / (t_ms * 1e-3) / 1e12
        ops[f"linear_M8192_K4096_N11008_{act or 'none'}"] = {
            "tflops": round(tf, 1), "frac_of_tensor_peak": round(tf / peaks["bf16_tflops"], 3), "ms": round(t_ms, 4)}
    del xs, ys, w, b
    for cols in (768, 4096):
        n_norm_sets = 12 if cols == 768 else 3  # 12 x 50 MB / 3 x 268 MB of inputs + outputs: > 2 x L2
        xn = [torch.randn((16384, cols), generator=g).half().to(dev) for _ in range(n_norm_sets)]
        yn = [torch.empty_like(t) for t in xn]  # outputs rotate with the inputs: no step finds its output lines in L2
        gm = (torch.rand((cols,), generator=g) + 0.5).half().to(dev)
        bt = (torch.randn((cols,), generator=g) * 0.1).half().to(dev)
        for rms in (False, True):
            t_ms = graph_time(lambda i: layer_norm(xn[i], gm, None if rms else bt, 1e-5, use_rms_norm=rms, out=yn[i]),
                              n_norm_sets, 4 * n_norm_sets, 3, min_total_ms=3.0, repeats=3)
            gbs = (4.0 * 16384 * cols + 4 * cols) / (t_ms * 1e-3) / 1e9
            ops[f"{'rmsnorm' if rms else 'layernorm'}_16384x{cols}"] = {
                "gbs": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 3), "ms": round(t_ms, 4)}
        del xn, yn
    _lib.device_status()

    cpu_sec, cores = time_cpu_attention(5, 2)
    cpu_tflops = flops / cpu_sec / 1e12

    per_launch_tflops = flops / (ms_local * 1e-3) / 1e12
    line = {
        "metric": "fused attention TFLOP/s", "value": value, "unit": "TFLOP/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {
            "workload": WORKLOAD_NAME,
            "per_gpu_batch": WORKLOAD["B"], "parallelism": f"replicas x{world} (batch-sharded, no collective)",
            "timing": "one CUDA-event pair around K back-to-back steps (CUDA-graph replays) on the launching stream; "
                      "steps cycle through 10 input sets (252 MB) so inputs are larger than L2, no flush in the timed region",
            "flops_per_step": flops,
            "note": "value counts the dense FLOPs of the shape; key blocks that are padding for a whole sequence are "
                    "skipped by the kernel (identical results), executed_fraction is the share actually multiplied",
            "executed_fraction": round(executed_fraction, 4),
        },
        "roofline": {
            "bound": "tensor", "achieved": per_launch_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
            "frac": per_launch_tflops / peaks["bf16_tflops"], "traffic": headline_traffic_bytes(),
            "peak_source": f"{peak_kind} cuBLAS bf16 burst (MEASURED_PEAKS.json)" if peak_kind == "measured" else "fallback 1590 TFLOP/s",
            "kernel": "attention_persist_kernel<half, row-broadcast mask>",
            "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one launch of this workload, " + TRAFFIC_PROFILE,
        },
        "cpu_baseline": {"value": cpu_tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": "5 full steps of the workload in fp32 (oracle restatement of the reference's eager attention)"},
        "e2e": {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                "latency_ms": e2e_latency_ms,
                "host_gbs_per_rank": (h2d + d2h) / (e2e_ms * 1e-3) / 1e9, "numa": numa,
                "api": "kernl_b200.host_pipeline.HostAttentionPipeline (two-deep: copies in both directions overlap)"},
        "gpu_launches": steps,
        "clocks": clocks,
        "ops": ops,
    }
    if tp is not None:
        line["tp"] = tp
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_sweep(args):
    """Per-shape kernel timings of the op configs (attention sweep, linear shapes, norms, decode),
    one JSON line per case: device time per launch (CUDA-graph replays cycling through input sets
    that together exceed twice the L2), achieved TFLOP/s or GB/s and the fraction of the measured
    peak that bounds the case. Not part of the default run."""
    import torch

    from kernl_b200 import _lib, build
    from kernl_b200.implementations.attention import attention_forward
    from kernl_b200.implementations.attention_skinny import skinny_attention_forward
    from kernl_b200.implementations.layer_norm import layer_norm
    from kernl_b200.implementations.linear_layer import linear_layer

    build.build()
    _lib.load()
    peaks, _ = load_peaks()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(0)
    iters, warm = args.steps, max(args.warmup, 3)
    want = lambda name: (args.sweep in ("all", name.split(":")[0])) and (args.case is None or args.case in name)

    def emit(name, ms_list, flops=None, nbytes=None):
        ms = statistics.mean(ms_list)
        rec = {"case": name, "ms": round(ms, 5), "ms_min": round(min(ms_list), 5)}
        if flops is not None:
            rec["tflops"] = round(flops / ms / 1e9, 1)
            rec["frac_tensor_peak"] = round(flops / ms / 1e9 / peaks["bf16_tflops"], 4)
        if nbytes is not None:
            rec["gbs"] = round(nbytes / ms / 1e6, 1)
            rec["frac_hbm_peak"] = round(nbytes / ms / 1e6 / peaks["hbm_gbs"], 4)
        print(json.dumps(rec), flush=True)

    def timed(make_set, bytes_per_set):
        """make_set() -> zero-argument callable over freshly allocated inputs; enough sets to
        exceed twice the L2."""
        n_sets = int(min(16, max(2, -(-256 * 1024 * 1024 // max(1, int(bytes_per_set))))))
        fns = [make_set() for _ in range(n_sets)]
        ms = graph_time(lambda i: fns[i](), n_sets, max(iters, n_sets), warm, min_total_ms=3.0, repeats=3)
        return [ms]

    for S in (128, 256, 512, 1024, 2048, 4096):
        for kind in ("full", "causal", "pad"):
            for (D, H, dt, tag) in ((64, 12, torch.float16, "f16"), (128, 32, torch.bfloat16, "bf16")):
                tokens = 4096 if D == 64 else 16384
                name = f"attention:{tag}_d{D}_s{S}_{kind}"
                if not want(name):
                    continue
                B = tokens // S
                causal = kind == "causal"

                def make_set():
                    q, k, v = (torch.randn((B, H, S, D), generator=g).to(dt).to(dev) for _ in range(3))
                    mask = None
                    if kind == "pad":
                        valid = torch.randint(min(64, S), S + 1, (B,), generator=g)
                        mask = torch.where(valid[:, None] > torch.arange(S)[None, :], 0.0, float("-inf")).reshape(B, 1, 1, S).to(dt).to(dev)
                    o = torch.empty_like(q)
                    return lambda: attention_forward(q, k, v, o, D ** -0.5, causal, mask)

                d = timed(make_set, 4 * B * H * S * D * 2)
                fl = 4.0 * B * H * D * (S * (S + 1) / 2 if causal else S * S)
                emit(name, d, flops=fl)
    # the same kernels with enough (batch x heads) to fill the GPU several times over: the sweep
    # above holds batch*seq at 4096 tokens, i.e. 192 CTAs on 148 SMs for head_dim 64
    for (B, H, S, D, dt, tag, causal) in ((8, 12, 4096, 64, torch.float16, "f16_d64_s4096_b8_full", False),
                                          (8, 12, 4096, 64, torch.float16, "f16_d64_s4096_b8_causal", True),
                                          (64, 12, 512, 64, torch.float16, "f16_d64_s512_b64_full", False),
                                          (8, 12, 4096, 64, torch.bfloat16, "bf16_d64_s4096_b8_full", False),
                                          (4, 32, 4096, 128, torch.float16, "f16_d128_s4096_b4_full", False)):
        name = f"attention_big:{tag}"
        if not want(name):
            continue

        def make_set():
            q, k, v = (torch.randn((B, H, S, D), generator=g).to(dt).to(dev) for _ in range(3))
            o = torch.empty_like(q)
            return lambda: attention_forward(q, k, v, o, D ** -0.5, causal, None)

        d = timed(make_set, 4 * B * H * S * D * 2)
        emit(name, d, flops=4.0 * B * H * D * (S * (S + 1) / 2 if causal else S * S))
    for M in (16, 128, 1024, 8192):
        for (K, N) in ((768, 768), (768, 3072), (3072, 768), (4096, 11008), (11008, 4096)):
            for act in ("", "gelu", "relu"):
                name = f"linear:M{M}_K{K}_N{N}_{act or 'none'}"
                if not want(name):
                    continue

                def make_set():
                    x = torch.randn((M, K), generator=g).half().to(dev)
                    w = (torch.randn((N, K), generator=g) * 0.02).half().to(dev)
                    b = (torch.randn((N,), generator=g) * 0.02).half().to(dev)
                    y = torch.empty((M, N), dtype=torch.float16, device=dev)
                    return lambda: linear_layer(x, w, b, act, out=y)

                nbytes = 2.0 * (M * K + N * K + M * N) + 2 * N
                emit(name, timed(make_set, nbytes), flops=2.0 * M * N * K, nbytes=nbytes)
    for cols in (768, 4096):
        for rms in (False, True):
            name = f"norm:{'rms' if rms else 'ln'}_16384x{cols}"
            if not want(name):
                continue

            def make_set():
                x = torch.randn((16384, cols), generator=g).half().to(dev)
                y = torch.empty_like(x)
                gm = (torch.rand((cols,), generator=g) + 0.5).half().to(dev)
                bt = (torch.randn((cols,), generator=g) * 0.1).half().to(dev)
                return lambda: layer_norm(x, gm, None if rms else bt, 1e-5, use_rms_norm=rms, out=y)

            nbytes = 4.0 * 16384 * cols + 4 * cols
            emit(name, timed(make_set, nbytes), nbytes=nbytes)
    for (B, H, N, D, dt, tag) in ((1, 12, 512, 64, torch.float16, "t5_cross"), (8, 32, 2048, 128, torch.bfloat16, "llama_decode"),
                                  (64, 32, 2048, 128, torch.bfloat16, "llama_decode_b64")):
        name = f"decode:{tag}"
        if not want(name):
            continue

        def make_set():
            q = torch.randn((B, H, 1, D), generator=g).to(dt).to(dev)
            k, v = (torch.randn((B, H, N, D), generator=g).to(dt).to(dev) for _ in range(2))
            o = torch.empty_like(q)
            return lambda: skinny_attention_forward(q, k, v, o, D ** -0.5)

        nbytes = 2.0 * 2 * B * H * N * D
        emit(name, timed(make_set, nbytes), nbytes=nbytes)
    _lib.device_status()


def run_bert(args):
    """Baseline config 1: BERT-base, random init (seed 0), batch 1 x seq 128, fp16 through
    optimize_model (graph rewrites + CUDA graph). Forward latency in ms; with --gpus N each rank
    runs its own replica (batch-sharded serving, no collective)."""
    import torch
    import torch._dynamo
    from transformers import BertConfig, BertModel

    from kernl_b200 import _lib
    from kernl_b200.model_optimization import optimize_model

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        # The tensor-parallel prefill overlaps its all-reduces with the other half-batch's GEMMs,
        # which leave 24 SMs free for them (LlamaTP.overlap_reserved_sms): the collective is told to
        # stay within that many CTAs (from four ranks on; two ranks measured better uncapped). Has to be
        # set before the communicator exists.
        if world >= 4:
            os.environ.setdefault("NCCL_MAX_CTAS", "24")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = torch.device("cuda", local_rank)
    torch.manual_seed(0)
    model = BertModel(BertConfig()).eval()
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 30522, (1, 128), generator=g)
    mask = torch.ones((1, 128), dtype=torch.long)
    cpu_ms = None
    if rank == 0:
        torch.set_num_threads(os.cpu_count() or 1)
        with torch.inference_mode():
            for _ in range(2):
                model(input_ids=ids, attention_mask=mask)
            t0 = time.perf_counter()
            for _ in range(5):
                ref = model(input_ids=ids, attention_mask=mask).last_hidden_state
            cpu_ms = (time.perf_counter() - t0) / 5 * 1e3
            # parity is checked against the fp32 model with the LayerNorm eps of the reference's
            # kernel path (eps raised to 1.6e-5 for fp16 inputs, layer_norm.py:295-296)
            for m in model.modules():
                if isinstance(m, torch.nn.LayerNorm):
                    m.eps = max(m.eps, 1.6e-5)
            ref = model(input_ids=ids, attention_mask=mask).last_hidden_state
    gm = model.half().to(dev)
    optimize_model(gm)
    ids_d, mask_d = ids.to(dev), mask.to(dev)
    steps, warmup = args.steps, max(args.warmup, 3)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.int8, device=dev)
    with torch.inference_mode():
        fwd = lambda: gm(input_ids=ids_d, attention_mask=mask_d)
        out = fwd()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        durs = event_time(fwd, steps, warmup, flush)
        out = fwd()
        # end to end: ids from pinned host memory, hidden state back to the host
        hid, hmask = ids.pin_memory(), mask.pin_memory()
        hout = torch.empty((1, 128, 768), dtype=torch.float16).pin_memory()

        def e2e():
            ids_d.copy_(hid, non_blocking=True)
            mask_d.copy_(hmask, non_blocking=True)
            hout.copy_(gm(input_ids=ids_d, attention_mask=mask_d).last_hidden_state, non_blocking=True)

        for _ in range(3):
            e2e()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            e2e()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) / steps * 1e3
    _lib.device_status()
    ms = statistics.mean(durs)
    if dist is not None:
        t = torch.tensor([ms, e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
    if rank == 0:
        from oracle import kernl_oracle as O

        par = O.parity(out.last_hidden_state, ref)
        print(json.dumps({
            "metric": "BERT-base forward latency", "value": ms, "unit": "ms", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms, "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {"workload": "BERT-base encoder forward, random init seed 0, batch 1 x seq 128, all-ones mask (baseline config 1)",
                       "parallelism": f"replicas x{world}", "sequences_per_s_all_gpus": world * 1e3 / ms,
                       "timing": "CUDA events per forward (one CUDA-graph replay), 256 MB L2 flush before each, outside the events"},
            "cpu_baseline": {"value": cpu_ms, "unit": "ms", "cores": os.cpu_count(), "kind": "reference",
                             "sample": "5 forwards of the same model in fp32 eager PyTorch (Hugging Face BertModel) on the host"},
            "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": 2 * 128 * 8, "d2h_bytes_per_step": 128 * 768 * 2},
            "parity_vs_fp32_cpu": par,
        }), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_t5(args):
    """Baseline config 4: T5-base-shaped encoder-decoder, random init (seed 0), batch B (default 1),
    encoder input 512 uniform-random ids, greedy decode of 128 tokens with the static KV cache under
    one CUDA graph, fp16. Value = latency of encode + 128 decode steps; with --gpus N each rank runs
    its own replica on its own batch (batch-sharded, no collective)."""
    import torch
    from transformers import T5Config, T5ForConditionalGeneration

    from kernl_b200 import _lib
    from kernl_b200.t5_generate import T5Kernl

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        # The tensor-parallel prefill overlaps its all-reduces with the other half-batch's GEMMs,
        # which leave 24 SMs free for them (LlamaTP.overlap_reserved_sms): the collective is told to
        # stay within that many CTAs (from four ranks on; two ranks measured better uncapped). Has to be
        # set before the communicator exists.
        if world >= 4:
            os.environ.setdefault("NCCL_MAX_CTAS", "24")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = torch.device("cuda", local_rank)
    torch.manual_seed(0)
    cfg = T5Config(d_model=768, d_ff=3072, num_layers=12, num_decoder_layers=12, num_heads=12, d_kv=64, vocab_size=32128,
                   feed_forward_proj="relu", relative_attention_num_buckets=32, decoder_start_token_id=0, pad_token_id=0,
                   eos_token_id=1)
    model = T5ForConditionalGeneration(cfg).eval()
    B, S, T = args.t5_batch, 512, 128
    ids = torch.randint(2, 32128, (B, S), generator=torch.Generator().manual_seed(rank)).to(dev)
    runner = T5Kernl(model, device=dev, dtype=torch.float16, max_new_tokens=T)
    del model
    steps, warmup = max(1, min(args.steps, 10)), 1
    with torch.inference_mode():
        for _ in range(warmup):
            toks = runner.generate(ids, T, use_cuda_graph=True)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            toks = runner.generate(ids, T, use_cuda_graph=True)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
    _lib.device_status()
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        print(json.dumps({
            "metric": "T5-base generate latency (encode 512 + 128 greedy tokens)", "value": ms, "unit": "ms", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"T5-base shape, random init seed 0, batch {B} per GPU, encoder 512 ids, 128 greedy decode "
                                   "steps with static KV cache, one CUDA graph per decode step (baseline config 4)",
                       "parallelism": f"replicas x{world}", "tokens_per_s_all_gpus": world * B * T / (ms * 1e-3),
                       "includes": "encoder, cross K/V projection, 128 graph replays; the decode graph is captured once (warm-up)",
                       "tokens_sample": toks[0, :8].tolist()}}), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def _make_comm(kind, rank, world, dev):
    import torch

    if world > 1 and kind == "peer":
        from kernl_b200.comm import PeerAllReduce

        return PeerAllReduce(rank, world, dev, torch.bfloat16)
    return None  # LlamaTP then uses NCCL (or nothing on one rank)


def measure_llama(world, rank, dev, dist, comm_kind, layers=32, decode_steps=256, prefill_reps=3):
    """Baseline config 5 on the ranks of this job as ONE tensor-parallel group: prefill 8 x 2048
    (causal), then `decode_steps` greedy steps replayed from one CUDA graph. Device-timed with CUDA
    events between barriers, max over ranks. Returns {"prefill_ms", "decode_ms_per_step", "tokens_sample"}."""
    import torch

    from kernl_b200 import _lib
    from kernl_b200.llama_tp import LlamaConfig, LlamaTP

    cfg = LlamaConfig(n_layers=layers)
    assert 2048 + decode_steps <= cfg.max_seq, f"prompt 2048 + {decode_steps} decode steps exceed the KV cache ({cfg.max_seq} slots)"
    comm = _make_comm(comm_kind, rank, world, dev)
    model = LlamaTP(cfg, rank=rank, world=world, device=dev, dtype=torch.bfloat16, seed=0, comm=comm)
    ids = torch.randint(0, cfg.vocab, (8, 2048), generator=torch.Generator().manual_seed(0)).to(dev)
    model.prefill(ids)  # warm-up
    torch.cuda.synchronize()
    pre = []
    for _ in range(max(1, prefill_reps)):
        if dist is not None:
            dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        model.prefill(ids)
        e.record()
        torch.cuda.synchronize()
        pre.append(s.elapsed_time(e))
    # decode: capture one step in a CUDA graph, then time `decode_steps` replays on the device
    tok = model.prefill(ids).float().argmax(-1)
    replay, static_tok, static_next = model.capture_decode(tok)
    static_tok.copy_(tok)
    for _ in range(3):
        replay()
        static_tok.copy_(static_next)
    model.prefill(ids)  # reset the cache position to the end of the prompt
    static_tok.copy_(tok)
    toks = []
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(decode_steps):
        replay()
        static_tok.copy_(static_next)
        toks.append(static_next.clone())
    e.record()
    torch.cuda.synchronize()
    dec_ms = s.elapsed_time(e)
    toks = torch.stack(toks, dim=1)
    _lib.device_status()
    t = torch.tensor([statistics.mean(pre), dec_ms], device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    result = {"prefill_ms": float(t[0]), "decode_ms_per_step": float(t[1]) / decode_steps,
              "tokens_sample": toks[0, :8].tolist()}
    # drop the captured graph (it holds NCCL work with the nccl communicator) before the caller
    # builds another model or tears NCCL down
    del replay, static_tok, static_next, model
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    if comm is not None:
        comm.close()
    torch.cuda.empty_cache()
    return result


def llama_tp_parity(world, rank, dev, dist, comm_kind, layers=2, prompt=2048, steps=4):
    """Logits of the tensor-parallel decoder against the same weights on ONE rank: a `layers`-deep
    slice of the 7B shape, prefill 8 x `prompt` plus `steps` teacher-forced decode steps (the decode
    steps are what the fused peer-memory kernel serves). Rank 0 evaluates the single-rank model and
    broadcasts its greedy tokens, every rank runs its shard. Returns max-abs / cosine per phase."""
    import torch

    from kernl_b200.llama_tp import LlamaConfig, LlamaTP

    cfg = LlamaConfig(n_layers=layers)
    ids = torch.randint(0, cfg.vocab, (8, prompt), generator=torch.Generator().manual_seed(1)).to(dev)
    ref_logits = None
    forced = torch.zeros((steps, 8), dtype=torch.long, device=dev)
    if rank == 0:
        single = LlamaTP(cfg, rank=0, world=1, device=dev, dtype=torch.bfloat16, seed=0)
        ref_logits = [single.prefill(ids).float()]
        for t in range(steps):
            forced[t] = ref_logits[-1].argmax(-1)
            ref_logits.append(single.decode_step(forced[t]).float())
        del single
        torch.cuda.empty_cache()
    if dist is not None:
        dist.broadcast(forced, src=0)
    comm = _make_comm(comm_kind, rank, world, dev)
    model = LlamaTP(cfg, rank=rank, world=world, device=dev, dtype=torch.bfloat16, seed=0, comm=comm)
    logits = [model.prefill(ids).float()]
    for t in range(steps):
        logits.append(model.decode_step(forced[t]).float())
    torch.cuda.synchronize()
    out = None
    if rank == 0:
        def cmp(a, b):
            a, b = torch.stack(a), torch.stack(b)
            return {"max_abs": float((a - b).abs().max()), "cos": float(torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0)),
                    "argmax_agree": float((a.argmax(-1) == b.argmax(-1)).float().mean())}
        out = {"prefill": cmp(logits[:1], ref_logits[:1]), "decode": cmp(logits[1:], ref_logits[1:]),
               "logit_abs_max": float(torch.stack(ref_logits).abs().max())}
    del model
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    if comm is not None:
        comm.close()
    torch.cuda.empty_cache()
    return out


def run_llama(args):
    """Baseline config 5: Llama-2-7B-shaped decoder, random init bf16, prefill 8 x 2048 then greedy
    decode with KV cache; tensor parallel over the ranks of this job (all-reduce after o_proj and
    down_proj: NCCL, or the fused peer-memory kernel for decode-size messages)."""
    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        # The tensor-parallel prefill overlaps its all-reduces with the other half-batch's GEMMs,
        # which leave 24 SMs free for them (LlamaTP.overlap_reserved_sms): the collective is told to
        # stay within that many CTAs (from four ranks on; two ranks measured better uncapped). Has to be
        # set before the communicator exists.
        if world >= 4:
            os.environ.setdefault("NCCL_MAX_CTAS", "24")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = torch.device("cuda", local_rank)
    kind = args.comm if world > 1 else "none"
    parity = llama_tp_parity(world, rank, dev, dist, kind) if world > 1 else None
    r = measure_llama(world, rank, dev, dist, kind, layers=args.layers, decode_steps=args.decode_steps,
                      prefill_reps=max(1, min(args.steps, 3)))
    if rank == 0:
        print(json.dumps({
            "metric": "Llama-7B-shape prefill latency", "value": r["prefill_ms"], "unit": "ms", "n_gpus": world,
            "steps": max(1, min(args.steps, 3)), "warmup": 1, "ms_per_step": r["prefill_ms"], "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"Llama-2-7B-shaped decoder ({args.layers} layers), prefill batch 8 x 2048 causal, then {args.decode_steps} greedy decode steps (baseline config 5)",
                       "parallelism": f"tp{world}", "all_reduce": ("fused peer-memory kernel for messages <= 1 MiB (decode), NCCL above"
                                                                    if kind == "peer" else "NCCL" if world > 1 else "none"),
                       "prefill_tokens_per_s": 8 * 2048 / r["prefill_ms"] * 1e3,
                       "decode_ms_per_step": r["decode_ms_per_step"], "decode_tokens_per_s": 8 / r["decode_ms_per_step"] * 1e3,
                       "tokens_sample": r["tokens_sample"],
                       "logits_vs_one_rank_2_layers": parity},
        }), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--sweep", choices=["all", "attention", "attention_big", "linear", "norm", "decode"], default=None,
                    help="per-shape kernel timings instead of the headline line")
    ap.add_argument("--case", default=None, help="with --sweep: only cases whose name contains this")
    ap.add_argument("--workload", choices=["attention", "bert", "llama", "t5"], default="attention",
                    help="attention = headline (default); bert / llama = the model configs")
    ap.add_argument("--no-pdl", action="store_true", help="model workloads: launch the light kernels without programmatic "
                    "dependent launch (A/B timing)")
    ap.add_argument("--t5-batch", type=int, default=1, help="t5 workload: sequences per GPU")
    ap.add_argument("--layers", type=int, default=32, help="llama workload: number of layers")
    ap.add_argument("--comm", choices=["nccl", "peer"], default="peer",
                    help="llama workload, N > 1: all-reduce through NCCL only, or the fused peer-memory kernel for decode-size messages")
    ap.add_argument("--decode-steps", type=int, default=256, help="llama workload: greedy decode steps")
    ap.add_argument("--no-tp", action="store_true", help="default run with N > 1: skip the tensor-parallel decoder measurement")
    args = ap.parse_args()
    if args.no_pdl:
        from kernl_b200 import _lib as _kb_lib

        _kb_lib.load().kb_debug_pdl(0)
    if args.workload == "bert":
        run_bert(args)
        return
    if args.workload == "t5":
        return run_t5(args)
    if args.workload == "llama":
        run_llama(args)
        return
    if args.sweep is not None:
        run_sweep(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
