"""Benchmark of the fused quantized matmul on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One JSON line on stdout (rank 0). A step is one pass of the hot path over one batch of
synthetic input: by default the prefill configuration, an int4 group-64 quantized matmul of
x[2048, 4096] (bf16, N(0,1)) against W[14336, 4096] (codes uniform 0..15, scales
U(0.002, 0.02), bias = -8*scale), bf16 output, float32 accumulation. `value` is the
whole-job TFLOP/s with inputs resident in HBM; `e2e` is the same metric through the public
call with pinned host buffers copied in and out inside the timed region; `roofline` compares
the kernel with the measured bf16 tensor peak; `cpu_baseline` is the CPU restatement of the
reference's fused dequantize-and-dot loop timed on the host cores on a bounded sample; `also`
carries the decode (M=1) configuration against the measured HBM bandwidth and the tokens/s of
whole Llama-3-8B-shaped decode steps (batch 1, 16, 64; weights sharded on N over the ranks).

With N > 1 (one process per GPU under torch.distributed.run) every rank runs the same
workload on its own token batch against replicated weights -- the path shards over
independent rows of x with no data-path collective -- so scaling is weak and `value` is the
sum over ranks divided by the slowest rank's time.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (M, K, N, group_size, bits, mode)
    "prefill_int4_g64_m2048_14336x4096": (2048, 4096, 14336, 64, 4, "affine"),
    "prefill_int4_g64_m2048_4096x14336": (2048, 14336, 4096, 64, 4, "affine"),
    "prefill_int8_g128_m2048_14336x4096": (2048, 4096, 14336, 128, 8, "affine"),
    "prefill_mxfp4_m4096_5760x2880": (4096, 2880, 5760, 32, 4, "mxfp4"),
    "decode_int4_g64_m1_4096x4096": (1, 4096, 4096, 64, 4, "affine"),
    "decode_mxfp4_m1_5760x2880": (1, 2880, 5760, 32, 4, "mxfp4"),
}
DEFAULT = "prefill_int4_g64_m2048_14336x4096"
DECODE = "decode_int4_g64_m1_4096x4096"
L2_BYTES = 126 * 1024 * 1024
# Whole decode steps of a Llama-3-8B-shaped model (32 layers, d 4096, 32/8 heads, ffn 14336,
# vocabulary 128256, int4 group-64 linears, bf16 KV cache of 2048 positions): name -> batch.
# The weights are sharded on N over the ranks, so these scale strongly.
DECODE_STEPS = {"decode_llama3_8b_b1": 1, "decode_llama3_8b_b16": 16, "decode_llama3_8b_b64": 64}
# The expert block of a Mixtral-8x7B-shaped mixture-of-experts layer: 4096 tokens, top-2 of 8
# experts, d 4096, ffn 14336, int4 group-64 expert weights; three grouped ragged products over
# 8192 (token, expert) pairs plus the routed weighted sum.
MOE_BLOCKS = {"moe_mixtral_t4096": (4096, 2, 8, 4096, 14336)}
# DRAM bytes (read + write) of one launch of the dominant kernel, from the ncu captures
# summarized under profiles/ (qmm_gemm_tc_int4_g64_m2048.md, qmm_gemv_int4_g64_m1_4096x4096.md).
MEASURED_TRAFFIC = {
    "prefill_int4_g64_m2048_14336x4096": 56048384 + 27941888,    # read + write; part of y is still in L2
    "decode_int4_g64_m1_4096x4096": 9480000,                      # every weight byte read once
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


def work_of(name):
    """Algorithmic flops and bytes of one call (weights + tables + activations + output)."""
    m, k, n, gs, bits, mode = WORKLOADS[name]
    flops = 2.0 * m * k * n
    tables = n * (k // gs) * (1 if mode == "mxfp4" else 4)      # E8M0 bytes, or bf16 scale + bias
    weight_bytes = n * k * bits // 8 + tables
    total_bytes = weight_bytes + m * k * 2 + m * n * 2
    return flops, weight_bytes, total_bytes


def make_inputs(name, seed, torch, device, sets):
    """`sets` independent synthetic problems of one workload, resident on `device`."""
    m, k, n, gs, bits, mode = WORKLOADS[name]
    g = torch.Generator(device=device).manual_seed(seed)
    out = []
    for _ in range(sets):
        x = torch.randn((m, k), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        words = n * k * bits // 32
        w = torch.randint(-(1 << 31), (1 << 31) - 1, (words,), generator=g, device=device,
                          dtype=torch.int64).to(torch.int32).reshape(n, -1).view(torch.uint32)
        if mode == "mxfp4":
            s = torch.randint(119, 128, (n, k // 32), generator=g, device=device).to(torch.uint8)
            b = None
        else:
            lo = 0.002 if m > 16 else 0.005
            s = (torch.rand((n, k // gs), generator=g, device=device) * (0.02 - lo) + lo).to(torch.bfloat16)
            b = (-(float(1 << (bits - 1))) * s.float()).to(torch.bfloat16)
        y = torch.empty((m, n), device=device, dtype=torch.bfloat16)
        out.append((x, w, s, b, y))
    return out


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while a timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "50"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
            time.sleep(0.3)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.1)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        return False

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.path or not os.path.exists(self.path):
            return out
        sm, smax, reasons = [], [], set()
        for line in open(self.path):
            f = [c.strip() for c in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            busy = [v for v in sm if v >= 0.5 * max(sm)] or sm
            out.update(sm_mhz=statistics.median(busy), sm_max_mhz=max(smax),
                       reasons=sorted(reasons), samples=len(sm))
        return out


def time_device(fn, steps, warmup, torch, dist=None):
    """`steps` calls of `fn(i)` between CUDA events on the current stream; ms total."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        fn(warmup + i)
    stop.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    return start.elapsed_time(stop)


def cpu_baseline(name, budget_rows=None):
    """The CPU restatement of the fused dequantize-and-dot, all host threads, on a bounded
    sample: the first `rows` rows of x against the whole weight."""
    from oracle import clib
    from oracle import qmm_oracle as O
    import ml_dtypes
    m, k, n, gs, bits, mode = WORKLOADS[name]
    clib.use_all_cores()
    rng = np.random.default_rng(0)
    rows = min(m, budget_rows or (64 if m > 1 else 1))
    w = rng.integers(0, 1 << 32, size=(n, k * bits // 32), dtype=np.uint64).astype(np.uint32)
    if mode == "mxfp4":
        s = rng.integers(119, 128, size=(n, k // 32)).astype(np.uint8)
        b = None
    else:
        s = rng.uniform(0.002, 0.02, size=(n, k // gs)).astype(ml_dtypes.bfloat16)
        b = (-(float(1 << (bits - 1))) * s.astype(np.float32)).astype(ml_dtypes.bfloat16)
    x = rng.standard_normal((rows, k)).astype(np.float32).astype(ml_dtypes.bfloat16)
    clib.qmm(x[:1], w, s, b, 1, k, n, gs, bits, mode)                  # warm the threads
    reps, t0 = 0, time.perf_counter()
    while True:
        clib.qmm(x, w, s, b, rows, k, n, gs, bits, mode)
        reps += 1
        dt = time.perf_counter() - t0
        if dt > 3.0 or reps >= 200:
            break
    per_call = dt / reps
    return {"seconds_per_sample": per_call, "rows": rows, "cores": clib.num_threads(),
            "flops": 2.0 * rows * k * n, "reps": reps}


def run_reference(args, rank):
    """The reference arm: the reference's CPU path for this op (its fused dequantize-and-dot,
    restated in oracle/qmm_oracle.c because the reference itself needs jax + mlx, which are
    not installed) on the host cores, same workload and metric, bounded sample per step."""
    if rank != 0:
        return
    name = args.workload
    if name in DECODE_STEPS:
        vals = [decode_step_cpu(DECODE_STEPS[name]) for _ in range(args.warmup + args.steps)][args.warmup:]
        value = statistics.mean(v["value"] for v in vals)
        cb = dict(vals[-1], value=value)
        print(json.dumps({
            "impl": "reference", "metric": "decode_tok_s", "value": value, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": DECODE_STEPS[name] / value * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": name, "batch": DECODE_STEPS[name]}, "cpu_baseline": cb,
            "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}), flush=True)
        return
    m, k, n, gs, bits, mode = WORKLOADS[name]
    flops, weight_bytes, _ = work_of(name)
    res = None
    per = []
    for i in range(args.warmup + args.steps):
        res = cpu_baseline(name)
        if i >= args.warmup:
            per.append(res["seconds_per_sample"])
    sec = statistics.mean(per)
    if m > 1:
        value, unit = res["flops"] / sec / 1e12, "TFLOP/s"
    else:
        value, unit = weight_bytes / sec / 1e9, "GB/s"
    sample = f"first {res['rows']} of {m} rows of x against the whole weight, {res['reps']} calls per step"
    line = {
        "impl": "reference", "metric": metric_name(name), "value": value, "unit": unit,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3 * (m / res["rows"]), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": name, "M": m, "K": k, "N": n, "group_size": gs, "bits": bits,
                   "mode": mode},
        "cpu_baseline": {"value": value, "unit": unit, "cores": res["cores"], "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def metric_name(name):
    m = WORKLOADS[name][0]
    return "qmm_tflops_m%d" % m if m > 1 else "qmm_weight_gbs_m1"


def measure(name, args, torch, qmm, _lib, dist, device):
    """Device-resident and end-to-end timing of one workload on this rank."""
    m, k, n, gs, bits, mode = WORKLOADS[name]
    flops, weight_bytes, total_bytes = work_of(name)
    per_set = total_bytes
    sets = max(2, int(2 * L2_BYTES // per_set) + 1)                   # rotate through > 2x L2
    sets = min(sets, 64)
    data = make_inputs(name, 1234 + int(os.environ.get("RANK", "0")), torch, device, sets)
    kw = dict(group_size=gs, bits=bits, mode=mode)

    def step(i):
        x, w, s, b, y = data[i % sets]
        qmm.quantized_matmul(x, w, s, b, out=y, **kw)

    steps = args.steps if m > 1 else args.steps * 50
    warm = max(args.warmup, 3)
    n0 = _lib.launch_count()
    ms = time_device(step, steps, warm, torch, dist)
    launches = _lib.launch_count() - n0 - warm
    if m > 1:
        # The same K steps replayed from one CUDA graph: with several ranks on one host the
        # per-call Python time of eight processes can exceed a 0.26 ms step and starve the GPU,
        # which measures the host, not the path. The smaller of the two times is reported.
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(steps):
                    step(warm + i)
        torch.cuda.current_stream().wait_stream(side)
        gms = time_device(lambda i: graph.replay(), 1, 3, torch, dist)
        timed = "stream launches"
        if gms < ms:
            ms, timed = gms, "cuda graph replay of the K steps"
    else:
        timed = "stream launches"
    res = {"ms_total": ms, "steps": steps, "ms_per_step": ms / steps, "launches": launches, "timed": timed,
           "sets": sets, "flops": flops, "weight_bytes": weight_bytes, "total_bytes": total_bytes}

    # decode calls are launch-latency sized: also time them replayed from one CUDA graph,
    # every node on a different weight set
    if m == 1:
        gsteps = sets
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            for i in range(3):
                step(i)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for i in range(gsteps):
                    step(i)
        torch.cuda.synchronize()
        reps = max(5, steps // gsteps)
        gms = time_device(lambda i: graph.replay(), reps, 3, torch, dist)
        res["graph_ms_per_step"] = gms / (reps * gsteps)

    # end to end: pinned host x in, y out, through the public call
    x, w, s, b, y = data[0]
    hx = [torch.empty_like(x, device="cpu").pin_memory().copy_(data[i % sets][0]) for i in range(2)]
    hy = torch.empty_like(y, device="cpu").pin_memory()
    dx = torch.empty_like(x)

    def e2e_step(i):
        dx.copy_(hx[i % 2], non_blocking=True)
        xx, ww, ss, bb, yy = data[i % sets]
        qmm.quantized_matmul(dx, ww, ss, bb, out=yy, **kw)
        hy.copy_(yy, non_blocking=True)
        torch.cuda.current_stream().synchronize()                     # the caller reads y

    esteps = max(3, min(steps, 20))
    ems = time_device(e2e_step, esteps, 3, torch, dist)
    res["e2e_ms_per_step"] = ems / esteps
    res["h2d"] = x.numel() * x.element_size()
    res["d2h"] = y.numel() * y.element_size()
    return res


def decode_step_bytes(batch, world):
    """Algorithmic HBM bytes one rank touches per decode step: its shard of the packed weights
    and tables, and its heads' KV cache of `batch` sequences."""
    from metaljax_b200 import llama
    sh = llama.LLAMA3_8B
    kv = 2 * sh.layers * batch * sh.kv_heads * sh.ctx * sh.head_dim * 2
    return sh.weight_bytes() / world, kv / world


def measure_decode_step(batch, steps, warmup, torch, dist, device):
    """One Llama-3-8B-shaped decode step per timed step, replayed from a CUDA graph: device
    time (tokens resident) and end to end (token ids from pinned host memory, next ids back)."""
    from metaljax_b200 import _lib, llama
    n0 = _lib.launch_count()
    step = llama.DecodeStep(llama.LLAMA3_8B, batch, device, seed=7)
    n1 = _lib.launch_count()
    step.capture(warmup=max(warmup, 3))
    per_step = (_lib.launch_count() - n1) // (max(warmup, 3) + 1)
    del n0
    ms = time_device(lambda i: step.replay(), steps, 3, torch, dist)
    host_in = torch.zeros((batch,), dtype=torch.int64).pin_memory()
    host_out = torch.zeros((batch,), dtype=torch.int64).pin_memory()

    def e2e_step(i):
        host_in.fill_(i % 1000)
        step.tokens.copy_(host_in, non_blocking=True)
        step.replay()
        host_out.copy_(step.next_tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    esteps = max(3, min(steps, 20))
    ems = time_device(e2e_step, esteps, 3, torch, dist)
    res = {"ms_per_step": ms / steps, "e2e_ms_per_step": ems / esteps, "launches_per_step": per_step,
           "h2d": batch * 8, "d2h": batch * 8, "steps": steps, "gather": step.gather_mode}
    del step
    torch.cuda.empty_cache()
    return res


def decode_step_cpu(batch):
    """The CPU port on one decoder layer's linears at `batch` rows, extrapolated to the whole
    step by parameter count (the other 31 layers and the lm_head repeat the same loop)."""
    from oracle import clib
    import ml_dtypes
    from metaljax_b200 import llama
    sh = llama.LLAMA3_8B
    clib.use_all_cores()
    rng = np.random.default_rng(0)
    shapes = [((sh.heads + 2 * sh.kv_heads) * sh.head_dim, sh.d_model), (sh.d_model, sh.heads * sh.head_dim),
              (2 * sh.ffn, sh.d_model), (sh.d_model, sh.ffn)]
    sec, params = 0.0, 0
    for n, k in shapes:
        w = rng.integers(0, 1 << 32, size=(n, k // 8), dtype=np.uint64).astype(np.uint32)
        s = rng.uniform(0.002, 0.02, size=(n, k // 64)).astype(ml_dtypes.bfloat16)
        b = (-8.0 * s.astype(np.float32)).astype(ml_dtypes.bfloat16)
        x = rng.standard_normal((batch, k)).astype(np.float32).astype(ml_dtypes.bfloat16)
        clib.qmm(x[:1], w, s, b, 1, k, n, 64, 4, "affine")
        t0 = time.perf_counter()
        clib.qmm(x, w, s, b, batch, k, n, 64, 4, "affine")
        sec += time.perf_counter() - t0
        params += n * k
    step_sec = sec * sh.linear_params() / params
    return {"value": batch / step_sec, "unit": "tok/s", "cores": clib.num_threads(), "kind": "port",
            "sample": f"the 4 fused linears of one of {sh.layers} layers at {batch} rows "
                      f"({sec:.2f} s), extrapolated to the step by parameter count; attention and glue not counted"}


def decode_step_line(name, args, torch, dist, device, world, pk, clk_fn=None):
    batch = DECODE_STEPS[name]
    res = measure_decode_step(batch, args.steps, args.warmup, torch, dist, device)
    t = torch.tensor([res["ms_per_step"], res["e2e_ms_per_step"]], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step, e2e_ms = float(t[0]), float(t[1])
    wb, kvb = decode_step_bytes(batch, world)
    achieved = (wb + kvb) / (res["ms_per_step"] * 1e-3) / 1e9
    return {
        "metric": "decode_tok_s", "value": batch / (ms_step * 1e-3), "unit": "tok/s", "n_gpus": world,
        "steps": res["steps"], "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": name, "batch": batch, "layers": 32, "d_model": 4096, "ffn": 14336, "vocab": 128256,
                   "context": 2048, "group_size": 64, "bits": 4,
                   "l2": f"one step streams {wb / 2**20:.0f} MiB of weights per GPU (> L2)",
                   "parallelism": f"tp{world}: every weight sharded on its output rows, all-gather after each linear"
                                  + {"none": "", "peer": " (one-shot peer-store kernel over NVLink)",
                                     "nccl": " (NCCL)", "skip": " (exchange left out: timing experiment)"}[res["gather"]],
                   "timed": "cuda graph replay of the whole step"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"],
                     "bytes": "this rank's packed weights + tables and its KV cache, read once per step"},
        "e2e": {"value": batch / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": res["h2d"],
                "d2h_bytes_per_step": res["d2h"], "ms_per_step": e2e_ms},
        "gpu_launches": int(res["launches_per_step"] * res["steps"]),
    }


def moe_line(name, args, torch, dist, device, world, pk):
    """One step = the whole expert block (`moe.moe_experts`) on this rank's own tokens."""
    from metaljax_b200 import _lib, moe
    t, k, e, d, f = MOE_BLOCKS[name]
    g = torch.Generator(device=device).manual_seed(11 + int(os.environ.get("RANK", "0")))

    def pack(n, kk):
        w = torch.randint(-(1 << 31), (1 << 31) - 1, (e, n, kk // 8), generator=g, device=device,
                          dtype=torch.int64).to(torch.int32).view(torch.uint32)
        s = (torch.rand((e, n, kk // 64), generator=g, device=device) * 0.018 + 0.002).to(torch.bfloat16)
        return w, s, (-8.0 * s.float()).to(torch.bfloat16)

    w1, w3, w2 = pack(f, d), pack(f, d), pack(d, f)
    sets = 3
    xs = [(torch.randn((t, d), generator=g, device=device) * 0.5).to(torch.bfloat16) for _ in range(sets)]
    logits = torch.randn((t, e), generator=g, device=device)
    wts, idx = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    wts = (wts / wts.sum(-1, keepdim=True)).float()
    flops = 2.0 * t * k * (3 * d * f)
    n0 = _lib.launch_count()
    ms = time_device(lambda i: moe.moe_experts(xs[i % sets], idx, wts, w1, w3, w2), args.steps, max(args.warmup, 3),
                     torch, dist)
    launches = (_lib.launch_count() - n0) * args.steps // (args.steps + max(args.warmup, 3))
    hx = torch.empty_like(xs[0], device="cpu").pin_memory().copy_(xs[0])
    hy = torch.empty_like(xs[0], device="cpu").pin_memory()
    dx = torch.empty_like(xs[0])

    def e2e_step(i):
        dx.copy_(hx, non_blocking=True)
        y = moe.moe_experts(dx, idx, wts, w1, w3, w2)
        hy.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    esteps = max(3, min(args.steps, 10))
    ems = time_device(e2e_step, esteps, 3, torch, dist)
    tt = torch.tensor([ms / args.steps, ems / esteps], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms_step, e2e_ms = float(tt[0]), float(tt[1])
    achieved = flops / (ms / args.steps * 1e-3) / 1e12
    return {
        "metric": "moe_block_tflops", "value": world * flops / (ms_step * 1e-3) / 1e12, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": name, "tokens": t, "top_k": k, "experts": e, "d_model": d, "ffn": f, "group_size": 64,
                   "bits": 4, "l2": f"{3 * e * d * f // 2 >> 20} MiB of expert weights per step (> L2)",
                   "parallelism": f"dp{world}: every rank routes its own tokens against replicated experts",
                   "includes": "pair sort, 3 grouped ragged products, SwiGLU, routed weighted sum"},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": achieved / pk["bf16_tflops"], "traffic": None, "peak_source": pk["source"]},
        "e2e": {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": t * d * 2, "d2h_bytes_per_step": t * d * 2, "ms_per_step": e2e_ms},
        "gpu_launches": int(launches),
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=DEFAULT, choices=sorted(WORKLOADS) + sorted(DECODE_STEPS) + sorted(MOE_BLOCKS))
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-also", action="store_true", help="skip the decode side measurement")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    from metaljax_b200 import _lib, qmm
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the fused op has no CPU path")
    _lib.lib()
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=device)
        dist = dist_mod

    name = args.workload
    pk = peaks()
    if name in DECODE_STEPS or name in MOE_BLOCKS:
        with ClockSampler(local) as clocks:
            line = (decode_step_line if name in DECODE_STEPS else moe_line)(name, args, torch, dist, device, world, pk)
        line["clocks"] = clocks.summary()
        _lib.poll_status()
        if rank == 0 and not args.no_cpu and name in DECODE_STEPS:
            line["cpu_baseline"] = decode_step_cpu(DECODE_STEPS[name])
        if rank == 0:
            print(json.dumps(line), flush=True)
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return
    m, k, n, gs, bits, mode = WORKLOADS[name]
    with ClockSampler(local) as clocks:
        res = measure(name, args, torch, qmm, _lib, dist, device)
    clk = clocks.summary()
    _lib.poll_status()

    # max over ranks of the timed region; work summed over ranks
    t = torch.tensor([res["ms_per_step"], res["e2e_ms_per_step"]], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step, e2e_ms = float(t[0]), float(t[1])
    flops, weight_bytes, total_bytes = res["flops"], res["weight_bytes"], res["total_bytes"]
    if m > 1:
        unit = "TFLOP/s"
        value = world * flops / (ms_step * 1e-3) / 1e12
        e2e_value = world * flops / (e2e_ms * 1e-3) / 1e12
        achieved = flops / (res["ms_per_step"] * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": achieved, "peak": pk["bf16_tflops"], "unit": unit,
                "frac": achieved / pk["bf16_tflops"], "traffic": MEASURED_TRAFFIC.get(name),
                "peak_source": pk["source"],
                "frac_of_nominal_2250": achieved / 2250.0}
    else:
        unit = "GB/s"
        value = world * weight_bytes / (ms_step * 1e-3) / 1e9
        e2e_value = world * weight_bytes / (e2e_ms * 1e-3) / 1e9
        best = min(res["ms_per_step"], res.get("graph_ms_per_step", 1e9))
        achieved = total_bytes / (best * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": unit,
                "frac": achieved / pk["hbm_gbs"], "traffic": MEASURED_TRAFFIC.get(name),
                "peak_source": pk["source"], "frac_of_nominal_8000": achieved / 8000.0,
                "timed": "cuda graph replay" if best != res["ms_per_step"] else "stream launches"}

    line = {
        "metric": metric_name(name), "value": value, "unit": unit, "n_gpus": world,
        "steps": res["steps"], "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": name, "M": m, "K": k, "N": n, "group_size": gs, "bits": bits,
                   "mode": mode, "route": qmm.route(m, k, n, gs, bits, mode),
                   "l2": f"inputs rotate through {res['sets']} sets ({res['sets'] * total_bytes >> 20} MiB > 2x L2)",
                   "parallelism": f"dp{world}: rows of x sharded, weights replicated, no collective",
                   "timed": res.get("timed", "stream launches")},
        "roofline": roof,
        "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": res["h2d"],
                "d2h_bytes_per_step": res["d2h"], "ms_per_step": e2e_ms},
        "gpu_launches": int(res["launches"]),
        "clocks": clk,
    }

    if rank == 0 and not args.no_also and name == DEFAULT and world == 1:
        side = measure(DECODE, args, torch, qmm, _lib, None, device)
        _, wb, tb = work_of(DECODE)
        best = min(side["ms_per_step"], side.get("graph_ms_per_step", 1e9))
        line["also"] = [{
            "workload": DECODE, "metric": "qmm_weight_gbs_m1",
            "value": wb / (best * 1e-3) / 1e9, "unit": "GB/s",
            "us_per_call_stream": side["ms_per_step"] * 1e3,
            "us_per_call_graph": side.get("graph_ms_per_step", float("nan")) * 1e3,
            "route": qmm.route(1, 4096, 4096),
            "roofline": {"bound": "hbm", "achieved": tb / (best * 1e-3) / 1e9, "peak": pk["hbm_gbs"],
                         "unit": "GB/s", "frac": tb / (best * 1e-3) / 1e9 / pk["hbm_gbs"],
                         "traffic": MEASURED_TRAFFIC.get(DECODE), "peak_source": pk["source"]},
        }]

    if not args.no_also and name == DEFAULT:
        # the decode-step tokens/s at this N (weights sharded on N: strong scaling), all ranks
        for side_name in ("decode_llama3_8b_b1", "decode_llama3_8b_b16", "decode_llama3_8b_b64"):
            side_line = decode_step_line(side_name, args, torch, dist, device, world, pk)
            line.setdefault("also", []).append(
                {key: side_line[key] for key in ("metric", "value", "unit", "n_gpus", "ms_per_step", "scaling",
                                                 "config", "roofline", "e2e", "gpu_launches")})

    if rank == 0 and not args.no_cpu and world >= 1:
        cb = cpu_baseline(name)
        if m > 1:
            cval = cb["flops"] / cb["seconds_per_sample"] / 1e12
        else:
            cval = weight_bytes / cb["seconds_per_sample"] / 1e9
        line["cpu_baseline"] = {
            "value": cval, "unit": unit, "cores": cb["cores"], "kind": "port",
            "sample": f"first {cb['rows']} of {m} rows of x against the whole weight, "
                      f"{cb['reps']} calls in {cb['seconds_per_sample'] * cb['reps']:.1f} s"}

    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
