"""Benchmark of the fused quantized matmul and its decode-step caller on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]
                    [--decode-sharding auto|rows|weights]

One JSON line on stdout (rank 0). The default workload is the path that shards over GPUs: one
decode step of a Llama-3-8B-shaped model (32 layers, d 4096, 32/8 heads, ffn 14336, vocabulary
128256, every linear an int4 group-64 quantized matmul, bf16 KV cache of 2048 positions) at
batch 64. Over N ranks the step is split by its sequences where the batch divides by N (every
rank steps batch / N sequences with the whole weights and their KV cache, nothing exchanged:
above a few rows the step is bound by per-sequence work, not by the weight bytes), else by its
weights (the linears sharded on their output rows, q/k/v by head so that the KV cache and
attention stay local, the slices exchanged over NVLink); `--decode-sharding` forces one, and
`also` carries the weight-sharded step beside the sequence-sharded one. `value` is tokens/s of
the whole job with everything resident in HBM, the step replayed from one CUDA graph; `e2e` is
the same through the public call with token ids copied in from pinned host memory and the next
ids copied back inside the timed region; `roofline` is this rank's packed weights + tables + KV
cache per step against the measured HBM bandwidth; `cpu_baseline` is the CPU restatement of the
reference's fused dequantize-and-dot loop timed on the host cores on a bounded sample.

`also` carries, at N = 1, every other configuration of the path -- the single quantized matmul
at M = 1 (GB/s of weight bytes) and M = 2048 (TFLOP/s) in int4 / int8 at both Llama MLP shapes,
MXFP4 at M = 1 / 512 / 4096, the Mixtral-shaped expert block, the decode step at batch 1 and 16
-- each with its own roofline; at N > 1 the decode step at the other batches, the
expert-parallel expert block (rows exchanged through peer memory), and `parity`: the decode step
in both splits and the expert-parallel block checked at small shapes against their references
before anything is timed.
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
    "prefill_int8_g128_m2048_4096x14336": (2048, 14336, 4096, 128, 8, "affine"),
    "prefill_mxfp4_m512_5760x2880": (512, 2880, 5760, 32, 4, "mxfp4"),
    "prefill_mxfp4_m4096_5760x2880": (4096, 2880, 5760, 32, 4, "mxfp4"),
    "decode_int4_g64_m1_4096x4096": (1, 4096, 4096, 64, 4, "affine"),
    "decode_int4_g64_m1_28672x4096": (1, 4096, 28672, 64, 4, "affine"),
    "decode_int4_g64_m1_65536x4096": (1, 4096, 65536, 64, 4, "affine"),
    "decode_int4_g64_m8_28672x4096": (8, 4096, 28672, 64, 4, "affine"),     # what a rank runs with 64 sequences on 8 GPUs
    "decode_mxfp4_m1_5760x2880": (1, 2880, 5760, 32, 4, "mxfp4"),
}
L2_BYTES = 126 * 1024 * 1024
STREAM_ROWS = 16      # up to this many rows a product is a weight stream (GB/s against HBM), above it a GEMM (TFLOP/s)
# Whole decode steps of the Llama-3-8B-shaped model: name -> batch. The weights are sharded on N
# over the ranks, so these scale strongly.
DECODE_STEPS = {"decode_llama3_8b_b1": 1, "decode_llama3_8b_b8": 8, "decode_llama3_8b_b16": 16, "decode_llama3_8b_b32": 32,
                "decode_llama3_8b_b64": 64}
DEFAULT = "decode_llama3_8b_b64"
ALSO_STEPS = ["decode_llama3_8b_b1", "decode_llama3_8b_b16", "decode_llama3_8b_b64"]     # the batches the configs name
# The expert block of a Mixtral-8x7B-shaped mixture-of-experts layer: 4096 tokens, top-2 of 8
# experts, d 4096, ffn 14336, int4 group-64 expert weights; three grouped ragged products over
# 8192 (token, expert) pairs plus the routed weighted sum. Over N ranks: experts split, tokens
# split, pairs exchanged through peer memory (QMM_EP_EXCHANGE=nccl: by all-to-all collectives).
MOE_BLOCKS = {"moe_mixtral_t4096": (4096, 2, 8, 4096, 14336)}
ALSO_AT_ONE = ["decode_int4_g64_m1_4096x4096", "decode_int4_g64_m1_65536x4096", "prefill_int4_g64_m2048_14336x4096", "prefill_int4_g64_m2048_4096x14336",
               "prefill_int8_g128_m2048_14336x4096", "prefill_int8_g128_m2048_4096x14336", "decode_mxfp4_m1_5760x2880",
               "prefill_mxfp4_m512_5760x2880", "prefill_mxfp4_m4096_5760x2880", "moe_mixtral_t4096"]


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


def measured_traffic(name):
    """DRAM bytes (read + write) of one launch of the workload's dominant kernel, from the ncu
    capture recorded next to the profile summaries; None when no capture has been recorded."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        entry = json.load(f).get(name)
    return None if entry is None else entry["bytes_per_launch"]


def work_of(name):
    """Algorithmic flops and bytes of one call (weights + tables + activations + output)."""
    m, k, n, gs, bits, mode = WORKLOADS[name]
    flops = 2.0 * m * k * n
    tables = n * (k // gs) * (1 if mode == "mxfp4" else 4)      # E8M0 bytes, or bf16 scale + bias
    weight_bytes = n * k * bits // 8 + tables
    total_bytes = weight_bytes + m * k * 2 + m * n * 2
    return flops, weight_bytes, total_bytes


DECODE_SHARDING = "auto"      # --decode-sharding


def decode_sharding(batch, world):
    """How a decode step of `batch` sequences is split over `world` ranks: "rows" (every rank steps
    batch / N sequences with the whole weights, nothing exchanged) where the batch divides, else
    "weights" (every linear split on its output rows, every rank steps every sequence). Above a few
    rows a step is bound by per-sequence work -- the KV cache and the tensor-core kernel's cost per
    weight block -- not by the weight bytes, which is why the sequences are what to split."""
    if world == 1:
        return "weights"
    if DECODE_SHARDING != "auto":
        return DECODE_SHARDING
    return "rows" if batch % world == 0 else "weights"


def config_of(name, world, sharding=None):
    """What the workload is; both arms print exactly this."""
    if name in DECODE_STEPS:
        sharding = sharding or decode_sharding(DECODE_STEPS[name], world)
        return {"workload": name, "batch": DECODE_STEPS[name], "layers": 32, "d_model": 4096, "heads": 32, "kv_heads": 8,
                "ffn": 14336, "vocab": 128256, "context": 2048, "group_size": 64, "bits": 4,
                "weights": "N(0, 0.02) quantized per group of 64: scale = (max - min)/15, zero = round(-min/scale)",
                "parallelism": (f"dp{world}: the sequences split over the ranks (batch / N each), whole weights on every rank, "
                                "nothing exchanged" if sharding == "rows" else
                                f"tp{world}: every linear sharded on its output rows, slices exchanged after it"),
                "l2": ("one step streams the packed weights (4.2 GB) and this rank's sequences' KV cache: far more than L2"
                       if sharding == "rows" else
                       "one step streams this rank's packed weights (4.2 GB / N) and KV cache: far more than L2")}
    if name in MOE_BLOCKS:
        t, k, e, d, f = MOE_BLOCKS[name]
        return {"workload": name, "tokens": t, "top_k": k, "experts": e, "d_model": d, "ffn": f, "group_size": 64, "bits": 4,
                "parallelism": f"ep{world}: experts and tokens split over the ranks, pairs exchanged between them"
                if world > 1 else "ep1",
                "l2": f"{3 * e * d * f // 2 >> 20} MiB of expert weights per step (> L2)"}
    m, k, n, gs, bits, mode = WORKLOADS[name]
    _, _, total = work_of(name)
    sets = rotation_sets(total)
    return {"workload": name, "M": m, "K": k, "N": n, "group_size": gs, "bits": bits, "mode": mode,
            "parallelism": f"dp{world}: rows of x sharded, weights replicated, no collective",
            "l2": f"inputs rotate through {sets} sets ({sets * total >> 20} MiB > 2x L2)"}


def rotation_sets(total_bytes):
    return min(64, max(2, int(2 * L2_BYTES // total_bytes) + 1))


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


PROFILE_WINDOW = False


def time_device(fn, steps, warmup, torch, dist=None):
    """`steps` calls of `fn(i)` between CUDA events on the current stream; ms total."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if PROFILE_WINDOW:                 # a profiler started with --profile-from-start off sees the timed steps only
        torch.cuda.profiler.start()
    start.record()
    for i in range(steps):
        fn(warmup + i)
    stop.record()
    torch.cuda.synchronize()
    if PROFILE_WINDOW:
        torch.cuda.profiler.stop()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    return start.elapsed_time(stop)


def max_over_ranks(values, torch, dist, device):
    t = torch.tensor(values, device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t]


# ---- the CPU legs ----------------------------------------------------------------------------


def cpu_qmm_sample(name, budget_rows=None):
    """The CPU restatement of the fused dequantize-and-dot, all host threads, on a bounded
    sample: the first `rows` rows of x against the whole weight."""
    from oracle import clib
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
    return {"seconds_per_sample": dt / reps, "rows": rows, "cores": clib.num_threads(),
            "flops": 2.0 * rows * k * n, "reps": reps}


def cpu_baseline_of(name):
    """`cpu_baseline` object of one workload (value in the workload's own unit)."""
    if name in DECODE_STEPS:
        return decode_step_cpu(DECODE_STEPS[name])
    if name in MOE_BLOCKS:
        return moe_block_cpu(name)
    m = WORKLOADS[name][0]
    _, weight_bytes, _ = work_of(name)
    cb = cpu_qmm_sample(name)
    val = cb["flops"] / cb["seconds_per_sample"] / 1e12 if m > STREAM_ROWS else weight_bytes / cb["seconds_per_sample"] / 1e9
    return {"value": val, "unit": "TFLOP/s" if m > STREAM_ROWS else "GB/s", "cores": cb["cores"], "kind": "port",
            "sample": f"first {cb['rows']} of {m} rows of x against the whole weight, "
                      f"{cb['reps']} calls in {cb['seconds_per_sample'] * cb['reps']:.1f} s"}


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


def moe_block_cpu(name):
    """The CPU port on 16 of the block's 8192 pair rows through one expert's three projections."""
    from oracle import clib
    import ml_dtypes
    t, k, e, d, f = MOE_BLOCKS[name]
    clib.use_all_cores()
    rng = np.random.default_rng(0)
    rows, sec = 16, 0.0
    for n, kk in ((f, d), (f, d), (d, f)):
        w = rng.integers(0, 1 << 32, size=(n, kk // 8), dtype=np.uint64).astype(np.uint32)
        s = rng.uniform(0.002, 0.02, size=(n, kk // 64)).astype(ml_dtypes.bfloat16)
        b = (-8.0 * s.astype(np.float32)).astype(ml_dtypes.bfloat16)
        x = rng.standard_normal((rows, kk)).astype(np.float32).astype(ml_dtypes.bfloat16)
        clib.qmm(x[:1], w, s, b, 1, kk, n, 64, 4, "affine")
        t0 = time.perf_counter()
        clib.qmm(x, w, s, b, rows, kk, n, 64, 4, "affine")
        sec += time.perf_counter() - t0
    flops = 2.0 * rows * 3 * d * f
    return {"value": flops / sec / 1e12, "unit": "TFLOP/s", "cores": clib.num_threads(), "kind": "port",
            "sample": f"{rows} of {t * k} pair rows through one expert's three projections ({sec:.2f} s)"}


def metric_of(name):
    if name in DECODE_STEPS:
        return "decode_tok_s", "tok/s"
    if name in MOE_BLOCKS:
        return "moe_block_tflops", "TFLOP/s"
    m = WORKLOADS[name][0]
    return ("qmm_tflops_m%d" % m, "TFLOP/s") if m > STREAM_ROWS else ("qmm_weight_gbs_m%d" % m, "GB/s")


def run_reference(args, rank):
    """The reference arm: the reference's CPU path for this workload (its fused
    dequantize-and-dot, restated in oracle/qmm_oracle.c because the reference itself needs jax +
    mlx, which are not installed) on the host cores, same workload and metric, a bounded sample
    per step."""
    if rank != 0:
        return
    name = args.workload
    metric, unit = metric_of(name)
    vals = []
    cb = None
    for i in range(args.warmup + args.steps):
        cb = cpu_baseline_of(name)
        if i >= args.warmup:
            vals.append(cb["value"])
    value = statistics.mean(vals)
    if name in DECODE_STEPS:
        ms = DECODE_STEPS[name] / value * 1e3
    elif name in MOE_BLOCKS:
        t, k, e, d, f = MOE_BLOCKS[name]
        ms = 2.0 * t * k * 3 * d * f / (value * 1e12) * 1e3
    else:
        flops, wb, _ = work_of(name)
        ms = (flops / (value * 1e12) if WORKLOADS[name][0] > STREAM_ROWS else wb / (value * 1e9)) * 1e3
    print(json.dumps({
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong" if name in DECODE_STEPS or name in MOE_BLOCKS else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": config_of(name, args.gpus),
        "cpu_baseline": dict(cb, value=value),
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}), flush=True)


# ---- the single quantized matmul ---------------------------------------------------------------


def measure_qmm(name, args, torch, qmm, _lib, dist, device):
    """Device-resident and end-to-end timing of one quantized-matmul workload on this rank."""
    m, k, n, gs, bits, mode = WORKLOADS[name]
    flops, weight_bytes, total_bytes = work_of(name)
    sets = rotation_sets(total_bytes)
    data = make_inputs(name, 1234 + int(os.environ.get("RANK", "0")), torch, device, sets)
    kw = dict(group_size=gs, bits=bits, mode=mode)

    def step(i):
        x, w, s, b, y = data[i % sets]
        qmm.quantized_matmul(x, w, s, b, out=y, **kw)

    steps = args.steps if m > STREAM_ROWS else args.steps * 50
    warm = max(args.warmup, 3)
    n0 = _lib.launch_count()
    ms = time_device(step, steps, warm, torch, dist)
    launches = _lib.launch_count() - n0 - warm
    # The same calls replayed from one CUDA graph (every node on a different weight set): a
    # decode call is launch-latency sized, and with several ranks on one host the per-call
    # Python time of eight processes can exceed a 0.26 ms step. The smaller time is reported.
    gsteps = steps if m > STREAM_ROWS else sets
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(gsteps):
                step(warm + i)
    torch.cuda.current_stream().wait_stream(side)
    reps = 1 if m > STREAM_ROWS else max(5, steps // gsteps)
    gms = time_device(lambda i: graph.replay(), reps, 3, torch, dist) / (reps * gsteps)
    timed = "stream launches"
    ms_step = ms / steps
    if gms < ms_step:
        ms_step, timed = gms, "cuda graph replay"
    res = {"steps": steps, "ms_per_step": ms_step, "launches": launches, "timed": timed, "sets": sets,
           "flops": flops, "weight_bytes": weight_bytes, "total_bytes": total_bytes}
    del graph

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


def qmm_line(name, args, torch, dist, device, world, pk):
    from metaljax_b200 import _lib, qmm
    m, k, n, gs, bits, mode = WORKLOADS[name]
    res = measure_qmm(name, args, torch, qmm, _lib, dist, device)
    ms_step, e2e_ms = max_over_ranks([res["ms_per_step"], res["e2e_ms_per_step"]], torch, dist, device)
    flops, weight_bytes, total_bytes = res["flops"], res["weight_bytes"], res["total_bytes"]
    metric, unit = metric_of(name)
    if m > STREAM_ROWS:
        value = world * flops / (ms_step * 1e-3) / 1e12
        e2e_value = world * flops / (e2e_ms * 1e-3) / 1e12
        achieved = flops / (res["ms_per_step"] * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": achieved, "peak": pk["bf16_tflops"], "unit": unit,
                "frac": achieved / pk["bf16_tflops"], "traffic": measured_traffic(name),
                "peak_source": pk["source"], "frac_of_nominal_2250": achieved / 2250.0}
    else:
        value = world * weight_bytes / (ms_step * 1e-3) / 1e9
        e2e_value = world * weight_bytes / (e2e_ms * 1e-3) / 1e9
        achieved = total_bytes / (res["ms_per_step"] * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": unit,
                "frac": achieved / pk["hbm_gbs"], "traffic": measured_traffic(name),
                "peak_source": pk["source"], "frac_of_nominal_8000": achieved / 8000.0,
                "us_per_call": res["ms_per_step"] * 1e3}
    return {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world,
        "steps": res["steps"], "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_of(name, world),
        "how": {"route": qmm.route(m, k, n, gs, bits, mode), "timed": res["timed"]},
        "roofline": roof,
        "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": res["h2d"],
                "d2h_bytes_per_step": res["d2h"], "ms_per_step": e2e_ms},
        "gpu_launches": int(res["launches"]),
    }


# ---- the decode step ------------------------------------------------------------------------------


def decode_step_bytes(batch, world, sharding="weights"):
    """Algorithmic HBM bytes one rank touches per decode step: its shard of the packed weights
    and tables (all of them when the sequences are what is split) and its share of the KV cache
    of `batch` sequences."""
    from metaljax_b200 import llama
    sh = llama.LLAMA3_8B
    kv = 2 * sh.layers * batch * sh.kv_heads * sh.ctx * sh.head_dim * 2
    return sh.weight_bytes() / (1 if sharding == "rows" else world), kv / world


def measure_decode_step(batch, steps, warmup, torch, dist, device, sharding="weights"):
    """One Llama-3-8B-shaped decode step per timed step, replayed from a CUDA graph: device
    time (tokens resident) and end to end (token ids from pinned host memory, next ids back;
    with the sequences split over the ranks every rank copies its own)."""
    from metaljax_b200 import _lib, llama
    step = llama.DecodeStep(llama.LLAMA3_8B, batch, device, seed=7, weights="normal", shard=sharding)
    batch_here = step.batch
    n1 = _lib.launch_count()
    step.capture(warmup=max(warmup, 3))
    per_step = (_lib.launch_count() - n1) // (max(warmup, 3) + 1)
    ms = time_device(lambda i: step.replay(), steps, 3, torch, dist)
    host_in = torch.zeros((batch_here,), dtype=torch.int64).pin_memory()
    host_out = torch.zeros((batch_here,), dtype=torch.int64).pin_memory()

    def e2e_step(i):
        host_in.fill_(i % 1000)
        step.tokens.copy_(host_in, non_blocking=True)
        step.replay()
        host_out.copy_(step.next_tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    esteps = max(3, min(steps, 20))
    ems = time_device(e2e_step, esteps, 3, torch, dist)
    res = {"ms_per_step": ms / steps, "e2e_ms_per_step": ems / esteps, "launches_per_step": per_step,
           "h2d": batch * 8, "d2h": batch * 8, "steps": steps, "exchange": step.exchange_description()}
    del step
    torch.cuda.empty_cache()
    return res


def decode_step_line(name, args, torch, dist, device, world, pk, sharding=None):
    batch = DECODE_STEPS[name]
    sharding = sharding or decode_sharding(batch, world)
    res = measure_decode_step(batch, args.steps, args.warmup, torch, dist, device, sharding)
    ms_step, e2e_ms = max_over_ranks([res["ms_per_step"], res["e2e_ms_per_step"]], torch, dist, device)
    wb, kvb = decode_step_bytes(batch, world, sharding)
    achieved = (wb + kvb) / (res["ms_per_step"] * 1e-3) / 1e9
    return {
        "metric": "decode_tok_s", "value": batch / (ms_step * 1e-3), "unit": "tok/s", "n_gpus": world,
        "steps": res["steps"], "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_of(name, world, sharding),
        "how": {"timed": "cuda graph replay of the whole step", "exchange": res["exchange"]},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"],
                     "bytes": ("the packed weights + tables and this rank's sequences' KV cache, read once per step"
                               if sharding == "rows" else
                               "this rank's packed weights + tables and its KV cache, read once per step")},
        "e2e": {"value": batch / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": res["h2d"],
                "d2h_bytes_per_step": res["d2h"], "ms_per_step": e2e_ms},
        "gpu_launches": int(res["launches_per_step"] * res["steps"]),
    }


# ---- the expert block -------------------------------------------------------------------------------


def moe_line(name, args, torch, dist, device, world, pk):
    """One step = the whole expert block: at N = 1 `moe.moe_experts` on all tokens, at N > 1
    `parallel.ExpertParallelMoE` with the tokens and the experts split over the ranks."""
    from metaljax_b200 import _lib, moe, parallel
    t, k, e, d, f = MOE_BLOCKS[name]
    rank = int(os.environ.get("RANK", "0"))
    g = torch.Generator(device=device).manual_seed(11)                     # the same experts on every rank
    gl = torch.Generator(device=device).manual_seed(100 + rank)            # this rank's tokens
    el = e // world if world > 1 else e

    def pack(n, kk):                                                        # this rank's experts only
        ws = []
        for ex in range(e):
            w = torch.randint(-(1 << 31), (1 << 31) - 1, (n, kk // 8), generator=g, device=device,
                              dtype=torch.int64).to(torch.int32).view(torch.uint32)
            s = (torch.rand((n, kk // 64), generator=g, device=device) * 0.018 + 0.002).to(torch.bfloat16)
            if world == 1 or ex // el == rank:
                ws.append((w, s))
        w = torch.stack([a for a, _ in ws])
        s = torch.stack([b_ for _, b_ in ws])
        return w, s, (-8.0 * s.float()).to(torch.bfloat16)

    w1, w3, w2 = pack(f, d), pack(f, d), pack(d, f)
    tl = t // world
    sets = 3
    xs = [(torch.randn((tl, d), generator=gl, device=device) * 0.5).to(torch.bfloat16) for _ in range(sets)]
    logits = torch.randn((tl, e), generator=gl, device=device)
    wts, idx = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    wts = (wts / wts.sum(-1, keepdim=True)).float()
    if world > 1:
        exchange = os.environ.get("QMM_EP_EXCHANGE", "peer")               # "nccl": all-to-all collectives
        block = parallel.ExpertParallelMoE(w1, w3, w2, group=None, local_experts=True,
                                           capacity_pairs=tl * k if exchange == "peer" else None)
        if exchange == "peer":
            # one call before anything is timed: if the exchange over peer memory does not come up on
            # every rank (no symmetric memory, a wait that ran out), every rank uses the collectives
            good = torch.ones((), device=device, dtype=torch.int32)
            try:
                block(xs[0], idx, wts)
                _lib.poll_status()
                if not block._peer:
                    good.zero_()
            except Exception:                                               # noqa: BLE001 -- decided together below
                good.zero_()
            dist.all_reduce(good, op=dist.ReduceOp.MIN)
            if int(good.item()) == 0:
                block = parallel.ExpertParallelMoE(w1, w3, w2, group=None, local_experts=True)
        run = lambda x: block(x, idx, wts)                                  # noqa: E731
    else:
        run = lambda x: moe.moe_experts(x, idx, wts, w1, w3, w2)            # noqa: E731
    flops = 2.0 * t * k * (3 * d * f)                                       # whole job
    warm = max(args.warmup, 3)
    n0 = _lib.launch_count()
    ms = time_device(lambda i: run(xs[i % sets]), args.steps, warm, torch, dist)
    launches = (_lib.launch_count() - n0) * args.steps // (args.steps + warm)
    hx = torch.empty_like(xs[0], device="cpu").pin_memory().copy_(xs[0])
    hy = torch.empty_like(xs[0], device="cpu").pin_memory()
    dx = torch.empty_like(xs[0])

    def e2e_step(i):
        dx.copy_(hx, non_blocking=True)
        y = run(dx)
        hy.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    esteps = max(3, min(args.steps, 10))
    ems = time_device(e2e_step, esteps, 3, torch, dist)
    ms_step, e2e_ms = max_over_ranks([ms / args.steps, ems / esteps], torch, dist, device)
    achieved = flops / world / (ms / args.steps * 1e-3) / 1e12               # this rank's share
    return {
        "metric": "moe_block_tflops", "value": flops / (ms_step * 1e-3) / 1e12, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_of(name, world),
        "how": {"includes": "pair sort, token exchange, 3 grouped ragged products, SwiGLU, routed weighted sum",
                "timed": "stream launches",
                "exchange": None if world == 1 else ("peer memory" if getattr(block, "_peer", None) else "nccl all-to-all")},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": achieved / pk["bf16_tflops"], "traffic": None, "peak_source": pk["source"]},
        "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": tl * d * 2, "d2h_bytes_per_step": tl * d * 2, "ms_per_step": e2e_ms},
        "gpu_launches": int(launches),
    }


# ---- parity of the sharded forms, checked before anything is timed (N > 1) ---------------------------


def parity_check(torch, dist, device, world, rank):
    """The N-sharded decode step against its float reference and the expert-parallel block
    against the oracle, at small shapes; returns the two relative errors (max over ranks)."""
    from metaljax_b200 import llama, parallel
    from oracle import qmm_oracle as O
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import activations, affine_case, to_numpy, to_torch
    shape = llama.Shape(layers=2, d_model=1024, heads=8, kv_heads=8, head_dim=64, ffn=2048, vocab=4096, ctx=64)
    errs = []
    for batch in (1, 5):
        fw = llama.random_full_weights(shape, batch, device, seed=3)                # identical on every rank
        step = llama.DecodeStep(shape, batch, device, full_weights=fw)
        tokens = torch.arange(batch, device=device) * 11 % shape.vocab
        step.tokens.copy_(tokens)
        first = step.step().clone()
        got = step.logits()
        want = llama.reference_logits(fw, shape, tokens, batch)
        errs.append((got - want).abs().max().item() / want.abs().max().item())
        for _ in range(3):                                                          # slots and flags cycle
            if not torch.equal(step.step(), first):
                errs.append(float("inf"))
        del step
    # the same step with the sequences split over the ranks (two and seventeen per rank: the fused
    # single-row path does not apply, the multi-row and the tensor-core kernels both do)
    for per_rank in (2, 17):
        batch = per_rank * world
        fw = llama.random_full_weights(shape, batch, device, seed=5)
        step = llama.DecodeStep(shape, batch, device, full_weights=fw, shard="rows")
        tokens = torch.arange(batch, device=device) * 13 % shape.vocab
        mine = slice(step.rows_rank * step.batch, (step.rows_rank + 1) * step.batch)
        step.tokens.copy_(tokens[mine])
        step.step()
        got = step.logits()
        want = llama.reference_logits(fw, shape, tokens, batch)[mine]
        errs.append((got - want).abs().max().item() / want.abs().max().item())
        del step
    rng = np.random.default_rng(0)
    e, kk, d, f, t = 8, 2, 256, 512, 64 + 8 * rank
    packs = [affine_case(rng, f, d, 64, 4, "bf16", lead=(e,))[1:], affine_case(rng, f, d, 64, 4, "bf16", lead=(e,))[1:],
             affine_case(rng, d, f, 64, 4, "bf16", lead=(e,))[1:]]
    block = parallel.ExpertParallelMoE(*[tuple(to_torch(a, device) for a in p) for p in packs],
                                       capacity_pairs=256 if os.environ.get("QMM_EP_EXCHANGE", "peer") == "peer" else None)
    rr = np.random.default_rng(100 + rank)
    x = activations(rr, (t, d), "bf16", 0.5)
    idx, wts = O.topk_router(rr.standard_normal((t, e)).astype(np.float32), kk)
    routed = (to_torch(x, device), torch.from_numpy(idx).to(device), torch.from_numpy(wts).to(device))
    good = torch.ones((), device=device, dtype=torch.int32)
    try:
        y = block(*routed)
        torch.cuda.synchronize(device)
    except Exception:                                       # noqa: BLE001 -- the ranks decide together below
        good.zero_()
    dist.all_reduce(good, op=dist.ReduceOp.MIN)
    if int(good.item()) == 0:                               # the peer exchange did not come up somewhere: collectives
        block = parallel.ExpertParallelMoE(*[tuple(to_torch(a, device) for a in p) for p in packs])
        y = block(*routed)
    tidx, eidx = np.repeat(np.arange(t), kk), idx.reshape(-1)
    gate = O.gather_qmm_exact(x[:, None, :], *packs[0], tidx, eidx)[:, 0]
    up = O.gather_qmm_exact(x[:, None, :], *packs[1], tidx, eidx)[:, 0]
    act = (gate / (1 + np.exp(-gate))) * up
    down = O.gather_qmm_exact(act[:, None, :], *packs[2], np.arange(len(tidx)), eidx)[:, 0]
    moe_err = O.rel_err(to_numpy(y).astype(np.float32), O.moe_combine_exact(down, wts))
    step_err, moe_err = max_over_ranks([max(errs), moe_err], torch, dist, device)
    return {"decode_step": step_err, "ep_moe": moe_err, "bounds": {"decode_step": 3e-2, "ep_moe": 2e-2},
            "what": "decode step (2 layers, d 1024) with the weights sharded (batch 1 and 5) and with the sequences "
                    "sharded (2 and 17 per rank) vs the float32 step on the dequantized weights; expert-parallel "
                    "SwiGLU block (8 experts, top-2) vs the oracle's pair-space product"}


def line_of(name, args, torch, dist, device, world, pk):
    if name in DECODE_STEPS:
        return decode_step_line(name, args, torch, dist, device, world, pk)
    if name in MOE_BLOCKS:
        return moe_line(name, args, torch, dist, device, world, pk)
    return qmm_line(name, args, torch, dist, device, world, pk)


ALSO_KEYS = ("metric", "value", "unit", "n_gpus", "ms_per_step", "scaling", "config", "how", "roofline", "e2e",
             "gpu_launches")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=DEFAULT, choices=sorted(WORKLOADS) + sorted(DECODE_STEPS) + sorted(MOE_BLOCKS))
    ap.add_argument("--decode-sharding", default="auto", choices=["auto", "rows", "weights"],
                    help="decode steps at N > 1: split the sequences, or the weights (auto: sequences where the batch divides)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-also", action="store_true", help="only the headline workload")
    ap.add_argument("--profile-window", action="store_true",
                    help="bracket the timed steps with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    args = ap.parse_args()
    global PROFILE_WINDOW, DECODE_SHARDING
    PROFILE_WINDOW = args.profile_window
    DECODE_SHARDING = args.decode_sharding

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    from metaljax_b200 import _lib
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
    parity = parity_check(torch, dist, device, world, rank) if world > 1 else None
    with ClockSampler(local) as clocks:
        line = line_of(name, args, torch, dist, device, world, pk)
    line["clocks"] = clocks.summary()
    _lib.poll_status()
    if parity is not None:
        line["parity"] = parity

    if not args.no_also and name == DEFAULT:
        if world == 1:
            sides = [w for w in ALSO_AT_ONE] + [w for w in ALSO_STEPS if w != name]
        else:
            sides = [w for w in ALSO_STEPS if w != name] + sorted(MOE_BLOCKS)
        for side_name in sides:
            side = line_of(side_name, args, torch, dist, device, world, pk)
            line.setdefault("also", []).append({key: side[key] for key in ALSO_KEYS})
        if world > 1 and DECODE_SHARDING == "auto":
            # the other way to split the headline and the batch-16 step: the weights instead of the sequences
            for side_name in (w for w in reversed(ALSO_STEPS) if decode_sharding(DECODE_STEPS[w], world) == "rows"):
                side = decode_step_line(side_name, args, torch, dist, device, world, pk, sharding="weights")
                line["also"].append({key: side[key] for key in ALSO_KEYS})
        _lib.poll_status()

    if rank == 0 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline_of(name)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
