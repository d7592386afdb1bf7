"""Host-side pieces of bench.py that need no GPU: how a decode step is split over N ranks, that
both arms describe the workload with the same `config`, the algorithmic byte counts behind the
roofline, and the reference arm's JSON line (a short run of the CPU restatement)."""

import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_decode_sharding_choice():
    assert bench.decode_sharding(64, 1) == "weights"
    for world in (2, 4, 8):
        assert bench.decode_sharding(64, world) == "rows"            # the batch divides: split the sequences
        assert bench.decode_sharding(16, world) == "rows"
        assert bench.decode_sharding(1, world) == "weights"          # one row: only the weights can be split
    assert bench.decode_sharding(5, 4) == "weights"
    bench.DECODE_SHARDING = "weights"
    try:
        assert bench.decode_sharding(64, 8) == "weights"
    finally:
        bench.DECODE_SHARDING = "auto"


def test_config_names_the_split_and_both_arms_agree():
    c = bench.config_of("decode_llama3_8b_b64", 8)
    assert c["workload"] == "decode_llama3_8b_b64" and c["batch"] == 64 and c["parallelism"].startswith("dp8")
    assert bench.config_of("decode_llama3_8b_b1", 8)["parallelism"].startswith("tp8")
    assert bench.config_of("decode_llama3_8b_b64", 8, "weights")["parallelism"].startswith("tp8")
    assert bench.config_of("moe_mixtral_t4096", 4)["parallelism"].startswith("ep4")
    assert bench.config_of("prefill_int4_g64_m2048_14336x4096", 1)["M"] == 2048


def test_algorithmic_bytes_of_the_configs():
    # C1: codes 8,388,608 + scale and bias tables 1,048,576 = 9,437,184 weight bytes; + x and y rows
    flops, wbytes, total = bench.work_of("decode_int4_g64_m1_4096x4096")
    assert (flops, wbytes, total) == (33554432.0, 9437184, 9437184 + 8192 + 8192)
    flops, _, _ = bench.work_of("prefill_int4_g64_m2048_14336x4096")
    assert flops == 240518168576.0
    pytest.importorskip("torch")
    wb, kv = bench.decode_step_bytes(64, 1)
    assert wb == 4221370368 and kv == 64 * 268435456
    wb8, kv8 = bench.decode_step_bytes(64, 8, "rows")
    assert wb8 == wb and kv8 == kv / 8                               # whole weights, an eighth of the sequences
    wbt, kvt = bench.decode_step_bytes(64, 8, "weights")
    assert wbt == wb / 8 and kvt == kv / 8


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                          "--gpus", "2", "--workload", "decode_int4_g64_m1_4096x4096"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-500:]
    line = json.loads([ln for ln in out.stdout.splitlines() if ln.startswith("{")][-1])
    assert line["impl"] == "reference" and line["metric"] == "qmm_weight_gbs_m1" and line["n_gpus"] == 2
    assert line["config"] == bench.config_of("decode_int4_g64_m1_4096x4096", 2)
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["cpu_baseline"]["kind"] in ("port", "reference")
    assert line["value"] > 0 and line["higher_is_better"] is True
