"""The C++ PJRT entry (`plugin/qmm_pjrt.cc`, `GetPjrtApi`) driven by a C++ host the way jaxlib
drives the reference's dylib (plugin/metal_pjrt.cc:1276): compile a StableHLO text program,
move host arrays in, execute, move the result out. Without a GPU: the table, the client, the
compile metadata and the error mapping. With one: the sub-channel int4 Dense program of the
reference's tests executed through PJRT against the oracle (the fused path must have run)."""

import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PLUGIN = os.path.join(ROOT, "plugin", "libqmm_pjrt.so")
DRIVER = os.path.join(ROOT, "plugin", "pjrt_driver")


def _built():
    import importlib.util
    spec = importlib.util.spec_from_file_location("plugin_build", os.path.join(ROOT, "plugin", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()                                   # (a no-op when the PJRT header is not on this machine)
    if not (os.path.exists(PLUGIN) and os.path.exists(DRIVER)):
        pytest.skip("the PJRT entry is not built here (pjrt_c_api.h not found and no prebuilt plugin in the tree)")


def _run(program_text, tmp_path, out_prefix, specs=()):
    prog = tmp_path / "program.mlir"
    prog.write_text(program_text)
    env = dict(os.environ)
    env.setdefault("QMM_PJRT_PYTHON", "python3")
    res = subprocess.run([DRIVER, PLUGIN, str(prog), out_prefix, *specs], capture_output=True, text=True, env=env, timeout=300)
    lines = dict(l.split("=", 1) for l in res.stdout.splitlines() if "=" in l and not l.startswith("FAILED"))
    assert res.returncode == 0 and lines.get("done") == "1", res.stdout + res.stderr
    return lines


def test_table_client_compile_and_error_mapping(tmp_path):
    from programs import SUB_CHANNEL
    _built()
    out = _run(SUB_CHANNEL, tmp_path, "-")
    assert out["api_version"] == "0.114" and out["platform"] == "qmm_b200" and out["devices"] == "1"
    assert out["name"] == "jit_dense_sub" and out["num_outputs"] == "1"
    assert out["output0"] == "type 13 dims 5 16"                       # PJRT_Buffer_Type_BF16, [5, 16]
    assert out["bytecode_code"] == "12" and out["format_code"] == "12"   # UNIMPLEMENTED (plugin/metal_pjrt.cc:185-226)
    assert out["garbage_code"] in ("3", "13")                            # INVALID_ARGUMENT / INTERNAL: a Python error
    assert out["topology_code"].startswith("12 ") and "PJRT_Client_TopologyDescription" in out["topology_code"]


@pytest.mark.gpu
def test_sub_channel_program_through_pjrt(tmp_path):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from helpers import BF16, to_numpy
    from programs import SUB_CHANNEL, sub_channel_inputs
    _built()
    x, codes, scales, zeros = sub_channel_inputs(seed=3)
    specs = []
    for name, t, enum in (("x", x, 13), ("codes", codes, 2), ("scales", scales, 13), ("zeros", zeros, 13)):
        path = tmp_path / f"{name}.bin"
        path.write_bytes(to_numpy(t).tobytes())
        specs.append(f"{path}:{enum}:" + "x".join(str(d) for d in t.shape))
    out = _run(SUB_CHANNEL, tmp_path, str(tmp_path / "y"), specs)
    assert out["result0_bytes"] == str(5 * 16 * 2) and out["short_call_code"] == "3"      # INVALID_ARGUMENT
    assert "B200" in out["device_kind"] or "NVIDIA" in out["device_kind"]
    got = np.frombuffer((tmp_path / "y.0.bin").read_bytes(), dtype=np.uint16).view(BF16).astype(np.float32).reshape(5, 16)
    w = (codes.double() - zeros.double().repeat_interleave(64, dim=1)) * scales.double().repeat_interleave(64, dim=1)
    want = (x.double() @ w.T).numpy()
    assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max()
