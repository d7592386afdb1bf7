"""ctypes front of the C restatement `qmm_oracle.c` (TEST INFRASTRUCTURE).

Used by the test-suite (to cross-check the numpy restatement) and by the
benchmark's CPU-baseline leg (a fused dequantize-and-dot loop over all host
threads is the stronger CPU figure; a CPU backend fuses the reconstruction into
the dot's operand loop, eterevsky/metaljax src/metaljax/qmm.py:11-13).
Builds the shared object with `make` on first use when it is missing.
"""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libqmm_oracle.so")
_lib = None

BF16, F32 = 0, 2


def build(force: bool = False) -> str:
    if force or not os.path.exists(_SO) or (
            os.path.getmtime(_SO) < os.path.getmtime(os.path.join(_HERE, "qmm_oracle.c"))):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B"])
    return _SO


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def use_all_cores() -> int:
    """Run the C loops on every host core, whatever OMP_NUM_THREADS a launcher exported."""
    lib().oracle_set_threads(os.cpu_count() or 1)
    return num_threads()


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def _ptr(a):
    return None if a is None else ctypes.c_void_p(a.ctypes.data)


def _code(a) -> int:
    return F32 if a.dtype == np.float32 else BF16


def _raw(a):
    """bf16 (ml_dtypes) arrays cross as their uint16 bit patterns."""
    if a is None:
        return None
    a = np.ascontiguousarray(a)
    if a.dtype.itemsize == 2 and a.dtype != np.uint16:
        return a.view(np.uint16)
    return a


def qmm(x, w, scales, biases, M, K, N, gs, bits, mode="affine", out_f32=False):
    """`y[M,N] = x[M,K] . deq(w)[N,K]^T`; returns float32 or bf16 bits (uint16)."""
    xr, wr, sr, br = _raw(x), np.ascontiguousarray(w, np.uint32), _raw(scales), _raw(biases)
    y = np.empty((M, N), np.float32 if out_f32 else np.uint16)
    mx = 1 if mode == "mxfp4" else 0
    rc = lib().oracle_qmm(_ptr(xr), _code(xr), _ptr(wr), _ptr(sr), _ptr(br),
                          F32 if (not mx and sr.dtype == np.float32) else BF16,
                          _ptr(y), F32 if out_f32 else BF16,
                          ctypes.c_long(M), ctypes.c_long(K), ctypes.c_long(N),
                          int(gs), int(bits), mx)
    if rc:
        raise RuntimeError(f"oracle_qmm failed: {rc}")
    return y


def dequantize(w, scales, biases, N, K, gs, bits, mode="affine"):
    wr, sr, br = np.ascontiguousarray(w, np.uint32), _raw(scales), _raw(biases)
    out = np.empty((N, K), np.float32)
    mx = 1 if mode == "mxfp4" else 0
    rc = lib().oracle_dequantize(_ptr(wr), _ptr(sr), _ptr(br),
                                 F32 if (not mx and sr.dtype == np.float32) else BF16,
                                 _ptr(out), ctypes.c_long(N), ctypes.c_long(K),
                                 int(gs), int(bits), mx)
    if rc:
        raise RuntimeError(f"oracle_dequantize failed: {rc}")
    return out


def qmm_ragged(x, w, scales, biases, group_sizes, M, K, N, gs, bits, mode="affine",
               out_f32=False):
    xr, wr, sr, br = _raw(x), np.ascontiguousarray(w, np.uint32), _raw(scales), _raw(biases)
    g = np.ascontiguousarray(group_sizes, np.int32)
    y = np.empty((M, N), np.float32 if out_f32 else np.uint16)
    mx = 1 if mode == "mxfp4" else 0
    rc = lib().oracle_qmm_ragged(_ptr(xr), _code(xr), _ptr(wr), _ptr(sr), _ptr(br),
                                 F32 if (not mx and sr.dtype == np.float32) else BF16,
                                 _ptr(y), F32 if out_f32 else BF16, _ptr(g),
                                 ctypes.c_long(len(g)), ctypes.c_long(M), ctypes.c_long(K),
                                 ctypes.c_long(N), int(gs), int(bits), mx)
    if rc:
        raise RuntimeError(f"oracle_qmm_ragged failed: {rc}")
    return y
