"""ctypes binding of libqmm.so: DLPack views in, status codes out.

Every tensor crosses as a DLPack `DLTensor` (taken from the tensor's own `__dlpack__`
capsule), which is the `qmm_tensor` of include/qmm.h. The library is looked up next to
this file; it is never built implicitly and there is no fallback when it is missing.
"""

from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("QMM_LIBRARY") or os.path.join(_HERE, "libqmm.so")     # (a development build can be named)

MODE = {"affine": 0, "mxfp4": 1}
ROUTES = {0: "none", 1: "gemv", 2: "gemm_tc", 3: "simt", 4: "gemv_fmma"}
ELEM = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2, torch.uint8: 3,
        torch.uint32: 4, torch.int32: 5}


class QmmError(RuntimeError):
    """A non-zero status from libqmm (`.status` holds the qmm_status value)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"libqmm status {status}: {message}")
        self.status = status


class Problem(ctypes.Structure):
    """`qmm_problem` of include/qmm.h."""

    _fields_ = [
        ("struct_size", ctypes.c_uint32), ("mode", ctypes.c_int32), ("bits", ctypes.c_int32),
        ("group_size", ctypes.c_int32), ("x_dtype", ctypes.c_int32),
        ("table_dtype", ctypes.c_int32), ("y_dtype", ctypes.c_int32),
        ("num_weights", ctypes.c_int32),
        ("batch", ctypes.c_int64), ("M", ctypes.c_int64), ("K", ctypes.c_int64),
        ("N", ctypes.c_int64),
        ("x", ctypes.c_void_p), ("w", ctypes.c_void_p), ("scales", ctypes.c_void_p),
        ("biases", ctypes.c_void_p), ("y", ctypes.c_void_p),
        ("x_batch_stride", ctypes.c_int64), ("w_batch_stride", ctypes.c_int64),
        ("y_batch_stride", ctypes.c_int64),
        ("lhs_idx", ctypes.c_void_p), ("rhs_idx", ctypes.c_void_p),
        ("group_sizes", ctypes.c_void_p),
        ("x_batches", ctypes.c_int64),
    ]


class Exchange(ctypes.Structure):
    """`qmm_exchange` of include/qmm_decode.h."""

    _fields_ = [("peer_bufs", ctypes.POINTER(ctypes.c_void_p)), ("epoch", ctypes.c_void_p),
                ("slot_bytes", ctypes.c_int64), ("rank", ctypes.c_int32), ("world", ctypes.c_int32)]


class EpExchange(ctypes.Structure):
    """`qmm_ep_exchange` of include/qmm_ep.h."""

    _fields_ = [("peer_counts", ctypes.POINTER(ctypes.c_void_p)), ("peer_flags", ctypes.POINTER(ctypes.c_void_p)),
                ("peer_recv", ctypes.POINTER(ctypes.c_void_p)), ("peer_ret", ctypes.POINTER(ctypes.c_void_p)),
                ("epoch", ctypes.c_void_p), ("scratch", ctypes.c_void_p),
                ("capacity_rows", ctypes.c_int64), ("max_pairs", ctypes.c_int64),
                ("rank", ctypes.c_int32), ("world", ctypes.c_int32), ("experts", ctypes.c_int32)]


class DecodeFusion(ctypes.Structure):
    """`qmm_decode_fusion` of include/qmm_decode.h."""

    _fields_ = [("prologue", ctypes.c_int32), ("wait_slot", ctypes.c_int32), ("wait_site", ctypes.c_int32),
                ("push_slot", ctypes.c_int32), ("push_site", ctypes.c_int32),
                ("residual_in", ctypes.c_void_p), ("residual_out", ctypes.c_void_p),
                ("norm_weight", ctypes.c_void_p), ("eps", ctypes.c_float), ("epilogue", ctypes.c_int32), ("epilogue_out", ctypes.c_void_p)]


_lib = None

ctypes.pythonapi.PyCapsule_GetPointer.restype = ctypes.c_void_p
ctypes.pythonapi.PyCapsule_GetPointer.argtypes = [ctypes.py_object, ctypes.c_char_p]

_T = ctypes.c_void_p  # const qmm_tensor*
_SIGNATURES = {
    "qmm_version": (ctypes.c_int, []),
    "qmm_last_error": (ctypes.c_char_p, []),
    "qmm_launch_count": (ctypes.c_uint64, []),
    "qmm_alloc_count": (ctypes.c_uint64, []),
    "qmm_poll_status": (ctypes.c_int, [ctypes.POINTER(ctypes.c_int)]),
    "qmm_poll_status_static": (ctypes.c_int, [ctypes.POINTER(ctypes.c_int)]),
    "qmm_set_wait_limit": (ctypes.c_int, [ctypes.c_longlong]),
    "qmm_set_route_override": (ctypes.c_int, [ctypes.c_int]),
    "qmm_quantized_matmul": (ctypes.c_int, [_T, _T, _T, _T, _T, ctypes.c_int, ctypes.c_int,
                                            ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
    "qmm_quantized_matmul_static": (ctypes.c_int, [_T, _T, _T, _T, _T, ctypes.c_int, ctypes.c_int,
                                                   ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
    "qmm_check_quantized_matmul": (ctypes.c_int, [_T, _T, _T, _T, _T, ctypes.c_int, ctypes.c_int,
                                                  ctypes.c_int, ctypes.c_int]),
    "qmm_gather_qmm": (ctypes.c_int, [_T, _T, _T, _T, _T, _T, _T, ctypes.c_int, ctypes.c_int,
                                      ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
    "qmm_ragged_dot": (ctypes.c_int, [_T, _T, _T, _T, _T, _T, ctypes.c_int, ctypes.c_int,
                                      ctypes.c_int, ctypes.c_void_p]),
    "qmm_ragged_mm": (ctypes.c_int, [_T, _T, _T, _T, ctypes.c_void_p]),
    "qmm_dequantize": (ctypes.c_int, [_T, _T, _T, _T, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                      ctypes.c_void_p]),
    "qmm_pack_codes": (ctypes.c_int, [_T, _T, ctypes.c_int, ctypes.c_void_p]),
    "qmm_moe_silu_mul": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                        ctypes.c_int, ctypes.c_void_p]),
    "qmm_moe_routed_sum": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.c_int64, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                          ctypes.c_void_p]),
    "qmm_launch": (ctypes.c_int, [ctypes.POINTER(Problem), ctypes.c_void_p]),
    # include/qmm_decode.h
    "qmm_decode_add_rmsnorm": (ctypes.c_int, [ctypes.c_void_p] * 5 + [ctypes.c_int64, ctypes.c_int64,
                                                                     ctypes.c_float, ctypes.c_void_p]),
    "qmm_decode_rope_kv": (ctypes.c_int, [ctypes.c_void_p] * 4 + [ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                                                                 ctypes.c_int, ctypes.c_int64, ctypes.c_int64,
                                                                 ctypes.c_float, ctypes.c_void_p]),
    "qmm_decode_silu_mul": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                           ctypes.c_void_p]),
    "qmm_decode_argmax_scratch_bytes": (ctypes.c_int64, [ctypes.c_int64]),
    "qmm_decode_argmax": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                         ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]),
    "qmm_decode_allgather": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p),
                                            ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_int,
                                            ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int64,
                                            ctypes.c_int64, ctypes.c_void_p]),
    "qmm_decode_step_begin": (ctypes.c_int, [ctypes.POINTER(Exchange), ctypes.c_void_p]),
    "qmm_decode_linear": (ctypes.c_int, [ctypes.POINTER(Problem), ctypes.POINTER(DecodeFusion),
                                         ctypes.POINTER(Exchange), ctypes.c_void_p]),
    "qmm_decode_attention_scratch_bytes": (ctypes.c_int64, [ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                            ctypes.c_int64]),
    "qmm_decode_attention": (ctypes.c_int, [ctypes.c_void_p] * 5 + [ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                                                                   ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_float,
                                                                   ctypes.c_int, ctypes.c_int, ctypes.POINTER(Exchange),
                                                                   ctypes.c_void_p]),
    "qmm_route": (ctypes.c_int, [ctypes.POINTER(Problem)]),
    # include/qmm_ep.h
    "qmm_ep_dispatch": (ctypes.c_int, [ctypes.POINTER(EpExchange), ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                       ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]),
    "qmm_ep_combine": (ctypes.c_int, [ctypes.POINTER(EpExchange), ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]),
}


def exported_symbols() -> list[str]:
    """Every entry point include/*.h declares (and this binding expects)."""
    return sorted(_SIGNATURES)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m metaljax_b200.build`. "
                "There is no fallback path for the fused quantized matmul.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        if handle.qmm_version() != 1:
            raise RuntimeError(f"libqmm ABI version {handle.qmm_version()} != 1")
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status:
        raise QmmError(status, lib().qmm_last_error().decode(errors="replace"))


class Views:
    """DLPack views of a call's tensors, kept alive until the call returns."""

    def __init__(self):
        self._caps = []

    def __call__(self, t):
        if t is None:
            return None
        # stream=-1: the producer inserts no synchronization; libqmm enqueues on the
        # caller's current stream, which is where the tensor's pending work already is.
        cap = t.__dlpack__(stream=-1)
        self._caps.append(cap)
        # DLManagedTensor begins with its DLTensor, so the capsule pointer is the view.
        return ctypes.pythonapi.PyCapsule_GetPointer(cap, b"dltensor")


def stream_ptr(t) -> int:
    """The current CUDA stream of `t`'s device (work is enqueued there, unsynchronized)."""
    if t.is_cuda:
        return torch.cuda.current_stream(t.device).cuda_stream
    return 0


class force_route:
    """Context manager for tests: every launch inside goes to one kernel family
    ("gemv", "gemm_tc", "simt"; "gemv_fmma" = the decode family's floating-point mma.sync kernel
    even for a single row) or fails with status 7 if that family declines it."""

    def __init__(self, name: str):
        self.route = {v: k for k, v in ROUTES.items()}[name]

    def __enter__(self):
        check(lib().qmm_set_route_override(self.route))
        return self

    def __exit__(self, *exc):
        lib().qmm_set_route_override(0)
        return False


def poll_status() -> int:
    """Synchronizes the device; raises QmmError(9) if a kernel gave up on a bounded wait."""
    st = ctypes.c_int(0)
    check(lib().qmm_poll_status(ctypes.byref(st)))
    return int(st.value)


def poll_status_static() -> int:
    """The same for the status word of `qmm_quantized_matmul_static` alone (allocates nothing)."""
    st = ctypes.c_int(0)
    check(lib().qmm_poll_status_static(ctypes.byref(st)))
    return int(st.value)


def launch_count() -> int:
    return int(lib().qmm_launch_count())


def alloc_count() -> int:
    """Device-memory allocations libqmm itself has made since it was loaded."""
    return int(lib().qmm_alloc_count())
