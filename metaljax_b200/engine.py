"""The Python side of the PJRT entry: compile / execute / buffer transfers.

The reference's C++ dylib trampolines every PJRT call into `metaljax.engine`
(plugin/metal_pjrt.cc:523-601, 960-1043; src/metaljax/engine.py:133-159, 325-400): a program
arrives as StableHLO, is kept as an interpreter object, and every execute first runs the
quantized-matmul prologue (pack once, rewrite the matched dots) and then walks the program.
This module is that surface for the B200 build, with the same function names, argument order
and buffer attributes (`.data`, `.type_enum`, `.dims`, `.nbytes`), so that
`plugin/qmm_pjrt.cc` stands where `plugin/metal_pjrt.cc` stands:

    compile_program(code: bytes, fmt: str, options: bytes | None) -> Program
    execute(program, buffers) -> list[DeviceBuffer]
    buffer_from_host(view, type_enum, dims, byte_strides, offset) -> DeviceBuffer
    to_host(buffer) -> bytes        buffer_pointer(buffer) -> int
    device_kind() -> str            stablehlo_version() -> str

Programs are StableHLO **text** (what `jax.jit(f).lower(...).as_text()` prints); the portable
bytecode artifact jax hands a plugin is decoded by `jaxlib.mlir` in the reference and is refused
here with an "Unsupported" error (jaxlib is not a dependency). Buffers live on the current CUDA
device as torch tensors; the fused ops run through libqmm, everything else through the literal
evaluator of `hlo.py`.
"""

from __future__ import annotations

import hashlib
import re

import torch

from . import hlo, recognizer


class UnsupportedProgramError(RuntimeError):
    """Maps to PJRT_Error_Code_UNIMPLEMENTED in the C++ entry (class name contains
    "Unsupported", plugin/metal_pjrt.cc:185-226)."""


# PJRT_Buffer_Type values (pjrt_c_api.h) <-> (torch storage dtype, StableHLO element type).
# 4-bit integers are held one per byte, as the reference widens them (src/metaljax/dtypes.py:207-212).
_TYPES = {
    1: (torch.bool, "i1"), 2: (torch.int8, "i8"), 3: (torch.int16, "i16"), 4: (torch.int32, "i32"),
    5: (torch.int64, "i64"), 6: (torch.uint8, "ui8"), 10: (torch.float16, "f16"), 11: (torch.float32, "f32"),
    12: (torch.float64, "f64"), 13: (torch.bfloat16, "bf16"),
}
_S4, _U4 = 21, 22
_EL_TO_ENUM = {el: enum for enum, (_, el) in _TYPES.items()}
_EL_TO_ENUM.update({"i4": _S4, "ui4": _U4})


def _device():
    if not torch.cuda.is_available():
        raise RuntimeError("the B200 engine needs a CUDA device")
    return torch.device("cuda", torch.cuda.current_device())


class DeviceBuffer:
    """A device array with the attributes the C++ entry reads (plugin/metal_pjrt.cc:284-299)."""

    __slots__ = ("data", "type_enum", "dims", "nbytes")

    def __init__(self, data: torch.Tensor, type_enum: int):
        self.data, self.type_enum = data, int(type_enum)
        self.dims = tuple(int(d) for d in data.shape)
        self.nbytes = data.numel() * data.element_size()


class Program:
    """What `compile_program` returns: the interpreter plus the metadata PJRT asks for."""

    def __init__(self, name, text):
        self.name = name
        self.fingerprint = hashlib.sha256(text.encode()).hexdigest()
        self.interp = recognizer.Interpreter(text)
        fn = self.interp.func
        self.num_params = len(fn.args)
        self.num_outputs = len(fn.returns)
        self.out_types = [_EL_TO_ENUM[v.type.el] for v in fn.returns]
        self.out_dims = [tuple(v.type.shape) for v in fn.returns]
        self.donated_params = sorted(fn.donated)
        self.param_types = [a.type for a in fn.args]
        self.executions = 0


def stablehlo_version() -> str:
    return "1.0.0"


def device_kind() -> str:
    return torch.cuda.get_device_name(torch.cuda.current_device()) if torch.cuda.is_available() else "no CUDA device"


def compile_program(code, fmt="mlir", options=None) -> Program:
    raw = bytes(code)
    if fmt != "mlir":
        raise UnsupportedProgramError(f"program format {fmt!r}: only 'mlir' (StableHLO) is accepted")
    if raw[:4] == b"ML\xefR":
        raise UnsupportedProgramError(
            "the program is MLIR bytecode (a StableHLO portable artifact); decoding it needs jaxlib.mlir, "
            "which this build does not depend on: pass the StableHLO text instead")
    text = raw.decode("utf-8")
    m = re.search(r"module\s+@([\w.$-]+)", text)
    try:
        return Program(m.group(1) if m else "main", text)
    except NotImplementedError as exc:
        raise UnsupportedProgramError(str(exc)) from exc


def buffer_from_host(view, type_enum, dims, byte_strides=None, offset=0) -> DeviceBuffer:
    """A device buffer from host memory: `view` exposes the bytes, element (i0, i1, ...) sits at
    `offset + sum(i_k * byte_strides[k])` (None = dense row-major), strides may be negative
    (plugin/metal_pjrt.cc:603-675)."""
    type_enum = int(type_enum)
    if type_enum in (_S4, _U4):
        dtype = torch.int8 if type_enum == _S4 else torch.uint8       # one code per byte on the host too
    elif type_enum in _TYPES:
        dtype = _TYPES[type_enum][0]
    else:
        raise UnsupportedProgramError(f"PJRT buffer type {type_enum}")
    dims = tuple(int(d) for d in dims)
    numel = 1
    for d in dims:
        numel *= d
    if view is None or numel == 0:
        return DeviceBuffer(torch.zeros(dims, dtype=dtype, device=_device()), type_enum)
    flat = torch.frombuffer(bytearray(bytes(view)), dtype=torch.uint8)
    esize = torch.empty((), dtype=dtype).element_size()
    if byte_strides is None:
        host = flat[offset: offset + numel * esize].view(dtype).reshape(dims)
    else:
        strides = tuple(int(s) for s in byte_strides)
        if any(s % esize for s in strides) or offset % esize:
            raise UnsupportedProgramError("host strides that are not multiples of the element size")
        typed = flat[: (flat.numel() // esize) * esize].view(dtype)
        # negative strides: index arithmetic on an explicit gather (as_strided refuses them)
        idx = torch.full(dims, offset // esize, dtype=torch.int64)
        for k, (d, s) in enumerate(zip(dims, strides)):
            shape = [1] * len(dims)
            shape[k] = d
            idx = idx + (torch.arange(d, dtype=torch.int64) * (s // esize)).reshape(shape)
        host = typed[idx.reshape(-1)].reshape(dims)
    return DeviceBuffer(host.to(_device()), type_enum)


def to_host(buf: DeviceBuffer) -> bytes:
    t = buf.data.detach().contiguous().cpu()
    return t.view(torch.uint8).numpy().tobytes() if t.numel() else b""


def buffer_pointer(buf: DeviceBuffer) -> int:
    return int(buf.data.data_ptr())


def execute(program: Program, buffers) -> list:
    """Runs the program on device buffers: the pack prologue on the first call (and whenever a
    weight buffer changes identity), the fused ops in place of the matched chains, the rest
    literally (src/metaljax/engine.py:385-400)."""
    if len(buffers) != program.num_params:
        raise ValueError(f"{program.name} takes {program.num_params} arguments, got {len(buffers)}")
    args = []
    for b, t in zip(buffers, program.param_types):
        if tuple(b.dims) != tuple(t.shape):
            raise ValueError(f"argument of shape {tuple(b.dims)} for a parameter of type {t}")
        args.append(b.data)
    outs = program.interp.execute(args)
    program.executions += 1
    fn = program.interp.func
    res = []
    for v, t in zip(fn.returns, outs):
        res.append(DeviceBuffer(t.contiguous(), _EL_TO_ENUM[v.type.el]))
    return res


def stats(program: Program) -> dict:
    """Counters a test can assert on, like the reference's STATS dicts (src/metaljax/qmm.py:176-187)."""
    return {"executions": program.executions, "fused_calls": program.interp.fused_calls,
            "rejections": list(program.interp.rejections)}
