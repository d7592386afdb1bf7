"""Host side of the fused quantized matmul, with the reference recognizer's interface.

Mirrors `metaljax.qmm` of eterevsky/metaljax 0.11.3 for the part of it that sits on the
hot path -- same names, argument meaning and error behaviour -- with torch tensors in
place of MLX arrays and `libqmm.so` (CUDA, sm_100a) in place of `mx.quantized_matmul`:

  pack primitives   pack_codes (src/metaljax/qmm.py:206-232), pack_exact / _scale_bias /
                    _lossless (:235-286), mxfp4_codes (:300-332), mxfp4_scale_bytes
                    (:335-357), _group_const / _group_heads / _pick_group /
                    _pick_group_heads (:1204-1247), _regroup / _column_keys / _take_k
                    (:390-464)
  metadata          Match, _Pack, State (:588-699), STATS / stats / reset_stats (:176-187)
  runtime           values / push / pop / pack_arrays (:2395-2421), emit_reads (:2424-2442),
                    emit_bytes (:2445-2466), emit (:2469-2501)
  the op itself     quantized_matmul / dequantize stand where the reference calls
                    mx.quantized_matmul (:2491) and mx.dequantize (tests/test_qmm.py:121)

The structural matcher (`analyze`) needs an MLIR front end and is outside this module.
There is no literal-chain fallback: a pack that cannot be built raises `_Reject`, and the
fused ops raise when libqmm or a CUDA device is missing.
"""

from __future__ import annotations

import math
import os
import weakref

import numpy as np
import torch

from . import _lib

QMM_ENABLED = os.environ.get("METALJAX_QMM", "1") != "0"
ENABLED = QMM_ENABLED or os.environ.get("METALJAX_MOE", "1") != "0"
_DEBUG = os.environ.get("METALJAX_DEBUG", "") == "1"

_GROUP_SIZES = (128, 64, 32)
_MAX_PACKS = int(os.environ.get("METALJAX_QMM_CACHE", "2"))
_MAX_REPACKS = int(os.environ.get("METALJAX_QMM_REPACKS", "8"))
_SCALE_WIDTH = os.environ.get("METALJAX_QMM_SCALES", "auto")
_BATCH = os.environ.get("METALJAX_QMM_BATCH", "1") != "0"

_E2M1_MAGS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_MXFP4_GROUP = 32

STATS = {"recognized": 0, "packs": 0, "fallbacks": 0, "perms": 0, "mxfp4": 0,
         "batched": 0, "shared": 0, "blocked": 0, "build_hits": 0, "build_declines": 0}

_FLOATS = (torch.float32, torch.float16, torch.bfloat16)


def stats() -> dict:
    return dict(STATS)


def reset_stats():
    for k in STATS:
        STATS[k] = 0


class _Reject(Exception):
    """A candidate cannot be represented (or trusted). The reference then runs the chain
    literally; this build has no literal chain, so callers surface the rejection."""


# --------------------------------------------------------------------------------------
# packing
# --------------------------------------------------------------------------------------


def _as_u32(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.uint32 else t.view(torch.uint32)


def pack_codes(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """Unsigned codes `[..., K]` -> uint32 words `[..., K*bits//32]`.

    Each row is one little-endian bit stream, LSB first: element i occupies bits
    [i*bits, (i+1)*bits). Codes are masked to `bits` so an out-of-range value cannot
    spill into its neighbour. Device tensors are packed by libqmm's kernel; host tensors
    by integer arithmetic here (the pack prologue may run before weights are moved).
    """
    if 32 % bits:
        raise ValueError(f"pack_codes: bits={bits} does not divide 32")
    per = 32 // bits
    k = codes.shape[-1]
    if k % per:
        raise ValueError(f"pack_codes: K={k} not a multiple of {per}")
    lead = list(codes.shape[:-1])
    if codes.is_cuda and bits in (4, 8):
        c8 = codes.contiguous() if codes.dtype == torch.uint8 else \
            (codes.contiguous().to(torch.int64) & ((1 << bits) - 1)).to(torch.uint8)
        out = torch.empty(lead + [k // per], dtype=torch.uint32, device=codes.device)
        if out.numel():
            v = _lib.Views()
            _lib.check(_lib.lib().qmm_pack_codes(v(c8), v(out), bits, _lib.stream_ptr(out)))
        return out
    c = codes.contiguous().to(torch.int64).reshape(lead + [k // per, per]) & ((1 << bits) - 1)
    shifts = torch.arange(per, dtype=torch.int64, device=codes.device) * bits
    words = (c << shifts).sum(dim=-1)                       # < 2**32, exact in int64
    words = torch.where(words >= (1 << 31), words - (1 << 32), words)
    return words.to(torch.int32).view(torch.uint32)


def _lossless(x: torch.Tensor, dtype) -> bool:
    return bool(torch.all(x.to(dtype).to(torch.float32) == x).item())


def _scale_bias(scales, zeros, offset, scale_dtype):
    """`biases = -scale * (offset + zero)` in float32, narrowed to the source dtype only
    when nothing is lost ("auto"), always ("source") or never ("f32")."""
    s32 = scales.contiguous().to(torch.float32)
    z32 = zeros.contiguous().to(torch.float32) if zeros is not None else 0.0
    b32 = -(s32 * (z32 + float(offset)))
    if scale_dtype is not None and scale_dtype != torch.float32 and _SCALE_WIDTH != "f32":
        if _SCALE_WIDTH == "source" or (_lossless(s32, scale_dtype)
                                        and _lossless(b32, scale_dtype)):
            return s32.to(scale_dtype), b32.to(scale_dtype)
    return s32, b32


def pack_exact(codes, scales, zeros, bits: int, scale_dtype=None, offset=None):
    """Repack `w = scale * (code - zero)` (signed codes `[N, K]`, per-group tables
    `[N, K/group_size]`) into `(packed_u32, scales, biases)` for `quantized_matmul`:
    `q_hat = code + offset` (unsigned, must fit `bits`), `biases = -scale*(offset+zero)`;
    `offset` defaults to `2**(bits-1)`."""
    off = (1 << (bits - 1)) if offset is None else int(offset)
    packed = pack_codes(codes.contiguous().to(torch.int32) + off, bits)
    s, b = _scale_bias(scales, zeros, off, scale_dtype)
    return packed, s, b


# --------------------------------------------------------------------------------------
# MXFP4
# --------------------------------------------------------------------------------------


def _int_view(dtype):
    return {torch.float32: (torch.int32, 32), torch.bfloat16: (torch.int16, 16),
            torch.float16: (torch.int16, 16)}.get(dtype)


def mxfp4_codes(values: torch.Tensor) -> torch.Tensor:
    """4-bit MXFP4 codes (uint8) for values lying EXACTLY on the E2M1 grid; `_Reject`
    otherwise. Bit patterns are compared, so -0.0 is code 8 and +0.0 is code 0."""
    iv = _int_view(values.dtype)
    if iv is None:
        raise _Reject(f"MXFP4 values in {values.dtype}")
    itype, width = iv
    bits = values.contiguous().view(itype).to(torch.int64) & ((1 << width) - 1)
    sign = bits >> (width - 1)
    mag = bits & ((1 << (width - 1)) - 1)
    grid = (torch.tensor(_E2M1_MAGS, dtype=values.dtype).view(itype).to(torch.int64)
            & ((1 << width) - 1)).tolist()
    if len(set(grid)) != len(_E2M1_MAGS):
        raise _Reject(f"the E2M1 grid is not distinct in {values.dtype}")
    codes = torch.zeros(mag.shape, dtype=torch.int64, device=values.device)
    ok = torch.zeros(mag.shape, dtype=torch.bool, device=values.device)
    for i, g in enumerate(grid):
        hit = mag == g
        codes = torch.where(hit, i, codes)
        ok |= hit
    if not bool(ok.all().item()):
        raise _Reject("weight values are not on the MXFP4 (E2M1) grid")
    return (codes | (sign << 3)).to(torch.uint8)


def mxfp4_scale_bytes(scales: torch.Tensor) -> torch.Tensor:
    """E8M0 bytes for scales that are exact positive normal powers of two: the byte is
    the float32 exponent field; a set sign or mantissa bit, or field 0 / 255, rejects."""
    bits = scales.to(torch.float32).contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    exp = (bits >> 23) & 0xFF
    bad = ((bits & 0x807FFFFF) != 0) | (exp == 0) | (exp == 0xFF)
    if bool(bad.any().item()):
        raise _Reject("MXFP4 group scales are not exact positive powers of two")
    return exp.to(torch.uint8)


# --------------------------------------------------------------------------------------
# group detection and regrouping of an interleaved contraction axis
# --------------------------------------------------------------------------------------


def _group_const(x: torch.Tensor, gs: int) -> bool:
    k = x.shape[-1]
    v = x.reshape(-1, k // gs, gs)
    return bool(torch.all(v == v[:, :, :1]).item())


def _group_heads(x: torch.Tensor, gs: int) -> torch.Tensor:
    """The first element of each group: `[..., K] -> [..., K/gs]`."""
    k = x.shape[-1]
    return x.reshape(list(x.shape[:-1]) + [k // gs, gs])[..., 0].contiguous()


def _pick_group_heads(k, scale_heads, zero_heads):
    g0 = _GROUP_SIZES[-1]
    for g in _GROUP_SIZES:
        if g < g0 or k % g:
            continue
        r = g // g0
        if r == 1 or (_group_const(scale_heads, r)
                      and (zero_heads is None or _group_const(zero_heads, r))):
            return g
    return None


def _pick_group(k, scale_map, zero_map):
    """The largest legal group size (128, 64, 32) these full-size maps are constant in."""
    g0 = _GROUP_SIZES[-1]
    if k % g0 or not _group_const(scale_map, g0):
        return None
    if zero_map is not None and not _group_const(zero_map, g0):
        return None
    return _pick_group_heads(k, _group_heads(scale_map, g0),
                             None if zero_map is None else _group_heads(zero_map, g0))


_MIX = 2246822519


def _mix(u: np.ndarray) -> np.ndarray:
    u = (u * np.uint32(_MIX)).astype(np.uint32)
    return u ^ (u >> np.uint32(15))


def _bits_u32(x: torch.Tensor) -> np.ndarray:
    if x.dtype in _FLOATS:
        return x.to(torch.float32).cpu().numpy().view(np.uint32)
    return x.to(torch.int64).cpu().numpy().astype(np.uint32)


def _column_keys(x: torch.Tensor) -> np.ndarray:
    """Per-column digest `[K, 2]` (uint32): equal columns digest equally; a collision can
    only merge two groups, which the exact constancy check afterwards rejects."""
    k = x.shape[-1]
    u = _bits_u32(x.reshape(-1, k))
    rows = np.arange(u.shape[0], dtype=np.uint32).reshape(-1, 1)
    with np.errstate(over="ignore"):
        r = _mix(rows * np.uint32(0x9E3779B9) + np.uint32(1))
        v = _mix(u)
        h1 = (v * (r | np.uint32(1))).sum(axis=0, dtype=np.uint32)
        h2 = _mix(v ^ r).sum(axis=0, dtype=np.uint32)
    return np.stack([h1, h2], axis=1)


def _regroup(k: int, maps):
    """A permutation of K that un-interleaves the quantization groups, or None when the
    columns are already grouped or no legal group size divides every run."""
    keys = np.concatenate([_column_keys(x) for x in maps if x is not None], axis=1)
    _, first, inv = np.unique(keys, axis=0, return_index=True, return_inverse=True)
    inv = np.asarray(inv).reshape(-1)
    order = np.argsort(first)
    rank = np.empty(len(order), np.int64)
    rank[order] = np.arange(len(order))
    ids = rank[inv]
    g = 0
    for length in np.bincount(ids):
        g = math.gcd(g, int(length))
    if not any(g and g % s == 0 for s in _GROUP_SIZES):
        return None
    perm = np.argsort(ids, kind="stable").astype(np.int32)
    if np.array_equal(perm, np.arange(k, dtype=np.int32)):
        return None
    return perm


def _take_k(x: torch.Tensor, perm) -> torch.Tensor:
    idx = torch.as_tensor(np.asarray(perm), dtype=torch.int64, device=x.device)
    return x.index_select(-1, idx).contiguous()


# --------------------------------------------------------------------------------------
# the fused op (the kernel boundary)
# --------------------------------------------------------------------------------------


def _mode_id(mode: str) -> int:
    try:
        return _lib.MODE[mode]
    except KeyError:
        raise ValueError(f"unknown quantization mode {mode!r}") from None


def quantized_matmul(x, w, scales, biases=None, transpose=True, group_size=64, bits=4,
                     mode="affine", out=None, out_dtype=None):
    """`y[.., m, n] = sum_k x[.., m, k] * deq(w)[.., n, k]` on the GPU.

    Argument meaning follows `mx.quantized_matmul` as the reference calls it
    (src/metaljax/qmm.py:2491): `w` uint32 `[(B,) N, K*bits/32]`, `scales`/`biases`
    `[(B,) N, K/group_size]` (`biases=None` and uint8 E8M0 scales for mode="mxfp4"),
    float32 accumulation. The result has `x`'s dtype unless `out_dtype` / `out` says
    otherwise (the reference casts to the dot's result type right after the call).
    """
    lead = list(x.shape[:-2])
    m, k = x.shape[-2], x.shape[-1]
    n = w.shape[-2]
    if out is None:
        out = torch.empty(lead + [m, n], dtype=out_dtype or x.dtype, device=x.device)
    elif not out.is_contiguous() or list(out.shape) != lead + [m, n]:
        raise ValueError("quantized_matmul: `out` must be contiguous [.., M, N]")
    xc = x.contiguous()
    if not lead:
        x3, y3 = xc, out
    elif w.dim() == 3:                       # one weight per batch
        x3, y3 = xc.reshape(-1, m, k), out.reshape(-1, m, n)
    else:                                    # shared weight: batches are more rows
        x3, y3 = xc.reshape(-1, k), out.reshape(-1, n)
    v = _lib.Views()
    _lib.check(_lib.lib().qmm_quantized_matmul(
        v(x3), v(_as_u32(w)), v(scales), v(biases), v(y3), 1 if transpose else 0,
        int(group_size), int(bits), _mode_id(mode), _lib.stream_ptr(x)))
    return out


def dequantize(w, scales, biases=None, group_size=64, bits=4, mode="affine",
               dtype=torch.float32):
    """The dequantized weight `[.., N, K]` (stands where the reference's tests call
    `mx.dequantize`, tests/test_qmm.py:121 and tests/test_qmm_mxfp4.py:192)."""
    k = w.shape[-1] * 32 // bits
    out = torch.empty(list(w.shape[:-1]) + [k], dtype=dtype, device=w.device)
    v = _lib.Views()
    _lib.check(_lib.lib().qmm_dequantize(v(_as_u32(w)), v(scales), v(biases), v(out),
                                         int(group_size), int(bits), _mode_id(mode),
                                         _lib.stream_ptr(w)))
    return out


def route(M, K, N, group_size=64, bits=4, mode="affine", x_dtype=torch.bfloat16,
          table_dtype=None, y_dtype=None, batch=1, gather=False, ragged=False) -> str:
    """Name of the kernel family libqmm picks for a problem of this shape (no device
    work): "gemv", "gemm_tc", "simt" or "none"."""
    p = _lib.Problem()
    p.struct_size = _lib.ctypes.sizeof(_lib.Problem)
    p.mode, p.bits, p.group_size = _mode_id(mode), bits, group_size
    p.x_dtype = _lib.ELEM[x_dtype]
    p.table_dtype = _lib.ELEM[table_dtype or (torch.uint8 if mode == "mxfp4" else x_dtype)]
    p.y_dtype = _lib.ELEM[y_dtype or x_dtype]
    p.batch, p.M, p.K, p.N = batch, M, K, N
    p.w_batch_stride = N if (batch > 1 or gather or ragged) else 0
    if gather:
        p.lhs_idx = p.rhs_idx = 16
    if ragged:
        p.group_sizes = 16
    r = _lib.lib().qmm_route(_lib.ctypes.byref(p))
    if r < 0:
        _lib.check(-r)
    return _lib.ROUTES[r]


# --------------------------------------------------------------------------------------
# recognizer metadata
# --------------------------------------------------------------------------------------


class Match:
    """One recognized quantized matmul (same slots as the reference's `Match`)."""

    __slots__ = ("root", "key", "lhs", "codes", "zero", "scale", "recip", "post",
                 "bcast_dims", "ops", "arg_indices", "required", "lperm", "rperm", "rshape",
                 "bshape", "mshape", "nshape", "B", "M", "K", "N", "out_dtype", "disabled",
                 "slot", "gs", "bits", "packs", "repacks", "name", "sub_range", "has_perm",
                 "mode", "nvals", "swapped", "absorbed", "fp")

    def __init__(self):
        self.recip = False
        self.fp = None
        self.absorbed = False
        self.mode = "affine"
        self.zero = None
        self.sub_range = None
        self.post = []
        self.bcast_dims = None
        self.ops = {}
        self.required = []
        self.arg_indices = ()
        self.disabled = False
        self.slot = -1
        self.nvals = 0
        self.gs = 0
        self.bits = 0
        self.has_perm = False
        self.packs = []
        self.repacks = 0
        self.name = "?"
        self.bshape = []
        self.mshape = []
        self.nshape = []
        self.lperm = None
        self.B = 1
        self.swapped = False


class _Pack:
    """The packed arrays of one weight, keyed by the identity of the buffers they were
    built from (weak references: a pack never keeps its source alive)."""

    __slots__ = ("refs", "w", "scales", "biases", "perm", "gs", "bits", "mode", "blocked")

    def __init__(self, leaves, w, scales, biases, perm, gs, bits, mode="affine"):
        self.refs = [weakref.ref(a) for a in leaves]
        self.w, self.scales, self.biases = w, scales, biases
        self.perm = perm
        self.gs, self.bits = gs, bits
        self.mode = mode
        self.blocked = False

    def arrays(self):
        out = [self.w, self.scales]
        if self.biases is not None:
            out.append(self.biases)
        if self.perm is not None:
            out.append(self.perm)
        return out

    def matches(self, leaves) -> bool:
        if len(leaves) != len(self.refs):
            return False
        return all(r() is a for r, a in zip(self.refs, leaves))


class State:
    """Per-program recognizer state: matches, the skip set, root dispatch and the flat
    list of packed arrays `emit` reads by slot."""

    __slots__ = ("matches", "skip", "roots", "values", "active", "moe", "fn", "floats")

    def __init__(self):
        self.matches = []
        self.moe = []
        self.fn = None               # the program (set by the analysis that needs it)
        self.floats = {}             # dots over float expert weights, by op identity
        self.skip = frozenset()
        self.roots = {}
        self.values = []
        self.active = False

    def rebuild(self):
        live = [m for m in self.matches if not m.disabled]
        self.roots = {m.key: m for m in live if not m.absorbed}
        skip = set()
        for m in live:
            skip.update(m.ops)
        for g in self.moe:
            if g.disabled:
                continue
            self.roots[g.key] = g
            skip.update(g.skip_keys)
        self.skip = frozenset(skip)
        self.active = bool(self.roots)


def build_pack(m: Match, codes, scale_map, zero_map=None, leaves=()) -> _Pack:
    """The value-level half of the reference's pack prologue for one match
    (`_build_affine_pack`, src/metaljax/qmm.py:1773-1915; `_build_mxfp4_pack`,
    :1723-1770) on already-materialized operands laid out `[.., N, K]`:

    affine  integral codes -> 4 bits if their span is < 16, 8 if < 256; offset
            `2**(bits-1)` unless the codes do not fit it, then `-lo`; scale / zero maps
            constant within groups -> largest legal group; integer zero points;
            interleaved groups -> a K permutation applied to codes, maps and (at run
            time) activations.
    mxfp4   (`m.mode == "mxfp4"`) values on the E2M1 grid, scales exact powers of two
            constant within groups of 32.
    Fills `m.gs / m.bits / m.has_perm`, appends the pack to `m.packs` (LRU of
    `_MAX_PACKS`) and returns it. Raises `_Reject` when a check fails.
    """
    k = codes.shape[-1]
    if m.mode == "mxfp4":
        if k % _MXFP4_GROUP:
            raise _Reject(f"K={k} is not a multiple of 32")
        if not _group_const(scale_map, _MXFP4_GROUP):
            raise _Reject("MXFP4 scales are not constant within groups of 32")
        q = mxfp4_codes(codes)
        sb = mxfp4_scale_bytes(_group_heads(scale_map, _MXFP4_GROUP))
        pack = _Pack(leaves, pack_codes(q, 4), sb, None, None, _MXFP4_GROUP, 4, "mxfp4")
        STATS["mxfp4"] += 1
    else:
        c = codes
        if c.dtype in _FLOATS:
            if not bool(torch.all(c == torch.round(c)).item()):
                raise _Reject("codes are not integers")
        c = c.to(torch.int64)
        lo, hi = int(c.min().item()), int(c.max().item())
        span = hi - lo + 1
        bits = 4 if span <= 16 else (8 if span <= 256 else 0)
        if not bits:
            raise _Reject(f"codes span {span} values: more than 8 bits")
        half = 1 << (bits - 1)
        off = half if (lo >= -half and hi < half) else -lo
        perm = None
        gs = _pick_group(k, scale_map, zero_map)
        if gs is None:
            perm = _regroup(k, [scale_map, zero_map])
            if perm is None:
                raise _Reject("scale/zero maps are not constant within legal groups")
            c, scale_map = _take_k(c, perm), _take_k(scale_map, perm)
            zero_map = None if zero_map is None else _take_k(zero_map, perm)
            gs = _pick_group(k, scale_map, zero_map)
            if gs is None:
                raise _Reject("regrouped maps are still not group-constant")
            STATS["perms"] += 1
        zh = None
        if zero_map is not None:
            zh = _group_heads(zero_map, gs).to(torch.float32)
            if not bool(torch.all(zh == torch.round(zh)).item()):
                raise _Reject("zero points are not integers")
            if float(zh.abs().max().item()) > 32768:
                raise _Reject("zero points out of range")
            if m.sub_range is not None:
                # the graph subtracts in integer arithmetic, which wraps; only fuse when
                # nothing can wrap (src/metaljax/qmm.py:1889-1897)
                zlo, zhi = int(zh.min().item()), int(zh.max().item())
                if (lo - zhi) < m.sub_range[0] or (hi - zlo) > m.sub_range[1]:
                    raise _Reject("integer zero-point subtraction can wrap")
        sdt = scale_map.dtype if scale_map.dtype in _FLOATS else torch.float32
        w, s, b = pack_exact(c, _group_heads(scale_map, gs), zh, bits, scale_dtype=sdt,
                             offset=off)
        pack = _Pack(leaves, w, s, b,
                     None if perm is None else torch.as_tensor(perm, device=codes.device),
                     gs, bits, "affine")
    return _record_pack(m, pack)


def _record_pack(m: Match, pack: _Pack) -> _Pack:
    pack = _share(pack)
    m.gs, m.bits, m.has_perm = pack.gs, pack.bits, pack.perm is not None
    m.nvals = len(pack.arrays())
    m.packs.insert(0, pack)
    del m.packs[_MAX_PACKS:]
    STATS["packs"] += 1
    return pack


# Packs that are still alive, grouped by a digest of their contents. jax lowers a decode loop's
# prefill and its while body as two separate dots over one set of weights, and two programs of
# one model are handed the same weights in different buffers: without this a model's packed
# weights would be held once per chain (src/metaljax/qmm.py:1645-1704). Entries are weak.
_SHARED = {}
_MAX_SHARED = int(os.environ.get("METALJAX_QMM_SHARE", "512"))


def _digest(a: torch.Tensor) -> int:
    """A cheap content digest of a packed array; it only narrows the search."""
    u = a.contiguous().reshape(-1)
    if u.numel() == 0:
        return 0
    nbytes = u.numel() * u.element_size()
    u8 = u.view(torch.uint8)
    if nbytes % 4:
        u8 = torch.cat([u8, u8.new_zeros(4 - nbytes % 4)])
    v = u8.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    idx = torch.arange(v.numel(), device=v.device, dtype=torch.int64)
    mixed = ((v ^ ((idx * 2654435761) & 0xFFFFFFFF)) * _MIX) & 0xFFFFFFFF
    mixed = mixed ^ (mixed >> 15)
    return int(mixed.sum().item()) & 0xFFFFFFFFFFFF


def _share(pk: _Pack) -> _Pack:
    """Alias `pk`'s arrays onto an identical earlier pack's, if one is alive. Content-addressed:
    nothing is aliased until the arrays compare equal element for element, so two chains that
    reconstruct the same weight share one copy and two that do not can never be confused."""
    arrays = pk.arrays()
    key = (pk.mode, pk.gs, pk.bits, len(arrays), str(arrays[0].device),
           tuple((tuple(a.shape), a.dtype) for a in arrays), _digest(arrays[0]))
    bucket = _SHARED.get(key)
    if bucket is not None:
        for i, refs in enumerate(bucket):
            other = [r() for r in refs]
            if any(o is None for o in other):
                continue
            if all(a is b or bool(torch.equal(a, b)) for a, b in zip(arrays, other)):
                pk.w, pk.scales = other[0], other[1]
                rest = list(other[2:])
                if pk.biases is not None:
                    pk.biases = rest.pop(0)
                if pk.perm is not None:
                    pk.perm = rest.pop(0)
                bucket.insert(0, bucket.pop(i))
                STATS["shared"] = STATS.get("shared", 0) + 1
                return pk
    if len(_SHARED) > _MAX_SHARED:
        _SHARED.clear()                                  # coarse, and only ever costs a repack
    bucket = _SHARED.setdefault(key, [])
    bucket[:] = [refs for refs in bucket if all(r() is not None for r in refs)]
    bucket.insert(0, [weakref.ref(a) for a in arrays])
    return pk


class BlockedPacker:
    """`build_pack` for a weight that arrives one block of rows at a time (`add`), so that the
    reconstruction chain -- several times wider than the weight -- is never alive whole
    (src/metaljax/qmm.py:1360-1400, 1723-1915). Per block only what the final decisions need is
    kept: the codes (one byte or two per element until the bit width is known), the first scale
    and zero of every 32 columns, the running code range. `finish` takes the same decisions as
    `build_pack` from those and returns an identical pack.

    A block whose maps are not constant within groups of 32 would need the column regrouping,
    which looks at whole columns: `NeedsWhole` is raised and the caller evaluates whole.
    """

    class NeedsWhole(Exception):
        pass

    def __init__(self, m: Match, k: int):
        self.m, self.k = m, k
        self.codes, self.scale_heads, self.zero_heads = [], [], []
        self.lo, self.hi = None, None
        self.sdt = None
        if m.mode == "mxfp4" and k % _MXFP4_GROUP:
            raise _Reject(f"K={k} is not a multiple of 32")

    def add(self, codes, scale_map, zero_map=None):
        g0 = _GROUP_SIZES[-1]
        if self.m.mode == "mxfp4":
            if not _group_const(scale_map, _MXFP4_GROUP):
                raise _Reject("MXFP4 scales are not constant within groups of 32")
            self.codes.append(pack_codes(mxfp4_codes(codes), 4))
            self.scale_heads.append(mxfp4_scale_bytes(_group_heads(scale_map, _MXFP4_GROUP)))
            return
        c = codes
        if c.dtype in _FLOATS and not bool(torch.all(c == torch.round(c)).item()):
            raise _Reject("codes are not integers")
        c = c.to(torch.int64)
        lo, hi = int(c.min().item()), int(c.max().item())
        self.lo = lo if self.lo is None else min(self.lo, lo)
        self.hi = hi if self.hi is None else max(self.hi, hi)
        if self.hi - self.lo + 1 > 256:
            raise _Reject(f"codes span {self.hi - self.lo + 1} values: more than 8 bits")
        if lo < -32768 or hi > 32767:
            raise BlockedPacker.NeedsWhole("codes outside 16 bits")
        self.codes.append(c.to(torch.int16))
        if self.k % g0 or not _group_const(scale_map, g0) or (zero_map is not None and not _group_const(zero_map, g0)):
            raise BlockedPacker.NeedsWhole("maps are not constant within groups of 32 as laid out")
        self.sdt = scale_map.dtype if scale_map.dtype in _FLOATS else torch.float32
        self.scale_heads.append(_group_heads(scale_map, g0))
        if zero_map is not None:
            self.zero_heads.append(_group_heads(zero_map, g0))

    def finish(self, leaves, prefix) -> _Pack:
        """`prefix` is the shape in front of the last axis (`[B, N]` or `[N]`)."""
        m, k = self.m, self.k
        join = lambda parts: (parts[0] if len(parts) == 1 else torch.cat(parts, 0))
        fold = lambda t: t.reshape(list(prefix) + [t.shape[-1]])
        if m.mode == "mxfp4":
            pack = _Pack(leaves, fold(join(self.codes)), fold(join(self.scale_heads)), None, None, _MXFP4_GROUP, 4, "mxfp4")
            STATS["mxfp4"] += 1
            return _record_pack(m, pack)
        lo, hi = self.lo, self.hi
        span = hi - lo + 1
        bits = 4 if span <= 16 else 8
        half = 1 << (bits - 1)
        off = half if (lo >= -half and hi < half) else -lo
        g0 = _GROUP_SIZES[-1]
        sh = join(self.scale_heads)
        zh32 = join(self.zero_heads) if self.zero_heads else None
        gs = _pick_group_heads(k, sh, zh32)
        if gs is None:
            raise _Reject("scale/zero maps are not constant within legal groups")
        step = gs // g0
        sh = sh[..., ::step].contiguous()
        zh = None
        if zh32 is not None:
            zh = zh32[..., ::step].contiguous().to(torch.float32)
            if not bool(torch.all(zh == torch.round(zh)).item()):
                raise _Reject("zero points are not integers")
            if float(zh.abs().max().item()) > 32768:
                raise _Reject("zero points out of range")
            if m.sub_range is not None:
                zlo, zhi = int(zh.min().item()), int(zh.max().item())
                if (lo - zhi) < m.sub_range[0] or (hi - zlo) > m.sub_range[1]:
                    raise _Reject("integer zero-point subtraction can wrap")
        words = [pack_codes(c.to(torch.int32) + off, bits) for c in self.codes]
        self.codes = []
        s, b = _scale_bias(sh, zh, off, self.sdt)
        pack = _Pack(leaves, fold(join(words)), fold(s), fold(b), None, gs, bits, "affine")
        return _record_pack(m, pack)


# --------------------------------------------------------------------------------------
# on-wire formats: packs straight from what a checkpoint or a quantized keras layer stores
# --------------------------------------------------------------------------------------


def check_scale_range(scale_bytes: torch.Tensor, what: str = ""):
    """E8M0 bytes 0 (2**-127, a float32 subnormal) and 255 (NaN) are not usable scales
    (scripts/model_bench/mxfp4_gpt_oss.py:83-87)."""
    lo, hi = int(scale_bytes.min().item()), int(scale_bytes.max().item())
    if lo < 1 or hi > 254:
        raise ValueError(f"{what}: E8M0 bytes span [{lo}, {hi}]; 0 and 255 are not usable scales")


def from_hf_mxfp4(blocks: torch.Tensor, scales: torch.Tensor):
    """A Hugging Face MXFP4 expert weight as the fused op's operands, with no copy:
    `*_blocks` uint8 `[.., N, K/32, 16]` (byte j of a block holds elements 2j and 2j+1, low
    nibble first) and `*_scales` uint8 `[.., N, K/32]` (E8M0) -> `(w uint32 [.., N, K/8],
    scales uint8 [.., N, K/32])` for `mode="mxfp4"`. The byte order is already the packed
    stream's (scripts/model_bench/mxfp4_gpt_oss.py:216-240, :90-97)."""
    if blocks.dtype != torch.uint8 or scales.dtype != torch.uint8:
        raise TypeError("MXFP4 blocks and scales are uint8")
    if blocks.shape[-1] != 16 or tuple(blocks.shape[:-1]) != tuple(scales.shape):
        raise ValueError(f"blocks {tuple(blocks.shape)} do not go with scales {tuple(scales.shape)}")
    check_scale_range(scales, "MXFP4 scales")
    lead = list(scales.shape[:-1])
    flat = blocks.contiguous().reshape(lead + [scales.shape[-1] * 16])
    return flat.view(torch.uint32), scales.contiguous()


def unpack_keras_int4(packed: torch.Tensor, columns: int) -> torch.Tensor:
    """`keras.quantizers.unpack_int4` for the layout packed along the last axis: int8
    `[rows, ceil(columns/2)]`, byte j of a row = columns 2j (low nibble) and 2j+1 (high), each
    a 4-bit two's-complement code -> int8 `[rows, columns]` (tests/test_qmm.py:179-190)."""
    p = packed.to(torch.int16) & 0xFF
    lo, hi = p & 15, (p >> 4) & 15
    both = torch.stack([lo, hi], dim=-1).reshape(packed.shape[0], -1)[:, :columns]
    return ((both ^ 8) - 8).to(torch.int8)


def from_keras_int4(packed, scale, zero=None, g_idx=None, columns=None, out_dtype=None):
    """A keras int4 `Dense` kernel as the fused op's operands (`Dense._int4_call`,
    tests/test_qmm.py:193-199): `packed` int8 `[K, ceil(N/2)]` (two OUTPUT columns per byte),
    `scale` / `zero` `[G, N]` per group of input rows, `g_idx[K]` the group of every input row
    (default: `K/G` consecutive rows per group) -> a `_Pack` with `w [N, K*bits/32]`,
    `scales`, `biases [N, K/gs]` and, when the groups interleave, the K permutation to apply to
    the activations. The same checks as the recognizer's pack prologue (`build_pack`)."""
    k = packed.shape[0]
    n = int(columns if columns is not None else scale.shape[-1])
    codes = unpack_keras_int4(packed, n).t().contiguous()                      # [N, K]
    groups = scale.shape[0]
    if g_idx is None:
        if k % groups:
            raise _Reject(f"{groups} groups do not divide K={k}")
        g_idx = torch.arange(k, device=packed.device) // (k // groups)
    g = g_idx.to(torch.int64)
    scale_map = scale.index_select(0, g).t()                                    # [N, K], a view of [K, N]
    zero_map = None if zero is None else zero.index_select(0, g).t()
    m = Match()
    m.mode, m.N, m.K = "affine", n, k
    m.out_dtype = out_dtype or (scale.dtype if scale.dtype in _FLOATS else torch.bfloat16)
    return build_pack(m, codes, scale_map, zero_map, leaves=(packed, scale))


# --------------------------------------------------------------------------------------
# runtime
# --------------------------------------------------------------------------------------


def values(interp):
    """Packed arrays for the current context."""
    st = getattr(interp, "_qmm", None)
    return st.values if st is not None else ()


def push(interp, vals):
    """Rebind the packed arrays (a traced function's own inputs in the reference; a
    captured CUDA graph's static buffers here)."""
    st = getattr(interp, "_qmm", None)
    if st is None or not st.values:
        return None
    prev = st.values
    st.values = list(vals)
    return (prev,)


def pop(interp, token):
    if token is not None:
        interp._qmm.values = token[0]


def pack_arrays(interp, m):
    st = interp._qmm
    return st.values[m.slot:m.slot + m.nvals]


def emit_reads(m):
    """The `env` values `emit` reads: exactly the activation operand."""
    if not isinstance(m, Match):
        from . import moe as _moe
        return _moe.emit_reads(m)
    return (m.lhs,)


def emit_bytes(m) -> int:
    """Device bytes `emit` materializes beyond the root's result: one copy of the
    activation at most (transpose / cast / group permutation)."""
    if not isinstance(m, Match):
        from . import moe as _moe
        return _moe.emit_bytes(m)
    esize = torch.empty((), dtype=m.out_dtype).element_size() if m.out_dtype else 2
    return int(m.B * m.M * m.K * esize)


def emit(interp, m, env):
    """One fused `quantized_matmul` in place of the whole dequantize-and-dot."""
    if not isinstance(m, Match):
        from . import moe as _moe
        return _moe.emit(interp, m, env)
    st = interp._qmm
    vals = st.values[m.slot:m.slot + m.nvals]
    w, scales = vals[0], vals[1]
    biases = vals[2] if m.mode == "affine" else None
    x = env[m.lhs]
    if m.lperm is not None and list(m.lperm) != list(range(x.dim())):
        x = x.permute(*m.lperm)
    x = x.reshape([m.B, m.M, m.K] if m.bshape else [m.M, m.K])
    if x.dtype not in _FLOATS:
        x = x.to(m.out_dtype)
    if m.has_perm:
        x = x.index_select(-1, vals[-1].to(torch.int64))
    # The cast to the dot's result type happens in the kernel's epilogue.
    y = quantized_matmul(x, w, scales, biases, transpose=True, group_size=m.gs,
                         bits=m.bits, mode=m.mode, out_dtype=m.out_dtype)
    if m.swapped:
        y = y.transpose(-1, -2).reshape(list(m.bshape) + list(m.nshape) + list(m.mshape))
    else:
        y = y.reshape(list(m.bshape) + list(m.mshape) + list(m.nshape))
    return [y]
