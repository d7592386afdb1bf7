"""CPU restatement of the reference's quantized-matmul arithmetic (TEST INFRASTRUCTURE).

This module is the checker, not the product: only the test-suite, the smoke
check and the CPU-baseline leg of the benchmark may import it. Nothing under
`metaljax_b200/` imports it, and the product path raises when its CUDA library
is missing instead of falling back to anything here.

What it restates (reference = eterevsky/metaljax 0.11.3, paths inside that
project):

* the packed layouts the reference writes for MLX (`src/metaljax/qmm.py:206-232`
  `pack_codes`; `tests/test_qmm.py:60-73` `np_pack_codes` is the reference's own
  independent statement of the same bit stream),
* the affine repack algebra `q_hat = code + offset`,
  `biases = -scale * (offset + zero)` (`src/metaljax/qmm.py:235-282`),
* MXFP4: the E2M1 grid (`src/metaljax/qmm.py:172`), codes by integer bit
  equality (`:300-332`), E8M0 byte = f32 exponent field (`:335-357`), dequant
  (`tests/test_qmm_mxfp4.py:77-90`),
* the fused op itself: `mx.quantized_matmul(x, w, scales, biases,
  transpose=True, group_size, bits, mode)` as called at `src/metaljax/qmm.py:2491`
  -- `y[.., m, n] = sum_k x[.., m, k] * deq(w)[.., n, k]`, with
  `deq = scales * q + biases` evaluated as one FMA per element (affine,
  `src/metaljax/qmm.py:71-75`) or `E2M1[q] * 2**(s - 127)` (mxfp4),
* `mx.gather_qmm(x, w, scales, biases, lhs_idx, rhs_idx, transpose=True, ...)`
  as called at `src/metaljax/moe.py:1320-1322` and the weighted K-sum that
  follows it (`src/metaljax/moe.py:1448-1453`),
* the literal chains the recognizer replaces (what the CPU backend runs;
  `tests/test_qmm.py:193-199`, `tests/test_qmm_mxfp4.py:282-304`), evaluated in
  the activation dtype with per-op rounding, as the second oracle of the
  reference's own `_compare` rule (`tests/test_qmm.py:261-282`).

The arithmetic of `mx.quantized_matmul` lives in MLX (third party, pinned
`mlx>=0.32`, used at 0.32.0; not part of the reference tree). Parity is pinned
through the reference's tests at that boundary: the bit-stream formula, the
E2M1 table, the E8M0 round trips and reject sets, and the pack_exact algebra
cases; see `tests/golden/`.
"""

from __future__ import annotations

import numpy as np

try:  # bf16 for numpy
    import ml_dtypes
    bfloat16 = ml_dtypes.bfloat16
except Exception:  # pragma: no cover - ml_dtypes ships with the image
    bfloat16 = None

GROUP_SIZES = (128, 64, 32)          # src/metaljax/qmm.py:147
MXFP4_GROUP = 32                     # src/metaljax/qmm.py:173
E2M1_MAGS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)   # src/metaljax/qmm.py:172
# Indexed by the 4-bit code; bit 3 is the sign (tests/test_qmm_mxfp4.py:60-61).
E2M1 = np.array(list(E2M1_MAGS) + [-m for m in E2M1_MAGS], np.float32)


class Reject(Exception):
    """The reference's `_Reject` (src/metaljax/qmm.py:197): not representable."""


# --------------------------------------------------------------------------
# packing
# --------------------------------------------------------------------------


def pack_codes(codes: np.ndarray, bits: int) -> np.ndarray:
    """Unsigned codes `[..., K]` -> uint32 `[..., K*bits//32]`.

    Little-endian bit stream, LSB first: element i at bits [i*bits,(i+1)*bits)
    (src/metaljax/qmm.py:206-232). Written as the generic bit-stream loop of
    tests/test_qmm.py:60-73 so that it does not share structure with the
    product's packer.
    """
    if 32 % bits:
        raise ValueError(f"pack_codes: bits={bits} does not divide 32")
    per = 32 // bits
    c = np.ascontiguousarray(codes).astype(np.uint64)
    k = c.shape[-1]
    if k % per:
        raise ValueError(f"pack_codes: K={k} not a multiple of {per}")
    words = k * bits // 32
    flat = c.reshape(-1, k) & np.uint64((1 << bits) - 1)
    out = np.zeros((flat.shape[0], words), np.uint64)
    for i in range(k):
        w0, off = divmod(i * bits, 32)
        out[:, w0] |= (flat[:, i] << np.uint64(off)) & np.uint64(0xFFFFFFFF)
    return out.astype(np.uint32).reshape(*c.shape[:-1], words)


def unpack_codes(packed: np.ndarray, bits: int) -> np.ndarray:
    """Inverse of `pack_codes`: uint32 `[..., W]` -> uint8 `[..., W*32//bits]`."""
    per = 32 // bits
    p = np.ascontiguousarray(packed).astype(np.uint32)
    shifts = (np.arange(per, dtype=np.uint32) * np.uint32(bits))
    v = (p[..., None] >> shifts) & np.uint32((1 << bits) - 1)
    return v.reshape(*p.shape[:-1], p.shape[-1] * per).astype(np.uint8)


def pack_blocks(codes: np.ndarray) -> np.ndarray:
    """4-bit codes `[..., K]` -> HF-style bytes `[..., K//2]`: low nibble is the
    even element (tests/test_qmm_mxfp4.py:93-97)."""
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def scale_bias(scales, zeros, offset: int):
    """`biases = -scale * (offset + zero)` in float32
    (src/metaljax/qmm.py:262-272)."""
    s32 = np.asarray(scales, np.float32)
    z32 = (np.asarray(zeros).astype(np.float32) if zeros is not None
           else np.float32(0.0))
    return s32, (-(s32 * (z32 + np.float32(offset)))).astype(np.float32)


def lossless(x32: np.ndarray, dtype) -> bool:
    """src/metaljax/qmm.py:285-286."""
    return bool(np.all(x32.astype(dtype).astype(np.float32) == x32))


def pack_exact(codes, scales, zeros, bits: int, scale_dtype=None, offset=None,
               width: str = "auto"):
    """src/metaljax/qmm.py:235-282: signed codes `[N,K]`, per-group scales and
    zero points `[N,K/gs]` of `w = scale*(code - zero)` -> `(packed, s, b)`."""
    off = (1 << (bits - 1)) if offset is None else int(offset)
    packed = pack_codes(np.asarray(codes).astype(np.int64) + off, bits)
    s32, b32 = scale_bias(scales, zeros, off)
    if scale_dtype is not None and np.dtype(scale_dtype) != np.float32 \
            and width != "f32":
        if width == "source" or (lossless(s32, scale_dtype)
                                 and lossless(b32, scale_dtype)):
            return packed, s32.astype(scale_dtype), b32.astype(scale_dtype)
    return packed, s32, b32


# --------------------------------------------------------------------------
# MXFP4
# --------------------------------------------------------------------------


def _uint_view(dtype):
    dtype = np.dtype(dtype)
    if dtype == np.float32:
        return np.uint32, 32
    if dtype == np.float16 or (bfloat16 is not None and dtype == np.dtype(bfloat16)):
        return np.uint16, 16
    return None, 0


def mxfp4_codes(values: np.ndarray) -> np.ndarray:
    """4-bit codes of values lying exactly on the E2M1 grid, else `Reject`
    (src/metaljax/qmm.py:300-332). Sign is the top bit: -0.0 -> 8."""
    uint, width = _uint_view(values.dtype)
    if uint is None:
        raise Reject(f"MXFP4 values in {values.dtype}")
    bits = np.ascontiguousarray(values).view(uint)
    sign = (bits >> uint(width - 1)).astype(np.uint8)
    mag = bits & uint((1 << (width - 1)) - 1)
    grid = np.array(E2M1_MAGS, np.float32).astype(values.dtype).view(uint)
    codes = np.zeros(mag.shape, np.uint8)
    ok = np.zeros(mag.shape, bool)
    for i in range(len(E2M1_MAGS)):
        hit = mag == grid[i]
        codes[hit] = i
        ok |= hit
    if not ok.all():
        raise Reject("weight values are not on the MXFP4 (E2M1) grid")
    return codes | (sign << np.uint8(3))


def mxfp4_scale_bytes(scales: np.ndarray) -> np.ndarray:
    """E8M0 byte = f32 exponent field; sign/mantissa must be zero and the
    field must not be 0 or 255 (src/metaljax/qmm.py:335-357)."""
    bits = np.ascontiguousarray(np.asarray(scales, np.float32)).view(np.uint32)
    exp = (bits >> np.uint32(23)) & np.uint32(0xFF)
    bad = ((bits & np.uint32(0x807FFFFF)) != 0) | (exp == 0) | (exp == 0xFF)
    if bad.any():
        raise Reject("MXFP4 group scales are not exact positive powers of two")
    return exp.astype(np.uint8)


# --------------------------------------------------------------------------
# dequantization (what MLX's dequantize / the kernel's operand means)
# --------------------------------------------------------------------------


def dequant_affine(packed, scales, biases, group_size: int, bits: int) -> np.ndarray:
    """`scales*q + biases`, one FMA per element, float32 result
    (src/metaljax/qmm.py:71-75; pinned by tests/test_qmm.py:96-132).

    The FMA is emulated in float64: `s*q` is exact there (24+8 significant
    bits) and the single rounding to float32 happens on the way out.
    """
    q = unpack_codes(packed, bits).astype(np.float64)
    s = np.repeat(np.asarray(scales).astype(np.float64), group_size, axis=-1)
    b = np.repeat(np.asarray(biases).astype(np.float64), group_size, axis=-1)
    return (s * q + b).astype(np.float32)


def dequant_mxfp4(packed, scale_bytes) -> np.ndarray:
    """`E2M1[q] * 2**(byte-127)` (tests/test_qmm_mxfp4.py:77-90); exact in f32."""
    q = unpack_codes(packed, 4)
    vals = E2M1[q].astype(np.float64)
    sc = np.exp2(np.asarray(scale_bytes).astype(np.float64) - 127.0)
    out = vals * np.repeat(sc, MXFP4_GROUP, axis=-1)
    return out.astype(np.float32)


def dequantize(packed, scales, biases=None, group_size=64, bits=4, mode="affine"):
    if mode == "mxfp4":
        return dequant_mxfp4(packed, scales)
    return dequant_affine(packed, scales, biases, group_size, bits)


# --------------------------------------------------------------------------
# the fused op and its variants
# --------------------------------------------------------------------------


def _f64(x):
    return np.asarray(x).astype(np.float32).astype(np.float64)


def qmm_exact(x, packed, scales, biases=None, group_size=64, bits=4,
              mode="affine") -> np.ndarray:
    """Exact reference of `mx.quantized_matmul(..., transpose=True)`
    (src/metaljax/qmm.py:2491): dequantized weight in float32, products and
    sums in float64. `x` is `[..., M, K]`; `packed` `[(B,) N, K*bits/32]`.
    Returns float64 `[..., M, N]` -- callers round it as their case needs.
    """
    w = dequantize(packed, scales, biases, group_size, bits, mode).astype(np.float64)
    return np.matmul(_f64(x), np.swapaxes(w, -1, -2))


def qmm_literal(x, packed, scales, zeros_or_biases=None, group_size=64, bits=4,
                mode="affine", form="bias") -> np.ndarray:
    """The chain the recognizer replaces, evaluated the way a CPU backend runs
    it: every elementwise op in the activation dtype (one rounding per op),
    the dot upcast to float32 with the result rounded to the activation dtype.

    form="zero":  `(cvt(q) - cvt(zero)) * scale`   (tests/test_qmm.py:193-199)
    form="bias":  `cvt(q) * scale + bias`          (same value, spelled with
                  the folded bias -- the config-level `bias = -mid*scale`)
    mxfp4:        `E2M1[q] * 2**(byte-127)`        (tests/test_qmm_mxfp4.py:282-304)
    """
    dt = np.asarray(x).dtype
    if mode == "mxfp4":
        q = unpack_codes(packed, 4)
        vals = E2M1[q].astype(dt)
        sc = np.exp2(np.asarray(scales).astype(np.float32) - 127.0).astype(dt)
        w = (vals * np.repeat(sc, MXFP4_GROUP, axis=-1)).astype(dt)
    else:
        q = unpack_codes(packed, bits).astype(dt)
        s = np.repeat(np.asarray(scales).astype(dt), group_size, axis=-1)
        t = np.repeat(np.asarray(zeros_or_biases).astype(dt), group_size, axis=-1)
        if form == "zero":
            w = ((q - t).astype(dt) * s).astype(dt)
        else:
            w = ((q * s).astype(dt) + t).astype(dt)
    y = np.matmul(np.asarray(x).astype(np.float32),
                  np.swapaxes(w.astype(np.float32), -1, -2))
    return y.astype(dt)


def gather_qmm_exact(x, packed, scales, biases, lhs_idx, rhs_idx,
                     group_size=64, bits=4, mode="affine") -> np.ndarray:
    """`mx.gather_qmm` as called at src/metaljax/moe.py:1320-1322:
    `y[p] = x[lhs_idx[p]] @ deq(w[rhs_idx[p]]).T`, x `[T|P, M, K]`,
    w `[E, N, K*bits/32]` -> `[P, M, N]` (float64)."""
    w = dequantize(packed, scales, biases, group_size, bits, mode).astype(np.float64)
    xs = _f64(x)[np.asarray(lhs_idx, np.int64)]
    ws = w[np.asarray(rhs_idx, np.int64)]
    return np.matmul(xs, np.swapaxes(ws, -1, -2))


def ragged_qmm_exact(x, packed, scales, biases, group_sizes,
                     group_size=64, bits=4, mode="affine") -> np.ndarray:
    """`ragged_dot(lhs[m,k], rhs[g,k,n], group_sizes[g])` with a packed rhs:
    rows `[off[g], off[g+1])` of `x` meet expert g. This is `gather_qmm` with
    pairs sorted by expert. Rows past `sum(group_sizes)` are zero (the
    `lax.ragged_dot` convention)."""
    w = dequantize(packed, scales, biases, group_size, bits, mode).astype(np.float64)
    xs = _f64(x)
    out = np.zeros((xs.shape[0], w.shape[-2]), np.float64)
    lo = 0
    for g, n in enumerate(np.asarray(group_sizes).tolist()):
        out[lo:lo + n] = xs[lo:lo + n] @ w[g].T
        lo += n
    return out


def topk_router(logits: np.ndarray, k: int):
    """`top_k` (stable descending, lowest index wins ties:
    src/metaljax/ops/sort.py:206-214) then softmax over the selected values in
    float32 (tests/test_moe.py:60-66). Returns `(indices[T,k], weights[T,k])`."""
    lg = np.asarray(logits, np.float32)
    idx = np.argsort(-lg, axis=-1, kind="stable")[:, :k]
    vals = np.take_along_axis(lg, idx, axis=-1)
    e = np.exp(vals - vals.max(axis=-1, keepdims=True))
    return idx.astype(np.int32), (e / e.sum(axis=-1, keepdims=True)).astype(np.float32)


def moe_combine_exact(y_pairs: np.ndarray, weights: np.ndarray) -> np.ndarray:
    """`sum_k w[t,k] * y[t*K+k]` (src/metaljax/moe.py:1446-1453), float64."""
    t, k = weights.shape
    y = np.asarray(y_pairs, np.float64).reshape(t, k, -1)
    return (y * np.asarray(weights, np.float64)[..., None]).sum(axis=1)


# --------------------------------------------------------------------------
# group detection (what the pack prologue decides)
# --------------------------------------------------------------------------


def group_const(x: np.ndarray, gs: int) -> bool:
    """src/metaljax/qmm.py:1204-1207."""
    k = x.shape[-1]
    v = x.reshape(-1, k // gs, gs)
    return bool(np.all(v == v[:, :, :1]))


def pick_group(k: int, scale_map, zero_map=None):
    """Largest of (128, 64, 32) the maps are constant within, else None
    (src/metaljax/qmm.py:1219-1247)."""
    g0 = GROUP_SIZES[-1]
    if k % g0 or not group_const(scale_map, g0):
        return None
    if zero_map is not None and not group_const(zero_map, g0):
        return None
    for g in GROUP_SIZES:
        if k % g:
            continue
        if group_const(scale_map, g) and (zero_map is None or group_const(zero_map, g)):
            return g
    return None


# --------------------------------------------------------------------------
# error measures used by the parity gates
# --------------------------------------------------------------------------


def rel_err(got, exact) -> float:
    """`max|got - exact| / max|exact|` (tests/test_qmm.py:271-273)."""
    e = np.asarray(exact, np.float64)
    scale = np.abs(e).max()
    if scale == 0:
        scale = 1.0
    return float(np.abs(np.asarray(got).astype(np.float64) - e).max() / scale)
