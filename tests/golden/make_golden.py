"""Writes tests/golden/qmm_golden.json: known-answer vectors for the packed layouts and the
dequantization algebra, derived from the reference's own tests.

The reference (eterevsky/metaljax 0.11.3) cannot be imported where this runs -- its modules
need jax, jaxlib.mlir and mlx -- so the vectors are produced from the *independent
statements* its tests make of each contract, not from its implementation and not from the
oracle under test:

  nibble_stream   tests/test_qmm_mxfp4.py:162-174  word = sum(code[8w+i] << 4i)
  bit_stream      tests/test_qmm.py:76-83 (shapes, seed 0), here as one big integer per row,
                  `sum(code_i << (i*bits))`, cut into little-endian 32-bit words -- the
                  definition of src/metaljax/qmm.py:209-212
  e2m1            src/metaljax/qmm.py:172, tests/test_qmm_mxfp4.py:60-61
  e8m0            tests/test_qmm_mxfp4.py:136-151 (round trips and the reject set)
  off_grid        tests/test_qmm_mxfp4.py:154-159
  pack_exact      tests/test_qmm.py:96-132: want = scale * (code - zp) in float32 and which
                  cases must be bit-exact; tests/test_qmm.py:135-152 (arbitrary offsets)
  mxfp4_dequant   tests/test_qmm_mxfp4.py:77-108, 250-262

Large arrays are stored as SHA-256 digests of their little-endian bytes plus a short prefix;
the test regenerates the inputs from the recorded seeds.

    python tests/golden/make_golden.py
"""

import hashlib
import json
import os

import ml_dtypes
import numpy as np

E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
        -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]


def digest(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def bigint_words(row, bits):
    """One row of codes as a single little-endian integer, cut into uint32 words."""
    total = 0
    for i, c in enumerate(row):
        total |= (int(c) & ((1 << bits) - 1)) << (i * bits)
    n = len(row) * bits // 32
    return [(total >> (32 * j)) & 0xFFFFFFFF for j in range(n)]


def scale_kind(kind, shape, rng):
    s = (rng.random(shape).astype(np.float32) + 0.5) * 0.03
    if kind == "pow2":
        return np.exp2(rng.integers(-8, 2, size=shape)).astype(np.float32)
    if kind == "bf16":
        return s.astype(ml_dtypes.bfloat16).astype(np.float32)
    return s


def pack_exact_case(bits, gs, zp_kind, sk):
    rng = np.random.default_rng(bits * 100 + gs)
    n, k = 16, 256
    lo, hi = -(1 << (bits - 1)), (1 << (bits - 1)) - 1
    codes = rng.integers(lo, hi + 1, size=(n, k)).astype(np.int32)
    codes[0, :4] = [lo, hi, 0, -1]
    ng = k // gs
    scale = scale_kind(sk, (n, ng), rng)
    if zp_kind == "zero":
        zp = np.zeros((n, ng), np.int32)
    elif zp_kind == "const":
        zp = np.full((n, ng), 3, np.int32)
    else:
        zp = rng.integers(lo, hi + 1, size=(n, ng)).astype(np.int32)
    want = scale.repeat(gs, axis=1) * (codes.astype(np.float32)
                                       - zp.repeat(gs, axis=1).astype(np.float32))
    return codes, scale, zp, want


def random_mxfp4(shape_nk, rng, exp_lo=118, exp_hi=132):
    *lead, k = shape_nk
    codes = rng.integers(0, 16, size=tuple(lead) + (k,)).astype(np.uint8)
    codes.reshape(-1, k)[0, :16] = np.arange(16)
    sb = rng.integers(exp_lo, exp_hi, size=tuple(lead) + (k // 32,)).astype(np.uint8)
    vals = np.array(E2M1, np.float32)[codes]
    scale = np.exp2(sb.astype(np.float32) - 127.0)
    w = (vals.reshape(tuple(lead) + (k // 32, 32)) * scale[..., None]).reshape(codes.shape)
    return codes, sb, w.astype(np.float32)


def main():
    g = {}
    codes = (np.arange(32) % 16).astype(np.uint8)
    g["nibble_stream"] = {
        "codes": codes.tolist(),
        "words": [sum(int(codes[8 * w + i]) << (4 * i) for i in range(8)) for w in range(4)],
    }
    g["bit_stream"] = []
    for bits in (4, 8):
        for shape in ((1, 32), (5, 128), (3, 4, 64)):
            rng = np.random.default_rng(0)
            c = rng.integers(0, 1 << bits, size=shape).astype(np.uint32)
            flat = c.reshape(-1, shape[-1])
            words = np.array([bigint_words(r, bits) for r in flat], np.uint32)
            g["bit_stream"].append({
                "bits": bits, "shape": list(shape), "seed": 0,
                "codes_sha256": digest(c), "words_sha256": digest(words),
                "first_row_words": words[0].tolist()})
    g["e2m1"] = E2M1
    g["e2m1_neg_zero_code"] = 8
    g["e8m0"] = {
        "bytes": [1, 100, 127, 200, 254],
        "scale_f32_bits": [int(np.array(np.exp2(float(b) - 127.0), np.float32).view(np.uint32))
                           for b in (1, 100, 127, 200, 254)],
        "reject_f32_bits": [int(np.array(v, np.float32).view(np.uint32))
                            for v in (3.0, 0.0, -2.0, np.inf, np.nan, 1.5e-38)],
    }
    g["off_grid"] = [0.7, 5.0, 8.0, 0.25, float("nan")]
    g["pack_exact"] = []
    for bits in (4, 8):
        for gs in (32, 64, 128):
            for zp_kind in ("zero", "const", "random"):
                for sk in ("pow2", "bf16", "f32"):
                    codes, scale, zp, want = pack_exact_case(bits, gs, zp_kind, sk)
                    g["pack_exact"].append({
                        "bits": bits, "gs": gs, "zp_kind": zp_kind, "scale_kind": sk,
                        "must_be_exact": zp_kind == "zero" or sk in ("pow2", "bf16"),
                        "rel_tol": 1e-5,
                        "codes_sha256": digest(codes), "want_sha256": digest(want),
                        "want_prefix": [float(v) for v in want[0, :8]]})
    g["pack_exact_offset"] = []
    for shift in (0, 8, -20):
        rng = np.random.default_rng(2)
        codes = rng.integers(-8, 8, size=(4, 128)).astype(np.int32) + shift
        scale = ((rng.random((4, 1)).astype(np.float32) + 0.5) * 0.1).astype(
            ml_dtypes.bfloat16).astype(np.float32)
        want = scale * codes.astype(np.float32)
        g["pack_exact_offset"].append({
            "shift": shift, "offset": -int(codes.min()), "want_sha256": digest(want),
            "want_prefix": [float(v) for v in want[0, :8]]})
    g["mxfp4_dequant"] = []
    for shape in ((4, 64), (3, 2, 128)):
        rng = np.random.default_rng(7 + sum(shape))
        codes, sb, w = random_mxfp4(shape, rng)
        g["mxfp4_dequant"].append({
            "shape": list(shape), "seed": 7 + sum(shape), "codes_sha256": digest(codes),
            "scale_bytes_sha256": digest(sb), "weight_sha256": digest(w),
            "weight_prefix": [float(v) for v in w.reshape(-1)[:8]]})
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "qmm_golden.json")
    with open(out, "w") as f:
        json.dump(g, f, indent=1, allow_nan=True)
    print(out)


if __name__ == "__main__":
    main()
