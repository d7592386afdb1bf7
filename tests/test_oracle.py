"""The oracle against the reference's known answers (CPU only).

Every vector in tests/golden/qmm_golden.json comes from an independent statement in the
reference's own tests (see tests/golden/make_golden.py); the oracle is trusted only as far
as these pin it. The C restatement is then checked against the numpy one.
"""

import ml_dtypes
import numpy as np
import pytest

from helpers import BF16, activations, affine_case, digest, mxfp4_case
from oracle import clib
from oracle import qmm_oracle as O
from golden import make_golden as G


def test_nibble_stream(golden):
    g = golden["nibble_stream"]
    codes = np.array(g["codes"], np.uint8).reshape(1, 32)
    np.testing.assert_array_equal(O.pack_codes(codes, 4)[0], np.array(g["words"], np.uint32))
    np.testing.assert_array_equal(O.unpack_codes(np.array([g["words"]], np.uint32), 4), codes)


def test_bit_stream_matches_reference_statement(golden):
    for case in golden["bit_stream"]:
        rng = np.random.default_rng(case["seed"])
        codes = rng.integers(0, 1 << case["bits"], size=case["shape"]).astype(np.uint32)
        assert digest(codes) == case["codes_sha256"], "numpy draw changed: regenerate golden"
        got = O.pack_codes(codes, case["bits"])
        assert got.shape == tuple(case["shape"][:-1]) + (case["shape"][-1] * case["bits"] // 32,)
        flat = got.reshape(-1, got.shape[-1])
        assert flat[0].tolist() == case["first_row_words"]
        assert digest(flat) == case["words_sha256"]
        np.testing.assert_array_equal(O.unpack_codes(got, case["bits"]), codes.astype(np.uint8))


def test_e2m1_table(golden):
    np.testing.assert_array_equal(O.E2M1, np.array(golden["e2m1"], np.float32))
    assert np.signbit(O.E2M1[golden["e2m1_neg_zero_code"]]) and O.E2M1[8] == 0


@pytest.mark.parametrize("dtype", [np.float32, BF16, np.float16])
def test_mxfp4_codes_recovers_every_code(dtype):
    codes = np.tile(np.arange(16, dtype=np.uint8), 8).reshape(4, 32)
    np.testing.assert_array_equal(O.mxfp4_codes(O.E2M1[codes].astype(dtype)), codes)
    z = np.array([[0.0, -0.0] * 16], np.float32)
    np.testing.assert_array_equal(O.mxfp4_codes(z), np.array([[0, 8] * 16], np.uint8))


def test_e8m0_round_trip_and_rejects(golden):
    g = golden["e8m0"]
    for byte, sbits in zip(g["bytes"], g["scale_f32_bits"]):
        scale = np.full((2, 4), np.array(sbits, np.uint32).view(np.float32), np.float32)
        np.testing.assert_array_equal(O.mxfp4_scale_bytes(scale), np.full((2, 4), byte, np.uint8))
    for bad in g["reject_f32_bits"]:
        scale = np.array([[1.0, np.array(bad, np.uint32).view(np.float32)]], np.float32)
        with pytest.raises(O.Reject):
            O.mxfp4_scale_bytes(scale)


def test_off_grid_values_reject(golden):
    for bad in golden["off_grid"]:
        vals = np.concatenate([O.E2M1[:8], np.array([bad] * 8, np.float32)]).reshape(1, 16)
        with pytest.raises(O.Reject):
            O.mxfp4_codes(vals)


def test_pack_exact_matrix(golden):
    for case in golden["pack_exact"]:
        codes, scale, zp, want = G.pack_exact_case(case["bits"], case["gs"], case["zp_kind"],
                                                   case["scale_kind"])
        assert digest(codes) == case["codes_sha256"], "numpy draw changed: regenerate golden"
        assert digest(want) == case["want_sha256"]
        w, s, b = O.pack_exact(codes, scale, zp, case["bits"])
        got = O.dequant_affine(w, s, b, case["gs"], case["bits"])
        if case["must_be_exact"]:
            np.testing.assert_array_equal(got, want)
        else:
            assert np.abs(got - want).max() / np.abs(want).max() < case["rel_tol"]
        # the C restatement dequantizes to the same bits
        np.testing.assert_array_equal(
            clib.dequantize(w, s, b, codes.shape[0], codes.shape[1], case["gs"], case["bits"]), got)


def test_pack_exact_arbitrary_offset(golden):
    for case in golden["pack_exact_offset"]:
        rng = np.random.default_rng(2)
        codes = rng.integers(-8, 8, size=(4, 128)).astype(np.int32) + case["shift"]
        scale = ((rng.random((4, 1)).astype(np.float32) + 0.5) * 0.1).astype(BF16).astype(np.float32)
        w, s, b = O.pack_exact(codes, scale, None, 4, offset=case["offset"])
        got = O.dequant_affine(w, s, b, 128, 4)
        assert digest(got) == case["want_sha256"]


def test_pack_exact_keeps_source_dtype_when_lossless():
    rng = np.random.default_rng(1)
    codes = rng.integers(-8, 8, size=(8, 128)).astype(np.int32)
    scale = np.exp2(rng.integers(-6, 0, size=(8, 1))).astype(np.float32)
    _, s, b = O.pack_exact(codes, scale, None, 4, scale_dtype=BF16)
    assert s.dtype == np.dtype(BF16) and b.dtype == np.dtype(BF16)
    scale = rng.random((8, 1)).astype(np.float32) + 1.0
    _, s, b = O.pack_exact(codes, scale, np.full((8, 1), 3, np.int32), 4, scale_dtype=BF16)
    assert s.dtype == np.float32 and b.dtype == np.float32


def test_mxfp4_dequant_bit_exact(golden):
    for case in golden["mxfp4_dequant"]:
        rng = np.random.default_rng(case["seed"])
        codes, sb, w = G.random_mxfp4(tuple(case["shape"]), rng)
        assert digest(codes) == case["codes_sha256"], "numpy draw changed: regenerate golden"
        assert digest(w) == case["weight_sha256"]
        packed = O.pack_codes(codes, 4)
        got = O.dequant_mxfp4(packed, sb)
        np.testing.assert_array_equal(got, w)
        np.testing.assert_array_equal(got.astype(BF16).astype(np.float32), w)   # exact in bf16
        # HF `_blocks` bytes are the same stream: low nibble = even element
        np.testing.assert_array_equal(O.pack_blocks(codes).reshape(-1),
                                      packed.view(np.uint8).reshape(-1))


def test_group_picks():
    rng = np.random.default_rng(0)
    heads = rng.random((4, 2)).astype(np.float32)
    assert O.pick_group(256, np.repeat(heads, 128, axis=1)) == 128
    heads = rng.random((4, 8)).astype(np.float32)
    assert O.pick_group(256, np.repeat(heads, 32, axis=1)) == 32
    assert O.pick_group(256, rng.random((4, 256)).astype(np.float32)) is None
    assert O.pick_group(48, np.ones((4, 48), np.float32)) is None


@pytest.mark.parametrize("bits,gs,table", [(4, 64, "bf16"), (8, 128, "bf16"), (4, 32, "f32")])
def test_c_oracle_matches_numpy_oracle(bits, gs, table):
    rng = np.random.default_rng(bits + gs)
    n, k, m = 40, 256, 5
    _, w, s, b = affine_case(rng, n, k, gs, bits, table)
    x = activations(rng, (m, k))
    exact = O.qmm_exact(x, w, s, b, gs, bits)
    y32 = clib.qmm(x, w, s, b, m, k, n, gs, bits, out_f32=True)
    assert O.rel_err(y32, exact) < 1e-6
    ybf = clib.qmm(x, w, s, b, m, k, n, gs, bits).view(BF16).astype(np.float32)
    assert O.rel_err(ybf, exact) < 5e-3
    lit = O.qmm_literal(x, w, s, b, gs, bits).astype(np.float32)
    assert O.rel_err(lit, exact) < 1e-2


def test_c_oracle_mxfp4_and_ragged():
    rng = np.random.default_rng(5)
    n, k = 48, 128
    _, w, sb = mxfp4_case(rng, n, k, lead=(3,))
    x = activations(rng, (10, k))
    gsz = np.array([4, 0, 5], np.int32)                 # one row left over -> zero
    exact = O.ragged_qmm_exact(x, w, sb, None, gsz, 32, 4, "mxfp4")
    got = clib.qmm_ragged(x, w, sb, None, gsz, 10, k, n, 32, 4, "mxfp4", out_f32=True)
    assert O.rel_err(got, exact) < 1e-6
    assert not got[9].any()
    # gather in router order equals ragged in sorted order
    lhs = np.array([0, 1, 2, 3, 4, 5, 6, 7, 8]); rhs = np.array([0, 0, 0, 0, 2, 2, 2, 2, 2])
    gat = O.gather_qmm_exact(x[:, None, :], w, sb, None, lhs, rhs, 32, 4, "mxfp4")[:, 0]
    np.testing.assert_allclose(gat, exact[:9], rtol=0, atol=0)


def test_router_and_combine():
    logits = np.array([[0.5, 0.5, 0.1, 0.9], [1.0, 1.0, 1.0, 1.0]], np.float32)
    idx, wts = O.topk_router(logits, 2)
    assert idx.tolist() == [[3, 0], [0, 1]]             # ties: lowest index first
    np.testing.assert_allclose(wts.sum(axis=1), 1.0, rtol=1e-6)
    y = np.arange(8, dtype=np.float64).reshape(4, 2)
    np.testing.assert_allclose(O.moe_combine_exact(y, wts)[1], 0.5 * y[2] + 0.5 * y[3])
