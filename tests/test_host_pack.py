"""Host side of the drop-in (metaljax_b200.qmm on CPU tensors) against the oracle: the pack
primitives, the group detection and the pack builder keep the reference's behaviour
(tests/test_qmm.py:60-171, 510-571; tests/test_qmm_mxfp4.py:116-174)."""

import numpy as np
import pytest
import torch

from helpers import BF16, to_numpy, to_torch
from metaljax_b200 import qmm
from oracle import qmm_oracle as O
from golden import make_golden as G


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("shape", [(1, 32), (5, 128), (3, 4, 64)])
def test_pack_codes_matches_oracle(bits, shape):
    rng = np.random.default_rng(0)
    codes = rng.integers(0, 1 << bits, size=shape).astype(np.uint8)
    got = to_numpy(qmm.pack_codes(torch.from_numpy(codes), bits))
    np.testing.assert_array_equal(got, O.pack_codes(codes, bits))


def test_pack_codes_masks_and_rejects():
    codes = torch.full((1, 8), 0x1F, dtype=torch.int32)           # out-of-range: masked to 4 bits
    assert to_numpy(qmm.pack_codes(codes, 4))[0, 0] == 0xFFFFFFFF
    with pytest.raises(ValueError):
        qmm.pack_codes(torch.zeros((1, 6), dtype=torch.uint8), 4)
    with pytest.raises(ValueError):
        qmm.pack_codes(torch.zeros((1, 32), dtype=torch.uint8), 5)


def test_pack_exact_matrix_matches_golden(golden):
    for case in golden["pack_exact"]:
        codes, scale, zp, want = G.pack_exact_case(case["bits"], case["gs"], case["zp_kind"],
                                                   case["scale_kind"])
        w, s, b = qmm.pack_exact(torch.from_numpy(codes), torch.from_numpy(scale),
                                 torch.from_numpy(zp), case["bits"])
        ow, os_, ob = O.pack_exact(codes, scale, zp, case["bits"])
        np.testing.assert_array_equal(to_numpy(w), ow)
        np.testing.assert_array_equal(to_numpy(s), os_)
        np.testing.assert_array_equal(to_numpy(b), ob)
        got = O.dequant_affine(to_numpy(w), to_numpy(s), to_numpy(b), case["gs"], case["bits"])
        if case["must_be_exact"]:
            np.testing.assert_array_equal(got, want)


def test_pack_exact_scale_width_policy():
    if qmm._SCALE_WIDTH != "auto":
        pytest.skip("METALJAX_QMM_SCALES overrides the width policy")
    rng = np.random.default_rng(1)
    codes = torch.from_numpy(rng.integers(-8, 8, size=(8, 128)).astype(np.int32))
    scale = torch.from_numpy(np.exp2(rng.integers(-6, 0, size=(8, 1))).astype(np.float32))
    _, s, b = qmm.pack_exact(codes, scale, None, 4, scale_dtype=torch.bfloat16)
    assert s.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    scale = torch.from_numpy(rng.random((8, 1)).astype(np.float32) + 1.0)
    zp = torch.full((8, 1), 3, dtype=torch.int32)
    _, s, b = qmm.pack_exact(codes, scale, zp, 4, scale_dtype=torch.bfloat16)
    assert s.dtype == torch.float32 and b.dtype == torch.float32


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_mxfp4_codes(dtype, golden):
    codes = np.tile(np.arange(16, dtype=np.uint8), 8).reshape(4, 32)
    vals = torch.from_numpy(O.E2M1[codes]).to(dtype)
    np.testing.assert_array_equal(qmm.mxfp4_codes(vals).numpy(), codes)
    z = torch.tensor([[0.0, -0.0] * 16], dtype=dtype)
    np.testing.assert_array_equal(qmm.mxfp4_codes(z).numpy(), np.array([[0, 8] * 16], np.uint8))
    for bad in golden["off_grid"]:
        v = torch.tensor([list(O.E2M1[:8]) + [bad] * 8], dtype=dtype)
        with pytest.raises(qmm._Reject):
            qmm.mxfp4_codes(v)


def test_mxfp4_scale_bytes(golden):
    g = golden["e8m0"]
    for byte, sbits in zip(g["bytes"], g["scale_f32_bits"]):
        scale = torch.from_numpy(np.full((2, 4), np.array(sbits, np.uint32).view(np.float32)))
        np.testing.assert_array_equal(qmm.mxfp4_scale_bytes(scale).numpy(),
                                      np.full((2, 4), byte, np.uint8))
    for bad in g["reject_f32_bits"]:
        scale = torch.from_numpy(np.array([[1.0, np.array(bad, np.uint32).view(np.float32)]],
                                          np.float32))
        with pytest.raises(qmm._Reject):
            qmm.mxfp4_scale_bytes(scale)


def test_group_picks_and_regroup():
    rng = np.random.default_rng(3)
    heads = torch.from_numpy(rng.random((4, 2)).astype(np.float32))
    assert qmm._pick_group(256, heads.repeat_interleave(128, dim=1), None) == 128
    heads = torch.from_numpy(rng.random((4, 4)).astype(np.float32))
    smap = heads.repeat_interleave(64, dim=1)
    assert qmm._pick_group(256, smap, None) == 64
    assert qmm._pick_group(256, torch.from_numpy(rng.random((4, 256)).astype(np.float32)), None) is None
    # interleaved groups: column k belongs to group k % 4 -> a permutation brings them together
    inter = heads[:, torch.arange(256) % 4]
    assert qmm._pick_group(256, inter, None) is None
    perm = qmm._regroup(256, [inter, None])
    assert perm is not None and sorted(perm.tolist()) == list(range(256))
    assert qmm._pick_group(256, qmm._take_k(inter, perm), None) == 64
    assert qmm._regroup(256, [smap, None]) is None          # already grouped: identity stays free


def _match(mode="affine"):
    m = qmm.Match()
    m.mode = mode
    return m


def test_build_pack_affine_signed_and_unsigned_codes():
    qmm.reset_stats()
    rng = np.random.default_rng(4)
    n, k, gs = 8, 256, 64
    heads = (rng.random((n, k // gs)).astype(np.float32) + 0.5).astype(BF16).astype(np.float32)
    smap = torch.from_numpy(np.repeat(heads, gs, axis=1))
    zmap = torch.from_numpy(np.repeat(rng.integers(-3, 4, (n, k // gs)), gs, axis=1).astype(np.int8))
    for lo, hi, want_bits in ((-8, 8, 4), (0, 16, 4), (0, 256, 8), (-128, 128, 8)):
        codes = rng.integers(lo, hi, size=(n, k)).astype(np.int32)
        codes[0, :2] = [lo, hi - 1]
        m = _match()
        pack = qmm.build_pack(m, torch.from_numpy(codes), smap, zmap)
        assert (m.bits, m.gs, m.has_perm, m.nvals) == (want_bits, gs, False, 3)
        want = smap.numpy() * (codes.astype(np.float32) - zmap.numpy().astype(np.float32))
        got = O.dequant_affine(to_numpy(pack.w), to_numpy(pack.scales), to_numpy(pack.biases),
                               gs, want_bits)
        np.testing.assert_array_equal(got, want)
    assert qmm.stats()["packs"] == 4
    with pytest.raises(qmm._Reject):
        qmm.build_pack(_match(), torch.from_numpy(rng.integers(0, 300, (n, k)).astype(np.int32)),
                       smap, None)
    with pytest.raises(qmm._Reject):                     # non-integer zero point
        qmm.build_pack(_match(), torch.zeros((n, k), dtype=torch.int32), smap, zmap.float() + 0.5)
    m = _match()
    m.sub_range = (-128, 127)                            # int8 subtraction would wrap
    with pytest.raises(qmm._Reject):
        qmm.build_pack(m, torch.full((n, k), 127, dtype=torch.int32), smap,
                       torch.full((n, k), -3, dtype=torch.int8))


def test_build_pack_interleaved_groups_carry_a_permutation():
    qmm.reset_stats()
    rng = np.random.default_rng(6)
    n, k = 4, 256
    heads = torch.from_numpy((rng.random((n, 4)).astype(np.float32) + 0.5))
    smap = heads[:, torch.arange(k) % 4]
    codes = torch.from_numpy(rng.integers(-8, 8, (n, k)).astype(np.int32))
    m = _match()
    pack = qmm.build_pack(m, codes, smap, None)
    assert m.has_perm and m.nvals == 4 and qmm.stats()["perms"] == 1
    perm = pack.perm.numpy()
    got = O.dequant_affine(to_numpy(pack.w), to_numpy(pack.scales), to_numpy(pack.biases), m.gs, m.bits)
    np.testing.assert_array_equal(got, (smap * codes.float()).numpy()[:, perm])


def test_build_pack_mxfp4():
    qmm.reset_stats()
    rng = np.random.default_rng(8)
    codes, sb, w = G.random_mxfp4((6, 128), rng)
    vals = torch.from_numpy(O.E2M1[codes]).to(torch.bfloat16)
    smap = torch.from_numpy(np.repeat(np.exp2(sb.astype(np.float32) - 127), 32, axis=1))
    m = _match("mxfp4")
    pack = qmm.build_pack(m, vals, smap, None)
    assert (m.bits, m.gs, m.nvals) == (4, 32, 2) and pack.biases is None
    assert qmm.stats()["mxfp4"] == 1
    np.testing.assert_array_equal(pack.scales.numpy(), sb)
    np.testing.assert_array_equal(O.dequant_mxfp4(to_numpy(pack.w), sb), w)
    with pytest.raises(qmm._Reject):
        qmm.build_pack(_match("mxfp4"), vals, smap * 3, None)       # not a power of two
    with pytest.raises(qmm._Reject):
        qmm.build_pack(_match("mxfp4"), vals + 0.25, smap, None)    # off the grid


def test_pack_lru_and_identity():
    a, b = torch.zeros(1), torch.zeros(1)
    p = qmm._Pack([a, b], None, None, None, None, 64, 4)
    assert p.matches([a, b]) and not p.matches([b, a]) and not p.matches([a])
    assert len(p.arrays()) == 2
    st = qmm.State()
    m = _match(); m.key = "dot0"; m.ops = {"k1": 1}
    st.matches.append(m); st.rebuild()
    assert st.active and st.roots == {"dot0": m} and st.skip == frozenset({"k1"})
    m.disabled = True; st.rebuild()
    assert not st.active
