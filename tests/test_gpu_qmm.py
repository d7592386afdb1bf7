"""Parity of the CUDA path against the oracle, through the C ABI (needs a B200).

Gates, as the reference's own `_compare` / `_no_worse_than` state them
(tests/test_qmm.py:261-282, tests/test_qmm_mxfp4.py:319-336), with `exact` the float64
product against the exactly dequantized weight:

  * integer unpacking and dequantization: BIT-EXACT against the oracle;
  * 16-bit activations: max|y - exact| <= 1e-2 * max|exact|, and, when the output has the
    activation's type, err <= 1.5 * err_literal + 1e-6 where `literal` is the chain the
    recognizer replaces evaluated the way a CPU backend runs it;
  * float32 activations: max|y - exact| <= 1e-5 * max|exact|.
"""

import numpy as np
import pytest
import torch

from helpers import BF16, activations, affine_case, mxfp4_case, np_dtype, to_numpy, to_torch
from metaljax_b200 import _lib, moe, qmm
from oracle import clib
from oracle import qmm_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL16 = 1e-2       # north-star bound for bf16/f16 activations
TOL32 = 1e-5       # float32 activations (tests/test_qmm_mxfp4.py:333)
TDT = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}


@pytest.fixture(autouse=True)
def _device_ok():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    yield
    assert _lib.poll_status() == 0          # no bounded wait ran out, no sticky CUDA error


def _gate(got, exact, x_dtype, literal=None):
    err = O.rel_err(got, exact)
    if x_dtype == "f32":
        assert err <= TOL32, err
        return err
    assert err <= TOL16, err
    if literal is not None:
        err_lit = O.rel_err(literal.astype(np.float32), exact)
        assert err <= 1.5 * err_lit + 1e-6, (err, err_lit)
    return err


def _run_affine(rng, m, k, n, gs, bits, xdt="bf16", tdt="bf16", ydt=None, route=None, lead=()):
    _, w, s, b = affine_case(rng, n, k, gs, bits, tdt)
    x = activations(rng, tuple(lead) + (m, k), xdt)
    ydt = ydt or xdt
    if route == "gemv" and m > 16:
        pytest.skip("the decode kernel takes M <= 16")
    args = [to_torch(a, DEV) for a in (x, w, s, b)]
    kw = dict(group_size=gs, bits=bits, out_dtype=TDT[ydt])
    if route:
        with _lib.force_route(route):
            y = qmm.quantized_matmul(*args, **kw)
    else:
        y = qmm.quantized_matmul(*args, **kw)
    exact = O.qmm_exact(x, w, s, b, gs, bits)
    lit = O.qmm_literal(x, w, s, b, gs, bits) if (ydt == xdt and xdt != "f32") else None
    assert tuple(y.shape) == tuple(lead) + (m, n) and y.dtype == TDT[ydt]
    return _gate(to_numpy(y).astype(np.float32), exact, xdt, lit)


# ---- integer / dequant work: bit-exact ---------------------------------------------------


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("shape", [(1, 32), (5, 128), (3, 4, 64), (33, 4096)])
def test_pack_codes_kernel_bit_exact(bits, shape):
    rng = np.random.default_rng(0)
    codes = rng.integers(0, 1 << bits, size=shape).astype(np.uint8)
    got = to_numpy(qmm.pack_codes(torch.from_numpy(codes).to(DEV), bits))
    np.testing.assert_array_equal(got, O.pack_codes(codes, bits))
    wide = torch.from_numpy(codes.astype(np.int32) + (1 << bits)).to(DEV)      # masked to `bits`
    np.testing.assert_array_equal(to_numpy(qmm.pack_codes(wide, bits)), O.pack_codes(codes, bits))


@pytest.mark.parametrize("bits,gs", [(4, 32), (4, 64), (4, 128), (8, 32), (8, 64), (8, 128)])
@pytest.mark.parametrize("tdt", ["bf16", "f16", "f32"])
def test_dequantize_affine_bit_exact(bits, gs, tdt):
    rng = np.random.default_rng(bits * 10 + gs)
    n, k = 37, 384
    codes, w, s, b = affine_case(rng, n, k, gs, bits, tdt, lead=(2,))
    codes.reshape(-1, k)[0, : 1 << min(bits, 6)] = np.arange(1 << min(bits, 6))   # every low code
    w = O.pack_codes(codes, bits)
    got = to_numpy(qmm.dequantize(to_torch(w, DEV), to_torch(s, DEV), to_torch(b, DEV), gs, bits))
    np.testing.assert_array_equal(got, O.dequant_affine(w, s, b, gs, bits))
    np.testing.assert_array_equal(O.unpack_codes(w, bits), codes)


def test_dequantize_pack_exact_matrix(golden):
    """The reference's bit-exactness matrix (tests/test_qmm.py:96-132) on the GPU."""
    from golden import make_golden as G
    for case in golden["pack_exact"]:
        codes, scale, zp, want = G.pack_exact_case(case["bits"], case["gs"], case["zp_kind"],
                                                   case["scale_kind"])
        w, s, b = qmm.pack_exact(torch.from_numpy(codes).to(DEV), torch.from_numpy(scale).to(DEV),
                                 torch.from_numpy(zp).to(DEV), case["bits"])
        got = to_numpy(qmm.dequantize(w, s, b, case["gs"], case["bits"]))
        if case["must_be_exact"]:
            np.testing.assert_array_equal(got, want)
        else:
            assert np.abs(got - want).max() / np.abs(want).max() < case["rel_tol"]


@pytest.mark.parametrize("out", ["f32", "bf16", "f16"])
def test_dequantize_mxfp4_bit_exact(out, golden):
    from golden import make_golden as G
    for case in golden["mxfp4_dequant"]:
        rng = np.random.default_rng(case["seed"])
        codes, sb, wref = G.random_mxfp4(tuple(case["shape"]), rng)
        packed = qmm.pack_codes(torch.from_numpy(codes).to(DEV), 4)
        np.testing.assert_array_equal(to_numpy(packed), O.pack_codes(codes, 4))
        got = qmm.dequantize(packed, torch.from_numpy(sb).to(DEV), None, 32, 4, "mxfp4", dtype=TDT[out])
        if out == "f16":     # 2^-9..2^4 scales times E2M1 stay exactly representable here
            np.testing.assert_array_equal(to_numpy(got).astype(np.float32), wref.astype(np.float16).astype(np.float32))
        else:
            np.testing.assert_array_equal(to_numpy(got).astype(np.float32), wref)


# ---- the fused op --------------------------------------------------------------------------

SHAPES = [  # (M, K, N)
    (1, 64, 8), (1, 4096, 256), (2, 128, 40), (3, 96, 130), (5, 256, 200), (16, 512, 128),
    (17, 320, 136), (64, 256, 512), (100, 192, 384), (128, 1024, 256), (200, 2880, 264),
    (257, 512, 520), (600, 256, 128),
]


@pytest.mark.parametrize("route", ["simt", "gemm_tc", "gemv", None])
@pytest.mark.parametrize("m,k,n", SHAPES)
def test_qmm_affine4_g64(route, m, k, n):
    rng = np.random.default_rng(m * 7 + n)
    _run_affine(rng, m, k, n, 64 if k % 64 == 0 else 32, 4, route=route)


@pytest.mark.parametrize("route", ["simt", "gemm_tc", "gemv", None])
@pytest.mark.parametrize("bits,gs", [(4, 32), (4, 128), (8, 32), (8, 64), (8, 128)])
@pytest.mark.parametrize("m", [1, 7, 40, 300])
def test_qmm_affine_variants(route, bits, gs, m):
    rng = np.random.default_rng(bits + gs + m)
    _run_affine(rng, m, 384, 200, gs, bits, route=route)


@pytest.mark.parametrize("route", ["simt", "gemm_tc", "gemv", None])
@pytest.mark.parametrize("xdt,tdt,ydt", [("f16", "f16", "f16"), ("bf16", "f32", "bf16"),
                                         ("bf16", "bf16", "f32"), ("f16", "bf16", "bf16"),
                                         ("bf16", "f16", "f16")])
def test_qmm_dtype_combinations(route, xdt, tdt, ydt):
    rng = np.random.default_rng(11)
    for m in (2, 150):
        _run_affine(rng, m, 256, 136, 64, 4, xdt, tdt, ydt, route=route)
        _run_affine(rng, m, 256, 136, 128, 8, xdt, tdt, ydt, route=route)


@pytest.mark.parametrize("m", [1, 4, 33])
def test_qmm_float32_activations(m):
    rng = np.random.default_rng(12)
    assert _run_affine(rng, m, 512, 72, 64, 4, "f32", "f32") <= TOL32
    assert _run_affine(rng, m, 512, 72, 32, 8, "f32", "bf16") <= TOL32
    with _lib.force_route("gemm_tc"):
        with pytest.raises(_lib.QmmError) as e:
            _run_affine(rng, m, 512, 72, 64, 4, "f32", "f32")
        assert e.value.status == 7


@pytest.mark.parametrize("route", ["simt", "gemm_tc", "gemv", None])
@pytest.mark.parametrize("m", [1, 3, 64, 512])
@pytest.mark.parametrize("xdt", ["bf16", "f16", "f32"])
def test_qmm_mxfp4(route, m, xdt):
    if xdt == "f32" and route in ("gemm_tc", "gemv"):
        pytest.skip("float32 activations take the SIMT route")
    if route == "gemv" and m > 16:
        pytest.skip("the decode kernel takes M <= 16")
    rng = np.random.default_rng(m + 3)
    n, k = 192, 320
    codes, w, sb = mxfp4_case(rng, n, k)
    codes[0, :16] = np.arange(16)
    w = O.pack_codes(codes, 4)
    x = activations(rng, (m, k), xdt, 0.4)
    args = (to_torch(x, DEV), to_torch(w, DEV), to_torch(sb, DEV), None)
    kw = dict(group_size=32, bits=4, mode="mxfp4")
    if route:
        with _lib.force_route(route):
            y = qmm.quantized_matmul(*args, **kw)
    else:
        y = qmm.quantized_matmul(*args, **kw)
    exact = O.qmm_exact(x, w, sb, None, 32, 4, "mxfp4")
    lit = O.qmm_literal(x, w, sb, None, 32, 4, "mxfp4") if xdt != "f32" else None
    _gate(to_numpy(y).astype(np.float32), exact, xdt, lit)


def test_mxfp4_every_code_and_scale_extremes():
    """All 16 codes against one-hot activations recover the dequantized weight itself, for
    E8M0 bytes across the range the 16-bit kernels can represent."""
    k, n = 64, 16
    codes = np.tile(np.arange(16, dtype=np.uint8), (n, k // 16))
    sb = np.tile(np.array([[100, 127], [126, 128], [110, 134], [120, 121]], np.uint8), (n // 4, 1))
    w = O.pack_codes(codes, 4)
    wref = O.dequant_mxfp4(w, sb)
    x = np.eye(k, dtype=np.float32).astype(BF16)
    for route in ("simt", "gemm_tc", "gemv"):
        xs = x[:16] if route == "gemv" else x
        with _lib.force_route(route):
            y = qmm.quantized_matmul(to_torch(xs, DEV), to_torch(w, DEV), to_torch(sb, DEV), None,
                                     group_size=32, bits=4, mode="mxfp4", out_dtype=torch.float32)
        np.testing.assert_array_equal(to_numpy(y), wref.T[: len(xs)])


def test_affine_one_hot_recovers_dequantized_weight():
    """x = I makes y = deq(w)^T: exposes any K / feature / token permutation in a kernel."""
    rng = np.random.default_rng(21)
    k, n = 128, 136
    _, w, s, b = affine_case(rng, n, k, 64, 4, "bf16")
    x = np.eye(k, dtype=np.float32).astype(BF16)
    want = O.dequant_affine(w, s, b, 64, 4).T
    for route, exact_bits in (("simt", True), ("gemv", True), ("gemm_tc", False)):
        xs = x[16:32] if route == "gemv" else x
        with _lib.force_route(route):
            y = qmm.quantized_matmul(to_torch(xs, DEV), to_torch(w, DEV), to_torch(s, DEV),
                                     to_torch(b, DEV), group_size=64, bits=4, out_dtype=torch.float32)
        got = to_numpy(y)
        if route == "gemv":
            # one product per output: s*(128+q) + (b-128s), each term exact, one f32 rounding each
            np.testing.assert_allclose(got, want[16:32], rtol=0, atol=2e-6)
        elif exact_bits:
            np.testing.assert_array_equal(got, want)
        else:   # the tensor-core route rounds the dequantized weight once to bf16
            np.testing.assert_array_equal(got, want.astype(BF16).astype(np.float32))


@pytest.mark.parametrize("route", ["simt", "gemm_tc", "gemv", None])
def test_batched_and_shared_weights(route):
    rng = np.random.default_rng(5)
    b_, m, k, n = 3, (20 if route != "gemv" else 5), 256, 72
    _, w, s, bi = affine_case(rng, n, k, 64, 4, "bf16", lead=(b_,))
    x = activations(rng, (b_, m, k))
    tx = to_torch(x, DEV)

    def call(*a, **kw):
        if route:
            with _lib.force_route(route):
                return qmm.quantized_matmul(*a, **kw)
        return qmm.quantized_matmul(*a, **kw)

    y = call(tx, to_torch(w, DEV), to_torch(s, DEV), to_torch(bi, DEV), group_size=64, bits=4)
    _gate(to_numpy(y).astype(np.float32), O.qmm_exact(x, w, s, bi, 64, 4), "bf16")
    y = call(tx, to_torch(w[0], DEV), to_torch(s[0], DEV), to_torch(bi[0], DEV), group_size=64, bits=4)
    _gate(to_numpy(y).astype(np.float32), O.qmm_exact(x, w[0], s[0], bi[0], 64, 4), "bf16")


@pytest.mark.parametrize("mode", ["affine", "mxfp4"])
def test_gather_qmm(mode):
    rng = np.random.default_rng(9)
    e, t, kk, k, n = 4, 6, 2, 128, 72
    if mode == "affine":
        _, w, s, b = affine_case(rng, n, k, 64, 4, "bf16", lead=(e,))
        gs = 64
    else:
        _, w, s = mxfp4_case(rng, n, k, lead=(e,))
        b, gs = None, 32
    x = activations(rng, (t, 1, k))
    eidx = rng.integers(0, e, size=t * kk).astype(np.int32)
    tidx = np.repeat(np.arange(t, dtype=np.int32), kk)          # src/metaljax/moe.py:1432-1433
    y = moe.gather_qmm(to_torch(x, DEV), to_torch(w, DEV), to_torch(s, DEV),
                       None if b is None else to_torch(b, DEV), torch.from_numpy(tidx).to(DEV),
                       torch.from_numpy(eidx).to(DEV), group_size=gs, bits=4, mode=mode)
    exact = O.gather_qmm_exact(x, w, s, b, tidx, eidx, gs, 4, mode)
    assert tuple(y.shape) == (t * kk, 1, n)
    _gate(to_numpy(y).astype(np.float32), exact, "bf16")
    with pytest.raises(RuntimeError):                            # 2-D operand is refused
        moe.gather_qmm(to_torch(x[:, 0], DEV), to_torch(w, DEV), to_torch(s, DEV), None,
                       torch.from_numpy(tidx).to(DEV), torch.from_numpy(eidx).to(DEV))


@pytest.mark.parametrize("route", ["simt", "gemm_tc", "gemv", None])
@pytest.mark.parametrize("sizes", [[5, 0, 300, 7], [0, 0, 0, 0], [64, 64, 64, 64], [1, 1, 1, 1], [513, 0, 0, 2]])
def test_ragged_dot(route, sizes):
    if route == "gemv":
        pytest.skip("ragged rows go to the tensor-core kernel")
    rng = np.random.default_rng(sum(sizes) + 1)
    g, k, n = len(sizes), 192, 136
    total = sum(sizes) + 3                                       # three rows belong to no group
    _, w, s, b = affine_case(rng, n, k, 64, 4, "bf16", lead=(g,))
    x = activations(rng, (total, k))
    gsz = np.array(sizes, np.int32)
    args = (to_torch(x, DEV), to_torch(w, DEV), to_torch(s, DEV), to_torch(b, DEV),
            torch.from_numpy(gsz).to(DEV))
    if route:
        with _lib.force_route(route):
            y = moe.ragged_dot(*args, group_size=64, bits=4)
    else:
        y = moe.ragged_dot(*args, group_size=64, bits=4)
    exact = O.ragged_qmm_exact(x, w, s, b, gsz, 64, 4)
    got = to_numpy(y).astype(np.float32)
    assert not got[sum(sizes):].any()
    if sum(sizes):
        _gate(got, exact, "bf16")
    cref = clib.qmm_ragged(x, w, s, b, gsz, total, k, n, 64, 4).view(BF16).astype(np.float32)
    np.testing.assert_allclose(got, cref, rtol=2e-2, atol=1e-2 * max(np.abs(exact).max(), 1e-6))


def test_moe_experts_matches_pair_space_reference():
    """Router -> sorted pairs -> three ragged dots -> weighted K-sum, against the dense
    statement `sum_e S[t,e] * expert_e(x)` evaluated exactly on the selected pairs."""
    rng = np.random.default_rng(31)
    t, d, f, e, kk = 48, 128, 192, 8, 2
    x = activations(rng, (t, d), "bf16", 0.5)
    logits = rng.standard_normal((t, e)).astype(np.float32)
    idx, wts = O.topk_router(logits, kk)
    packs = [affine_case(rng, f, d, 64, 4, "bf16", lead=(e,))[1:],
             affine_case(rng, f, d, 64, 4, "bf16", lead=(e,))[1:],
             affine_case(rng, d, f, 64, 4, "bf16", lead=(e,))[1:]]
    dev = [tuple(to_torch(a, DEV) for a in p) for p in packs]
    y = moe.moe_experts(to_torch(x, DEV), torch.from_numpy(idx).to(DEV), torch.from_numpy(wts).to(DEV),
                        dev[0], dev[1], dev[2])
    tidx = np.repeat(np.arange(t), kk)
    eidx = idx.reshape(-1)
    x3 = x[:, None, :]
    gate = O.gather_qmm_exact(x3, *packs[0], tidx, eidx)[:, 0]
    up = O.gather_qmm_exact(x3, *packs[1], tidx, eidx)[:, 0]
    act = (gate / (1 + np.exp(-gate))) * up
    down = O.gather_qmm_exact(act[:, None, :], *packs[2], np.arange(t * kk), eidx)[:, 0]
    want = O.moe_combine_exact(down, wts)
    assert O.rel_err(to_numpy(y).astype(np.float32), want) <= 2e-2      # two bf16 hand-offs inside


def test_emit_through_the_recognizer_interface():
    """`emit` with a hand-built Match/State, as the reference's interpreter would call it
    (src/metaljax/interpreter.py:900-908): transposed activations, batch shape, swapped."""
    rng = np.random.default_rng(41)
    n, k = 96, 128
    codes = rng.integers(-8, 8, size=(n, k)).astype(np.int32)
    heads = (rng.random((n, k // 64)).astype(np.float32) + 0.5).astype(BF16)
    smap = np.repeat(heads, 64, axis=1)
    m = qmm.Match()
    m.key, m.lhs = "dot", "x"
    pack = qmm.build_pack(m, torch.from_numpy(codes).to(DEV), to_torch(smap, DEV), None)
    x = activations(rng, (k, 2, 5))                       # [K, a, b] -> canonical [a*b, K]
    m.lperm, m.B, m.M, m.K, m.N = [1, 2, 0], 1, 10, k, n
    m.mshape, m.nshape, m.bshape, m.out_dtype = [2, 5], [n], [], torch.float32
    m.slot = 0

    class Interp:
        pass

    it = Interp()
    it._qmm = qmm.State()
    it._qmm.values = pack.arrays()
    (y,) = qmm.emit(it, m, {"x": to_torch(x, DEV)})
    wref = smap.astype(np.float32) * codes.astype(np.float32)
    want = np.einsum("kab,nk->abn", x.astype(np.float64), wref.astype(np.float64))
    assert tuple(y.shape) == (2, 5, n) and y.dtype == torch.float32
    assert O.rel_err(to_numpy(y), want) <= TOL16
    m.swapped = True
    (y,) = qmm.emit(it, m, {"x": to_torch(x, DEV)})
    assert tuple(y.shape) == (n, 2, 5)
    assert O.rel_err(to_numpy(y), np.moveaxis(want, -1, 0)) <= TOL16
    assert qmm.emit_reads(m) == ("x",) and qmm.emit_bytes(m) == 10 * k * 4


def test_device_side_validation():
    x = torch.zeros(4, 128, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 16, dtype=torch.int32, device=DEV).view(torch.uint32)
    s = torch.zeros(8, 2, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(_lib.QmmError) as e:
        qmm.quantized_matmul(x, w, s, s.cpu(), group_size=64, bits=4)
    assert e.value.status == 5                                    # biases on another device
    xs = torch.zeros(4, 136, dtype=torch.bfloat16, device=DEV)[:, 8:]
    v = _lib.Views()
    y = torch.zeros(4, 8, dtype=torch.bfloat16, device=DEV)
    rc = _lib.lib().qmm_quantized_matmul(v(xs), v(w), v(s), v(s), v(y), 1, 64, 4, 0, None)
    assert rc == 4                                                # strided view
    empty = qmm.quantized_matmul(x[:0], w, s, s, group_size=64, bits=4)
    assert tuple(empty.shape) == (0, 8)


@pytest.mark.parametrize("m", list(range(1, 17)))
@pytest.mark.parametrize("kind", ["aff4g64", "aff4g32", "aff8g128", "mx4"])
def test_decode_kernel_every_m(m, kind):
    """The decode kernel for every M it accepts, N not a multiple of its 16-row tile, K that
    does not divide evenly among its eight warps, against the oracle and the SIMT route."""
    rng = np.random.default_rng(m)
    n, k = 83, 2880 if kind == "mx4" else 1152
    x = activations(rng, (m, k))
    if kind == "mx4":
        _, w, s = mxfp4_case(rng, n, k)
        b, gs, bits, mode = None, 32, 4, "mxfp4"
    else:
        bits = 8 if kind.startswith("aff8") else 4
        gs = int(kind.split("g")[1])
        _, w, s, b = affine_case(rng, n, k, gs, bits, "bf16")
        mode = "affine"
    args = (to_torch(x, DEV), to_torch(w, DEV), to_torch(s, DEV), None if b is None else to_torch(b, DEV))
    with _lib.force_route("gemv"):
        y = qmm.quantized_matmul(*args, group_size=gs, bits=bits, mode=mode, out_dtype=torch.float32)
    with _lib.force_route("simt"):
        ys = qmm.quantized_matmul(*args, group_size=gs, bits=bits, mode=mode, out_dtype=torch.float32)
    exact = O.qmm_exact(x, w, s, b, gs, bits, mode)
    assert O.rel_err(to_numpy(y), exact) <= 2e-5
    assert O.rel_err(to_numpy(y), to_numpy(ys).astype(np.float64)) <= 2e-5


def test_decode_kernel_long_k_and_wide_batch():
    """K longer than one staged pass (two passes at M <= 8, seven at M > 8) and a gather over
    many pairs."""
    rng = np.random.default_rng(77)
    n, k = 48, 14336
    _, w, s, b = affine_case(rng, n, k, 64, 4, "bf16")
    for m in (3, 12):
        x = activations(rng, (m, k))
        with _lib.force_route("gemv"):
            y = qmm.quantized_matmul(to_torch(x, DEV), to_torch(w, DEV), to_torch(s, DEV),
                                     to_torch(b, DEV), group_size=64, bits=4, out_dtype=torch.float32)
        assert O.rel_err(to_numpy(y), O.qmm_exact(x, w, s, b, 64, 4)) <= 2e-5


@pytest.mark.parametrize("m,k,n,gs,bits,mode", [(8, 4096, 1000, 64, 4, "affine"), (7, 4096, 272, 64, 4, "affine"),
                                                (8, 4096, 48, 128, 8, "affine"), (8, 4096, 80, 32, 4, "mxfp4"),
                                                (4, 8192, 64, 64, 4, "affine"), (8, 3584, 160, 32, 4, "affine"),
                                                (8, 14336, 336, 64, 4, "affine")])        # restaged passes with one box
def test_decode_kernel_with_a_single_box_ring(m, k, n, gs, bits, mode):
    """Rows and K at which the activations only stay resident (two CTAs per SM) with ONE box per
    warp in flight: the ring's slot and parity arithmetic at depth one, several tiles per CTA."""
    rng = np.random.default_rng(m * 31 + n)
    x = activations(rng, (m, k))
    if mode == "mxfp4":
        codes = rng.integers(0, 16, size=(n, k), dtype=np.uint8)
        w = O.pack_codes(codes, 4)
        s = rng.integers(119, 128, size=(n, k // 32), dtype=np.uint8)
        b = None
    else:
        _, w, s, b = affine_case(rng, n, k, gs, bits, "bf16")
    with _lib.force_route("gemv"):
        y = qmm.quantized_matmul(to_torch(x, DEV), to_torch(w, DEV), to_torch(s, DEV), None if b is None else to_torch(b, DEV),
                                 group_size=gs, bits=bits, mode=mode, out_dtype=torch.float32)
    assert O.rel_err(to_numpy(y), O.qmm_exact(x, w, s, b, gs, bits, mode)) <= (2e-5 if mode == "affine" and bits == 4 else 2e-3)
    assert _lib.poll_status() == 0


# ---- benchmark configurations at full size ---------------------------------------------------


def test_config1_decode_gemv_full_size():
    """int4 g64, M=1, K=N=4096: the whole output against the oracle."""
    rng = np.random.default_rng(0)
    _, w, s, b = affine_case(rng, 4096, 4096, 64, 4, "bf16")
    x = activations(rng, (1, 4096))
    y = qmm.quantized_matmul(to_torch(x, DEV), to_torch(w, DEV), to_torch(s, DEV), to_torch(b, DEV),
                             group_size=64, bits=4)
    exact = clib.qmm(x, w, s, b, 1, 4096, 4096, 64, 4, out_f32=True).astype(np.float64)
    lit = O.qmm_literal(x, w, s, b, 64, 4)
    _gate(to_numpy(y).astype(np.float32), exact, "bf16", lit)


@pytest.mark.parametrize("bits,gs,n,k", [(4, 64, 14336, 4096), (4, 64, 4096, 14336), (8, 128, 14336, 4096),
                                         (8, 128, 4096, 14336)])
def test_config2_prefill_full_size_sampled_rows_and_linearity(bits, gs, n, k):
    """M=2048 at Llama-3-8B MLP shapes (up/gate and down, 4- and 8-bit): token rows sampled from
    every 256-row token tile (first, last and interior rows of each: 72 rows) against the
    oracle, agreement of the tensor-core and SIMT routes on a row block, and linearity
    y(2x) == 2 y(x) bit for bit (a power-of-two scaling commutes with every rounding)."""
    rng = np.random.default_rng(2)
    m = 2048
    w = rng.integers(0, 1 << 32, size=(n, k * bits // 32), dtype=np.uint64).astype(np.uint32)   # uniform codes
    s = rng.uniform(0.002, 0.02, size=(n, k // gs)).astype(BF16)
    b = (-float(1 << (bits - 1)) * s.astype(np.float32)).astype(BF16)
    x = activations(rng, (m, k))
    tx, tw, ts, tb = (to_torch(a, DEV) for a in (x, w, s, b))
    y = qmm.quantized_matmul(tx, tw, ts, tb, group_size=gs, bits=bits)
    rows = np.unique(np.concatenate([t0 + np.array([0, 1, 31, 32, 100, 127, 128, 200, 255]) for t0 in range(0, m, 256)]))
    assert len(rows) >= 64
    exact = clib.qmm(x[rows], w, s, b, len(rows), k, n, gs, bits, out_f32=True).astype(np.float64)
    _gate(to_numpy(y[torch.from_numpy(rows).to(DEV)]).astype(np.float32), exact, "bf16")
    with _lib.force_route("simt"):
        ys = qmm.quantized_matmul(tx[:64], tw, ts, tb, group_size=gs, bits=bits)
    scale = float(np.abs(exact).max())
    assert float((ys.float() - y[:64].float()).abs().max()) <= 2e-2 * scale
    y2 = qmm.quantized_matmul(tx * 2, tw, ts, tb, group_size=gs, bits=bits)
    assert torch.equal(y2, y * 2)


@pytest.mark.parametrize("m", [1, 512, 4096])
def test_config3_mxfp4_full_size(m):
    rng = np.random.default_rng(3)
    n, k = 5760, 2880
    _, w, sb = mxfp4_case(rng, n, k)
    x = activations(rng, (m, k))
    y = qmm.quantized_matmul(to_torch(x, DEV), to_torch(w, DEV), to_torch(sb, DEV), None,
                             group_size=32, bits=4, mode="mxfp4")
    rows = np.unique(np.array([0, m // 2, m - 1]))
    exact = clib.qmm(x[rows], w, sb, None, len(rows), k, n, 32, 4, "mxfp4", out_f32=True).astype(np.float64)
    _gate(to_numpy(y[torch.from_numpy(rows).to(DEV)]).astype(np.float32), exact, "bf16")


# ---- config 5 at full size: the grouped ragged kernel and the expert block ------------------


def _boundary_rows(offsets, total):
    """First and last row of every expert, and the rows either side of every boundary."""
    rows = set()
    for lo, hi in zip(offsets[:-1], offsets[1:]):
        if hi > lo:
            rows.update({lo, min(lo + 1, hi - 1), (lo + hi) // 2, max(hi - 2, lo), hi - 1})
    return np.array(sorted(r for r in rows if 0 <= r < total))


def test_config5_moe_full_size_ragged_rows_and_expert_block():
    """Mixtral-8x7B expert shape: 4096 tokens, top-2 of 8, d 4096, ffn 14336, int4 group 64.
    The grouped ragged product at that size (about 1024 rows per expert, 256-row token tiles
    straddling expert boundaries) is checked on the rows at and around every expert boundary,
    the whole expert block on sampled tokens, both against the oracle."""
    rng = np.random.default_rng(5)
    t, e, kk, d, f, gs = 4096, 8, 2, 4096, 14336, 64
    x = activations(rng, (t, d))
    logits = rng.standard_normal((t, e)).astype(np.float32)
    idx, wts = O.topk_router(logits, kk)

    def pack(n, k):
        w = rng.integers(0, 1 << 32, size=(e, n, k // 8), dtype=np.uint64).astype(np.uint32)
        s = rng.uniform(0.002, 0.01, size=(e, n, k // gs)).astype(BF16)
        return w, s, (-8.0 * s.astype(np.float32)).astype(BF16)

    w1, w3, w2 = pack(f, d), pack(f, d), pack(d, f)
    dev = [tuple(to_torch(a, DEV) for a in p) for p in (w1, w3, w2)]
    tx, tidx = to_torch(x, DEV), torch.from_numpy(idx).to(DEV)
    # (1) the ragged product of the gate projection on the sorted pairs
    order, tok, gsz = moe.sort_pairs(tidx, e)
    xs = tx.index_select(0, tok)
    gate = moe.ragged_dot(xs, *dev[0], gsz, group_size=gs, bits=4)
    sizes = to_numpy(gsz)
    assert int(sizes.sum()) == t * kk
    offs = np.concatenate([[0], np.cumsum(sizes)])
    rows = _boundary_rows(offs, t * kk)
    xs_np = to_numpy(xs)
    expert_of = np.searchsorted(offs, rows, side="right") - 1
    want = np.stack([clib.qmm(xs_np[r:r + 1], w1[0][ex], w1[1][ex], w1[2][ex], 1, d, f, gs, 4, out_f32=True)[0]
                     for r, ex in zip(rows, expert_of)]).astype(np.float64)
    _gate(to_numpy(gate[torch.from_numpy(rows).to(DEV)]).astype(np.float32), want, "bf16")
    # (2) the expert block on sampled tokens
    y = moe.moe_experts(tx, tidx, torch.from_numpy(wts).to(DEV), dev[0], dev[1], dev[2], group_size=gs, bits=4)
    toks = np.array([0, 1, 255, 256, 1023, 2048, 3000, 4095])
    out = np.zeros((len(toks), d))
    for i, tk in enumerate(toks):
        for j in range(kk):
            ex = idx[tk, j]
            g_ = clib.qmm(x[tk:tk + 1], w1[0][ex], w1[1][ex], w1[2][ex], 1, d, f, gs, 4, out_f32=True)[0].astype(np.float64)
            u_ = clib.qmm(x[tk:tk + 1], w3[0][ex], w3[1][ex], w3[2][ex], 1, d, f, gs, 4, out_f32=True)[0].astype(np.float64)
            act = (g_ / (1 + np.exp(-g_)) * u_).astype(np.float32)[None, :]
            dn = clib.qmm(act, w2[0][ex], w2[1][ex], w2[2][ex], 1, f, d, gs, 4, out_f32=True)[0].astype(np.float64)
            out[i] += wts[tk, j] * dn
    got = to_numpy(y[torch.from_numpy(toks).to(DEV)]).astype(np.float32)
    assert O.rel_err(got, out) <= 2e-2                     # two bf16 hand-offs inside the block


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_moe_glue_kernels_match_the_two_step_forms(dtype):
    """`silu(gate) * up` and the routed K-sum as single passes against the eager forms they
    replace (bit for bit: the same roundings in the same order)."""
    from metaljax_b200 import _lib, moe
    g = torch.Generator(device=DEV).manual_seed(3)
    gate = (torch.randn((301, 192), generator=g, device=DEV) * 3).to(dtype)
    up = torch.randn((301, 192), generator=g, device=DEV).to(dtype)
    want = torch.nn.functional.silu(gate) * up
    got = moe.silu_mul(gate, up)
    # __expf against torch's expf: a unit in the last place of the storage type at most
    assert (got.float() - want.float()).abs().max() <= 2 ** -7 * want.float().abs().max()
    assert (got != want).float().mean() < 0.02
    t, k, e, d = 37, 3, 5, 136
    idx = torch.stack([torch.randperm(e, generator=g, device=DEV)[:k] for _ in range(t)])
    weights = torch.rand((t, k), generator=g, device=DEV)
    order, tok, sizes = moe.sort_pairs(idx, e)
    rows = torch.randn((t * k, d), generator=g, device=DEV).to(dtype)
    out = moe.routed_sum(rows, order, weights, t, k)
    # the same sum pair by pair in router order
    inv = torch.empty_like(order)
    inv[order] = torch.arange(t * k, device=DEV)
    acc = torch.zeros((t, d), device=DEV, dtype=torch.float32)
    for j in range(k):
        acc = acc + rows[inv.reshape(t, k)[:, j]].float() * weights[:, j:j + 1].float()
    assert torch.equal(out, acc.to(dtype))
    assert _lib.poll_status() == 0


@pytest.mark.parametrize("dtype,e,n,k,sizes,extra", [
    (torch.bfloat16, 5, 136, 200, [70, 0, 129, 1, 100], 4),        # an empty expert, a one-row expert, a K tail, rows past the groups
    (torch.float16, 3, 300, 64, [256, 257, 3], 0),                 # tiles that straddle expert boundaries
    (torch.bfloat16, 8, 512, 1024, [200] * 8, 0),
])
def test_ragged_mm_float_experts(dtype, e, n, k, sizes, extra):
    """The grouped product over FLOAT expert weights (the reference's `mx.gather_mm` once the
    pairs are sorted, src/metaljax/moe.py:1324-1336) against float64, with the reference's gate:
    within 1e-2 of the largest magnitude and no worse than 1.5x the literal bf16/f16 matmul."""
    g = torch.Generator(device=DEV).manual_seed(e * 1000 + n)
    rows = sum(sizes) + extra
    x = torch.randn((rows, k), generator=g, device=DEV).to(dtype)
    w = (torch.randn((e, n, k), generator=g, device=DEV) * 0.1).to(dtype)
    gs = torch.tensor(sizes, device=DEV, dtype=torch.int32)
    y = moe.ragged_mm(x, w, gs)
    assert y.shape == (rows, n) and y.dtype == dtype
    exact = torch.zeros((rows, n), device=DEV, dtype=torch.float64)
    literal = torch.zeros((rows, n), device=DEV, dtype=dtype)
    lo = 0
    for ex, sz in enumerate(sizes):
        exact[lo:lo + sz] = x[lo:lo + sz].double() @ w[ex].double().T
        literal[lo:lo + sz] = x[lo:lo + sz] @ w[ex].T
        lo += sz
    scale = exact.abs().max().item()
    err = (y.double() - exact).abs().max().item() / scale
    err_l = (literal.double() - exact).abs().max().item() / scale
    assert err <= 1e-2 and err <= 1.5 * err_l + 1e-6, (err, err_l)
    assert bool((y[sum(sizes):] == 0).all())                       # rows past the last group
    assert _lib.poll_status() == 0


def test_gather_mm_float_experts_in_router_order():
    g = torch.Generator(device=DEV).manual_seed(77)
    t, m, k, e, n, p = 9, 2, 128, 4, 72, 23
    x = torch.randn((t, m, k), generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn((e, n, k), generator=g, device=DEV) * 0.1).to(torch.bfloat16)
    lhs = torch.randint(0, t, (p,), generator=g, device=DEV)
    rhs = torch.randint(0, e, (p,), generator=g, device=DEV)
    y = moe.gather_mm(x, w, lhs, rhs)
    want = torch.einsum("pmk,pnk->pmn", x[lhs].double(), w[rhs].double())
    assert y.shape == (p, m, n)
    assert (y.double() - want).abs().max() <= 1e-2 * want.abs().max()
    with pytest.raises(RuntimeError):
        moe.gather_mm(x[0], w, lhs, rhs)                             # a 2-D operand has no batch to gather from
    with pytest.raises(_lib.QmmError):
        moe.ragged_mm(x.reshape(-1, k)[:, :60].contiguous(), w[:, :, :60].contiguous(), torch.tensor([18, 0, 0, 0], device=DEV, dtype=torch.int32))


@pytest.mark.parametrize("m,k,n,gs,xdt,tdt,ydt", [
    (64, 4096, 1024, 64, "bf16", "bf16", None),          # few tiles: every tile's K blocks split over CTAs
    (17, 512, 1000, 32, "bf16", "bf16", None),           # a feature tile that ends inside 32 columns
    (33, 4096, 6144, 64, "bf16", "bf16", "f32"),
    (64, 14336, 512, 128, "f16", "f16", None),           # long K
    (48, 2048, 40000, 64, "bf16", "f32", None),          # more tiles than SMs (persistent walk), wide tables
    (20, 64, 256, 64, "bf16", "bf16", None),             # a single K block
    (64, 1024, 28672, 64, "bf16", "bf16", None),         # 224 tiles on 148 SMs: the last wave's K blocks as one flat range
    (32, 4096, 28672 + 128 * 30, 64, "bf16", "bf16", "f32"),   # ... a fuller last wave, ranges across tile boundaries
])
def test_few_dozen_rows_take_the_tensor_core_kernel(m, k, n, gs, xdt, tdt, ydt):
    """17..64 rows (the decode step at a batch of a few dozen): the tensor-core kernel with narrow
    token tiles and the twelve-slot ring, the usual gate against the oracle."""
    rng = np.random.default_rng(m * 7 + n)
    assert qmm.route(m, k, n, gs, 4, "affine", TDT[xdt]) == "gemm_tc"
    _run_affine(rng, m, k, n, gs, 4, xdt=xdt, tdt=tdt, ydt=ydt, route="gemm_tc")
    assert _lib.poll_status() == 0
