"""The single-row (M = 1) decode kernel -- integer tensor-core path -- against the oracle and
against the decode family's floating-point kernel, through the C ABI (needs a B200).

The kernel carries the activation row as 24-bit fixed point relative to its largest magnitude,
so besides the parity gates of test_gpu_qmm.py these cases look at what that could break:
rows with outliers, tiny rows, rows with zeros, infinities, every K-tail and table layout.
"""

import numpy as np
import pytest
import torch

from helpers import BF16, activations, affine_case, mxfp4_case, to_numpy, to_torch
from metaljax_b200 import _lib, qmm
from oracle import clib
from oracle import qmm_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TDT = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}


@pytest.fixture(autouse=True)
def _device_ok():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    yield
    assert _lib.poll_status() == 0


def _call(x, w, s, b, gs, bits, mode="affine", out=torch.float32, route="gemv"):
    args = (to_torch(x, DEV), to_torch(w, DEV), to_torch(s, DEV), None if b is None else to_torch(b, DEV))
    if route is None:
        return to_numpy(qmm.quantized_matmul(*args, group_size=gs, bits=bits, mode=mode, out_dtype=out))
    with _lib.force_route(route):
        return to_numpy(qmm.quantized_matmul(*args, group_size=gs, bits=bits, mode=mode, out_dtype=out))


CASES = [  # (kind, group_size, K, N): K tails of every kind, N not a multiple of any tile
    ("aff4", 64, 4096, 256), ("aff4", 64, 2880, 83), ("aff4", 32, 1152, 40), ("aff4", 128, 1536, 100),
    ("aff4", 64, 64, 8), ("aff4", 32, 32, 3), ("aff4", 64, 14336, 48), ("aff4", 128, 128, 17),
    ("aff8", 128, 4096, 120), ("aff8", 64, 1088, 83), ("aff8", 32, 352, 19), ("aff8", 128, 14336, 24),
    ("mx4", 32, 2880, 83), ("mx4", 32, 512, 64), ("mx4", 32, 32, 5), ("mx4", 32, 4128, 33),
]


@pytest.mark.parametrize("kind,gs,k,n", CASES)
@pytest.mark.parametrize("xdt", ["bf16", "f16"])
def test_single_row_against_oracle_and_float_kernel(kind, gs, k, n, xdt):
    rng = np.random.default_rng(k + n)
    x = activations(rng, (1, k), xdt)
    if kind == "mx4":
        _, w, s = mxfp4_case(rng, n, k)
        b, bits, mode = None, 4, "mxfp4"
    else:
        bits, mode = (8 if kind == "aff8" else 4), "affine"
        _, w, s, b = affine_case(rng, n, k, gs, bits, "bf16")
    y = _call(x, w, s, b, gs, bits, mode)
    exact = O.qmm_exact(x, w, s, b, gs, bits, mode)
    assert O.rel_err(y, exact) <= 2e-5                     # float32 out: only accumulation order differs
    yf = _call(x, w, s, b, gs, bits, mode, route="gemv_fmma")
    assert O.rel_err(y, yf.astype(np.float64)) <= 1e-4         # (that kernel rounds f16 activations' group sums)
    # and in the activation's type, with the reference's "no worse than the literal chain" rule
    y16 = _call(x, w, s, b, gs, bits, mode, out=TDT[xdt]).astype(np.float32)
    err, err_lit = O.rel_err(y16, exact), O.rel_err(O.qmm_literal(x, w, s, b, gs, bits, mode).astype(np.float32), exact)
    assert err <= 1e-2 and err <= 1.5 * err_lit + 1e-6, (err, err_lit)


@pytest.mark.parametrize("tdt", ["bf16", "f16"])
@pytest.mark.parametrize("bits,gs", [(4, 64), (8, 128)])
def test_table_types(tdt, bits, gs):
    rng = np.random.default_rng(5)
    n, k = 72, 768
    _, w, s, b = affine_case(rng, n, k, gs, bits, tdt)
    b = (b.astype(np.float32) + rng.normal(0, 0.01, b.shape).astype(np.float32)).astype(b.dtype)   # zero points off mid-code
    x = activations(rng, (1, k))
    assert O.rel_err(_call(x, w, s, b, gs, bits), O.qmm_exact(x, w, s, b, gs, bits)) <= 2e-5


@pytest.mark.parametrize("kind", ["aff4", "aff8", "mx4"])
def test_one_hot_rows_recover_the_dequantized_weight(kind):
    """x = e_j gives y = deq(w)[:, j]: any K permutation, nibble order or group slot mistake in
    the kernel shows as a wrong column."""
    rng = np.random.default_rng(21)
    n, k = 40, 512
    if kind == "mx4":
        codes, w, s = mxfp4_case(rng, n, k)
        b, gs, bits, mode = None, 32, 4, "mxfp4"
        want = O.dequant_mxfp4(w, s)
    else:
        bits, gs, mode = (8, 128, "affine") if kind == "aff8" else (4, 64, "affine")
        _, w, s, b = affine_case(rng, n, k, gs, bits, "bf16")
        want = O.dequant_affine(w, s, b, gs, bits)
    for j in list(range(0, 72)) + [127, 128, 255, 256, 300, 511]:
        x = np.zeros((1, k), np.float32)
        x[0, j] = 1.0
        y = _call(x.astype(BF16), w, s, b, gs, bits, mode)
        np.testing.assert_allclose(y[0], want[:, j], rtol=0, atol=1e-6 * max(1.0, np.abs(want[:, j]).max()), err_msg=f"column {j}")


def test_rows_with_outliers_tiny_rows_and_zeros():
    rng = np.random.default_rng(8)
    n, k, gs, bits = 64, 2048, 64, 4
    _, w, s, b = affine_case(rng, n, k, gs, bits, "bf16")
    base = rng.standard_normal((1, k)).astype(np.float32)
    rows = {
        "outlier 1e4": np.where(np.arange(k) == 777, 1.0e4, base),
        "outlier 2^20 among 2^-6": np.where(np.arange(k) == 3, 2.0 ** 20, base * 2.0 ** -6),
        "tiny 1e-30": base * 1e-30,
        "huge 1e30": base * 1e30,
        "sparse": np.where(rng.random((1, k)) < 0.9, 0.0, base),
        "zeros": np.zeros((1, k), np.float32),
    }
    for name, xr in rows.items():
        x = xr.astype(np.float32).astype(BF16)
        y = _call(x, w, s, b, gs, bits)
        exact = O.qmm_exact(x, w, s, b, gs, bits)
        if name == "zeros":
            assert not y.any()
            continue
        # elements more than 2^16 below the row's largest lose low bits, as they would against a
        # float32 accumulator holding the largest term: the bound is relative to the row's result
        assert O.rel_err(y, exact) <= 2e-5, name
        yf = _call(x, w, s, b, gs, bits, route="gemv_fmma")
        assert O.rel_err(y, exact) <= 4 * O.rel_err(yf, exact) + 1e-6, name


def test_non_finite_activations_poison_the_row():
    rng = np.random.default_rng(9)
    n, k = 24, 256
    _, w, s, b = affine_case(rng, n, k, 64, 4, "bf16")
    x = activations(rng, (1, k)).astype(np.float32)
    x[0, 5] = np.inf
    y = _call(x.astype(BF16), w, s, b, 64, 4)
    assert np.isnan(y).all()


def test_down_projection_and_vocabulary_shapes():
    """K = 14336 (the staged row is 43 KB) and N = 128256 (8016 tiles), whole outputs."""
    rng = np.random.default_rng(4)
    for n, k in ((4096, 14336), (128256, 4096)):
        w = rng.integers(0, 1 << 32, size=(n, k // 8), dtype=np.uint64).astype(np.uint32)
        s = rng.uniform(0.002, 0.02, size=(n, k // 64)).astype(BF16)
        b = (-8.0 * s.astype(np.float32)).astype(BF16)
        x = activations(rng, (1, k))
        y = _call(x, w, s, b, 64, 4, out=torch.bfloat16, route=None).astype(np.float32)
        exact = clib.qmm(x, w, s, b, 1, k, n, 64, 4, out_f32=True).astype(np.float64)
        assert O.rel_err(y, exact) <= 1e-2
        y32 = _call(x, w, s, b, 64, 4, route=None)
        assert O.rel_err(y32, exact) <= 2e-5


def test_linearity_and_repeatability():
    """y(2x) == 2 y(x) and y(x) == y(x) bit for bit: the fixed-point row scales with x, the
    summation order is fixed (no atomics)."""
    rng = np.random.default_rng(6)
    n, k = 4096, 4096
    _, w, s, b = affine_case(rng, n, k, 64, 4, "bf16")
    x = activations(rng, (1, k))
    tw, ts, tb = (to_torch(a, DEV) for a in (w, s, b))
    tx = to_torch(x, DEV)
    y = qmm.quantized_matmul(tx, tw, ts, tb, group_size=64, bits=4, out_dtype=torch.float32)
    assert qmm.route(1, k, n) == "gemv"
    for _ in range(3):
        assert torch.equal(qmm.quantized_matmul(tx, tw, ts, tb, group_size=64, bits=4, out_dtype=torch.float32), y)
    assert torch.equal(qmm.quantized_matmul(tx * 2, tw, ts, tb, group_size=64, bits=4, out_dtype=torch.float32), y * 2)


def test_back_to_back_launches_on_one_stream():
    """A chain of dependent single-row products (each reads the previous one's output), as a
    decode step issues them: programmatic stream serialization must not let a kernel read its
    activations early."""
    rng = np.random.default_rng(12)
    d = 1024
    packs = []
    for _ in range(6):
        _, w, s, b = affine_case(rng, d, d, 64, 4, "bf16", scale_lo=0.004, scale_hi=0.008)
        packs.append((w, s, b))
    x0 = activations(rng, (1, d))
    dev = [tuple(to_torch(a, DEV) for a in p) for p in packs]
    x = to_torch(x0, DEV)
    for p in dev:
        x = qmm.quantized_matmul(x, *p, group_size=64, bits=4)
    ref = x0
    for w, s, b in packs:
        ref = O.qmm_exact(ref, w, s, b, 64, 4).astype(np.float32).astype(BF16)
    got = to_numpy(x).astype(np.float32)
    assert O.rel_err(got, ref.astype(np.float64)) <= 3e-2       # six bf16 hand-offs
