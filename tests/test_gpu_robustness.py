"""Failure reporting and edge handling of the CUDA path (needs a B200): a bounded wait that
runs out and returns, gather indices out of range, the glue kernels at their documented limits.
Nothing here faults, traps or hangs the device: every failure is made on the host side (a flag
nobody raises, an index the kernel clamps) and read back through the status word."""

import ctypes

import numpy as np
import pytest
import torch

from helpers import BF16, activations, affine_case, to_numpy, to_torch
from metaljax_b200 import _lib, llama, moe, qmm
from oracle import qmm_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(autouse=True)
def _device_ok():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    yield
    _lib.check(_lib.lib().qmm_set_wait_limit(4_000_000_000))
    assert _lib.poll_status() == 0


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def test_exchange_wait_runs_out_reports_and_recovers():
    """`qmm_decode_allgather` as rank 0 of a world of 2 whose second rank does not exist: its
    buffer and flag words are local memory that nobody signals. With the wait limit set to about
    a millisecond the kernel gives up, records 100 + (the silent rank) in the status word and
    returns; the next call skips its wait; a poll reports QMM_ERR_TIMEOUT and clears the word."""
    lib = _lib.lib()
    rows, slice_bytes = 4, 256
    slot_bytes = rows * slice_bytes * 2
    local = torch.arange(rows * slice_bytes // 2, device=DEV, dtype=torch.int16).view(torch.bfloat16)
    bufs = [torch.zeros(3 * slot_bytes, device=DEV, dtype=torch.uint8) for _ in range(2)]
    flags = [torch.zeros(24, device=DEV, dtype=torch.int32) for _ in range(2)]
    state = torch.zeros(16, device=DEV, dtype=torch.int32)
    peer_bufs = (ctypes.c_void_p * 2)(bufs[0].data_ptr(), bufs[1].data_ptr())
    peer_flags = (ctypes.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    _lib.check(lib.qmm_set_wait_limit(2_000_000))               # ~1 ms of SM clock
    stream = _lib.stream_ptr(local)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    _lib.check(lib.qmm_decode_allgather(_ptr(local), peer_bufs, peer_flags, _ptr(state), 0, 2, 0, rows, slice_bytes,
                                        slot_bytes, stream))
    stop.record()
    torch.cuda.synchronize()
    assert start.elapsed_time(stop) < 200.0                     # the kernel returned by itself
    # this rank's slice did land in both buffers, its own flag was raised
    want = local.view(torch.uint8).view(rows, slice_bytes)
    for r in range(2):
        got = bufs[r][:slot_bytes].view(rows, 2 * slice_bytes)[:, :slice_bytes]
        assert torch.equal(got, want)
        assert int(flags[r][0]) == 1
    assert int(flags[0][1]) == 0                                # rank 1 never arrived
    # the next call does not wait at all (status is already set)
    start.record()
    _lib.check(lib.qmm_decode_allgather(_ptr(local), peer_bufs, peer_flags, _ptr(state), 0, 2, 1, rows, slice_bytes,
                                        slot_bytes, stream))
    stop.record()
    torch.cuda.synchronize()
    assert start.elapsed_time(stop) < 50.0
    st = ctypes.c_int(0)
    rc = lib.qmm_poll_status(ctypes.byref(st))
    assert rc == 9 and st.value == 101, (rc, st.value)          # QMM_ERR_TIMEOUT, rank 1 silent
    assert b"wait ran out" in lib.qmm_last_error()
    assert _lib.poll_status() == 0                              # the poll cleared it
    # the library is usable afterwards
    rng = np.random.default_rng(0)
    _, w, s, b = affine_case(rng, 64, 128, 64, 4)
    x = activations(rng, (1, 128))
    y = qmm.quantized_matmul(to_torch(x, DEV), to_torch(w, DEV), to_torch(s, DEV), to_torch(b, DEV), group_size=64, bits=4)
    assert O.rel_err(to_numpy(y).astype(np.float32), O.qmm_exact(x, w, s, b, 64, 4)) <= 1e-2


@pytest.mark.parametrize("m", [1, 20])
def test_gather_with_indices_from_the_previous_kernel_and_out_of_range(m):
    """Indices written by a kernel launched directly before the call are honoured (the gather
    is not allowed to start early), and an index outside [0, E) / [0, T) is reported through the
    status word while that pair is computed with index 0 -- no out-of-bounds read."""
    rng = np.random.default_rng(3)
    e, t, k, n = 4, 6, 128, 72
    _, w, s, b = affine_case(rng, n, k, 64, 4, "bf16", lead=(e,))
    x = activations(rng, (t, m, k))
    dev = [to_torch(a, DEV) for a in (x, w, s, b)]
    p = 12
    seed = torch.arange(p, device=DEV, dtype=torch.int32)
    eidx = torch.zeros(p, device=DEV, dtype=torch.int32)
    tidx = torch.zeros(p, device=DEV, dtype=torch.int32)
    torch.remainder(seed * 7 + 1, e, out=eidx)                   # written by kernels just before the call
    torch.remainder(seed * 5 + 2, t, out=tidx)
    y = moe.gather_qmm(dev[0], dev[1], dev[2], dev[3], tidx, eidx, group_size=64, bits=4)
    exact = O.gather_qmm_exact(x, w, s, b, to_numpy(tidx), to_numpy(eidx), 64, 4)
    assert O.rel_err(to_numpy(y).astype(np.float32), exact) <= 1e-2
    assert _lib.poll_status() == 0
    bad_e, bad_t = eidx.clone(), tidx.clone()
    bad_e[3] = e + 5
    bad_t[7] = -1
    y = moe.gather_qmm(dev[0], dev[1], dev[2], dev[3], bad_t, bad_e, group_size=64, bits=4)
    st = ctypes.c_int(0)
    rc = _lib.lib().qmm_poll_status(ctypes.byref(st))
    assert rc == 3 and st.value == 200, (rc, st.value)           # QMM_ERR_SHAPE, QMM_DEVICE_BAD_INDEX
    fixed_e, fixed_t = to_numpy(eidx).copy(), to_numpy(tidx).copy()
    fixed_e[3], fixed_t[7] = 0, 0
    exact = O.gather_qmm_exact(x, w, s, b, fixed_t, fixed_e, 64, 4)
    assert O.rel_err(to_numpy(y).astype(np.float32), exact) <= 1e-2
    assert _lib.poll_status() == 0


def test_add_rmsnorm_at_its_largest_width():
    dim, rows = 24576, 3
    g = torch.Generator(device=DEV).manual_seed(1)
    x = torch.randn((rows, dim), generator=g, device=DEV).to(torch.bfloat16)
    res = torch.randn((rows, dim), generator=g, device=DEV).to(torch.bfloat16)
    wgt = (1 + 0.1 * torch.randn(dim, generator=g, device=DEV)).to(torch.bfloat16)
    out = torch.empty_like(x)
    res_in = res.clone()
    llama.add_rmsnorm(x, wgt, out, residual=res, eps=1e-5)
    h = (x.float() + res_in.float()).to(torch.bfloat16)
    assert torch.equal(res, h)
    hf = h.float()
    want = hf * torch.rsqrt((hf * hf).mean(-1, keepdim=True) + 1e-5) * wgt.float()
    assert float((out.float() - want).abs().max()) <= 2e-2 * float(want.abs().max())


def test_rotary_angles_at_long_positions():
    """pos ~ 1e5: the rotary frequency needs full float32 precision (its relative error is
    multiplied by the position). Against a float64 host reference."""
    heads, kv, hd, ctx, pos, theta = 2, 1, 128, 100_032, 100_001, 500000.0
    g = torch.Generator(device=DEV).manual_seed(2)
    qkv = torch.randn((1, (heads + 2 * kv) * hd), generator=g, device=DEV).to(torch.bfloat16)
    q = torch.empty((1, heads, 1, hd), device=DEV, dtype=torch.bfloat16)
    kc = torch.zeros((1, kv, ctx, hd), device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros((1, kv, ctx, hd), device=DEV, dtype=torch.bfloat16)
    llama.rope_kv(qkv, q, kc, vc, heads, kv, hd, pos, theta)
    v = qkv.double().cpu().numpy().reshape(heads + 2 * kv, hd)
    half = hd // 2
    ang = pos * theta ** (-2.0 * np.arange(half) / hd)
    c, s_ = np.cos(ang), np.sin(ang)

    def rot(a):
        lo, hi = a[:half], a[half:]
        return np.concatenate([lo * c - hi * s_, hi * c + lo * s_])

    for hh in range(heads):
        got = q[0, hh, 0].double().cpu().numpy()
        assert np.abs(got - rot(v[hh])).max() <= 3e-2 * np.abs(v[hh]).max()      # bf16 output + float32 angle
    got_k = kc[0, 0, pos].double().cpu().numpy()
    assert np.abs(got_k - rot(v[heads])).max() <= 3e-2 * np.abs(v[heads]).max()
    assert torch.equal(vc[0, 0, pos], qkv[0, (heads + kv) * hd:])


def test_two_devices_in_one_process():
    """Per-device state (status word, kernel attributes, SM count) is keyed by device: the same
    process drives cuda:0 and cuda:1 alternately."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    rng = np.random.default_rng(13)
    _, w, s, b = affine_case(rng, 256, 4096, 64, 4)
    exact = {}
    for m in (1, 8, 200):
        x = activations(rng, (m, 4096))
        for dev in ("cuda:1", "cuda:0", "cuda:1"):
            with torch.cuda.device(dev):
                y = qmm.quantized_matmul(to_torch(x, dev), to_torch(w, dev), to_torch(s, dev), to_torch(b, dev),
                                         group_size=64, bits=4)
                assert O.rel_err(to_numpy(y).astype(np.float32), O.qmm_exact(x, w, s, b, 64, 4)) <= 1e-2
                assert _lib.poll_status() == 0


def test_stamped_row_that_never_arrives():
    """A fused decode linear whose activation row is a gather slot nobody fills: the bounded wait
    of the consuming kernel runs out (limit about a millisecond), the status word reports 100,
    the call returns, and the library works afterwards."""
    g = torch.Generator(device=DEV).manual_seed(4)
    lin = llama._Linear(64, 256, DEV, g, 64, "normal")
    area = torch.zeros((2 * 256 * 4,), device=DEV, dtype=torch.uint8)
    state = torch.ones((8,), device=DEV, dtype=torch.int32)
    ex = _lib.Exchange()
    bufs = (ctypes.c_void_p * 1)(area.data_ptr())
    ex.peer_bufs = ctypes.cast(bufs, ctypes.POINTER(ctypes.c_void_p))
    ex.epoch, ex.slot_bytes, ex.rank, ex.world = state.data_ptr(), 256 * 4, 0, 1
    fz = _lib.DecodeFusion()
    fz.wait_slot, fz.wait_site, fz.push_slot = 0, 5, -1
    y = torch.zeros((1, 64), device=DEV, dtype=torch.bfloat16)
    p = lin.problem(None, y)
    lib = _lib.lib()
    _lib.check(lib.qmm_set_wait_limit(2_000_000))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    _lib.check(lib.qmm_decode_linear(ctypes.byref(p), ctypes.byref(fz), ctypes.byref(ex), _lib.stream_ptr(y)))
    stop.record()
    torch.cuda.synchronize()
    assert start.elapsed_time(stop) < 200.0
    st = ctypes.c_int(0)
    assert lib.qmm_poll_status(ctypes.byref(st)) == 9 and st.value == 100        # QMM_ERR_TIMEOUT
    assert _lib.poll_status() == 0
    x = torch.randn((1, 256), generator=g, device=DEV).to(torch.bfloat16)
    want = (x.float() @ lin.dense().float().T)
    lin(x, y)
    assert float((y.float() - want).abs().max()) <= 2e-2 * float(want.abs().max())
