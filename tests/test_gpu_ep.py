"""The expert-parallel dispatch / combine kernels (include/qmm_ep.h) on ONE GPU: the layout
arithmetic with a single rank (its own stores satisfy its own waits, in stream order), every
buffer bound, and a wait that nothing satisfies -- a second "rank" whose buffers are local memory
nobody writes -- which runs out after about a millisecond, reports through the status word and
returns. The two-rank exchange itself is tests/test_gpu_parallel.py. Nothing here faults, traps or
hangs the device."""

import ctypes

import pytest
import torch

from metaljax_b200 import _lib, moe

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(autouse=True)
def _device_ok():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    yield
    _lib.check(_lib.lib().qmm_set_wait_limit(4_000_000_000))
    assert _lib.poll_status() == 0


class _Exchange:
    """`world` sets of buffers in this device's memory, seen from `rank`."""

    def __init__(self, world, rank, experts, capacity_rows, max_pairs, row_bytes):
        self.counts = [torch.zeros((world * experts, 2), device=DEV, dtype=torch.int32) for _ in range(world)]
        self.flags = [torch.zeros((2 * world,), device=DEV, dtype=torch.int32) for _ in range(world)]
        self.recv = [torch.zeros((capacity_rows, row_bytes), device=DEV, dtype=torch.uint8) for _ in range(world)]
        self.ret = [torch.zeros((max_pairs, row_bytes), device=DEV, dtype=torch.uint8) for _ in range(world)]
        self.local = torch.zeros((64,), device=DEV, dtype=torch.int32)
        self.arrays = [(ctypes.c_void_p * world)(*[t.data_ptr() for t in ts])
                       for ts in (self.counts, self.flags, self.recv, self.ret)]
        ex = _lib.EpExchange()
        ex.peer_counts, ex.peer_flags, ex.peer_recv, ex.peer_ret = (
            ctypes.cast(a, ctypes.POINTER(ctypes.c_void_p)) for a in self.arrays)
        ex.epoch, ex.scratch = self.local.data_ptr(), self.local.data_ptr() + 16
        ex.capacity_rows, ex.max_pairs = capacity_rows, max_pairs
        ex.rank, ex.world, ex.experts = rank, world, experts
        self.ex = ex


@pytest.mark.parametrize("tokens,k,experts,width", [(40, 2, 4, 128), (1, 1, 8, 64), (257, 4, 16, 256), (9, 2, 4, 8)])
def test_single_rank_dispatch_and_combine_layout(tokens, k, experts, width):
    g = torch.Generator(device=DEV).manual_seed(tokens)
    x = torch.randn((tokens, width), generator=g, device=DEV).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(experts, generator=g, device=DEV)[:k] for _ in range(tokens)])
    order, tok, sizes = moe.sort_pairs(idx, experts)
    pairs, row_bytes = tokens * k, width * 2
    xc = _Exchange(1, 0, experts, pairs, pairs, row_bytes)
    out_sizes = torch.full((experts,), -1, device=DEV, dtype=torch.int32)
    lib, stream = _lib.lib(), _lib.stream_ptr(x)
    for call in range(3):                                   # the call counter and the CTA counters cycle
        xs = x if call != 1 else (x.float() * 2).to(torch.bfloat16)
        _lib.check(lib.qmm_ep_dispatch(ctypes.byref(xc.ex), xs.data_ptr(), tokens, row_bytes, tok.contiguous().data_ptr(),
                                       sizes.data_ptr(), pairs, out_sizes.data_ptr(), stream))
        rows = xc.recv[0].view(torch.bfloat16).view(pairs, width)
        assert torch.equal(out_sizes, sizes)
        assert torch.equal(rows, xs.index_select(0, tok))   # (expert, source order): the grouped product's layout
        back = (rows.float() + 1).to(torch.bfloat16)
        _lib.check(lib.qmm_ep_combine(ctypes.byref(xc.ex), back.data_ptr(), row_bytes, stream))
        assert torch.equal(xc.ret[0].view(torch.bfloat16).view(pairs, width), back)
    assert int(xc.local[0]) == 3
    assert _lib.poll_status() == 0


def test_rows_that_do_not_fit_are_dropped_and_reported():
    tokens, k, experts, width = 16, 2, 4, 64
    g = torch.Generator(device=DEV).manual_seed(1)
    x = torch.randn((tokens, width), generator=g, device=DEV).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(experts, generator=g, device=DEV)[:k] for _ in range(tokens)])
    order, tok, sizes = moe.sort_pairs(idx, experts)
    pairs = tokens * k
    xc = _Exchange(1, 0, experts, pairs - 5, pairs, width * 2)          # a receive buffer five rows short
    out_sizes = torch.zeros((experts,), device=DEV, dtype=torch.int32)
    lib = _lib.lib()
    _lib.check(lib.qmm_ep_dispatch(ctypes.byref(xc.ex), x.data_ptr(), tokens, width * 2, tok.contiguous().data_ptr(),
                                   sizes.data_ptr(), pairs, out_sizes.data_ptr(), _lib.stream_ptr(x)))
    st = ctypes.c_int(0)
    assert lib.qmm_poll_status(ctypes.byref(st)) != 0 and st.value != 0
    rows = xc.recv[0].view(torch.bfloat16).view(pairs - 5, width)
    assert torch.equal(rows, x.index_select(0, tok)[: pairs - 5])       # what fits is where it belongs
    assert _lib.poll_status() == 0
    # the host-side checks: more pairs than the return buffer, a misaligned row
    assert lib.qmm_ep_dispatch(ctypes.byref(xc.ex), x.data_ptr(), tokens, width * 2, tok.contiguous().data_ptr(),
                               sizes.data_ptr(), pairs + 1, out_sizes.data_ptr(), _lib.stream_ptr(x)) != 0
    assert lib.qmm_ep_dispatch(ctypes.byref(xc.ex), x.data_ptr(), tokens, 24, tok.contiguous().data_ptr(),
                               sizes.data_ptr(), pairs, out_sizes.data_ptr(), _lib.stream_ptr(x)) != 0


def test_counts_that_never_arrive_time_out_and_the_library_recovers():
    """Rank 0 of two, the other rank's buffers being local memory nobody writes: the wait for its
    pairs-per-expert table runs out (code 110), the flag wait is skipped, the call returns."""
    tokens, k, experts, width = 8, 2, 4, 64
    g = torch.Generator(device=DEV).manual_seed(2)
    x = torch.randn((tokens, width), generator=g, device=DEV).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(experts, generator=g, device=DEV)[:k] for _ in range(tokens)])
    order, tok, sizes = moe.sort_pairs(idx, experts)
    pairs = tokens * k
    xc = _Exchange(2, 0, experts, 2 * pairs, pairs, width * 2)
    out_sizes = torch.full((experts // 2,), -1, device=DEV, dtype=torch.int32)
    lib = _lib.lib()
    _lib.check(lib.qmm_set_wait_limit(2_000_000))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    _lib.check(lib.qmm_ep_dispatch(ctypes.byref(xc.ex), x.data_ptr(), tokens, width * 2, tok.contiguous().data_ptr(),
                                   sizes.data_ptr(), pairs, out_sizes.data_ptr(), _lib.stream_ptr(x)))
    stop.record()
    torch.cuda.synchronize()
    assert start.elapsed_time(stop) < 500.0
    st = ctypes.c_int(0)
    assert lib.qmm_poll_status(ctypes.byref(st)) == 9 and st.value == 110        # QMM_ERR_TIMEOUT
    assert torch.equal(out_sizes, torch.zeros_like(out_sizes))                   # no sizes from half a table
    assert _lib.poll_status() == 0
    # the library is usable afterwards: a single-rank exchange on fresh buffers
    _lib.check(lib.qmm_set_wait_limit(4_000_000_000))
    one = _Exchange(1, 0, experts, pairs, pairs, width * 2)
    full = torch.zeros((experts,), device=DEV, dtype=torch.int32)
    _lib.check(lib.qmm_ep_dispatch(ctypes.byref(one.ex), x.data_ptr(), tokens, width * 2, tok.contiguous().data_ptr(),
                                   sizes.data_ptr(), pairs, full.data_ptr(), _lib.stream_ptr(x)))
    assert torch.equal(one.recv[0].view(torch.bfloat16).view(pairs, width), x.index_select(0, tok))


def test_a_rank_that_is_sent_no_rows():
    """The collective form of the block on a rank whose experts nobody chose: empty arrays (no
    address) through the grouped products and the glue kernels."""
    import numpy as np
    from helpers import affine_case, to_torch
    rng = np.random.default_rng(0)
    e, d, f = 2, 128, 256
    w1 = tuple(to_torch(a, DEV) for a in affine_case(rng, f, d, 64, 4, "bf16", lead=(e,))[1:])
    w2 = tuple(to_torch(a, DEV) for a in affine_case(rng, d, f, 64, 4, "bf16", lead=(e,))[1:])
    rows = torch.empty((0, d), device=DEV, dtype=torch.bfloat16)
    sizes = torch.zeros((e,), device=DEV, dtype=torch.int32)
    gate = moe.ragged_dot(rows, *w1, sizes)
    up = moe.ragged_dot(rows, *w1, sizes)
    act = moe.silu_mul(gate, up)
    down = moe.ragged_dot(act, *w2, sizes)
    assert tuple(gate.shape) == (0, f) and tuple(act.shape) == (0, f) and tuple(down.shape) == (0, d)
    out = moe.routed_sum(torch.zeros((8, d), device=DEV, dtype=torch.bfloat16), torch.arange(0, device=DEV),
                         torch.zeros((0, 2), device=DEV), 0, 2)
    assert tuple(out.shape) == (0, d)
    assert _lib.poll_status() == 0
