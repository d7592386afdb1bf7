"""The multi-GPU host logic on CPU ranks (gloo, world_size 2): shard boundaries, the all-gather
assembly of a column-parallel product, and the expert-parallel dispatch / combine. The compute
calls are stood in for by the oracle (test infrastructure) so that only the sharding and the
collectives are under test; the GPU parity of the kernels themselves is in test_gpu_qmm.py."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import activations, affine_case, to_numpy, to_torch
from metaljax_b200 import parallel
from oracle import qmm_oracle as O


class OracleOps:
    """CPU stand-in for the CUDA ops: exact float64 products rounded to the output type."""

    @staticmethod
    def quantized_matmul(x, w, s, b, out_dtype=None, group_size=64, bits=4, mode="affine"):
        y = O.qmm_exact(to_numpy(x), to_numpy(w), to_numpy(s), None if b is None else to_numpy(b),
                        group_size, bits, mode)
        return torch.from_numpy(y.astype(np.float32)).to(out_dtype or x.dtype)

    @staticmethod
    def ragged_dot(x, w, s, b, group_sizes, group_size=64, bits=4, mode="affine", out_dtype=None):
        y = O.ragged_qmm_exact(to_numpy(x), to_numpy(w), to_numpy(s), None if b is None else to_numpy(b),
                               group_sizes.numpy(), group_size, bits, mode)
        return torch.from_numpy(y.astype(np.float32)).to(out_dtype or x.dtype)


def test_shard_rows_cover_and_align():
    for n, world in ((4096, 8), (14336, 8), (128256, 8), (100, 3), (16, 4)):
        spans = [parallel.shard_rows(n, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all(lo % 16 == 0 for lo, _ in spans)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, what, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(0)                   # identical draws on every rank
        if what == "linear":
            n, k, m = 200, 128, 3                        # 200 rows -> uneven shards (112 + 88)
            _, w, s, b = affine_case(rng, n, k, 64, 4, "f32")
            x = activations(rng, (m, k), "f32")
            lin = parallel.ColumnParallelLinear(to_torch(w), to_torch(s), to_torch(b), ops=OracleOps)
            y = lin(to_torch(x))
            want = O.qmm_exact(x, w, s, b, 64, 4)
            assert (lin.lo, lin.hi) == parallel.shard_rows(n, world, rank)
            np.testing.assert_allclose(y.numpy(), want, rtol=1e-5, atol=1e-5)
            n = 256                                      # equal shards take the single all-gather
            _, w, s, b = affine_case(rng, n, k, 64, 4, "f32")
            lin = parallel.ColumnParallelLinear(to_torch(w), to_torch(s), to_torch(b), ops=OracleOps)
            np.testing.assert_allclose(lin(to_torch(x)).numpy(), O.qmm_exact(x, w, s, b, 64, 4),
                                       rtol=1e-5, atol=1e-5)
        else:
            e, kk, d, f, t = 4, 2, 64, 128, 10
            packs = [affine_case(rng, f, d, 64, 4, "f32", lead=(e,))[1:],
                     affine_case(rng, f, d, 64, 4, "f32", lead=(e,))[1:],
                     affine_case(rng, d, f, 64, 4, "f32", lead=(e,))[1:]]
            tp = [tuple(to_torch(a) for a in p) for p in packs]
            moe = parallel.ExpertParallelMoE(*tp, ops=OracleOps)
            rng_r = np.random.default_rng(100 + rank)    # every rank has its own tokens
            x = activations(rng_r, (t + rank, d), "f32", 0.5)
            idx, wts = O.topk_router(rng_r.standard_normal((t + rank, e)).astype(np.float32), kk)
            y = moe(to_torch(x), torch.from_numpy(idx), torch.from_numpy(wts))
            tidx, eidx = np.repeat(np.arange(len(x)), kk), idx.reshape(-1)
            x3 = x[:, None, :]
            gate = O.gather_qmm_exact(x3, *packs[0], tidx, eidx)[:, 0]
            up = O.gather_qmm_exact(x3, *packs[1], tidx, eidx)[:, 0]
            act = ((gate / (1 + np.exp(-gate))) * up).astype(np.float32)
            down = O.gather_qmm_exact(act[:, None, :], *packs[2], np.arange(len(tidx)), eidx)[:, 0]
            want = O.moe_combine_exact(down, wts)
            np.testing.assert_allclose(y.numpy(), want, rtol=2e-4, atol=2e-4)
            # every pair of every rank to the experts of rank 0: rank 1 is sent nothing
            idx0 = np.tile(np.array([[0, 1]], dtype=idx.dtype), (len(x), 1))
            y0 = moe(to_torch(x), torch.from_numpy(idx0), torch.from_numpy(wts))
            eidx0 = idx0.reshape(-1)
            gate = O.gather_qmm_exact(x3, *packs[0], tidx, eidx0)[:, 0]
            up = O.gather_qmm_exact(x3, *packs[1], tidx, eidx0)[:, 0]
            act = ((gate / (1 + np.exp(-gate))) * up).astype(np.float32)
            down = O.gather_qmm_exact(act[:, None, :], *packs[2], np.arange(len(tidx)), eidx0)[:, 0]
            np.testing.assert_allclose(y0.numpy(), O.moe_combine_exact(down, wts), rtol=2e-4, atol=2e-4)
        ret[rank] = "ok"
    except Exception as exc:                             # surfaced by the parent
        ret[rank] = repr(exc)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("what", ["linear", "moe"])
def test_two_cpu_ranks(what):
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, what, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert not p.is_alive(), "rank did not finish"
    assert dict(ret) == {0: "ok", 1: "ok"}, dict(ret)


def _failing_worker(rank, world, port, ret):
    """Rank 1 fails on the host between two calls (it raises instead of joining the second one);
    rank 0 must come back from its collective with an error, not wait for ever."""
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    try:
        rng = np.random.default_rng(0)
        e, kk, d, f, t = 4, 2, 64, 128, 6
        packs = [affine_case(rng, f, d, 64, 4, "f32", lead=(e,))[1:], affine_case(rng, f, d, 64, 4, "f32", lead=(e,))[1:],
                 affine_case(rng, d, f, 64, 4, "f32", lead=(e,))[1:]]
        moe = parallel.ExpertParallelMoE(*[tuple(to_torch(a) for a in p) for p in packs], ops=OracleOps)
        x = activations(np.random.default_rng(rank), (t, d), "f32", 0.5)
        idx, wts = O.topk_router(np.random.default_rng(rank).standard_normal((t, e)).astype(np.float32), kk)
        args = (to_torch(x), torch.from_numpy(idx), torch.from_numpy(wts))
        moe(*args)                                        # a healthy first call on both ranks
        if rank == 1:
            ret[rank] = "left between calls"
            return                                        # (no collective in flight: the rank just never joins again)
        t0 = time.time()
        try:
            moe(*args)
            ret[rank] = "the second call returned without its peer"
        except Exception as exc:                          # noqa: BLE001 -- whatever the backend raises
            ret[rank] = f"error after {time.time() - t0:.0f} s: {type(exc).__name__}"
    finally:
        try:
            dist.destroy_process_group()
        except Exception:                                 # noqa: BLE001 -- the group is already broken on rank 0
            pass


def test_a_rank_that_leaves_ends_the_others_collective_with_an_error():
    """Failure detection without touching a GPU: the failure is made on the host (a rank that
    never joins), and the survivor's next collective ends with an error inside the process
    group's timeout instead of hanging."""
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    stuck = [p for p in procs if p.is_alive()]
    for p in stuck:                                       # exactly the processes started above
        p.terminate()
    assert not stuck, dict(ret)
    assert ret.get(1) == "left between calls"
    assert str(ret.get(0, "")).startswith("error after"), dict(ret)
