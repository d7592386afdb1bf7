"""The multi-GPU shardings on real GPUs (NCCL, one process per GPU): a column-parallel decode
product with its all-gather and the expert-parallel mixture-of-experts block with its token
all-to-all, each against the oracle, and the N-sharded Llama-shaped decode step against its
float reference. Skipped when fewer than two GPUs are visible."""

import os
import socket
import time

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    from helpers import activations, affine_case, to_numpy, to_torch
    from metaljax_b200 import _lib, parallel
    from oracle import qmm_oracle as O

    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    # a rank that fails leaves the others in a collective: a short timeout ends those with an error
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=45))
    stage = "start"
    try:
        rng = np.random.default_rng(0)                   # identical draws on every rank
        # column-parallel linear at decode and prefill sizes
        n, k = 1000, 512
        _, w, s, b = affine_case(rng, n, k, 64, 4, "bf16")
        lin = parallel.ColumnParallelLinear(to_torch(w, dev), to_torch(s, dev), to_torch(b, dev))
        for m in (1, 7, 96):
            x = activations(rng, (m, k))
            y = lin(to_torch(x, dev))
            err = O.rel_err(to_numpy(y).astype(np.float32), O.qmm_exact(x, w, s, b, 64, 4))
            assert tuple(y.shape) == (m, n) and err <= 1e-2, (m, err)
        stage = "column-parallel done"
        # expert-parallel MoE: every rank routes its own tokens
        e, kk, d, f, t = 4, 2, 128, 256, 40 + 8 * rank
        packs = [affine_case(rng, f, d, 64, 4, "bf16", lead=(e,))[1:],
                 affine_case(rng, f, d, 64, 4, "bf16", lead=(e,))[1:],
                 affine_case(rng, d, f, 64, 4, "bf16", lead=(e,))[1:]]
        moe = parallel.ExpertParallelMoE(*[tuple(to_torch(a, dev) for a in p) for p in packs])
        rr = np.random.default_rng(100 + rank)
        x = activations(rr, (t, d), "bf16", 0.5)
        idx, wts = O.topk_router(rr.standard_normal((t, e)).astype(np.float32), kk)
        y = moe(to_torch(x, dev), torch.from_numpy(idx).to(dev), torch.from_numpy(wts).to(dev))
        tidx, eidx = np.repeat(np.arange(t), kk), idx.reshape(-1)
        gate = O.gather_qmm_exact(x[:, None, :], *packs[0], tidx, eidx)[:, 0]
        up = O.gather_qmm_exact(x[:, None, :], *packs[1], tidx, eidx)[:, 0]
        act = (gate / (1 + np.exp(-gate))) * up
        down = O.gather_qmm_exact(act[:, None, :], *packs[2], np.arange(len(tidx)), eidx)[:, 0]
        want = O.moe_combine_exact(down, wts)
        err = O.rel_err(to_numpy(y).astype(np.float32), want)
        assert err <= 2e-2, err                           # two bf16 hand-offs inside the block
        stage = "expert-parallel done"
        # the same block with the rows exchanged through peer memory: the same bits, call after call
        peer = parallel.ExpertParallelMoE(*[tuple(to_torch(a, dev) for a in p) for p in packs], capacity_pairs=128)
        for call in range(3):
            y2 = peer(to_torch(x, dev), torch.from_numpy(idx).to(dev), torch.from_numpy(wts).to(dev))
            assert peer._peer, peer._peer_error
            assert torch.equal(y2, y), (call, (y2.float() - y.float()).abs().max().item())
        # every pair of every rank to the experts of rank 0: the other rank receives nothing
        idx0 = np.tile(np.array([[0, 1]], dtype=idx.dtype), (t, 1))
        args0 = (to_torch(x, dev), torch.from_numpy(idx0).to(dev), torch.from_numpy(wts).to(dev))
        assert torch.equal(peer(*args0), moe(*args0))
        torch.cuda.synchronize(dev)
        assert _lib.poll_status() == 0
        stage = "expert-parallel over peer memory done"
        # the Llama-shaped decode step sharded over the ranks: same logits as the float reference
        from metaljax_b200 import llama
        shape = llama.Shape(layers=2, d_model=256, heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=1000, ctx=48)
        for batch, gather in ((1, "peer"), (5, "peer"), (5, "nccl")):
            fw = llama.random_full_weights(shape, batch, dev, seed=3)         # identical on every rank
            step = llama.DecodeStep(shape, batch, dev, full_weights=fw, gather=gather)
            tokens = torch.arange(batch, device=dev) * 11 % shape.vocab
            step.tokens.copy_(tokens)
            nxt = step.step().clone()
            got = step.logits()
            want = llama.reference_logits(fw, shape, tokens, batch)
            err = (got - want).abs().max().item() / want.abs().max().item()
            assert err <= 3e-2, ("decode step", batch, err)
            top2 = want.topk(2, dim=-1).values
            clear = (top2[:, 0] - top2[:, 1]) > 2 * 3e-2 * want.abs().max()
            assert torch.equal(nxt[clear], want.argmax(-1)[clear])
            for _ in range(3):                                                # slots and flags cycle correctly
                assert torch.equal(step.step(), nxt)
            stage = f"decode step batch {batch} ({gather}) done"
        # the same step with the sequences split over the ranks instead of the weights
        batch = 6
        fw = llama.random_full_weights(shape, batch, dev, seed=4)
        step = llama.DecodeStep(shape, batch, dev, full_weights=fw, shard="rows")
        assert step.batch == batch // world and step.world == 1
        tokens = torch.arange(batch, device=dev) * 7 % shape.vocab
        mine = slice(rank * step.batch, (rank + 1) * step.batch)
        step.tokens.copy_(tokens[mine])
        step.step()
        want = llama.reference_logits(fw, shape, tokens, batch)[mine]
        err = (step.logits() - want).abs().max().item() / want.abs().max().item()
        assert err <= 3e-2, ("decode step, sequences split", err)
        stage = "decode step with the sequences split done"
        assert _lib.poll_status() == 0
        ret[rank] = "ok"
    except Exception as exc:                              # surfaced by the parent
        ret[rank] = f"after '{stage}': {exc!r}"
    finally:
        dist.destroy_process_group()


def test_two_gpu_ranks():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    deadline = time.time() + 180
    for p in procs:
        p.join(max(1.0, deadline - time.time()))
    stuck = [p for p in procs if p.is_alive()]
    for p in stuck:                                       # exactly the processes started above
        p.terminate()
    assert not stuck, f"ranks did not finish: {dict(ret)}"
    assert dict(ret) == {0: "ok", 1: "ok"}, dict(ret)
