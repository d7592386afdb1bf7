"""Multi-GPU forms of the fused quantized matmul: one process per GPU, torch.distributed.

The reference is single-device (`plugin/metal_pjrt.cc:478-482`; every collective is an
identity, `src/metaljax/ops/collectives.py:40-85`), so both shardings here are new. They are
the two ways this path partitions:

* `ColumnParallelLinear` -- a packed weight `[N, K*bits/32]` split on N. Packing is per output
  row and quantization groups run along K, so a shard is a plain row slice of `w`, `scales` and
  `biases`; every rank computes `y[:, N/g]` from the replicated activations and the slices are
  all-gathered on the last axis.
* `ExpertParallelMoE` -- the experts of a mixture-of-experts layer split over ranks. Every rank
  routes its own tokens, sends each (token, expert) pair's activation row to the rank that
  owns the expert (all-to-all), runs the grouped ragged product on what it received, and
  sends the results back (all-to-all) for the weighted K-sum
  (`src/metaljax/moe.py:1446-1453`).

The compute calls go through an `ops` object with `quantized_matmul` and `ragged_dot`
(default: this package's CUDA ops); the collectives are torch.distributed's (NCCL on GPUs).
"""

from __future__ import annotations

import torch
import torch.distributed as dist


class _CudaOps:
    """The package's own fused ops (CUDA only)."""

    @staticmethod
    def quantized_matmul(*a, **k):
        from . import qmm
        return qmm.quantized_matmul(*a, **k)

    @staticmethod
    def ragged_dot(*a, **k):
        from . import moe
        return moe.ragged_dot(*a, **k)

    @staticmethod
    def silu_mul(gate, up):
        from . import moe
        return moe.silu_mul(gate, up)

    @staticmethod
    def routed_sum(rows, order, weights, tokens, k):
        from . import moe
        return moe.routed_sum(rows, order, weights, tokens, k)


def shard_rows(n: int, world: int, rank: int, multiple: int = 16):
    """Rows `[lo, hi)` of an N-row weight owned by `rank`: contiguous, sized in multiples of
    `multiple` rows (so every shard keeps the kernels' 16-byte alignment), the last rank
    taking the remainder."""
    per = -(-n // world)
    per = -(-per // multiple) * multiple
    lo = min(n, rank * per)
    return lo, min(n, lo + per)


class ColumnParallelLinear:
    """`y = x . deq(w)^T` with `w` split on its output rows over the process group."""

    def __init__(self, w, scales, biases, group_size=64, bits=4, mode="affine", group=None,
                 ops=None, full=True):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.ops = ops or _CudaOps
        self.kw = dict(group_size=group_size, bits=bits, mode=mode)
        self.n = w.shape[-2] if full else None
        if full:
            lo, hi = shard_rows(self.n, self.world, self.rank)
            self.lo, self.hi = lo, hi
            self.w = w[lo:hi].contiguous()
            self.scales = scales[lo:hi].contiguous()
            self.biases = None if biases is None else biases[lo:hi].contiguous()
        else:  # already a local shard
            self.w, self.scales, self.biases = w, scales, biases
            self.lo = self.hi = None
        sizes = [shard_rows(self.n, self.world, r) for r in range(self.world)] if full else None
        self.sizes = None if sizes is None else [b - a for a, b in sizes]

    def local(self, x, out_dtype=None):
        """This rank's slice `y[:, lo:hi]`."""
        return self.ops.quantized_matmul(x, self.w, self.scales, self.biases, out_dtype=out_dtype,
                                         **self.kw)

    def __call__(self, x, out_dtype=None):
        y = self.local(x, out_dtype)
        if self.world == 1:
            return y
        m = y.shape[0]
        if len(set(self.sizes)) == 1:
            # equal shards: one all-gather into [world, M, N/world], then interleave on N
            buf = torch.empty((self.world * m, y.shape[1]), dtype=y.dtype, device=y.device)
            dist.all_gather_into_tensor(buf, y.contiguous(), group=self.group)
            return buf.view(self.world, m, -1).permute(1, 0, 2).reshape(m, self.n)
        # uneven shards: pad every slice to the widest, gather once, cut the padding out
        widest = max(self.sizes)
        padded = torch.zeros((m, widest), dtype=y.dtype, device=y.device)
        padded[:, : y.shape[1]] = y
        buf = torch.empty((self.world * m, widest), dtype=y.dtype, device=y.device)
        dist.all_gather_into_tensor(buf, padded, group=self.group)
        buf = buf.view(self.world, m, widest)
        return torch.cat([buf[r, :, :s] for r, s in enumerate(self.sizes)], dim=-1)


class ExpertParallelMoE:
    """SwiGLU mixture-of-experts block with the experts split over the process group.

    `w1, w3, w2` are `(w, scales, biases)` packs of ALL experts, `[E, ffn, d*bits/32]`,
    `[E, ffn, ...]`, `[E, d, ffn*bits/32]`; each rank keeps experts `[rank*E/g, (rank+1)*E/g)`.
    """

    def __init__(self, w1, w3, w2, group_size=64, bits=4, mode="affine", group=None, ops=None,
                 local_experts=False, capacity_pairs=None):
        """With `local_experts` the packs already hold only this rank's E/g experts. With
        `capacity_pairs` (the most (token, expert) pairs any rank brings to a call; the same number
        on every rank) rows travel through peer memory (`qmm_ep_dispatch` / `qmm_ep_combine`:
        stores over NVLink into symmetric buffers, sizes kept on the devices, nothing read back by
        the host) instead of through all-to-all collectives."""
        self.group = group
        self.capacity_pairs = capacity_pairs
        self._peer = None                     # the peer-memory exchange, set up at the first call
        self._peer_error = None
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.ops = ops or _CudaOps
        self.kw = dict(group_size=group_size, bits=bits, mode=mode)
        self.e = w1[0].shape[0] * (self.world if local_experts else 1)
        if self.e % self.world:
            raise ValueError(f"{self.e} experts do not split over {self.world} ranks")
        self.el = self.e // self.world
        lo = self.rank * self.el

        def take(pack):
            if local_experts:
                return tuple(pack)
            return tuple(None if a is None else a[lo:lo + self.el].contiguous() for a in pack)

        self.w1, self.w3, self.w2 = take(w1), take(w3), take(w2)

    def _peer_setup(self, x):
        """Symmetric buffers of the peer-memory exchange for rows like x's; on any failure every
        rank falls back to the collectives together."""
        import ctypes
        from . import _lib
        d, dev = x.shape[1], x.device
        row_bytes = d * x.element_size()
        ok = torch.ones((), device=dev, dtype=torch.int32)
        state = None
        try:
            if row_bytes % 16 or x.dtype not in (torch.bfloat16, torch.float16):
                raise ValueError("rows must be 16-bit and a multiple of 16 bytes")
            import torch.distributed._symmetric_memory as symm_mem
            cap_rows = self.world * self.capacity_pairs
            sizes = [self.world * self.e * 8, 2 * self.world * 4, cap_rows * row_bytes, self.capacity_pairs * row_bytes]
            offs, total = [], 0
            for sz in sizes:
                offs.append(total)
                total += -(-sz // 256) * 256
            buf = symm_mem.empty((total,), dtype=torch.uint8, device=dev)
            buf[: offs[2]].zero_()
            hdl = symm_mem.rendezvous(buf, self.group if self.group is not None else dist.group.WORLD)
            bases = [int(p) for p in hdl.buffer_ptrs]
            arrays = [(ctypes.c_void_p * self.world)(*[b + o for b in bases]) for o in offs]
            local = torch.zeros((64,), device=dev, dtype=torch.int32)            # [0] the call counter, [4..] CTA counters
            ex = _lib.EpExchange()
            ex.peer_counts, ex.peer_flags, ex.peer_recv, ex.peer_ret = (
                ctypes.cast(a, ctypes.POINTER(ctypes.c_void_p)) for a in arrays)
            ex.epoch, ex.scratch = local.data_ptr(), local.data_ptr() + 16
            ex.capacity_rows, ex.max_pairs = cap_rows, self.capacity_pairs
            ex.rank, ex.world, ex.experts = self.rank, self.world, self.e
            state = dict(ex=ex, buf=buf, hdl=hdl, arrays=arrays, local=local, row_bytes=row_bytes, d=d, dtype=x.dtype,
                         recv=buf[offs[2]: offs[2] + cap_rows * row_bytes].view(x.dtype).view(cap_rows, d),
                         ret=buf[offs[3]: offs[3] + self.capacity_pairs * row_bytes].view(x.dtype).view(self.capacity_pairs, d),
                         sizes=torch.zeros((self.el,), device=dev, dtype=torch.int32))
        except Exception as exc:                                  # noqa: BLE001 -- any setup failure
            self._peer_error = repr(exc)
            ok.zero_()
        torch.cuda.synchronize(dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        self._peer = state if int(ok.item()) == 1 else False

    def _call_peer(self, x, indices, weights):
        import ctypes
        from . import _lib, moe
        st = self._peer
        t, k = indices.shape
        pairs = t * k
        if pairs > self.capacity_pairs:
            raise ValueError(f"{pairs} pairs on this rank, the exchange was sized for {self.capacity_pairs}")
        eidx = indices.reshape(-1).to(torch.int64)
        order = torch.sort(eidx, stable=True).indices
        tok = (order // k).contiguous()
        counts = torch.bincount(eidx, minlength=self.e).to(torch.int32)
        x = x.contiguous()
        stream = _lib.stream_ptr(x)
        lib = _lib.lib()
        _lib.check(lib.qmm_ep_dispatch(ctypes.byref(st["ex"]), x.data_ptr(), t, st["row_bytes"], tok.data_ptr(),
                                       counts.data_ptr(), pairs, st["sizes"].data_ptr(), stream))
        rows, sizes = st["recv"], st["sizes"]
        act = moe.silu_mul(moe.ragged_dot(rows, *self.w1, sizes, **self.kw), moe.ragged_dot(rows, *self.w3, sizes, **self.kw))
        down = moe.ragged_dot(act, *self.w2, sizes, **self.kw)
        _lib.check(lib.qmm_ep_combine(ctypes.byref(st["ex"]), down.data_ptr(), st["row_bytes"], stream))
        return moe.routed_sum(st["ret"][:pairs], order, weights, t, k).to(x.dtype)

    def __call__(self, x, indices, weights, sum_dtype=torch.float32):
        """x `[T, d]` (this rank's tokens), router `indices[T, K]` (global expert ids) and
        `weights[T, K]` -> `[T, d]`."""
        if self.capacity_pairs and self.world > 1 and x.is_cuda and self.ops is _CudaOps and sum_dtype == torch.float32:
            if self._peer is None:
                self._peer_setup(x)
            if self._peer and x.shape[1] == self._peer["d"] and x.dtype == self._peer["dtype"] and x.shape[1] % 8 == 0:
                return self._call_peer(x, indices, weights)
        t, k = indices.shape
        eidx = indices.reshape(-1).to(torch.int64)
        order = torch.sort(eidx, stable=True).indices          # pairs sorted by global expert
        tok = order // k
        xs = x.index_select(0, tok)                            # rows in destination order
        counts = torch.bincount(eidx, minlength=self.e)        # pairs per global expert
        if self.world > 1:
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts, group=self.group)   # [world * el]
            send_rows = counts.reshape(self.world, self.el).sum(1).tolist()
            recv_mat = recv_counts.reshape(self.world, self.el)             # [src rank, local expert]
            recv_rows = recv_mat.sum(1).tolist()
            got = torch.empty((sum(recv_rows), x.shape[1]), dtype=x.dtype, device=x.device)
            dist.all_to_all_single(got, xs.contiguous(), recv_rows, send_rows, group=self.group)
            # received rows are ordered (source rank, local expert); the grouped product wants
            # (local expert, source rank)
            src_expert = torch.repeat_interleave(
                torch.arange(self.world * self.el, device=x.device) % self.el, recv_mat.reshape(-1))
            perm = torch.sort(src_expert, stable=True).indices
            rows = got.index_select(0, perm)
            group_sizes = recv_mat.sum(0).to(torch.int32)
        else:
            rows, group_sizes, perm = xs, counts.to(torch.int32), None
        gate = self.ops.ragged_dot(rows, *self.w1, group_sizes, **self.kw)
        up = self.ops.ragged_dot(rows, *self.w3, group_sizes, **self.kw)
        silu_mul = getattr(self.ops, "silu_mul", None)
        act = silu_mul(gate, up) if silu_mul is not None else torch.nn.functional.silu(gate) * up
        del gate, up
        down = self.ops.ragged_dot(act, *self.w2, group_sizes, **self.kw)
        if self.world > 1:
            back = torch.empty_like(down)
            back[perm] = down                                   # undo the local regrouping
            ret = torch.empty((xs.shape[0], down.shape[1]), dtype=down.dtype, device=x.device)
            dist.all_to_all_single(ret, back.contiguous(), send_rows, recv_rows, group=self.group)
        else:
            ret = down
        routed_sum = getattr(self.ops, "routed_sum", None)
        if routed_sum is not None and sum_dtype == torch.float32 and ret.dtype in (torch.bfloat16, torch.float16) \
                and ret.shape[1] % 8 == 0:
            return routed_sum(ret, order, weights, t, k).to(x.dtype)
        wsorted = weights.reshape(-1).index_select(0, order).to(sum_dtype)
        out = torch.zeros((t, ret.shape[1]), dtype=sum_dtype, device=x.device)
        out.index_add_(0, tok, ret.to(sum_dtype) * wsorted[:, None])
        return out.to(x.dtype)
