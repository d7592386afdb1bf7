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
                 local_experts=False):
        """With `local_experts` the packs already hold only this rank's E/g experts."""
        self.group = group
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

    def __call__(self, x, indices, weights, sum_dtype=torch.float32):
        """x `[T, d]` (this rank's tokens), router `indices[T, K]` (global expert ids) and
        `weights[T, K]` -> `[T, d]`."""
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
