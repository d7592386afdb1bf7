"""A Llama-shaped decode step built on the fused quantized linears: the caller of the hot path
at decode time, used to measure 4-bit decode tokens/s on 1..8 GPUs.

One step takes `batch` token ids at context position `ctx - 1` and returns the next ids:
embedding -> per layer [RMSNorm, fused q/k/v linear, rotary + KV append, GQA attention over
the cache, output linear, residual + RMSNorm, fused gate/up linear, SwiGLU, down linear] ->
final norm -> lm_head -> argmax. Every linear is an int4 group-64 `quantized_matmul`; the
element-wise glue is this package's three small CUDA kernels (include/qmm_decode.h);
attention over the cache is the library's own kernel (`QMM_DECODE_ATTENTION=sdpa`: torch's
scaled_dot_product_attention). Nothing here runs on the CPU.

Weights are synthetic: either packed random codes with U(0.002, 0.02) scales and
bias = -8*scale (`weights="codes"`, what the benchmark uses), or N(0, 0.02) values quantized
per group of 64 to uint4 with scale = (max - min)/15, zero = round(-min/scale),
bias = -scale*zero (`weights="normal"`, `quantize_affine4` below).

With a process group of g ranks the step is sharded on the output rows of every weight
(packing is per output row, so a shard is a row slice): q/k/v by attention head (attention
and the KV cache stay local), the other linears on N, each followed by an all-gather of the
`[batch, N/g]` slices; lm_head shards the vocabulary and the argmax is reduced from per-rank
(max, index) pairs. The all-gathers are this package's one-shot peer-store kernel
(`qmm_decode_allgather`: every rank writes its slice straight into every rank's buffer over
NVLink and raises a flag; symmetric memory from torch.distributed) or, with `gather="nccl"`,
NCCL's; the final argmax reduction is NCCL's.
"""

from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import _lib, qmm


@dataclass(frozen=True)
class Shape:
    layers: int
    d_model: int
    heads: int
    kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    ctx: int
    eps: float = 1e-5
    theta: float = 500000.0
    group_size: int = 64

    def linear_params(self) -> int:
        per_layer = (self.heads + 2 * self.kv_heads) * self.head_dim * self.d_model \
            + self.d_model * self.heads * self.head_dim + 3 * self.ffn * self.d_model
        return self.layers * per_layer + self.vocab * self.d_model

    def weight_bytes(self) -> int:
        """Packed codes plus bf16 scale and bias tables of every linear: what one step streams."""
        p = self.linear_params()
        return p // 2 + (p // self.group_size) * 4


LLAMA3_8B = Shape(layers=32, d_model=4096, heads=32, kv_heads=8, head_dim=128, ffn=14336,
                  vocab=128256, ctx=2048)


def quantize_affine4(w: torch.Tensor, group_size: int = 64):
    """Float `[N, K]` -> (packed uint32 `[N, K/8]`, scales, biases) with codes in 0..15,
    scale = (max - min)/15 and zero = round(-min/scale) per group of `group_size` along K,
    biases = -scale*zero, tables in bf16 (so `scale*q + bias` reconstructs the weight)."""
    n, k = w.shape
    g = w.float().reshape(n, k // group_size, group_size)
    lo, hi = g.amin(-1), g.amax(-1)
    scale = ((hi - lo) / 15.0).clamp_min(1e-8).to(torch.bfloat16).float()
    zero = torch.round(-lo / scale).clamp(0, 15)
    codes = torch.round(g / scale[..., None] + zero[..., None]).clamp(0, 15).to(torch.uint8)
    biases = (-scale * zero).to(torch.bfloat16)
    return qmm.pack_codes(codes.reshape(n, k), 4), scale.to(torch.bfloat16), biases


def _ptr(t) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def add_rmsnorm(x, weight, out, residual=None, eps=1e-5, write_residual=True):
    """`h = x (+ residual)`; `residual <- h` in place when `write_residual`; `out = rmsnorm(h) * weight`."""
    rows, dim = x.shape
    res_out = residual if (residual is not None and write_residual) else None
    _lib.check(_lib.lib().qmm_decode_add_rmsnorm(_ptr(x), _ptr(residual), _ptr(weight), _ptr(out), _ptr(res_out),
                                                 rows, dim, float(eps), _lib.stream_ptr(x)))
    return out


def rope_kv(qkv, q_out, k_cache, v_cache, heads, kv_heads, head_dim, pos, theta):
    batch, ctx = qkv.shape[0], k_cache.shape[2]
    _lib.check(_lib.lib().qmm_decode_rope_kv(_ptr(qkv), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), batch, heads,
                                             kv_heads, head_dim, ctx, int(pos), float(theta), _lib.stream_ptr(qkv)))


def decode_attention(qkv, k_cache, v_cache, out, scratch, heads, kv_heads, head_dim, pos, theta, push=None, ex=None):
    """Rotary embedding, cache append and attention of the decode position in one kernel
    (`qmm_decode_attention`); `push` = (slot, site) sends the row to every rank's gather slot."""
    batch, ctx = qkv.shape[0], k_cache.shape[2]
    slot, site = push if push is not None else (-1, 0)
    _lib.check(_lib.lib().qmm_decode_attention(
        _ptr(qkv), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(scratch), scratch.numel() * scratch.element_size(), batch,
        heads, kv_heads, head_dim, ctx, int(pos), float(theta), slot, site, None if ex is None else ctypes.byref(ex),
        _lib.stream_ptr(qkv)))
    return out


def silu_mul(gate_up, out):
    rows, two_f = gate_up.shape
    _lib.check(_lib.lib().qmm_decode_silu_mul(_ptr(gate_up), _ptr(out), rows, two_f // 2, _lib.stream_ptr(gate_up)))
    return out


class _Linear:
    """One quantized weight (this rank's rows)."""

    def __init__(self, n, k, device, gen, group_size, weights, pack=None):
        if pack is not None:
            self.w, self.s, self.b = (t.contiguous() for t in pack)
        elif weights == "normal":
            self.w, self.s, self.b = quantize_affine4(torch.randn((n, k), generator=gen, device=device) * 0.02,
                                                      group_size)
        else:
            self.w = torch.randint(-(1 << 31), (1 << 31) - 1, (n, k // 8), generator=gen, device=device,
                                   dtype=torch.int64).to(torch.int32).view(torch.uint32)
            s = torch.rand((n, k // group_size), generator=gen, device=device) * 0.018 + 0.002
            self.s = s.to(torch.bfloat16)
            self.b = (-8.0 * self.s.float()).to(torch.bfloat16)
        self.gs = group_size
        self.n = n

    def __call__(self, x, out):
        return qmm.quantized_matmul(x, self.w, self.s, self.b, out=out, group_size=self.gs, bits=4)

    def dense(self):
        return qmm.dequantize(self.w, self.s, self.b, group_size=self.gs, bits=4)

    def problem(self, x, y):
        """`qmm_problem` of this weight against one bf16 row `x` (or None: the row comes from a
        gather slot) into `y` (or None: the result only goes to the other ranks)."""
        p = _lib.Problem()
        p.struct_size = ctypes.sizeof(_lib.Problem)
        p.mode, p.bits, p.group_size = 0, 4, self.gs
        p.x_dtype = p.table_dtype = p.y_dtype = _lib.ELEM[torch.bfloat16]
        p.batch, p.M, p.K, p.N = 1, 1, self.w.shape[1] * 8, self.n
        p.x = None if x is None else x.data_ptr()
        p.w, p.scales, p.biases = self.w.data_ptr(), self.s.data_ptr(), self.b.data_ptr()
        p.y = None if y is None else y.data_ptr()
        p.x_batch_stride, p.y_batch_stride = p.K, p.N
        return p


class DecodeStep:
    """Weights, KV cache and buffers of one rank, and the step itself."""

    def __init__(self, shape: Shape, batch: int, device, group=None, seed: int = 0, weights: str = "codes",
                 full_weights=None, gather: str = "peer", shard: str = "weights"):
        """`shard="weights"`: every linear is split on its output rows over the ranks and every rank
        steps all `batch` sequences. `shard="rows"`: the sequences are split instead -- rank r steps
        rows `[r * batch / N, (r + 1) * batch / N)` with the whole weights and its own sequences' KV
        cache, and nothing is exchanged; `self.batch` is then this rank's share."""
        self.shape, self.device, self.group = shape, torch.device(device), group
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.shard, self.global_batch = shard, batch
        self.rows_world, self.rows_rank = 1, 0
        if shard == "rows" and self.world > 1:
            if batch % self.world:
                raise ValueError(f"{batch} sequences do not split over {self.world} ranks")
            self.rows_world, self.rows_rank = self.world, self.rank
            batch //= self.world
            self.world, self.rank = 1, 0                     # as far as the weights are concerned
        elif shard not in ("weights", "rows"):
            raise ValueError("shard is 'weights' or 'rows'")
        self.batch = batch
        sh, g, r = shape, self.world, self.rank
        if sh.heads % g or sh.kv_heads % g or sh.ffn % (16 * g) or sh.d_model % (16 * g):
            raise ValueError(f"shape does not split over {g} ranks")
        self.h_l, self.kv_l = sh.heads // g, sh.kv_heads // g
        self.ffn_l, self.d_l = sh.ffn // g, sh.d_model // g
        v_per = -(-sh.vocab // g)
        v_per = -(-v_per // 16) * 16
        self.v_lo = min(sh.vocab, r * v_per)
        self.v_l = max(0, min(sh.vocab, self.v_lo + v_per) - self.v_lo)
        gen = torch.Generator(device=self.device).manual_seed(seed * 1000 + r)
        shared = torch.Generator(device=self.device).manual_seed(seed)     # replicated tensors
        dev, gs = self.device, sh.group_size
        hd = sh.head_dim

        def make(n, k, src):
            return _Linear(n, k, dev, gen, gs, weights, src)

        fw = full_weights                                                  # optional full packs to shard
        self.layers = []
        for li in range(sh.layers):
            src = {} if fw is None else self._slices(fw["layers"][li])
            self.layers.append({
                "qkv": make((self.h_l + 2 * self.kv_l) * hd, sh.d_model, src.get("qkv")),
                "o": make(self.d_l, sh.heads * hd, src.get("o")),
                "gate_up": make(2 * self.ffn_l, sh.d_model, src.get("gate_up")),
                "down": make(self.d_l, sh.ffn, src.get("down")),
                "ln1": (torch.ones(sh.d_model, device=dev) if fw is None else fw["layers"][li]["ln1"]).to(torch.bfloat16),
                "ln2": (torch.ones(sh.d_model, device=dev) if fw is None else fw["layers"][li]["ln2"]).to(torch.bfloat16),
            })
        self.final_norm = (torch.ones(sh.d_model, device=dev) if fw is None else fw["final_norm"]).to(torch.bfloat16)
        self.lm_head = make(self.v_l, sh.d_model,
                            None if fw is None else tuple(t[self.v_lo:self.v_lo + self.v_l] for t in fw["lm_head"]))
        if fw is None:
            self.embedding = (torch.randn((sh.vocab, sh.d_model), generator=shared, device=dev) * 0.5).to(torch.bfloat16)
        else:
            self.embedding = fw["embedding"].to(torch.bfloat16)
        # KV cache of this rank's heads, filled up to (not including) the decode position
        kv_shape = (sh.layers, batch, self.kv_l, sh.ctx, hd)
        rows = slice(self.rows_rank * batch, (self.rows_rank + 1) * batch)           # of a full cache's sequences
        if self.rows_world > 1:
            gen = torch.Generator(device=self.device).manual_seed(seed * 1000 + 500 + self.rows_rank)   # its own sequences
        self.k_cache = (torch.randn(kv_shape, generator=gen, device=dev, dtype=torch.float32) * 0.5).to(torch.bfloat16) \
            if fw is None else fw["k_cache"][:, rows, r * self.kv_l:(r + 1) * self.kv_l].contiguous()
        self.v_cache = (torch.randn(kv_shape, generator=gen, device=dev, dtype=torch.float32) * 0.5).to(torch.bfloat16) \
            if fw is None else fw["v_cache"][:, rows, r * self.kv_l:(r + 1) * self.kv_l].contiguous()
        bf = dict(device=dev, dtype=torch.bfloat16)
        b = batch
        self.res = torch.empty((b, sh.d_model), **bf)
        self.normed = torch.empty((b, sh.d_model), **bf)
        self.qkv = torch.empty((b, (self.h_l + 2 * self.kv_l) * hd), **bf)
        self.q = torch.empty((b, self.h_l, 1, hd), **bf)
        self.attn_full = torch.empty((b, sh.heads * hd), **bf)
        self.o_l = torch.empty((b, self.d_l), **bf)
        self.o_full = torch.empty((b, sh.d_model), **bf)
        self.gate_up = torch.empty((b, 2 * self.ffn_l), **bf)
        self.act_l = torch.empty((b, self.ffn_l), **bf)
        self.act_full = torch.empty((b, sh.ffn), **bf)
        self.down_l = torch.empty((b, self.d_l), **bf)
        self.down_full = torch.empty((b, sh.d_model), **bf)
        self.logits_l = torch.empty((b, max(self.v_l, 1)), **bf)
        widest = g * b * max(sh.ffn // g, sh.d_model // g, self.h_l * hd)            # elements of one gathered matrix
        self.gather_buf = torch.empty((widest,), **bf) if g > 1 else None
        # QMM_DECODE_GATHER overrides the mode for experiments: "peer", "nccl", or "skip" (no
        # exchange at all: timing of the compute alone, the results are meaningless)
        self.gather_mode = os.environ.get("QMM_DECODE_GATHER", gather) if g > 1 else "none"
        self._site = 0
        self._sites_per_step = 4 * sh.layers
        if self.gather_mode == "peer":
            # one symmetric allocation per rank: 24 flag words, then three gather slots; every
            # rank maps every other rank's allocation (CUDA IPC under torch's symmetric memory).
            # If any rank cannot set that up, every rank uses NCCL's all-gather instead.
            ok = torch.ones((), device=dev, dtype=torch.int32)
            try:
                import torch.distributed._symmetric_memory as symm_mem
                self._slot_bytes = -(-widest * 2 // 256) * 256
                self._symm = symm_mem.empty((256 + 3 * self._slot_bytes,), dtype=torch.uint8, device=dev)
                self._symm.zero_()
                self._symm_hdl = symm_mem.rendezvous(self._symm, group if group is not None else dist.group.WORLD)
                ptrs = [int(p_) for p_ in self._symm_hdl.buffer_ptrs]
                self._peer_flags = (ctypes.c_void_p * g)(*ptrs)
                self._peer_bufs = (ctypes.c_void_p * g)(*[p_ + 256 for p_ in ptrs])
                self._ag_state = torch.zeros((16,), device=dev, dtype=torch.int32)
                self._slots = [self._symm[256 + i * self._slot_bytes: 256 + (i + 1) * self._slot_bytes].view(torch.bfloat16)
                               for i in range(3)]
            except Exception as exc:                              # noqa: BLE001 -- any setup failure
                self._peer_error = repr(exc)
                ok.zero_()
            torch.cuda.synchronize(dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)   # also: every rank's flags are zero now
            if int(ok.item()) == 0:
                self.gather_mode = "nccl"
        # A single row takes the fused step: norms, SwiGLU and the exchange of every sharded linear
        # happen inside the linears' kernels (qmm_decode_linear). QMM_DECODE_FUSED=0 turns it off.
        self.fused = b == 1 and os.environ.get("QMM_DECODE_FUSED", "1") != "0" and self.gather_mode in ("none", "peer")
        self._ex = None
        if self.fused:
            self.res2 = torch.empty((2, b, sh.d_model), **bf)                 # the residual stream, ping-pong
            self.emb_row = torch.empty((b, sh.d_model), **bf)
            self.attn_l = torch.empty((b, self.h_l * hd), **bf)
            nbytes = _lib.lib().qmm_decode_attention_scratch_bytes(b, self.h_l, self.kv_l, hd, sh.ctx)
            self.attn_scratch = torch.zeros((nbytes,), device=dev, dtype=torch.uint8)
            if g > 1:
                ok = torch.ones((), device=dev, dtype=torch.int32)
                try:
                    import torch.distributed._symmetric_memory as symm_mem
                    # two gather slots of the widest row, [gate | up], as stamped units (4 bytes per value)
                    self._fslot_bytes = -(-(2 * sh.ffn * 4) // 256) * 256
                    self._fsymm = symm_mem.empty((2 * self._fslot_bytes,), dtype=torch.uint8, device=dev)
                    self._fsymm.zero_()
                    hdl = symm_mem.rendezvous(self._fsymm, group if group is not None else dist.group.WORLD)
                    self._fsymm_hdl = hdl
                    self._fpeer_bufs = (ctypes.c_void_p * g)(*[int(p_) for p_ in hdl.buffer_ptrs])
                    self._fstate = torch.zeros((8,), device=dev, dtype=torch.int32)       # [0] the step counter
                    ex = _lib.Exchange()
                    ex.peer_bufs = ctypes.cast(self._fpeer_bufs, ctypes.POINTER(ctypes.c_void_p))
                    ex.epoch = self._fstate.data_ptr()
                    ex.slot_bytes, ex.rank, ex.world = self._fslot_bytes, r, g
                    self._ex = ex
                except Exception as exc:                          # noqa: BLE001 -- any setup failure
                    self._peer_error = repr(exc)
                    ok.zero_()
                torch.cuda.synchronize(dev)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
                if int(ok.item()) == 0:
                    self.fused = False
        # Above one row too, rotary + append + attention are one kernel of the library (its streaming
        # tensor-core form once a slice of the context is a few hundred positions long);
        # QMM_DECODE_ATTENTION=sdpa runs the rotary kernel followed by torch's scaled_dot_product_attention.
        self.own_attention = not self.fused and os.environ.get("QMM_DECODE_ATTENTION", "own") != "sdpa"
        if self.own_attention:
            self.attn_l = torch.empty((b, self.h_l * hd), **bf)
            nbytes = _lib.lib().qmm_decode_attention_scratch_bytes(b, self.h_l, self.kv_l, hd, sh.ctx)
            self.attn_scratch = torch.zeros((nbytes,), device=dev, dtype=torch.uint8)
        if self.fused:
            # the fused gate/up kernel applies SwiGLU in its epilogue: its rows alternate gate_j, up_j
            idx = torch.stack([torch.arange(self.ffn_l, device=dev), torch.arange(self.ffn_l, device=dev) + self.ffn_l],
                              dim=1).reshape(-1)
            for layer in self.layers:
                lin = layer["gate_up"]
                lin.w = lin.w.view(torch.int32).index_select(0, idx).contiguous().view(torch.uint32)
                lin.s, lin.b = lin.s.index_select(0, idx).contiguous(), lin.b.index_select(0, idx).contiguous()
        self._argmax_scratch = torch.zeros((_lib.lib().qmm_decode_argmax_scratch_bytes(b),), device=dev, dtype=torch.uint8)
        self._argmax_val = torch.empty((b,), device=dev, dtype=torch.float32)
        self._argmax_idx = torch.empty((b,), device=dev, dtype=torch.int64)
        self.graph = None
        self.tokens = torch.zeros((b,), device=dev, dtype=torch.int64)
        self.next_tokens = torch.zeros((b,), device=dev, dtype=torch.int64)

    def _slices(self, layer):
        """This rank's rows of one layer's full packs `(w, scales, biases)`: q/k/v by head, the
        rest on N. A row slice of a pack is the pack of the row slice."""
        r, hd = self.rank, self.shape.head_dim

        def rows(name, lo, hi):
            return tuple(t[lo:hi] for t in layer[name])

        def cat(*packs):
            return tuple(torch.cat(ts) for ts in zip(*packs))

        return {"qkv": cat(rows("q", r * self.h_l * hd, (r + 1) * self.h_l * hd),
                           rows("k", r * self.kv_l * hd, (r + 1) * self.kv_l * hd),
                           rows("v", r * self.kv_l * hd, (r + 1) * self.kv_l * hd)),
                "o": rows("o", r * self.d_l, (r + 1) * self.d_l),
                "gate_up": cat(rows("gate", r * self.ffn_l, (r + 1) * self.ffn_l),
                               rows("up", r * self.ffn_l, (r + 1) * self.ffn_l)),
                "down": rows("down", r * self.d_l, (r + 1) * self.d_l)}

    # ---- collectives ----
    def _gather(self, local, full):
        """`[batch, n/g]` slices of every rank -> `full [batch, n]` (rank-major on the last axis)."""
        if self.world == 1:
            return local
        b, n_l = local.shape
        if self.gather_mode == "peer":
            # consecutive calls use different slots (a slot is rewritten by the peers as soon as
            # they have seen this rank's flag of the call after it)
            site, total = self._site, self._sites_per_step
            slot = 1 if (total % 3 == 1 and site == total - 1) else site % 3
            self._site = (site + 1) % total
            _lib.check(_lib.lib().qmm_decode_allgather(
                _ptr(local), self._peer_bufs, self._peer_flags, _ptr(self._ag_state), self.rank, self.world, slot,
                b, n_l * 2, self._slot_bytes, _lib.stream_ptr(local)))
            return self._slots[slot][: b * self.world * n_l].view(b, self.world * n_l)
        buf = self.gather_buf[: self.world * b * n_l].view(self.world * b, n_l)
        if self.gather_mode == "skip":
            return buf.view(b, self.world * n_l)
        dist.all_gather_into_tensor(buf, local, group=self.group)
        if b == 1:
            return buf.view(1, self.world * n_l)
        full.view(b, self.world, n_l).copy_(buf.view(self.world, b, n_l).permute(1, 0, 2))
        return full

    # ---- the step ----
    def _fused_linear(self, lin, x, y, prologue=0, wait=None, push=None, residual_in=None, residual_out=None,
                      norm_weight=None, swiglu_out=None, swiglu=False):
        """One `qmm_decode_linear`: `wait` / `push` are (slot, site) pairs or None; with `swiglu`
        the weight's rows alternate gate, up and silu(gate) * up is what leaves the kernel."""
        f = _lib.DecodeFusion()
        f.prologue = prologue
        f.epilogue = 1 if swiglu else 0
        f.epilogue_out = None if swiglu_out is None else swiglu_out.data_ptr()
        f.wait_slot, f.wait_site = wait if wait is not None else (-1, 0)
        f.push_slot, f.push_site = push if push is not None else (-1, 0)
        f.residual_in = None if residual_in is None else residual_in.data_ptr()
        f.residual_out = None if residual_out is None else residual_out.data_ptr()
        f.norm_weight = None if norm_weight is None else norm_weight.data_ptr()
        f.eps = float(self.shape.eps)
        p = lin.problem(x, y)
        _lib.check(_lib.lib().qmm_decode_linear(ctypes.byref(p), ctypes.byref(f),
                                                None if self._ex is None else ctypes.byref(self._ex),
                                                _lib.stream_ptr(self.res)))

    def _step_fused(self, tok):
        """The single-row step: five kernels per layer (qkv, attention, o, gate/up, down). Every sharded linear writes its slice into
        all ranks' gather slots from its own epilogue and the kernel that consumes the row waits for
        the flags itself; RMS norms and SwiGLU are computed by the consuming linear while it stages
        its activation row."""
        sh, hd, g = self.shape, self.shape.head_dim, self.world
        stream = _lib.stream_ptr(self.res)
        torch.index_select(self.embedding, 0, tok, out=self.emb_row)
        if self._ex is not None:
            _lib.check(_lib.lib().qmm_decode_step_begin(ctypes.byref(self._ex), stream))
        pos = sh.ctx - 1
        site = 0                      # exchanges of this step so far; exchange i uses slot i % 2
        down_wait = None              # (slot, site) of the previous layer's down projection
        x_in = self.emb_row
        for li, layer in enumerate(self.layers):
            # qkv <- rmsnorm(residual + previous down) ; the residual stream moves R0 -> R1
            self._fused_linear(layer["qkv"], None if down_wait else x_in, self.qkv, prologue=1, wait=down_wait,
                               residual_in=None if li == 0 else self.res2[0], residual_out=self.res2[1],
                               norm_weight=layer["ln1"])
            at_push = (site % 2, site) if g > 1 else None
            decode_attention(self.qkv, self.k_cache[li], self.v_cache[li], None if g > 1 else self.attn_l, self.attn_scratch,
                             self.h_l, self.kv_l, hd, pos, sh.theta, push=at_push, ex=self._ex)
            site += g > 1
            # o ; gate_up <- rmsnorm(residual + o) ; R1 -> R0 ; down <- silu(gate) * up
            o_push = (site % 2, site) if g > 1 else None
            self._fused_linear(layer["o"], None if g > 1 else self.attn_l, None if g > 1 else self.o_l, wait=at_push, push=o_push)
            site += g > 1
            gu_push = (site % 2, site) if g > 1 else None
            # (gate/up rows are interleaved in the fused layout: SwiGLU happens in that kernel's epilogue)
            self._fused_linear(layer["gate_up"], None if g > 1 else self.o_l, None, prologue=1,
                               wait=o_push, push=gu_push, residual_in=self.res2[1], residual_out=self.res2[0],
                               norm_weight=layer["ln2"], swiglu=True, swiglu_out=None if g > 1 else self.act_l)
            site += g > 1
            dn_push = (site % 2, site) if g > 1 else None
            self._fused_linear(layer["down"], None if g > 1 else self.act_l, None if g > 1 else self.down_l,
                               wait=gu_push, push=dn_push)
            site += g > 1
            down_wait, x_in = dn_push, self.down_l
        self._fused_linear(self.lm_head, None if down_wait else x_in, self.logits_l, prologue=1, wait=down_wait,
                           residual_in=self.res2[0], residual_out=self.res2[1], norm_weight=self.final_norm)

    def step(self, tokens=None):
        sh, b, hd = self.shape, self.batch, self.shape.head_dim
        tok = self.tokens if tokens is None else tokens
        self._site = 0
        if self.fused:
            self._step_fused(tok)
            return self._finish_step()
        torch.index_select(self.embedding, 0, tok, out=self.res)
        pos = sh.ctx - 1
        add_rmsnorm(self.res, self.layers[0]["ln1"], self.normed, eps=sh.eps)
        for li, layer in enumerate(self.layers):
            layer["qkv"](self.normed, self.qkv)
            if self.own_attention:
                attn = decode_attention(self.qkv, self.k_cache[li], self.v_cache[li], self.attn_l, self.attn_scratch,
                                        self.h_l, self.kv_l, hd, pos, sh.theta)
            else:
                rope_kv(self.qkv, self.q, self.k_cache[li], self.v_cache[li], self.h_l, self.kv_l, hd, pos, sh.theta)
                attn = F.scaled_dot_product_attention(self.q, self.k_cache[li], self.v_cache[li], enable_gqa=True)
            attn_full = self._gather(attn.reshape(b, self.h_l * hd), self.attn_full)
            layer["o"](attn_full, self.o_l)
            o_full = self._gather(self.o_l, self.o_full)
            add_rmsnorm(o_full, layer["ln2"], self.normed, residual=self.res, eps=sh.eps)
            layer["gate_up"](self.normed, self.gate_up)
            silu_mul(self.gate_up, self.act_l)
            act_full = self._gather(self.act_l, self.act_full)
            layer["down"](act_full, self.down_l)
            down_full = self._gather(self.down_l, self.down_full)
            last = li + 1 == sh.layers
            nxt = self.final_norm if last else self.layers[li + 1]["ln1"]
            add_rmsnorm(down_full, nxt, self.normed, residual=self.res, eps=sh.eps)
        self.lm_head(self.normed, self.logits_l)
        return self._finish_step()

    def _finish_step(self):
        b = self.batch
        val, idx = self._argmax_val, self._argmax_idx
        if self.v_l > 0:
            _lib.check(_lib.lib().qmm_decode_argmax(_ptr(self.logits_l), b, self.v_l, self.logits_l.shape[1], self.v_lo,
                                                    _ptr(val), _ptr(idx), _ptr(self._argmax_scratch),
                                                    self._argmax_scratch.numel(), _lib.stream_ptr(self.logits_l)))
        else:                                                     # a rank without vocabulary rows never wins
            val.fill_(float("-inf"))
            idx.zero_()
        if self.world > 1:
            pair = torch.stack([val, idx.float()], dim=-1).contiguous()            # [b, 2]
            allp = torch.empty((self.world,) + tuple(pair.shape), device=self.device, dtype=pair.dtype)
            dist.all_gather_into_tensor(allp.view(-1, 2), pair, group=self.group)
            best = torch.argmax(allp[..., 0], dim=0)                                 # [b]
            idx = allp[best, torch.arange(b, device=self.device), 1].to(torch.int64)
        self.next_tokens.copy_(idx)
        return self.next_tokens

    def logits(self):
        """Full `[batch, vocab]` logits of the last step (float32), gathered over ranks."""
        if self.world == 1:
            return self.logits_l[:, : self.v_l].float()
        v_per = -(-(-(-self.shape.vocab // self.world)) // 16) * 16            # as in __init__
        sizes = [max(0, min(self.shape.vocab, (r + 1) * v_per) - min(self.shape.vocab, r * v_per))
                 for r in range(self.world)]
        widest = max(sizes)
        padded = torch.zeros((self.batch, widest), device=self.device, dtype=torch.float32)
        padded[:, : self.v_l] = self.logits_l[:, : self.v_l].float()
        buf = torch.empty((self.world * self.batch, widest), device=self.device, dtype=torch.float32)
        dist.all_gather_into_tensor(buf, padded, group=self.group)
        buf = buf.view(self.world, self.batch, widest)
        return torch.cat([buf[r, :, :s] for r, s in enumerate(sizes)], dim=-1)

    def exchange_description(self) -> str:
        """How the slices of a sharded linear reach the other ranks (for benchmark records)."""
        if self.rows_world > 1:
            return "none: the sequences are split over the ranks, every rank holds the whole weights"
        if self.fused and self.world > 1:
            return ("stamped peer stores from the epilogue of each sharded kernel (attention, o, gate/up, down), read "
                    "as they arrive by the kernel that consumes the row")
        return {"none": "none (one rank)", "peer": "one-shot peer-store kernel over NVLink after each sharded linear",
                "nccl": "NCCL all-gather after each sharded linear",
                "skip": "left out (timing experiment)"}[self.gather_mode]

    def capture(self, warmup: int = 3):
        """Warm up and capture the step in a CUDA graph; `replay()` then runs it."""
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                self.step()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                self.step()
        torch.cuda.current_stream(self.device).wait_stream(stream)
        self.graph = graph
        return graph

    def replay(self):
        self.graph.replay()
        return self.next_tokens


def reference_logits(fw, shape: Shape, tokens, batch):
    """The same step in float32 torch on the dequantized packs (for tests): `[batch, vocab]`.
    The hand-offs between kernels are rounded to bf16 as the kernels do."""
    sh, hd = shape, shape.head_dim

    def dense(pack):
        return qmm.dequantize(*pack, group_size=sh.group_size, bits=4)

    def norm(x, w):
        return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + sh.eps) * w.to(torch.bfloat16).float()

    def rope(x, pos):                      # [b, heads, hd]
        half = hd // 2
        j = torch.arange(half, device=x.device, dtype=torch.float32)
        ang = pos * sh.theta ** (-2.0 * j / hd)
        c, s = torch.cos(ang), torch.sin(ang)
        lo, hi = x[..., :half], x[..., half:]
        return torch.cat([lo * c - hi * s, hi * c + lo * s], dim=-1)

    def bf(t):
        return t.to(torch.bfloat16).float()

    res = fw["embedding"].to(torch.bfloat16).float()[tokens]
    pos = sh.ctx - 1
    for li in range(sh.layers):
        L = fw["layers"][li]
        y = bf(norm(res, L["ln1"]))
        q = bf(y @ dense(L["q"]).T).view(batch, sh.heads, hd)
        k = bf(y @ dense(L["k"]).T).view(batch, sh.kv_heads, hd)
        v = bf(y @ dense(L["v"]).T).view(batch, sh.kv_heads, hd)
        q, k = bf(rope(q, pos)), bf(rope(k, pos))
        kc = fw["k_cache"][li].float().clone()
        vc = fw["v_cache"][li].float().clone()
        kc[:, :, pos], vc[:, :, pos] = k, v
        rep = sh.heads // sh.kv_heads
        kc, vc = kc.repeat_interleave(rep, dim=1), vc.repeat_interleave(rep, dim=1)
        att = torch.softmax(torch.einsum("bhd,bhtd->bht", q, kc) / hd ** 0.5, dim=-1)
        a = bf(torch.einsum("bht,bhtd->bhd", att, vc)).reshape(batch, sh.heads * hd)
        res = bf(res + bf(a @ dense(L["o"]).T))
        y = bf(norm(res, L["ln2"]))
        gate, up = bf(y @ dense(L["gate"]).T), bf(y @ dense(L["up"]).T)
        act = bf(gate / (1 + torch.exp(-gate)) * up)
        res = bf(res + bf(act @ dense(L["down"]).T))
    y = bf(norm(res, fw["final_norm"]))
    return y @ dense(fw["lm_head"]).T


def random_full_weights(shape: Shape, batch, device, seed=0):
    """Full (unsharded) packs, norms, embedding and caches for small tests; pass the result as
    `full_weights` to `DecodeStep` on every rank and to `reference_logits`."""
    g = torch.Generator(device=device).manual_seed(seed)
    sh, hd = shape, shape.head_dim

    def pack(n, k):
        return quantize_affine4(torch.randn((n, k), generator=g, device=device) * 0.05, sh.group_size)

    def ln():
        return 1 + 0.1 * torch.randn(sh.d_model, generator=g, device=device)

    layers = []
    for _ in range(sh.layers):
        layers.append({"q": pack(sh.heads * hd, sh.d_model), "k": pack(sh.kv_heads * hd, sh.d_model),
                       "v": pack(sh.kv_heads * hd, sh.d_model), "o": pack(sh.d_model, sh.heads * hd),
                       "gate": pack(sh.ffn, sh.d_model), "up": pack(sh.ffn, sh.d_model),
                       "down": pack(sh.d_model, sh.ffn), "ln1": ln(), "ln2": ln()})
    kv = (sh.layers, batch, sh.kv_heads, sh.ctx, hd)
    return {"layers": layers, "final_norm": ln(), "lm_head": pack(sh.vocab, sh.d_model),
            "embedding": torch.randn((sh.vocab, sh.d_model), generator=g, device=device).to(torch.bfloat16),
            "k_cache": (torch.randn(kv, generator=g, device=device) * 0.5).to(torch.bfloat16),
            "v_cache": (torch.randn(kv, generator=g, device=device) * 0.5).to(torch.bfloat16)}
