"""Expert-gather side of the fused quantized matmul (mirror of `metaljax.moe`'s runtime).

The reference re-plans a dense mixture-of-experts block in pair space (`P = T*K` selected
(token, expert) pairs) and emits `mx.gather_qmm(x, w, scales, biases, lhs_idx, rhs_idx,
transpose=True, ...)` per expert dot (eterevsky/metaljax src/metaljax/moe.py:1283-1340),
then multiplies by the routing weights and sums over K (:1425-1461). This module provides
the same calls on the GPU: `gather_qmm` (router order), `ragged_dot` (pairs sorted by
expert, walked by per-expert row offsets), `sort_pairs` that turns the one into the other,
and `moe_experts`, the gathered SwiGLU expert block of a Mixtral-style layer.
"""

from __future__ import annotations

import torch

from . import _lib
from .qmm import _as_u32, _mode_id

STATS = {"recognized": 0, "gather_qmm": 0, "gather_mm": 0, "ragged_dot": 0}


def stats() -> dict:
    return dict(STATS)


def reset_stats():
    for k in STATS:
        STATS[k] = 0


def gather_qmm(x, w, scales, biases, lhs_idx, rhs_idx, transpose=True, group_size=64,
               bits=4, mode="affine", out_dtype=None):
    """`y[p] = x[lhs_idx[p]] @ deq(w[rhs_idx[p]]).T`: x `[T, M, K]`, w `[E, N, K*bits/32]`,
    indices `[P]` -> `[P, M, N]` (src/metaljax/moe.py:1320-1322)."""
    if x.dim() != 3:
        # the reference refuses the same thing: a 2-D operand would be read as [M, K]
        # with no batch and the indices broadcast against it (src/metaljax/moe.py:1303-1306)
        raise RuntimeError("moe: gather operand is not [batch, M, K]")
    p = lhs_idx.shape[0]
    y = torch.empty((p, x.shape[1], w.shape[-2]), dtype=out_dtype or x.dtype, device=x.device)
    v = _lib.Views()
    _lib.check(_lib.lib().qmm_gather_qmm(
        v(x.contiguous()), v(_as_u32(w)), v(scales), v(biases),
        v(lhs_idx.to(torch.int32).contiguous()), v(rhs_idx.to(torch.int32).contiguous()), v(y),
        1 if transpose else 0, int(group_size), int(bits), _mode_id(mode), _lib.stream_ptr(x)))
    STATS["gather_qmm"] += 1
    return y


def ragged_dot(x, w, scales, biases, group_sizes, group_size=64, bits=4, mode="affine",
               out_dtype=None):
    """`ragged_dot(lhs[m,k], rhs[g,k,n], group_sizes[g])` with a packed rhs `[G, N, words]`:
    rows `[off[g], off[g+1])` of `x` meet expert g; rows past `sum(group_sizes)` are zero."""
    y = torch.empty((x.shape[0], w.shape[-2]), dtype=out_dtype or x.dtype, device=x.device)
    v = _lib.Views()
    _lib.check(_lib.lib().qmm_ragged_dot(
        v(x.contiguous()), v(_as_u32(w)), v(scales), v(biases),
        v(group_sizes.to(torch.int32).contiguous()), v(y), int(group_size), int(bits),
        _mode_id(mode), _lib.stream_ptr(x)))
    STATS["ragged_dot"] += 1
    return y


def ragged_mm(x, w, group_sizes, out_dtype=None):
    """`ragged_dot` for float experts: `w [G, N, K]` holds values of x's type."""
    y = torch.empty((x.shape[0], w.shape[-2]), dtype=out_dtype or x.dtype, device=x.device)
    v = _lib.Views()
    _lib.check(_lib.lib().qmm_ragged_mm(v(x.contiguous()), v(w.contiguous()), v(group_sizes.to(torch.int32).contiguous()),
                                        v(y), _lib.stream_ptr(x)))
    STATS["ragged_dot"] += 1
    return y


def gather_mm(x, w, lhs_idx, rhs_idx, out_dtype=None):
    """`y[p] = x[lhs_idx[p]] @ w[rhs_idx[p]].T` for float experts: x `[T, M, K]`, w `[E, N, K]`
    (the reference hands MLX the lazily transposed `[E, K, N]` view of the same array,
    src/metaljax/moe.py:1324-1336), indices `[P]` -> `[P, M, N]`. The pairs are sorted by expert,
    the sorted rows go through one grouped product, the result is put back in pair order."""
    if x.dim() != 3:
        raise RuntimeError("moe: gather operand is not [batch, M, K]")
    e, n = w.shape[0], w.shape[1]
    p, m = lhs_idx.shape[0], x.shape[1]
    eidx = rhs_idx.reshape(-1).to(torch.int64)
    order = torch.sort(eidx, stable=True).indices
    sizes = torch.bincount(eidx, minlength=e).to(torch.int32) * m
    rows = x.index_select(0, lhs_idx.reshape(-1).to(torch.int64).index_select(0, order)).reshape(p * m, x.shape[2])
    ys = ragged_mm(rows, w, sizes, out_dtype=out_dtype)
    y = torch.empty((p, m, n), dtype=ys.dtype, device=x.device)
    y[order] = ys.reshape(p, m, n)
    STATS["gather_mm"] += 1
    return y


def sort_pairs(indices: torch.Tensor, num_experts: int):
    """Router output `indices[T, K]` -> the sorted pair layout `ragged_dot` walks.

    Returns `(order, token_of_row, group_sizes)`: `order[r]` is the pair (in router order,
    `p = t*K + k`, src/metaljax/moe.py:1432-1433) that lands on sorted row r -- a stable
    sort by expert, so rows of one expert keep token order -- `token_of_row[r] = order[r]//K`
    and `group_sizes[e]` the number of pairs routed to expert e."""
    t, k = indices.shape
    eidx = indices.reshape(-1).to(torch.int64)
    order = torch.sort(eidx, stable=True).indices
    group_sizes = torch.bincount(eidx, minlength=num_experts).to(torch.int32)
    return order, order // k, group_sizes


def moe_experts(x, indices, weights, w1, w3, w2, group_size=64, bits=4, mode="affine",
                sum_dtype=torch.float32):
    """The gathered expert block of a SwiGLU mixture-of-experts layer.

    x `[T, d]`; router `indices[T, K]`, `weights[T, K]`; packed expert weights
    `w1, w3 = (w, scales, biases)` each `[E, ffn, d*bits/32]`, `w2` `[E, d, ffn*bits/32]`.
    Pairs are sorted by expert and every projection is one `ragged_dot`; the routing
    weights are applied and the K terms summed in `sum_dtype` as the reference does
    after its gathered dots (src/metaljax/moe.py:1446-1453).
    """
    t, k = indices.shape
    e = w1[0].shape[0]
    order, tok, group_sizes = sort_pairs(indices, e)
    xs = x.index_select(0, tok)
    kw = dict(group_size=group_size, bits=bits, mode=mode)
    gate = ragged_dot(xs, *w1, group_sizes, **kw)
    up = ragged_dot(xs, *w3, group_sizes, **kw)
    act = silu_mul(gate, up)
    del gate, up
    down = ragged_dot(act, *w2, group_sizes, **kw)
    if sum_dtype == torch.float32 and down.dtype in _GLUE_DTYPES and down.shape[1] % 8 == 0:
        return routed_sum(down, order, weights, t, k)
    wsorted = weights.reshape(-1).index_select(0, order).to(sum_dtype)
    contrib = down.to(sum_dtype) * wsorted[:, None]
    out = torch.zeros((t, down.shape[1]), dtype=sum_dtype, device=x.device)
    out.index_add_(0, tok, contrib)
    return out.to(x.dtype)


def moe_experts_float(x, indices, weights, w1, w3, w2, sum_dtype=torch.float32):
    """`moe_experts` over FLOAT expert weights `w1, w3 [E, ffn, d]`, `w2 [E, d, ffn]` of x's
    type: the same pair sort, three grouped products (`ragged_mm`), SwiGLU and routed sum."""
    t, k = indices.shape
    order, tok, group_sizes = sort_pairs(indices, w1.shape[0])
    xs = x.index_select(0, tok)
    act = silu_mul(ragged_mm(xs, w1, group_sizes), ragged_mm(xs, w3, group_sizes))
    down = ragged_mm(act, w2, group_sizes)
    if sum_dtype == torch.float32 and down.dtype in _GLUE_DTYPES and down.shape[1] % 8 == 0:
        return routed_sum(down, order, weights, t, k)
    wsorted = weights.reshape(-1).index_select(0, order).to(sum_dtype)
    out = torch.zeros((t, down.shape[1]), dtype=sum_dtype, device=x.device)
    out.index_add_(0, tok, down.to(sum_dtype) * wsorted[:, None])
    return out.to(x.dtype)


_GLUE_DTYPES = (torch.bfloat16, torch.float16)


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """`silu(gate) * up` in one pass (the SwiGLU between the grouped products)."""
    if gate.dtype not in _GLUE_DTYPES or gate.numel() % 8 or gate.shape != up.shape or gate.numel() == 0:
        return torch.nn.functional.silu(gate) * up
    gate, up = gate.contiguous(), up.contiguous()
    out = torch.empty_like(gate)
    _lib.check(_lib.lib().qmm_moe_silu_mul(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel(),
                                           _lib.ELEM[gate.dtype], _lib.stream_ptr(gate)))
    return out


def routed_sum(rows: torch.Tensor, order: torch.Tensor, weights: torch.Tensor, tokens: int, k: int) -> torch.Tensor:
    """Every token's K expert outputs times their routing weights, added in float32 in k order
    (src/metaljax/moe.py:1446-1453): `rows` are the pair outputs sorted by expert, `order[r]` the
    pair (router order) on sorted row r."""
    rows = rows.contiguous()
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel(), device=order.device, dtype=order.dtype)
    w32 = weights.reshape(tokens, k).to(torch.float32).contiguous()
    out = torch.empty((tokens, rows.shape[1]), dtype=rows.dtype, device=rows.device)
    _lib.check(_lib.lib().qmm_moe_routed_sum(rows.data_ptr(), inv.data_ptr(), w32.data_ptr(), out.data_ptr(), tokens, k,
                                             rows.shape[1], rows.shape[0], _lib.ELEM[rows.dtype], _lib.stream_ptr(rows)))
    return out


# ---- recognizer-facing hooks (metaljax.moe.emit_reads / emit_bytes / emit) ------------------


class Match:
    """A recognized expert gather: what `emit` needs of the reference's `moe.Match`
    (router values, pair-space sizes and the packed projections it reads)."""

    __slots__ = ("key", "skip_keys", "disabled", "router_indices", "router_weights", "lhs",
                 "T", "K", "E", "P", "packs", "sum_dtype", "out_dtype", "bytes")

    def __init__(self):
        self.skip_keys = ()
        self.disabled = False
        self.bytes = 0
        self.sum_dtype = torch.float32
        self.out_dtype = None


def emit_reads(m):
    reads = getattr(m, "reads", None)           # a planned region lists what it gathers
    if reads is not None:
        return tuple(reads)
    return (m.lhs, m.router_indices, m.router_weights)


def emit_bytes(m) -> int:
    return int(m.bytes)


def emit(interp, m, env):
    """The gathered expert dispatch in place of the dense weighted sum: packs are read
    through `qmm.pack_arrays` exactly as `_emit_dot` does (src/metaljax/moe.py:1308-1315)."""
    from . import qmm
    idx, wgt = env[m.router_indices], env[m.router_weights]
    x = env[m.lhs]
    packs = []
    for pm in m.packs:
        vals = qmm.pack_arrays(interp, pm)
        packs.append((vals[0], vals[1], vals[2] if pm.mode == "affine" else None))
    pm = m.packs[0]
    y = moe_experts(x, idx, wgt, packs[0], packs[1], packs[2], group_size=pm.gs, bits=pm.bits,
                    mode=pm.mode, sum_dtype=m.sum_dtype)
    if m.out_dtype is not None and y.dtype != m.out_dtype:
        y = y.to(m.out_dtype)
    return [y]
