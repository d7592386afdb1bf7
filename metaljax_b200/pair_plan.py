"""Pair-space plan of a dense mixture-of-experts region (the reference's `_Planner` with its
`_Ext / _Elem / _View / _Dot` nodes, src/metaljax/moe.py:450-810, and the evaluation half of its
`emit`, :1260-1340, 1425-1461).

A dense expert block computes, for every (expert, token), a value `Y[.., e, .., t, ..]` and then
sums it against the routing matrix. Only T*K of the E*T (expert, token) pairs carry weight, so
the region is re-run over those pairs alone. Starting at Y with its expert axis `ea` and token axis
`ta`, the planner walks the producers backwards and gives every value a node:

  ext    computed outside the region (no expert axis: token-only work is not repeated K times, and
         nothing without the expert axis can depend on region work): read from `env` when the
         block is emitted and gathered by (expert of the pair, token of the pair)
  const  a splat constant inside the region: a scalar
  elem   an element-wise op (or a concatenate along a trailing axis) on pair-space operands
  view   broadcast / transpose / reshape / slice acting on the trailing axes only
  dot    a per-expert matmul: a quantized match of `recognizer.analyze` (fused onto the grouped
         ragged product), or a 16-bit float weight computed from the program's arguments

A pair-space array is `[P, *trailing]`, `trailing` being the dense shape without the expert and
token axes; a value that has neither axis keeps its dense shape and broadcasts against the rest.
Where the reference keeps the pairs in router order and hands `mx.gather_qmm` an index per pair,
the pairs here are sorted by expert once (`moe.sort_pairs`), so that every dot of the region is a
grouped product over contiguous row runs (`qmm_ragged_dot` / `qmm_ragged_mm`), and the weighted
sum over a token's K pairs reads through the inverse of that sort (`qmm_moe_routed_sum`).
"""

from __future__ import annotations

import torch

from . import hlo, moe
from .qmm import _Reject

ELEMENTWISE = frozenset((
    "stablehlo.add", "stablehlo.subtract", "stablehlo.multiply", "stablehlo.divide", "stablehlo.maximum",
    "stablehlo.minimum", "stablehlo.negate", "stablehlo.abs", "stablehlo.exponential", "stablehlo.rsqrt",
    "stablehlo.logistic", "stablehlo.sqrt", "stablehlo.tanh", "stablehlo.log", "stablehlo.power",
    "stablehlo.convert", "stablehlo.compare", "stablehlo.select", "stablehlo.clamp", "stablehlo.and",
    "stablehlo.or", "stablehlo.xor"))


class Node:
    """One value of the region in pair space. `ea` / `ta`: the dense value's expert / token axis
    (None when it has none); `shape`: the dense shape."""

    __slots__ = ("kind", "ea", "ta", "shape", "value", "op", "srcs", "arg", "match")

    def __init__(self, kind, ea, ta, shape, value=None, op=None, srcs=(), arg=None, match=None):
        self.kind, self.ea, self.ta, self.shape = kind, ea, ta, tuple(shape)
        self.value, self.op, self.srcs, self.arg, self.match = value, op, tuple(srcs), arg, match

    @property
    def paired(self):
        return self.ea is not None or self.ta is not None

    @property
    def trailing(self):
        return [s for i, s in enumerate(self.shape) if i not in (self.ea, self.ta)]


def _tpos(ea, ta, axis):
    """Position of dense `axis` among the trailing axes."""
    return sum(1 for i in range(axis) if i not in (ea, ta))


def _prod(xs):
    out = 1
    for x in xs:
        out *= int(x)
    return out


class Planner:
    def __init__(self, st, E, T, find_match):
        self.st, self.E, self.T = st, E, T
        self.find_match = find_match       # dot op -> qmm.Match (quantized or float) or _Reject
        self.nodes = {}                    # (value, ea, ta) -> Node
        self.order = []                    # nodes, operands before users
        self.region = {}                   # id(op) -> op: the dense ops the plan replaces
        self.reads = []                    # outside values the emission reads
        self.matches = []                  # the quantized / float matches of the region's dots

    def plan(self, v, ea, ta) -> Node:
        key = (v, ea, ta)
        hit = self.nodes.get(key)
        if hit is None:
            hit = self._build(v, ea, ta)
            self.nodes[key] = hit
            self.order.append(hit)
        return hit

    def _build(self, v, ea, ta):
        shape = tuple(v.type.shape)
        if ea is not None and shape[ea] != self.E:
            raise _Reject("expert axis size disagrees")
        if ta is not None and shape[ta] != self.T:
            raise _Reject("token axis size disagrees")
        o = v.op
        # THE BOUNDARY: only values that carry the expert axis are region work
        if o is None or ea is None:
            if o is not None and (o.opaque or o.name == "stablehlo.while"):
                raise _Reject("a region input is produced by an op with regions")
            self.reads.append(v)
            return Node("ext", ea, ta, shape, value=v)
        name = o.name
        if name == "stablehlo.constant":
            t = hlo._dense(o.text, v.type)
            flat = t.reshape(-1)
            if flat.numel() == 0 or not bool((flat == flat[0]).all()):
                raise _Reject("a per-expert constant inside the region")
            self.region[id(o)] = o
            return Node("const", None, None, (), value=flat[0].clone())
        if name == "stablehlo.iota":
            raise _Reject("a per-expert iota inside the region")
        if o.opaque or o.regions:
            raise _Reject(f"{name} is not modelled in pair space")
        m = self._match_rooted_at(o)
        if m is not None:
            return self._dot(o, m, ea, ta, shape)
        self.region[id(o)] = o
        if name in ELEMENTWISE:
            srcs = []
            for x in o.operands:
                xs = tuple(x.type.shape)
                if xs == shape:
                    srcs.append(self.plan(x, ea, ta))
                elif not xs:
                    srcs.append(self.plan(x, None, None))
                else:
                    raise _Reject(f"{name} operand shape {xs} != {shape}")
            return Node("elem", ea, ta, shape, op=o, srcs=srcs)
        if name == "stablehlo.concatenate":
            if o.attrs["dim"] in (ea, ta):
                raise _Reject("concatenate along the expert or token axis")
            return Node("elem", ea, ta, shape, op=o, srcs=[self.plan(x, ea, ta) for x in o.operands])
        if name == "stablehlo.broadcast_in_dim":
            return self._bcast(o, ea, ta, shape)
        if name == "stablehlo.transpose":
            perm = o.attrs["dims"]
            src = o.operands[0]
            bea = perm[ea] if ea is not None else None
            bta = perm[ta] if ta is not None else None
            node = self.plan(src, bea, bta)
            order = [_tpos(bea, bta, perm[i]) for i in range(len(shape)) if i not in (ea, ta)]
            return Node("view", ea, ta, shape, srcs=[node], arg=("perm", order))
        if name == "stablehlo.reshape":
            src = o.operands[0]
            sshape = tuple(src.type.shape)
            lead = max(a for a in (ea, ta) if a is not None) + 1
            if len(sshape) < lead or sshape[:lead] != shape[:lead]:
                raise _Reject("reshape crosses the expert / token axes")
            return Node("view", ea, ta, shape, srcs=[self.plan(src, ea, ta)], arg=("reshape", None))
        if name == "stablehlo.slice":
            src = o.operands[0]
            sshape = tuple(src.type.shape)
            spec = [tuple(s) + (1,) * (3 - len(s)) for s in o.attrs["slices"]]
            for a in (ea, ta):
                if a is not None and (spec[a][0], spec[a][1], spec[a][2]) != (0, sshape[a], 1):
                    raise _Reject("slice cuts the expert or token axis")
            keep = [spec[i] for i in range(len(sshape)) if i not in (ea, ta)]
            return Node("view", ea, ta, shape, srcs=[self.plan(src, ea, ta)], arg=("slice", keep))
        if name == "stablehlo.dot_general":
            return self._dot(o, self.find_match(o), ea, ta, shape)
        raise _Reject(f"{name} is not modelled in pair space")

    def _match_rooted_at(self, o):
        for m in self.st.matches:
            if not m.disabled and m.root is o:
                return m
        return None

    def _bcast(self, o, ea, ta, shape):
        bd = list(o.attrs["dims"])
        if bd != sorted(bd):
            raise _Reject("broadcast dimensions are not increasing")
        src = o.operands[0]
        sshape = tuple(src.type.shape)
        bea = bta = None
        drop = set()
        for j, d in enumerate(bd):
            if d not in (ea, ta):
                continue
            full = self.E if d == ea else self.T
            # a UNIT source axis is a broadcast, never the axis itself (the two readings overlap
            # when T == 1, every decode step; src/metaljax/moe.py:637-647)
            if sshape[j] == 1:
                drop.add(j)
            elif sshape[j] == full:
                if d == ea:
                    bea = j
                else:
                    bta = j
            else:
                raise _Reject("expert / token axis broadcast from a part")
        node = self.plan(src, bea, bta)
        keep = []                                   # per source trailing axis: its trailing place in the result, None = dropped
        for j in range(len(sshape)):
            if j in (bea, bta):
                continue
            keep.append(None if j in drop else _tpos(ea, ta, bd[j]))
        dest = [k for k in keep if k is not None]
        if dest != sorted(dest):
            raise _Reject("broadcast reorders the trailing axes")
        return Node("view", ea, ta, shape, srcs=[node], arg=("bcast", keep))

    def _dot(self, o, m, ea, ta, shape):
        """A per-expert matmul on match `m` (dimension bookkeeping of `recognizer._finish`:
        `lperm` lists the data operand's axes as batching, free, contracting; the result lists
        batching, then the lhs operand's free axes, then the rhs operand's)."""
        if ta is None:
            raise _Reject("per-expert dot without a token axis")
        nb, nm, nn = len(m.bshape), len(m.mshape), len(m.nshape)
        if len(shape) != nb + nm + nn:
            raise _Reject("the dot's result does not list batching, free and free axes")
        d0, w0 = (nb + nn, nb) if m.swapped else (nb, nb + nm)       # first data-free / weight-free result axis
        if not d0 <= ta < d0 + nm:
            raise _Reject("the token axis is not a free axis of the data operand")
        tdim = m.lperm[nb + (ta - d0)]
        if ea < nb:                                                  # the experts batch the dot
            if nb != 1 or m.bshape[0] != self.E:
                raise _Reject("the dot batches over more than the experts")
            ddim, n_rest = m.lperm[0], list(m.nshape)
            n_keep = list(range(nn))
        elif w0 <= ea < w0 + nn:                                     # the experts lead the weight's output features
            if nb or ea != w0:
                raise _Reject("the expert axis is not the weight's leading axis")
            ddim, n_rest = None, list(m.nshape[1:])
            n_keep = list(range(1, nn))
        else:
            raise _Reject("the expert axis belongs to the data operand only")
        data_v = m.lhs
        data = self.plan(data_v, ddim, tdim)
        # data trailing axes (dense order) -> [M..., K...] in the match's order
        dorder = [_tpos(ddim, tdim, d) for d in m.lperm[nb:] if d != tdim]
        mshape = [s for j, s in enumerate(m.mshape) if nb + j != nb + (ta - d0)]
        M, N, K = _prod(mshape), _prod(n_rest), int(m.K)
        if M == 0 or N == 0:
            raise _Reject("empty per-expert dot")
        # result trailing axes in dense order, as indices into [mshape..., n_rest...]
        perm = []
        for i in range(len(shape)):
            if i in (ea, ta):
                continue
            if d0 <= i < d0 + nm:
                j = i - d0
                perm.append(j - (1 if j > ta - d0 else 0))
            else:
                perm.append(len(mshape) + n_keep.index(i - w0))
        self.matches.append(m)
        for op in m.ops.values() if isinstance(m.ops, dict) else ():
            self.region[id(op)] = op
        self.region[id(m.root)] = m.root
        return Node("dot", ea, ta, shape, op=o, srcs=[data], match=m,
                    arg=dict(dorder=dorder, mshape=mshape, nshape=n_rest, M=M, N=N, K=K, perm=perm,
                             dtype=o.results[0].type.dtype))

    def bytes(self, P):
        """Device bytes the emission materializes: every paired node's `[P, *trailing]` array."""
        total = 0
        for n in self.order:
            if n.paired and n.kind != "view":
                total += P * _prod(n.trailing) * 2
        return total


# ---------------------------------------------------------------------------------------
# evaluation
# ---------------------------------------------------------------------------------------


def evaluate(nodes, env, pairs, experts, weight_of, ragged=None):
    """Run the planned nodes over the sorted pairs. `pairs` = (token_of_row, expert_of_row,
    group_sizes); `weight_of(match)` returns the match's per-expert weight: a `(w, scales, biases)`
    pack with `[E, N, ...]` arrays or a float `[E, N, K]` array; `ragged(rows, weight, sizes, match)`
    is the grouped product (default: the library's). Returns {id(node): array}."""
    tok, eor, sizes = pairs
    P = tok.shape[0]
    out = {}
    for n in nodes:
        k = n.kind
        if k == "ext":
            t = hlo.evaluate_value(n.value, env)
            if n.paired:
                lead = [a for a in (n.ea, n.ta) if a is not None]
                t = t.movedim(lead, list(range(len(lead))))
                t = t[eor, tok] if len(lead) == 2 else t.index_select(0, eor if n.ea is not None else tok)
            out[id(n)] = t
        elif k == "const":
            out[id(n)] = n.value.to(tok.device)
        elif k == "elem":
            ins = [out[id(s)] for s in n.srcs]
            if n.op.name == "stablehlo.concatenate":
                ins = [x if s.paired else x.expand([P] + list(s.trailing)) for x, s in zip(ins, n.srcs)]
                out[id(n)] = torch.cat(ins, dim=1 + _tpos(n.ea, n.ta, n.op.attrs["dim"]))
            else:
                out[id(n)] = hlo.EVAL[n.op.name](n.op, *ins)
        elif k == "view":
            src = n.srcs[0]
            x = out[id(src)]
            off = 1 if src.paired else 0
            head = list(x.shape[:off])
            what, arg = n.arg
            if what == "perm":
                x = x.permute(list(range(off)) + [off + a for a in arg])
            elif what == "reshape":
                x = x.reshape(head + n.trailing)
            elif what == "slice":
                x = x[(slice(None),) * off + tuple(slice(a, b, c) for a, b, c in arg)]
            else:                                                   # bcast
                for i in reversed(range(len(arg))):
                    if arg[i] is None:
                        x = x.squeeze(off + i)
                tshape = n.trailing
                view = [1] * len(tshape)
                for place, size in zip([a for a in arg if a is not None], x.shape[off:]):
                    view[place] = size
                x = x.reshape(head + view).expand(head + tshape)
            out[id(n)] = x
        else:                                                       # dot
            a = n.arg
            x = out[id(n.srcs[0])]
            if not n.srcs[0].paired:
                raise _Reject("the data of a per-expert dot has no pair axis")
            x = x.permute([0] + [1 + d for d in a["dorder"]]).reshape(P * a["M"], a["K"])
            if x.dtype != a["dtype"]:
                x = x.to(a["dtype"])
            w = weight_of(n.match)
            rows_per_expert = sizes * a["M"] if a["M"] != 1 else sizes
            if ragged is not None:
                y = ragged(x.contiguous(), w, rows_per_expert, n.match)
            elif isinstance(w, tuple):
                y = moe.ragged_dot(x.contiguous(), w[0], w[1], w[2], rows_per_expert, group_size=n.match.gs,
                                   bits=n.match.bits, mode=n.match.mode)
            else:
                y = moe.ragged_mm(x.contiguous(), w, rows_per_expert)
            y = y.reshape([P] + a["mshape"] + a["nshape"])
            if a["perm"] != list(range(len(a["perm"]))):
                y = y.permute([0] + [1 + j for j in a["perm"]])
            out[id(n)] = y
    return out


def weighted_sum(y_pair, order, weights, T, K, out_dtype, sum_dtype=torch.float32):
    """`out[t] = sum_k weights[t, k] * y_pair[row of pair (t, k)]`, k ascending, in `sum_dtype`
    (the reference's weighted K-sum, src/metaljax/moe.py:1425-1461)."""
    width = _prod(y_pair.shape[1:])
    rows = y_pair.reshape(y_pair.shape[0], width)
    if rows.is_cuda and rows.dtype in (torch.bfloat16, torch.float16) and width % 8 == 0 and sum_dtype == torch.float32:
        return moe.routed_sum(rows.contiguous(), order, weights.to(torch.float32), T, K).to(out_dtype)
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel(), device=order.device)
    picked = rows.index_select(0, inv).reshape(T, K, width).to(sum_dtype)
    acc = torch.zeros((T, width), dtype=sum_dtype, device=rows.device)
    for k in range(K):
        acc = acc + (weights[:, k, None].to(sum_dtype) * picked[:, k]).to(sum_dtype)
    return acc.to(out_dtype)
