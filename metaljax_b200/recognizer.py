"""The quantized-matmul recognizer over StableHLO: structural analysis, the pack prologue and
the interpreter hook that puts one fused `quantized_matmul` where a dequantize-and-dot chain
stood. Mirrors the fused-root protocol of the reference (src/metaljax/qmm.py):

    analyze(interp) -> State            once per program, never touches values   (:1042-1091)
    prologue(interp, args) -> bool      eager, on concrete buffers: verify + pack (:2305-2387)
    emit(interp, match, env) -> [y]     the fused op                              (:2469-2501)

over the IR of `metaljax_b200/hlo.py` (the reference walks jaxlib.mlir objects). `Match`,
`State`, `_Pack`, `build_pack`, `emit` and the liveness hooks live in `metaljax_b200/qmm.py`.

Three forms are recognized, on either operand of a `dot_general` (the right-hand side first,
src/metaljax/qmm.py:902-917):

    sub-channel   dot(x, [shape ops](mul(sub(cvt(codes), cvt(zeros)), scales)))   (:920-950)
    MXFP4         dot(x, [shape ops](mul(values, broadcast(one scale per 32))))   (:868-899)
    per-channel   divide(dot(x, [shape ops](cvt(codes))), broadcast(scale))       (:953-982)

The chain under the codes / scale / zero operands is not matched op by op: the three subtrees
are recorded, required to depend only on `@main`'s non-donated arguments through ops without
regions, and evaluated once at the first execute, where every value-level question is settled
(`qmm.build_pack`). A failed check disables that one match; analysis never raises.

`Interpreter` is the small host that the reference's engine is to its recognizers: it owns the
parsed function, the recognizer state (`_qmm`) and `execute(args)`, which runs the prologue and
then the ops in order — skipped ones not at all, fused roots through `emit`, everything else
literally (`hlo.eval_op`).
"""

from __future__ import annotations

import os
import re
import weakref

import torch

from . import hlo, qmm
from .qmm import Match, State, _Reject

SHAPE_OPS = ("stablehlo.reshape", "stablehlo.transpose", "stablehlo.broadcast_in_dim")
GROUP_SIZES = (128, 64, 32)
MXFP4_GROUP = 32
ENABLED = True

# Finished packs shared across programs: a model compiled once per sequence length hands every
# shape its own program and recognizer state, and would otherwise verify and repack the same
# weights again (src/metaljax/qmm.py:2208-2302). Key: the canonical text of the reconstruction
# subtree plus the identity of the buffers it reads; an entry dies with its buffers.
_BUILD_CACHE = {}
_BUILD_CACHE_MAX = 256


# ---------------------------------------------------------------------------------------
# structural helpers
# ---------------------------------------------------------------------------------------


def _strip(v, names):
    """Walk down through ops of kind `names`; returns (base, ops outermost last)."""
    chain = []
    while v.op is not None and v.op.name in names:
        chain.append(v.op)
        v = v.op.operands[0]
    return v, chain[::-1]


def _is_int(v):
    return v.type.el in hlo.INT_ELS


def _is_float(v):
    return v.type.el in hlo.FLOAT_ELS


def _prod(xs):
    p = 1
    for x in xs:
        p *= x
    return p


_SIGNED_WIDTH = {"i4": 4, "i8": 8, "i16": 16, "i32": 32, "i64": 64}


def _parse_codes(v):
    """`v` as an integer-code operand -> (codes, zero point or None, integer subtract range or
    None); None when it is not one. A subtraction done in integer arithmetic wraps, so its range
    is remembered and checked against the values later (src/metaljax/qmm.py:531-555)."""
    base, _ = _strip(v, ("stablehlo.convert",))
    if base.op is not None and base.op.name == "stablehlo.subtract":
        c, _ = _strip(base.op.operands[0], ("stablehlo.convert",))
        if not _is_int(c):
            return None
        rng = None
        if _is_int(base):
            w = _SIGNED_WIDTH.get(base.type.el)
            if w is None:
                return None
            rng = (-(1 << (w - 1)), (1 << (w - 1)) - 1)
        return c, base.op.operands[1], rng
    return (base, None, None) if _is_int(base) else None


def _broadcast_base(v):
    """Peel broadcast_in_dim / convert chains: (base, dims) with dims[i] the dimension of `v`
    that base's dimension i lands in, or (v, None) when nothing was broadcast."""
    dims = list(range(len(v.type.shape)))
    seen = False
    while v.op is not None:
        if v.op.name == "stablehlo.broadcast_in_dim":
            dims = [dims[j] for j in v.op.attrs["dims"]]
            v = v.op.operands[0]
            seen = True
        elif v.op.name == "stablehlo.convert":
            v = v.op.operands[0]
        else:
            break
    return (v, dims) if seen else (v, None)


def _has_int_leaf(v, limit=64):
    """Does the subtree bottom out on an integer tensor? (a cheap guard that keeps the MXFP4
    branch from adopting `x @ (w * mask)`, src/metaljax/qmm.py:844-865)"""
    stack, seen = [v], set()
    while stack and len(seen) < limit:
        cur = stack.pop()
        if cur in seen:
            continue
        seen.add(cur)
        if _is_int(cur):
            return True
        if cur.op is not None and not cur.op.opaque:
            stack.extend(cur.op.operands)
    return False


def _split_scaled(mul):
    """(values, scale) of `values * broadcast(per-32 scale)`: the scale is the operand broadcast
    from a tensor holding exactly one value per 32 (an RMS norm's `x * broadcast(rsqrt)` has one
    per row and is not adopted)."""
    total = _prod(mul.results[0].type.shape)
    cands = []
    for i in (0, 1):
        v = mul.operands[i]
        if not _is_float(v):
            raise _Reject(f"multiply operand element type {v.type.el}")
        base, dims = _broadcast_base(v)
        if dims is not None and _prod(base.type.shape) * MXFP4_GROUP == total:
            cands.append(i)
    if len(cands) != 1:
        raise _Reject("no single operand broadcasts one scale per 32 values")
    return mul.operands[1 - cands[0]], mul.operands[cands[0]]


def _closure(values, fn, ops, arg_indices, register=()):
    """Backward closure of `values`: every leaf must be an argument of `@main`; no op with
    regions inside (src/metaljax/qmm.py:743-777)."""
    for o in register:
        ops[id(o)] = o
    stack, seen = list(values), set()
    while stack:
        v = stack.pop()
        if v in seen:
            continue
        seen.add(v)
        if v.op is None:
            if v.is_main_argument:
                arg_indices.add(v.index)
                continue
            # a loop's closed-over weight arrives as a carry the body returns unchanged: follow
            # it out to the value the loop was handed (src/metaljax/qmm.py:714-740)
            outer = hlo.invariant_init(v)
            if outer is None:
                raise _Reject("operand depends on an inner block argument")
            stack.append(outer)
            continue
        if v.op.opaque or v.op.regions:
            raise _Reject(f"operand subtree contains {v.op.name}")
        ops.setdefault(id(v.op), v.op)
        stack.extend(v.op.operands)


def _finish(fn, m, root, absorb, dot, qside=1, required=(), register=()):
    """Dimension bookkeeping for a dot whose operand `qside` is the quantized one: B, M, K, N,
    the permutations that bring both operands to [B, rows, K], and the absorbed op set
    (src/metaljax/qmm.py:780-841)."""
    (lb, rb), (lc, rc) = dot.attrs["batching"], dot.attrs["contracting"]
    (qb, qc), (ab, ac) = ((rb, rc), (lb, lc)) if qside == 1 else ((lb, lc), (rb, rc))
    quant, act = dot.operands[qside], dot.operands[1 - qside]
    if not _is_float(act):
        raise _Reject(f"activation element type {act.type.el}")
    if not _is_float(root.results[0]):
        raise _Reject(f"result element type {root.results[0].type.el}")
    qshape, ashape = list(quant.type.shape), list(act.type.shape)
    if [ashape[d] for d in ab] != [qshape[d] for d in qb]:
        raise _Reject("batching dimensions disagree")
    afree = [d for d in range(len(ashape)) if d not in ac and d not in ab]
    qfree = [d for d in range(len(qshape)) if d not in qc and d not in qb]
    m.B = _prod(ashape[d] for d in ab)
    m.M, m.K, m.N = _prod(ashape[d] for d in afree), _prod(ashape[d] for d in ac), _prod(qshape[d] for d in qfree)
    if 0 in (m.B, m.M, m.K, m.N):
        raise _Reject("empty matmul")
    if m.K % GROUP_SIZES[-1]:
        raise _Reject(f"K={m.K} is not a multiple of {GROUP_SIZES[-1]}")
    if m.K != _prod(qshape[d] for d in qc):
        raise _Reject("contracting dimensions disagree")
    m.root, m.key, m.lhs, m.swapped = root, id(root), act, qside == 0
    m.lperm, m.rperm, m.rshape = ab + afree + ac, qb + qfree + qc, qshape
    m.bshape, m.mshape, m.nshape = [ashape[d] for d in ab], [ashape[d] for d in afree], [qshape[d] for d in qfree]
    m.out_dtype = root.results[0].type.dtype
    m.name = (f"{m.M}x{m.K}x{m.N}" if not m.bshape else f"{'x'.join(map(str, m.bshape))}|{m.M}x{m.K}x{m.N}") \
        + ("'" if m.swapped else "")
    arg_indices = set()
    _closure(absorb, fn, m.ops, arg_indices, register)
    if arg_indices & fn.donated:
        raise _Reject("quantized operand is donated (its buffer may be reused)")
    m.arg_indices = tuple(sorted(arg_indices))
    m.required = [id(o) for o in required] + [id(o) for o in m.post]
    return m


def _try_scaled_side(fn, dot, qside):
    """Forms `mul(sub(cvt(codes), cvt(zeros)), scales)` and MXFP4 on operand `qside`."""
    qop = dot.operands[qside]
    base, post = _strip(qop, SHAPE_OPS + ("stablehlo.convert",))
    mul = base.op
    if mul is None or mul.name != "stablehlo.multiply":
        raise _Reject("the operand is not a multiply")
    parsed = scale = None
    for i in (0, 1):
        parsed = _parse_codes(mul.operands[i])
        if parsed is not None:
            scale = mul.operands[1 - i]
            break
    m = Match()
    if parsed is None:
        values, scale = _split_scaled(mul)
        if not _has_int_leaf(values):
            raise _Reject("the scaled operand holds no integer codes")
        m.mode, m.codes = "mxfp4", values
    else:
        m.codes, m.zero, m.sub_range = parsed
    if not _is_float(scale):
        raise _Reject(f"scale element type {scale.type.el}")
    m.scale = scale
    m.post = [o for o in post if o.name in SHAPE_OPS]
    return _finish(fn, m, dot, [qop], dot, qside=qside, required=(mul,))


def _try_scaled(fn, dot):
    first = None
    for qside in (1, 0):
        try:
            return _try_scaled_side(fn, dot, qside)
        except _Reject as e:
            first = first or e
    raise first


def _try_perchannel(fn, div):
    """`divide(dot(x, [shape ops](cvt(codes))), broadcast(scale))`."""
    num, den = div.operands
    dot = num.op
    if dot is None or dot.name != "stablehlo.dot_general":
        raise _Reject("divide numerator is not a dot")
    codes, post = _strip(dot.operands[1], SHAPE_OPS + ("stablehlo.convert",))
    if not _is_int(codes):
        raise _Reject("dot rhs is not an integer code tensor")
    scale, dims = _broadcast_base(den)
    if dims is None or not _is_float(scale):
        raise _Reject("divisor is not a broadcast float")
    (lb, rb), (lc, _) = dot.attrs["batching"], dot.attrs["contracting"]
    if lb or rb:
        raise _Reject("batching dimensions")
    nm = len(dot.operands[0].type.shape) - len(lc)          # leading output (M) dimensions
    if any(d < nm for d in dims):
        raise _Reject("divisor depends on the batch axis")
    m = Match()
    m.recip, m.codes, m.scale = True, codes, scale
    m.bcast_dims = [d - nm for d in dims]
    m.post = [o for o in post if o.name in SHAPE_OPS]
    return _finish(fn, m, div, [dot.operands[1], den], dot, required=(dot,), register=(dot,))


def _prune(cands):
    """Which absorbed ops may really be skipped: an op only if every consumer of every result is
    itself skipped or is a rewritten root; a candidate whose required ops cannot be skipped is
    dropped, which can un-skip ops others counted on, so iterate to a fixed point
    (src/metaljax/qmm.py:991-1039)."""
    live = list(cands)
    while True:
        roots = {m.key for m in live}
        skip = {}
        for m in live:
            skip.update(m.ops)
        changed = True
        while changed:
            changed = False
            for key, op in list(skip.items()):
                for r in op.results:
                    for user, _ in r.uses:
                        if id(user) not in skip and id(user) not in roots:
                            del skip[key]
                            changed = True
                            break
                    if key not in skip:
                        break
        keep = [m for m in live if all(k in skip for k in m.required)]
        if len(keep) == len(live):
            for m in live:
                m.ops = {k: o for k, o in m.ops.items() if k in skip}
            return live
        live = keep


def analyze(interp) -> State:
    """Structural analysis of a program, once. Never touches values, never raises."""
    st = interp._qmm
    if st is not None:
        return st
    st = State()
    interp._qmm = st
    try:
        if not ENABLED:
            raise _Reject("recognizer disabled")
        fn = interp.func
        cands = []
        for op in fn.walk():
            try:
                if op.name == "stablehlo.dot_general":
                    cands.append(_try_scaled(fn, op))
                elif op.name == "stablehlo.divide":
                    cands.append(_try_perchannel(fn, op))
            except _Reject:
                pass
        absorbed = set()
        for m in cands:
            absorbed.update(m.ops)
        cands = [m for m in cands if m.key not in absorbed]      # a dot inside another's subtree
        st.matches = _prune(cands) if cands else []
        qmm.STATS["recognized"] += len(st.matches)
    except Exception:                                            # analysis must never break a program
        st.matches = []
    # Expert-gather rewrites are found on top of the quantized ones: a dense mixture-of-experts
    # block whose dots were matched here adopts those matches (src/metaljax/qmm.py:1085-1091).
    from . import moe_recognizer
    moe_recognizer.analyze(interp, st)
    st.rebuild()
    return st


# ---------------------------------------------------------------------------------------
# first execute: verification + packing
# ---------------------------------------------------------------------------------------


def _to_nk(t, m):
    """An operand-shaped tensor -> `[B?, N, K]` (src/metaljax/qmm.py:1188-1201)."""
    t = t.permute(*m.rperm)
    return t.reshape([m.B, m.N, m.K] if m.bshape else [m.N, m.K])


def _replay(t, post):
    for op in post:
        if op.name == "stablehlo.reshape":
            t = t.reshape(op.results[0].type.shape)
        elif op.name == "stablehlo.transpose":
            t = t.permute(*op.attrs["dims"])
        else:
            t = hlo.EVAL[op.name](op, t)
    return t


def _fingerprint(m):
    """Canonical text of the reconstruction subtree: ops in program order, operands named by
    position among the subtree's values or by argument number."""
    ops = sorted(m.ops.values(), key=lambda o: o.position)
    names = {}
    lines = []
    for o in ops:
        ins = []
        for v in o.operands:
            ins.append((f"a{v.index}" if v.is_main_argument else f"b{v.name}") if v.op is None
                       else names.get(v, f"x{v.name}"))
        for r in o.results:
            names[r] = f"v{len(names)}"
        lines.append(f"{o.name}({','.join(ins)})[{sorted(o.attrs.items())}]{[r.type for r in o.results]}"
                     + (o.text if o.name == "stablehlo.constant" else ""))
    return "\n".join(lines) + f"|{m.mode}|{m.recip}|{m.rperm}|{m.B},{m.N},{m.K}"


def _leaf_key(leaves):
    return tuple((t.data_ptr(), tuple(t.shape), t.dtype, t._version) for t in leaves)


def _cached_build(key, leaves):
    ent = _BUILD_CACHE.get(key)
    if ent is None:
        return None
    refs, pack = ent
    if len(refs) != len(leaves) or any(r() is not t for r, t in zip(refs, leaves)):
        del _BUILD_CACHE[key]                                    # a buffer died and its address was reused
        return None
    return pack


# Weight elements evaluated per block: the reconstruction chain is several times wider than its
# result, so a block of 2^24 elements keeps the transient within a few hundred MB
# (src/metaljax/qmm.py:1253-1259).
_BLOCK_ELEMS = int(os.environ.get("METALJAX_QMM_BLOCK", str(1 << 24)))
# Ceiling on a value the blocking reads WHOLE for every block (a decode table, a splat): a big
# one means the blocking misread the graph, and evaluating whole is the honest answer.
_WHOLE_MAX = 1 << 22

# Ops whose evaluator is a pure function of the arrays it is handed, so that a slice of the
# leading axis of every operand gives that slice of the result (src/metaljax/qmm.py:1274-1292).
_ROW_LOCAL = frozenset("""
    stablehlo.abs stablehlo.add stablehlo.and stablehlo.ceil stablehlo.clamp stablehlo.compare
    stablehlo.convert stablehlo.divide stablehlo.exponential stablehlo.floor stablehlo.log
    stablehlo.maximum stablehlo.minimum stablehlo.multiply stablehlo.negate stablehlo.not
    stablehlo.or stablehlo.power stablehlo.round_nearest_even stablehlo.rsqrt stablehlo.select
    stablehlo.shift_left stablehlo.shift_right_arithmetic stablehlo.shift_right_logical
    stablehlo.sign stablehlo.sqrt stablehlo.subtract stablehlo.tanh stablehlo.xor
    stablehlo.bitcast_convert
""".split())


class _NotBlockable(Exception):
    """The subtree cannot be evaluated one block of rows at a time. Not a `_Reject`: the weight
    still packs, from a whole evaluation."""


class _RowBlocks:
    """A match's operand subtrees evaluated one slice of the weight's leading axis at a time
    (src/metaljax/qmm.py:1360-1631). Every op on the way has to be row-local: the slice of its
    result must be its result on the slices. That is free for an element-wise op and a rule
    about the dimension attributes of the others (`_ev`). A value read through a gather (a
    decode table) or broadcast along the leading axis is wanted whole by every block, and has
    to be small. Anything else raises `_NotBlockable`."""

    def __init__(self, interp, m, args):
        self.m = m
        self.env = dict(zip(interp.func.args, args))
        self.whole = dict(self.env)                              # memo of the small whole-evaluated values
        self.lead = int(m.rshape[0]) if m.rshape else 0
        per = _prod(m.rshape[1:]) if m.rshape else 0
        self.step = None
        if m.rshape and list(m.rperm)[:1] == [0] and self.lead > 1 and self.lead * per > _BLOCK_ELEMS:
            self.step = max(1, _BLOCK_ELEMS // max(per, 1))

    def blocks(self):
        return [(lo, min(lo + self.step, self.lead)) for lo in range(0, self.lead, self.step)]

    def rows(self, value, lo, hi, memo, like=None):
        """`value`'s rows of block [lo, hi) as a `[rows, K]` matrix (batch and row axes folded);
        `like` is the shape the chain broadcasts the value to before the post ops."""
        m = self.m
        t = self._ev(value, True, lo, hi, memo)
        if like is not None and list(t.shape[1:]) != list(like[1:]):
            t = t.expand([hi - lo] + list(like[1:]))
        for op in m.post:                                        # reshapes / transposes after the multiply
            shape = list(op.results[0].type.shape)
            if not shape or shape[0] != self.lead:
                raise _NotBlockable(f"{op.name} folds the leading axis")
            if op.name == "stablehlo.reshape":
                t = t.reshape([hi - lo] + shape[1:])
            elif op.name == "stablehlo.transpose":
                if op.attrs["dims"][0] != 0:
                    raise _NotBlockable("a transpose moves the leading axis")
                t = t.permute(*op.attrs["dims"])
            elif op.name in _ROW_LOCAL and op.name in hlo.EVAL:
                t = hlo.EVAL[op.name](op, t)
            else:
                raise _NotBlockable(op.name)
        if list(t.shape) != [hi - lo] + list(m.rshape[1:]):
            raise _NotBlockable(f"a block evaluated to {list(t.shape)}")
        return t.permute(*m.rperm).reshape(-1, m.K)

    def _whole(self, v):
        if _prod(v.type.shape) > _WHOLE_MAX:
            raise _NotBlockable(f"a value of {_prod(v.type.shape)} elements is wanted whole by every block")
        return hlo.evaluate_value(v, self.whole)

    def _ev(self, v, row, lo, hi, memo):
        if not row:
            return self._whole(v)
        got = memo.get(v)
        if got is not None:
            return got
        shape = list(v.type.shape)
        if not shape or shape[0] != self.lead:
            raise _NotBlockable(f"%{v.name} of shape {shape} has no row axis")
        bshape = [hi - lo] + shape[1:]
        if v.op is None:
            t = self.env.get(v)
            if t is None:
                outer = hlo.invariant_init(v)
                if outer is None:
                    raise _Reject("unbound value in operand subtree")
                out = self._ev(outer, True, lo, hi, memo)
            else:
                out = t[lo:hi]
            memo[v] = out
            return out
        op, n = v.op, v.op.name
        ev = lambda o, r=True: self._ev(o, r, lo, hi, memo)
        if n in _ROW_LOCAL and n in hlo.EVAL:
            out = hlo.EVAL[n](op, *[ev(o) for o in op.operands])
        elif n == "stablehlo.constant":
            if re.search(r"dense<\s*[^\[\]<>]+\s*>", op.text):  # a splat: one value however big the type
                one = hlo._dense(op.text, hlo.TensorType((), v.type.el))
                dev = next((t.device for t in self.env.values()), None)
                out = one.to(dev).reshape([1] * len(bshape)).expand(bshape)
            else:
                out = self._whole(v)[lo:hi]
        elif n == "stablehlo.broadcast_in_dim":
            dims, src = list(op.attrs["dims"]), op.operands[0]
            sshape = list(src.type.shape)
            rowwise = 0 in dims and sshape[dims.index(0)] == self.lead
            if rowwise and dims.index(0) != 0:
                raise _NotBlockable("a broadcast moves the leading axis")
            x = ev(src, rowwise)
            view = [1] * len(bshape)
            for i, d in enumerate(dims):
                view[d] = x.shape[i]
            out = x.reshape(view).expand(bshape)
        elif n == "stablehlo.reshape":
            src = op.operands[0]
            if not src.type.shape or src.type.shape[0] != self.lead:
                raise _NotBlockable("a reshape folds the leading axis")
            out = ev(src).reshape(bshape)
        elif n == "stablehlo.transpose":
            if op.attrs["dims"][0] != 0:
                raise _NotBlockable("a transpose moves the leading axis")
            out = ev(op.operands[0]).permute(*op.attrs["dims"])
        elif n == "stablehlo.gather":
            a = op.attrs
            table, idx = op.operands
            if a["collapsed_slice_dims"] != [0] or a["start_index_map"] != [0] or a.get("operand_batching_dims") \
                    or a["slice_sizes"][1:] != list(table.type.shape[1:]):
                raise _NotBlockable("a gather that is not a row take")
            tb, ix = ev(table, False), ev(idx)
            ivd = a["index_vector_dim"]
            ix = ix.select(ivd, 0) if ivd < ix.dim() else ix
            out = tb[ix.to(torch.int64).clamp(0, tb.shape[0] - 1)].reshape(bshape)
        elif n == "stablehlo.concatenate":
            if op.attrs["dim"] == 0:
                raise _NotBlockable("a concatenation along the leading axis")
            out = torch.cat([ev(o) for o in op.operands], dim=op.attrs["dim"])
        elif n == "stablehlo.slice":
            sl = op.attrs["slices"]
            if not sl or tuple(sl[0][:2]) != (0, self.lead) or (len(sl[0]) > 2 and sl[0][2] != 1):
                raise _NotBlockable("a slice of the leading axis")
            x = ev(op.operands[0])
            out = x[(slice(None),) + tuple(slice(*s) for s in sl[1:])]
        else:
            raise _NotBlockable(n)
        if list(out.shape) != bshape:
            raise _NotBlockable(f"{n} evaluated to {list(out.shape)} for a block of {bshape}")
        memo[v] = out
        return out


def _build_blocked(src, m, leaves):
    """The pack from row blocks: the same decisions as `qmm.build_pack`, the same arrays."""
    packer = qmm.BlockedPacker(m, m.K)
    like = None
    if not m.recip and m.required:
        like = list(m.ops[m.required[0]].results[0].type.shape)
    inv = None
    if m.recip:                                                  # one scale per output channel, small
        s = hlo.evaluate_value(m.scale, src.whole)
        dims = list(m.bcast_dims)
        if dims != sorted(dims):
            order = sorted(range(len(dims)), key=lambda i: dims[i])
            s, dims = s.permute(*order), sorted(dims)
        interim = [1] * len(m.nshape)
        for i, d in enumerate(dims):
            interim[d] = s.shape[i]
        inv = (1.0 / s.reshape(interim).expand(m.nshape).reshape(m.N, 1).to(torch.float32))
    rows_per = _prod(m.rshape[1:]) // m.K
    for lo, hi in src.blocks():
        memo = {}
        codes = src.rows(m.codes, lo, hi, memo, None if m.recip else like)
        if m.recip:
            if m.bshape:
                raise _NotBlockable("a batched per-channel weight")
            packer.add(codes, inv[lo * rows_per: hi * rows_per].expand(-1, m.K), None)
        else:
            scale = src.rows(m.scale, lo, hi, memo, like)
            zero = None if m.zero is None else src.rows(m.zero, lo, hi, memo, like)
            packer.add(codes, scale, zero)
        del memo
    qmm.STATS["blocked"] = qmm.STATS.get("blocked", 0) + 1
    return packer.finish(leaves, [m.B, m.N] if m.bshape else [m.N])


def _build(interp, m, args, leaves):
    src = _RowBlocks(interp, m, args)
    if src.step is not None:
        try:
            return _build_blocked(src, m, leaves)
        except (_NotBlockable, qmm.BlockedPacker.NeedsWhole, NotImplementedError) as why:
            qmm.STATS["unblocked"] = qmm.STATS.get("unblocked", 0) + 1
            if qmm._DEBUG:
                print(f"[metaljax] qmm: {m.name} packs from a whole evaluation ({why})", flush=True)
    return _build_whole(interp, m, args, leaves)


def _build_whole(interp, m, args, leaves):
    fn = interp.func
    env = dict(zip(fn.args, args))
    shape = m.codes.type.shape if not m.post else None

    def full(v):                                                 # operand subtree -> [B?, N, K]
        t = hlo.evaluate_value(v, env)
        mul_shape = m.required and m.ops[m.required[0]].results[0].type.shape if not m.recip else None
        if mul_shape is not None and tuple(t.shape) != tuple(mul_shape):
            t = t.expand(mul_shape)
        return _to_nk(_replay(t, m.post), m)

    del shape
    if m.recip:
        codes = _to_nk(_replay(hlo.evaluate_value(m.codes, env), m.post), m)
        s = hlo.evaluate_value(m.scale, env)
        dims = list(m.bcast_dims)
        if dims != sorted(dims):
            order = sorted(range(len(dims)), key=lambda i: dims[i])
            s, dims = s.permute(*order), sorted(dims)
        interim = [1] * len(m.nshape)
        for i, d in enumerate(dims):
            interim[d] = s.shape[i]
        s = s.reshape(interim).expand(m.nshape).reshape(m.N, 1)
        # the graph divides the output by a per-output-channel scale: fold the reciprocal into
        # the weight scale (1/s computed once in float32, src/metaljax/qmm.py:1804-1827)
        scale_map = (1.0 / s.to(torch.float32)).expand(m.N, m.K)
        return qmm.build_pack(m, codes, scale_map, None, leaves)
    codes = full(m.codes)
    scale_map = full(m.scale)
    zero_map = None if m.zero is None else full(m.zero)
    return qmm.build_pack(m, codes, scale_map, zero_map, leaves)


def _resolve(interp, m, args):
    """The pack of match `m` for these argument buffers: the match's own recent packs, then the
    cross-program build cache, then a fresh build."""
    leaves = [args[i] for i in m.arg_indices]
    for pk in m.packs:
        if pk.matches(leaves):
            return pk
    if m.fp is None:
        m.fp = _fingerprint(m)
    key = (m.fp, _leaf_key(leaves))
    pk = _cached_build(key, leaves)
    if pk is not None:
        m.gs, m.bits, m.has_perm = pk.gs, pk.bits, pk.perm is not None
        m.nvals = len(pk.arrays())
        m.packs.insert(0, pk)
        qmm.STATS["cache_hits"] = qmm.STATS.get("cache_hits", 0) + 1
        return pk
    if m.packs:
        m.repacks += 1
    pk = _build(interp, m, args, leaves)
    if len(_BUILD_CACHE) >= _BUILD_CACHE_MAX:
        _BUILD_CACHE.pop(next(iter(_BUILD_CACHE)))
    _BUILD_CACHE[key] = ([weakref.ref(t) for t in leaves], pk)
    return pk


def prologue(interp, args) -> bool:
    """Resolve every live match against the argument buffers and lay the packed arrays out in
    `st.values` (`m.slot`, `m.nvals`). Returns True when the set of live rewrites changed
    (a match was disabled), so that a caller that caches a traced program can retrace."""
    st = analyze(interp)
    if not st.matches and not st.moe:
        return False
    from . import moe_recognizer
    changed = moe_recognizer.prologue(interp, st, args[0].device if args else None)
    vals = []
    for m in st.matches:
        if m.disabled:
            continue
        try:
            pk = _resolve(interp, m, args)
        except _Reject as e:
            m.disabled, changed = True, True
            qmm.STATS["rejected"] = qmm.STATS.get("rejected", 0) + 1
            interp.rejections.append((m.name, str(e)))
            continue
        m.slot = len(vals)
        arrays = pk.arrays()
        m.nvals = len(arrays)
        vals.extend(arrays)
    if changed:
        st.rebuild()
    st.values = vals
    return changed


# ---------------------------------------------------------------------------------------
# what a host that traces / compiles blocks asks the recognizer
# ---------------------------------------------------------------------------------------

_UNKNOWN_TRIP = 1024            # a loop whose bound is not static is charged this many bodies


def _scalar_constant(v):
    if v is None or v.op is None or v.op.name != "stablehlo.constant" or _prod(v.type.shape) != 1:
        return None
    try:
        return int(hlo._dense(v.op.text, v.type).reshape(()).item())
    except Exception:
        return None


def static_trip(loop):
    """Iterations of a counted `stablehlo.while` (carry i starts at a constant, the condition is
    `carry_i < constant`, the body returns `carry_i + 1`), or None (src/metaljax/ops/control.py:289-301)."""
    if loop.name != "stablehlo.while" or len(loop.regions) != 2:
        return None
    cond, body = loop.regions
    if len(cond.returns) != 1 or cond.returns[0].op is None:
        return None
    cmp_ = cond.returns[0].op
    if cmp_.name != "stablehlo.compare" or cmp_.attrs.get("direction") != "LT":
        return None
    counter, bound = cmp_.operands
    end = _scalar_constant(bound)
    if end is None or counter.op is not None or counter not in cond.args:
        return None
    i = cond.args.index(counter)
    start = _scalar_constant(loop.operands[i])
    nxt = body.returns[i].op if i < len(body.returns) else None
    if start is None or nxt is None or nxt.name != "stablehlo.add":
        return None
    a, b = nxt.operands
    step = _scalar_constant(b) if a is body.args[i] else _scalar_constant(a) if b is body.args[i] else None
    if step != 1:
        return None
    return max(end - start, 1)


def _state_of(interp):
    st = analyze(interp)
    return st if st is not None and (st.matches or st.moe) else None


def block_cost(interp, block) -> int:
    """Approximate op count of `block` when it is traced with loops unrolled: an op the rewrite
    absorbed costs nothing (it never runs), a fused root costs 2 units (one kernel plus the
    activation reshuffle), a loop its body times the trip count -- 1024 when the bound is not
    static, so that an unknown loop can never look cheap (src/metaljax/ops/control.py:251-312)."""
    st = _state_of(interp)
    cost = 0
    for op in block.ops:
        if st is not None:
            if id(op) in st.roots:
                cost += 2
                continue
            if id(op) in st.skip:
                continue
        cost += 1
        if op.name == "stablehlo.while" and len(op.regions) == 2:
            trip = static_trip(op)
            cost += (trip if trip is not None else _UNKNOWN_TRIP) * block_cost(interp, op.regions[1])
        else:
            for region in op.regions:
                cost += block_cost(interp, region)
    return cost


def value_bytes(v) -> int:
    t = v.type
    bits = 8 if t.el == "i1" else int(re.sub(r"\D", "", t.el) or 8)
    return (_prod(t.shape) * bits + 7) // 8


def op_bytes(op) -> int:
    """Declared result bytes; a splat constant is one element however big its type says
    (src/metaljax/interpreter.py:162-199)."""
    if op.name == "stablehlo.constant" and re.search(r"dense<\s*[-+0-9.eE xa-fA-Fin]+\s*>", op.text):
        return sum((value_bytes(r) // max(_prod(r.type.shape), 1)) or 1 for r in op.results)
    return sum(value_bytes(r) for r in op.results)


def block_bytes(interp, block) -> int:
    """Approximate device bytes materialized when `block` is traced: the same walk as
    `block_cost`, absorbed ops charged nothing, a fused root its result plus what the emission
    builds in the chain's place (`emit_bytes`: one copy of the activation; for an expert block
    the pair-space intermediates), loops unrolled (src/metaljax/ops/control.py:317-423)."""
    st = _state_of(interp)
    total = 0
    for op in block.ops:
        if st is not None:
            root = st.roots.get(id(op))
            if root is not None:
                total += op_bytes(op)
                try:
                    total += qmm.emit_bytes(root)
                except Exception:                                # an unsizable plan must not zero the block
                    pass
                continue
            if id(op) in st.skip:
                continue
        total += op_bytes(op)
        if op.name == "stablehlo.while" and len(op.regions) == 2:
            trip = static_trip(op)
            total += (trip if trip is not None else _UNKNOWN_TRIP) * block_bytes(interp, op.regions[1])
        else:
            for region in op.regions:
                total += block_bytes(interp, region)
    return total


def free_values(block):
    """Values `block` reads but neither defines nor takes as arguments, in first-use order
    (what a compiled body must be handed explicitly)."""
    own = set(block.args)
    free, seen = [], set()

    def rec(b):
        for op in b.ops:
            for v in op.operands:
                if v not in own and v not in seen:
                    seen.add(v)
                    free.append(v)
            for region in op.regions:
                own.update(region.args)
                rec(region)
            own.update(op.results)
    rec(block)
    return free


def captures(interp, env, free):
    """The buffers a compiled body takes besides its carries: its free values, then the packed
    arrays of every live rewrite -- those travel as explicit inputs so that a repack reaches a
    body that was already compiled. A free value the rewrite absorbed in the enclosing block has
    no buffer; nothing in the body can read it (its consumers are absorbed too), so a stand-in
    keeps the body's arity stable (src/metaljax/ops/control.py:700-725)."""
    st = interp._qmm
    skipped = set()
    if st is not None and (st.matches or st.moe):
        skipped = st.skip
    caps = []
    for v in free:
        t = env.get(v)
        if t is None and v.op is not None and id(v.op) in skipped:
            t = _ABSORBED
        elif t is None:
            t = env[v]                                           # missing for another reason: raise
        caps.append(t)
    caps.extend(qmm.values(interp))
    return caps


_ABSORBED = torch.zeros((), dtype=torch.uint8)


# ---------------------------------------------------------------------------------------
# the host
# ---------------------------------------------------------------------------------------


class Interpreter:
    """A parsed program with its recognizer state. `execute(args)` returns the function's
    results; with `fused=False` every op runs literally."""

    def __init__(self, text_or_func):
        self.func = hlo.parse(text_or_func) if isinstance(text_or_func, str) else text_or_func
        self._qmm = None
        self.rejections = []
        self.fused_calls = 0

    def execute(self, args, fused=True):
        fn = self.func
        if not fused:
            return hlo.evaluate(fn, args)
        prologue(self, args)
        st = self._qmm
        env = dict(zip(fn.args, args))

        def hook(op, env):
            key = id(op)
            root = st.roots.get(key)
            if root is not None:
                from . import moe_recognizer
                fused = (moe_recognizer.emit if isinstance(root, moe_recognizer.ExpertBlock) else qmm.emit)
                for r, t in zip(op.results, fused(self, root, env)):
                    env[r] = t
                self.fused_calls += 1
                return True
            return key in st.skip

        hlo.run_block(fn, env, hook, args[0].device if args else None)
        return [env[v] for v in fn.returns]
