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


def _build(interp, m, args, leaves):
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
    if not st.matches:
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
