"""Recognizer that maps a DENSE mixture-of-experts dispatch onto the gathered expert block.

A layer written against `jax.numpy` runs every expert for every token and lets routing weights
that are zero off the top-k selection null the rest (src/metaljax/moe.py:1-60). This module
recognizes that structure on the IR of `metaljax_b200/hlo.py` and replaces the dense region with
`moe.moe_experts` (pairs sorted by expert, three grouped ragged products on the packed expert
weights, the routed K-sum):

  root     reduce(add over the expert axis)( multiply(Y, broadcast(S)) )      (:859-1073)
  router   S = reduce(add over k)( one_hot(indices, E) * broadcast(w) ) with `one_hot` matched
           down to `compare EQ (broadcast(indices), iota)`, `indices` and the values behind `w`
           coming from one `chlo.top_k`; so S[t, e] = sum_k [indices[t, k] == e] * w[t, k] is an
           identity, not a guess                                                  (:249-442)
  verify   the router tail from `top_k` down to S is evaluated on synthetic logits in the
           prologue and compared, exactly, against `w` scattered at `indices`    (:1112-1191)
  plan     Y must be the SwiGLU expert block on weights the quantized-matmul recognizer has
           already matched: down( silu(gate(x)) * up(x) ), gate / up being dots of the tokens
           against [E, ffn, d] weights (expert axis leading the output features) and down a dot
           batched over the expert axis. The reference plans arbitrary element-wise regions in
           pair space (`_Planner`, :450-810); this build plans that one block, which is the
           block every model in the reference's own benchmarks has, and rejects the rest.

Anything not understood rejects the match and the dense region runs as before. The three
quantized matches the block adopts are marked absorbed (they are no longer roots of their own).
"""

from __future__ import annotations

import torch

from . import hlo, moe, qmm
from .qmm import _Reject

STATS = {"recognized": 0, "verified": 0, "rejected": 0}
VERIFY_DRAWS = 3


class Router:
    """`S[t, e] = sum_k [indices[t, k] == e] * w[t, k]`, with the values it was matched from."""

    __slots__ = ("S", "top_k", "indices", "weights", "T", "K", "E", "t_axis", "e_axis", "ops")

    def __init__(self):
        self.ops = {}


def _peel(v, names=("stablehlo.convert", "stablehlo.broadcast_in_dim")):
    """Peel converts and broadcasts: (base, dims) with dims[j] = the axis of `v` that base axis j
    lands in."""
    dims = list(range(len(v.type.shape)))
    while v.op is not None and v.op.name in names:
        if v.op.name == "stablehlo.broadcast_in_dim":
            dims = [dims[d] for d in v.op.attrs["dims"]]
        v = v.op.operands[0]
    return v, dims


def _zero_sum_axis(op):
    """The reduced axis of a `reduce(add, init = 0)` over one axis; `_Reject` otherwise."""
    if op is None or op.name != "stablehlo.reduce" or op.attrs.get("applies") != "stablehlo.add":
        raise _Reject("not a sum")
    if len(op.attrs["dims"]) != 1:
        raise _Reject("the sum spans more than one axis")
    init = op.operands[1]
    if init.op is None or init.op.name != "stablehlo.constant":
        raise _Reject("the sum does not start at a constant")
    if float(hlo._dense(init.op.text, init.type).reshape(-1)[0]) != 0.0:
        raise _Reject("the sum does not start at zero")
    return op.attrs["dims"][0]


def match_router(S) -> Router:
    """Prove that `S` is a top-k routing matrix (src/metaljax/moe.py:249-442)."""
    red = S.op
    k_axis = _zero_sum_axis(red)
    mul = red.operands[0].op
    if mul is None or mul.name != "stablehlo.multiply":
        raise _Reject("the summand is not a product")
    r = Router()
    r.S = S
    for hot_side in (0, 1):
        hot, _ = _peel(mul.operands[hot_side], ("stablehlo.convert",))
        cmp_op = hot.op
        if cmp_op is None or cmp_op.name != "stablehlo.compare" or cmp_op.attrs.get("direction") != "EQ":
            continue
        for idx_side in (0, 1):
            idx, idx_dims = _peel(cmp_op.operands[idx_side])
            iota, iota_dims = _peel(cmp_op.operands[1 - idx_side])
            if iota.op is None or iota.op.name != "stablehlo.iota":
                continue
            if idx.op is None or idx.op.name != "chlo.top_k" or idx.index != 1:
                continue
            e_axis = iota_dims[iota.op.attrs["dim"]]
            w, w_dims = _peel(mul.operands[1 - hot_side], ("stablehlo.broadcast_in_dim",))
            if len(idx.type.shape) != 2 or tuple(w.type.shape) != tuple(idx.type.shape) or w_dims != idx_dims:
                raise _Reject("weights and indices are not laid out alike")
            t_axis, kk = idx_dims
            if kk != k_axis or e_axis in (t_axis, kk):
                raise _Reject("the sum is not over the selection axis")
            # w may depend on nothing but the selected values (and constants)
            seen, stack = set(), [w]
            while stack:
                cur = stack.pop()
                if cur in seen:
                    continue
                seen.add(cur)
                if cur.op is None:
                    raise _Reject("routing weights depend on something other than the selection")
                if cur.op is idx.op:
                    continue
                if cur.op.opaque or cur.op.regions:
                    raise _Reject(f"routing weights go through {cur.op.name}")
                stack.extend(cur.op.operands)
            r.top_k, r.indices, r.weights = idx.op, idx, w
            r.T, r.K = idx.type.shape
            r.E = mul.results[0].type.shape[e_axis]
            if idx.op.operands[0].type.shape != (r.T, r.E):
                raise _Reject("top_k is not taken over the expert axis of [tokens, experts] logits")
            out_axes = [a for a in range(len(mul.results[0].type.shape)) if a != k_axis]
            r.t_axis, r.e_axis = out_axes.index(t_axis), out_axes.index(e_axis)
            return r
    raise _Reject("no one-hot of top-k indices in the product")


def verify_router(r: Router, device=None, draws=VERIFY_DRAWS) -> bool:
    """Evaluate the router tail on synthetic logits and compare S, exactly, with `w` scattered at
    `indices`, a few draws (src/metaljax/moe.py:1112-1153). The draws are the reference's: one
    generator seeded 20260803, standard normal `[T, E]`; every draw after the first is rounded to
    halves, because exact ties are where a top-k and a hand-rolled scatter would most easily
    disagree (`:1128-1131`). A token with more than K nonzero routing weights also fails the
    match (`:1144-1152`). Fails closed: an axis misread, an op the evaluator lacks -> False."""
    import numpy as np
    logits = r.top_k.operands[0]
    rng = np.random.default_rng(20260803)
    k = r.indices.type.shape[-1]
    for d in range(max(1, draws)):
        raw = rng.standard_normal(tuple(logits.type.shape)).astype(np.float32)
        if d:
            raw = np.round(raw * 2.0) / 2.0
        draw = torch.from_numpy(raw).to(logits.type.dtype).to(device)
        env = {logits: draw}
        try:
            S = hlo.evaluate_value(r.S, env)
            idx = env[r.indices].to(torch.int64)
            w = hlo.evaluate_value(r.weights, env)
        except (KeyError, NotImplementedError):
            return False
        got = S if r.t_axis < r.e_axis else S.transpose(0, 1)
        if tuple(got.shape) != (r.T, r.E):
            return False
        want = torch.zeros((r.T, r.E), dtype=got.dtype, device=S.device)
        want.index_put_((torch.arange(r.T, device=S.device)[:, None].expand_as(idx), idx), w.to(got.dtype), accumulate=True)
        if not torch.equal(got, want):
            return False
        if int((got != 0).sum(dim=1).max().item()) > k:
            return False
    STATS["verified"] += 1
    return True


class ExpertBlock(moe.Match):
    """A recognized dense expert block (what `emit` reads)."""

    __slots__ = ("root", "router", "x", "gate", "up", "down", "out_shape", "ops", "name", "verified")

    def __init__(self):
        super().__init__()
        self.verified = False

    def matches(self):
        """The quantized / float matches the block runs on (no longer roots of their own)."""
        return (self.gate, self.up, self.down)


class ExpertRegion(ExpertBlock):
    """A dense expert region planned node by node in pair space (`pair_plan`): any element-wise
    work between any number of per-expert dots. `y` is the node of the weighted value, `dots` the
    matches its dots run on."""

    __slots__ = ("planner", "y", "dots", "e_axis", "t_axis", "reads")

    def matches(self):
        return tuple(self.dots)


def _float_match(st, dot):
    """A dot whose weight operand is a FLOAT array computed from `@main`'s arguments alone (an
    unquantized expert weight, possibly converted / transposed on the way): the dimension
    bookkeeping of a quantized match with nothing to dequantize. The reference plans these onto
    `mx.gather_mm` (src/metaljax/moe.py:1324-1336). Cached per dot in `st`."""
    from . import recognizer
    cache = st.floats
    if id(dot) in cache:
        return cache[id(dot)]
    last = None
    for qside in (1, 0):
        m = qmm.Match()
        m.mode = "float"
        w = dot.operands[qside]
        try:
            if w.type.el not in ("bf16", "f16") or dot.operands[1 - qside].type.el != w.type.el:
                raise _Reject("float experts are taken in the activations' 16-bit type only")
            recognizer._finish(st.fn, m, dot, [w], dot, qside=qside)
            if not m.arg_indices:
                raise _Reject("the weight operand does not come from an argument")
        except _Reject as why:
            last = why
            continue
        m.codes = w
        cache[id(dot)] = m
        return m
    raise last or _Reject("no float expert weight under this dot")


def _find_match(st, value, through=("stablehlo.transpose", "stablehlo.reshape", "stablehlo.convert"), floats=False):
    """The quantized match whose root produces `value` (looking through shape ops); with
    `floats`, a plain dot over a float expert weight counts too."""
    v = value
    while v.op is not None and v.op.name in through:
        v = v.op.operands[0]
    if v.op is None:
        raise _Reject("expert activations do not come from a recognized quantized dot")
    for m in st.matches:
        if not m.disabled and m.root is v.op:
            return m
    if floats and v.op.name == "stablehlo.dot_general":
        return _float_match(st, v.op)
    raise _Reject("expert activations do not come from a recognized quantized dot")


def _plan_swiglu(st, Y, r: Router) -> ExpertBlock:
    """Y = down( silu(gate(x)) * up(x) ) on three matches of the quantized recognizer."""
    down = _find_match(st, Y, floats=True)
    if down.bshape != [r.E] or down.M != r.T or down.swapped or down.mode not in ("affine", "mxfp4", "float"):
        raise _Reject("the last expert dot is not batched over the experts with the tokens as rows")
    act = down.lhs
    while act.op is not None and act.op.name in ("stablehlo.transpose", "stablehlo.reshape", "stablehlo.convert"):
        act = act.op.operands[0]
    prod = act.op
    if prod is None or prod.name != "stablehlo.multiply":
        raise _Reject("the expert activation is not a gated product")

    def silu_of(v):
        """g when v = g * logistic(g) (either order), else None."""
        o = v.op
        if o is None or o.name != "stablehlo.multiply":
            return None
        for i in (0, 1):
            lg = o.operands[i].op
            if lg is not None and lg.name == "stablehlo.logistic" and lg.operands[0] is o.operands[1 - i]:
                return o.operands[1 - i]
        return None

    for i in (0, 1):
        g = silu_of(prod.operands[i])
        if g is None:
            continue
        gate, up = _find_match(st, g, floats=True), _find_match(st, prod.operands[1 - i], floats=True)
        if len({m.mode == "float" for m in (gate, up, down)}) != 1:
            raise _Reject("float and quantized projections in one expert block")
        for m in (gate, up):
            if m.bshape or m.swapped or m.M != r.T or len(m.nshape) != 2 or m.nshape[0] != r.E:
                raise _Reject("an expert projection does not lead its output features with the expert axis")
        if gate.lhs is not up.lhs or gate.nshape != up.nshape or gate.K != up.K:
            raise _Reject("gate and up do not read the same tokens")
        if down.K != gate.nshape[1] or down.N != gate.K:
            raise _Reject("the down projection does not close the block")
        b = ExpertBlock()
        b.router, b.x, b.gate, b.up, b.down = r, gate.lhs, gate, up, down
        b.T, b.K, b.E, b.P = r.T, r.K, r.E, r.T * r.K
        return b
    raise _Reject("no silu(gate) * up under the last expert dot")


def _plan_region(st, Y, r: Router, e_axis, t_axis) -> ExpertRegion:
    """The general plan: whatever element-wise region and per-expert dots produce Y
    (src/metaljax/moe.py:450-810)."""
    from . import pair_plan

    def find(dot):
        return _float_match(st, dot)

    planner = pair_plan.Planner(st, r.E, r.T, find)
    y = planner.plan(Y, e_axis, t_axis)
    if not planner.matches:
        raise _Reject("no per-expert dot in the region")
    modes = {m.mode == "float" for m in planner.matches}
    b = ExpertRegion()
    b.router, b.planner, b.y, b.dots = r, planner, y, list(dict.fromkeys(planner.matches))
    b.e_axis, b.t_axis = e_axis, t_axis
    b.x = b.gate = b.up = b.down = None
    b.reads = tuple(dict.fromkeys(planner.reads))
    b.T, b.K, b.E, b.P = r.T, r.K, r.E, r.T * r.K
    b.bytes = planner.bytes(b.P)
    del modes
    return b


def analyze(interp, st) -> None:
    """Find dense expert blocks on top of the quantized matches in `st` (the reference chains
    its recognizers the same way, src/metaljax/qmm.py:1085-1091). Never raises."""
    fn = interp.func
    st.fn = fn
    try:
        for op in fn.walk():
            if op.name != "stablehlo.reduce" or op.attrs.get("applies") != "stablehlo.add":
                continue
            try:
                e_axis = _zero_sum_axis(op)
                mul = op.operands[0].op
                if mul is None or mul.name != "stablehlo.multiply":
                    raise _Reject("the summand is not a product")
                block = None
                for s_side in (0, 1):
                    S, s_dims = _peel(mul.operands[s_side])
                    if S.op is None or S.op.name != "stablehlo.reduce":
                        continue
                    r = match_router(S)
                    if s_dims[r.e_axis] != e_axis:
                        raise _Reject("the outer sum is not over the expert axis")
                    Y = mul.operands[1 - s_side]
                    try:
                        block = _plan_swiglu(st, Y, r)             # the one-launch-per-projection block
                    except _Reject:
                        block = _plan_region(st, Y, r, e_axis, s_dims[r.t_axis])
                    break
                if block is None:
                    continue
                block.root, block.key = op, id(op)
                block.out_shape = list(op.results[0].type.shape)
                block.out_dtype = op.results[0].type.dtype
                block.name = f"moe {block.T}x{block.K}/{block.E}"
                # The region: the three projections with everything they absorbed, the
                # element-wise ops between them, the weighting product -- and whatever only
                # fed those (the one-hot, S and its broadcast are dead once the block is
                # gathered; src/metaljax/moe.py:870-930). The router's own outputs, which the
                # gathered block reads, and everything they are computed from stay.
                needed = set()
                stack = [r.indices, r.weights]
                while stack:
                    v = stack.pop()
                    if v.op is None or id(v.op) in needed:
                        continue
                    needed.add(id(v.op))
                    stack.extend(v.op.operands)
                skip = {id(mul): mul}
                roots = {id(m.root) for m in block.matches()}
                for m in block.matches():
                    skip.update(m.ops)
                    skip[id(m.root)] = m.root
                if isinstance(block, ExpertRegion):
                    skip.update(block.planner.region)              # exactly the ops the plan replaces
                else:
                    stack = [mul.operands[1 - s_side]]             # Y back to the projections
                    while stack:
                        v = stack.pop()
                        if v is block.x or v.op is None or id(v.op) in skip:
                            continue
                        skip[id(v.op)] = v.op
                        stack.extend(v.op.operands)
                grew = True
                while grew:                                         # dead sweep
                    grew = False
                    for o in list(skip.values()):
                        for v in o.operands:
                            p = v.op
                            if p is None or id(p) in skip or id(p) in needed or p.regions and p.name != "stablehlo.reduce":
                                continue
                            if all(id(u) in skip or u is op for res in p.results for u, _ in res.uses):
                                skip[id(p)] = p
                                grew = True
                changed = True
                while changed:                                      # nothing read from outside
                    changed = False
                    for key, o in list(skip.items()):
                        if any(id(u) not in skip and u is not op for res in o.results for u, _ in res.uses):
                            del skip[key]
                            changed = True
                if not roots <= set(skip) or id(mul) not in skip:
                    raise _Reject("a value of the expert region is also read outside it")
                block.ops = skip
                block.skip_keys = tuple(skip)
                for m in block.matches():
                    m.absorbed = True
                st.moe.append(block)
                STATS["recognized"] += 1
            except _Reject:
                STATS["rejected"] += 1
    except Exception:                                            # analysis must never break a program
        pass


def prologue(interp, st, device=None) -> bool:
    """Numeric check of every block's router, once; a failure disables the block and releases
    its three projections to be fused on their own."""
    changed = False
    for b in st.moe:
        if b.disabled or b.verified:
            continue
        if verify_router(b.router, device):
            b.verified = True
            continue
        b.disabled = True
        for m in b.matches():
            m.absorbed = False
        changed = True
    return changed


def _expert_pack(interp, m, E):
    """The packed arrays of match `m` as per-expert stacks `[E, rows, ...]`."""
    vals = qmm.pack_arrays(interp, m)
    w, s = vals[0], vals[1]
    b = vals[2] if m.mode == "affine" else None
    if m.has_perm:
        raise _Reject("a permuted contraction axis inside an expert block")

    def stack(t):
        return None if t is None else t.reshape(E, -1, t.shape[-1])

    return stack(w), stack(s), stack(b)


def _float_weight(interp, m, env, E):
    """The float expert weight of `m` as `[E, rows, K]`, contiguous: evaluated from the argument
    buffers once and kept while those buffers are the same objects (like a pack)."""
    from . import recognizer
    fn = interp.func
    leaves = [env[fn.args[i]] for i in m.arg_indices]
    for pk in m.packs:
        if pk.matches(leaves):
            return pk.w
    t = hlo.evaluate_value(m.codes, {a: env[a] for a in fn.args if a in env})
    w = recognizer._to_nk(recognizer._replay(t, m.post), m).contiguous()
    w = w.reshape(E, -1, w.shape[-1])
    pk = qmm._Pack(leaves, w, None, None, None, 0, 16, "float")
    m.packs.insert(0, pk)
    del m.packs[2:]
    return w


def emit(interp, b: ExpertBlock, env):
    """The gathered expert block in place of the dense region."""
    r = b.router
    idx = hlo.evaluate_value(r.indices, env).to(torch.int64)
    wts = hlo.evaluate_value(r.weights, env)
    if isinstance(b, ExpertRegion):
        return [_emit_region(interp, b, env, idx, wts)]
    x = env[b.x]
    if list(b.gate.lperm) != list(range(x.dim())):
        x = x.permute(*b.gate.lperm)
    x = x.reshape(b.T, b.gate.K)
    if b.gate.mode == "float":
        y = moe.moe_experts_float(x.to(b.out_dtype) if x.dtype != b.out_dtype else x, idx, wts,
                                  _float_weight(interp, b.gate, env, b.E), _float_weight(interp, b.up, env, b.E),
                                  _float_weight(interp, b.down, env, b.E))
        return [y.reshape(b.out_shape).to(b.out_dtype)]
    kw = dict(group_size=b.gate.gs, bits=b.gate.bits, mode=b.gate.mode)
    if (b.up.gs, b.up.bits, b.down.gs, b.down.bits) != (b.gate.gs, b.gate.bits, b.gate.gs, b.gate.bits):
        raise _Reject("the three projections are packed differently")
    y = moe.moe_experts(x.to(b.out_dtype) if x.dtype != b.out_dtype else x, idx, wts,
                        _expert_pack(interp, b.gate, b.E), _expert_pack(interp, b.up, b.E),
                        _expert_pack(interp, b.down, b.E), **kw)
    return [y.reshape(b.out_shape).to(b.out_dtype)]


def _emit_region(interp, b: ExpertRegion, env, idx, wts, ragged=None):
    """A planned region over the routed pairs: sort the pairs by expert, evaluate the plan's nodes
    on `[P, ...]` arrays, weight and add every token's K results."""
    from . import pair_plan
    order, tok, sizes = moe.sort_pairs(idx, b.E)
    eor = torch.repeat_interleave(torch.arange(b.E, device=idx.device), sizes.to(torch.int64), output_size=b.P)

    def weight_of(m):
        return _float_weight(interp, m, env, b.E) if m.mode == "float" else _expert_pack(interp, m, b.E)

    vals = pair_plan.evaluate(b.planner.order, env, (tok, eor, sizes), b.E, weight_of, ragged)
    y = vals[id(b.y)]
    if not b.y.paired or y.shape[0] != b.P:
        raise _Reject("the weighted value has no pair axis")
    trailing = b.y.trailing
    out = pair_plan.weighted_sum(y.reshape([b.P] + trailing), order, wts, b.T, b.K, b.out_dtype)
    out = out.reshape([b.T] + trailing)
    # the root's result is Y's shape without the expert axis: put the token axis where it belongs
    t_out = b.t_axis - (1 if b.e_axis < b.t_axis else 0)
    if t_out:
        out = out.movedim(0, t_out)
    return out.reshape(b.out_shape).to(b.out_dtype)
