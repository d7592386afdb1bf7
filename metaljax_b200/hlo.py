"""A small StableHLO front end: text as jax prints it -> an in-memory IR, plus a literal
evaluator on torch tensors.

The reference's recognizers walk `jaxlib.mlir` objects (`ir.Value`, `ir.OpResult`,
`ir.BlockArgument`, `op.operands/.results/.attributes`, `ir.RankedTensorType`;
src/metaljax/interpreter.py:325-395, src/metaljax/qmm.py:472-500). `jaxlib` is not a dependency
here, so this module provides the same surface for the part of the language the quantized-matmul
recognizer meets: straight-line `func.func @main` bodies of element-wise, shape, constant,
gather and dot ops. Ops with regions (while, reduce, ...) are parsed as opaque: the recognizer
refuses to look through them (as the reference does, src/metaljax/qmm.py:710-711) and the
evaluator refuses to run them.

The evaluator exists for two callers: the recognizer's pack prologue, which evaluates the
codes / scale / zero-point subtrees once on concrete buffers (src/metaljax/qmm.py:1130-1176),
and tests, which compare a fused program with its literal evaluation.
"""

from __future__ import annotations

import ast
import re

import torch

# ---------------------------------------------------------------------------------------
# IR
# ---------------------------------------------------------------------------------------

_DTYPES = {
    "f64": torch.float64, "f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16,
    "i1": torch.bool, "i8": torch.int8, "i16": torch.int16, "i32": torch.int32, "i64": torch.int64,
    "ui8": torch.uint8, "i4": torch.int8, "ui4": torch.uint8,
}
FLOAT_ELS = ("f64", "f32", "f16", "bf16")
INT_ELS = ("i4", "ui4", "i8", "ui8", "i16", "i32", "i64")


class TensorType:
    __slots__ = ("shape", "el")

    def __init__(self, shape, el):
        self.shape, self.el = tuple(shape), el

    @property
    def dtype(self):
        try:
            return _DTYPES[self.el]
        except KeyError:
            raise NotImplementedError(f"element type {self.el}") from None

    def __repr__(self):
        return "tensor<" + "x".join([*map(str, self.shape), self.el]) + ">"

    def __eq__(self, other):
        return isinstance(other, TensorType) and (self.shape, self.el) == (other.shape, other.el)

    def __hash__(self):
        return hash((self.shape, self.el))


class Value:
    """An SSA value: a function argument (`op is None`, `index` = argument number) or result
    `index` of `op`. Hashable by identity; `uses` lists the `(op, operand position)` pairs."""

    __slots__ = ("name", "type", "op", "index", "uses", "block")

    def __init__(self, name, type_, op, index, block=None):
        self.name, self.type, self.op, self.index = name, type_, op, index
        self.uses = []
        self.block = block           # the Block whose argument this is (None for op results)

    @property
    def is_argument(self):
        return self.op is None

    @property
    def is_main_argument(self):
        return self.op is None and (self.block is None or self.block.owner is None)

    def __repr__(self):
        return f"%{self.name}: {self.type}"


class Op:
    __slots__ = ("name", "operands", "results", "attrs", "text", "opaque", "position", "regions")

    def __init__(self, name, operands, attrs, text, opaque=False):
        self.name, self.operands, self.attrs, self.text, self.opaque = name, operands, attrs, text, opaque
        self.results = []
        self.position = -1
        self.regions = []            # Blocks (stablehlo.while: [cond, body]); other region ops are opaque

    def __repr__(self):
        return f"<{self.name} -> {[r.name for r in self.results]}>"


class Block:
    """Arguments, ops in program order and the values its terminator returns. `owner` is the op
    whose region this is (None for a function body)."""

    def __init__(self, owner=None):
        self.owner = owner
        self.args, self.ops, self.returns = [], [], []
        self.return_op = None


class Func(Block):
    """`func.func @main`: a Block plus the argument numbers the caller donates
    (`tf.aliasing_output` / `jax.buffer_donor`)."""

    def __init__(self, name):
        super().__init__(None)
        self.name = name
        self.donated = set()

    def walk(self):
        """Every op, those inside while regions included, in program order."""
        def rec(block):
            for op in block.ops:
                yield op
                for region in op.regions:
                    yield from rec(region)
        return rec(self)


def invariant_init(v):
    """For an argument of a while region that the loop hands on unchanged (jax lowers a loop's
    closed-over weights as such carries, src/metaljax/qmm.py:714-740): the while's initial
    operand. None when `v` is anything else."""
    if v.op is not None or v.block is None or v.block.owner is None:
        return None
    loop = v.block.owner
    if loop.name != "stablehlo.while" or len(loop.regions) != 2:
        return None
    body = loop.regions[1]
    if v.index >= len(body.returns) or body.returns[v.index] is not body.args[v.index]:
        return None
    return loop.operands[v.index]


# ---------------------------------------------------------------------------------------
# parsing
# ---------------------------------------------------------------------------------------

_TYPE_RE = re.compile(r"tensor<([^<>]*)>")


def parse_type(text: str) -> TensorType:
    m = _TYPE_RE.search(text)
    if not m:
        raise ValueError(f"not a ranked tensor type: {text!r}")
    parts = m.group(1).split("x")
    return TensorType([int(p) for p in parts[:-1]], parts[-1].strip())


def _top_level_split(text, sep):
    """Split at `sep` outside (), [], {} and <> (the `>` of `->` does not close anything)."""
    out, depth, start, i = [], 0, 0, 0
    while i < len(text):
        c = text[i]
        if text.startswith("->", i):
            i += 2
            continue
        if c in "([{<":
            depth += 1
        elif c in ")]}>":
            depth -= 1
        elif depth == 0 and text.startswith(sep, i):
            out.append(text[start:i])
            start = i + len(sep)
            i += len(sep)
            continue
        i += 1
    out.append(text[start:])
    return out


def _int_list(text):
    text = text.strip()
    return [] if text in ("", "[]") else [int(t) for t in text.strip("[]").split(",")]


def _attr(text, key, default=None):
    m = re.search(r"\b" + re.escape(key) + r"\s*=\s*(\[[^\]]*\]|array<i64(?::[^>]*)?>|-?\d+)", text)
    if not m:
        return default
    v = m.group(1)
    if v.startswith("array<i64"):
        body = v[len("array<i64"):-1].lstrip(":")
        return _int_list("[" + body + "]")
    return _int_list(v) if v.startswith("[") else int(v)


def _pair(text, key):
    m = re.search(r"\b" + key + r"\s*=\s*(\[[^\]]*\])\s*x\s*(\[[^\]]*\])", text)
    return ([], []) if not m else (_int_list(m.group(1)), _int_list(m.group(2)))


def _dense(text, type_):
    """The payload of `dense<...>` as a tensor of `type_`."""
    m = re.search(r"dense<(.*)>\s*$", text.strip(), re.S)
    if not m:
        raise ValueError(f"unsupported constant: {text[:60]!r}")
    body = m.group(1).strip()
    if body.startswith('"0x'):
        raw = bytes.fromhex(body.strip('"')[2:])
        return torch.frombuffer(bytearray(raw), dtype=type_.dtype).reshape(type_.shape).clone()
    body = body.replace("true", "True").replace("false", "False")
    body = re.sub(r"(?<![\w.])(-?)(nan|inf)\b", lambda mm: f'"{mm.group(1)}{mm.group(2).lower()}"', body, flags=re.I)

    def number(x):
        if isinstance(x, (list, tuple)):
            return [number(y) for y in x]
        return float(x) if isinstance(x, str) else x

    data = number(ast.literal_eval(body))
    t = torch.tensor(data, dtype=torch.float64 if type_.el in FLOAT_ELS else torch.int64)
    return t.to(type_.dtype).expand(type_.shape).contiguous() if t.dim() == 0 else t.to(type_.dtype).reshape(type_.shape)


def _signature(head):
    """`(name, type, attribute text)` of every argument in a `func.func` header line."""
    sig = head[head.index("(") + 1:]
    depth, end = 1, 0
    for end, c in enumerate(sig):
        depth += c == "("
        depth -= c == ")"
        if depth == 0:
            break
    out = []
    for piece in (p for p in _top_level_split(sig[:end], ",") if p.strip()):
        m = re.match(r"\s*%([\w.$-]+)\s*:\s*(tensor<[^>]*>)(.*)", piece, re.S)
        if not m:
            raise ValueError(f"cannot parse argument {piece!r}")
        out.append((m.group(1), parse_type(m.group(2)), m.group(3)))
    return out


def parse(text: str) -> Func:
    """The first `func.func ... @main` (or the first function) of a module. Calls of the module's
    other functions (`func.call @callee(...)`, `stablehlo.composite ... {decomposition = @callee}`:
    jax outlines helpers such as `take` and `dynamic_index_in_dim` as private functions) are
    inlined where they stand, so the recognizer
    sees one flat graph, as the reference does by following callees (src/metaljax/qmm.py:743-777)."""
    lines = text.splitlines()
    heads = [i for i, ln in enumerate(lines) if re.search(r"\bfunc\.func\b", ln)]
    start = next((i for i in heads if "@main" in lines[i]), None)
    if start is None:
        start = heads[0] if heads else None
    if start is None:
        raise ValueError("no func.func in the module")
    funcs = {}
    for i in heads:
        if i != start:
            m = re.search(r"@([\w.$-]+)", lines[i])
            if m:
                funcs[m.group(1)] = i
    head = lines[start]
    fn = Func(re.search(r"@([\w.$-]+)", head).group(1))
    env = {}
    for i, (name, type_, attrs) in enumerate(_signature(head)):
        v = Value(name, type_, None, i)
        if "tf.aliasing_output" in attrs or "jax.buffer_donor" in attrs:
            fn.donated.add(i)
        fn.args.append(v)
        env[v.name] = v
        v.block = fn
    counter = [0, funcs, 0]          # next op position, the module's other functions, inlining depth
    _parse_block(lines, start + 1, env, fn, counter)
    return fn


def _inline_call(lines, callee_line, operands, block, counter):
    """The body of the function whose header is `lines[callee_line]`, parsed into `block` with its
    arguments bound to `operands`; returns the Values it returns."""
    if counter[2] >= 32:
        raise ValueError("function calls nest too deeply (recursion?)")
    sig = _signature(lines[callee_line])
    if len(sig) != len(operands):
        raise ValueError(f"call with {len(operands)} operands of a function of {len(sig)}")
    cenv = {name: v for (name, _, _), v in zip(sig, operands)}
    tmp = Block(block.owner)
    counter[2] += 1
    _parse_block(lines, callee_line + 1, cenv, tmp, counter)
    counter[2] -= 1
    block.ops.extend(tmp.ops)
    for k, v in enumerate(tmp.returns):                            # the callee's return is no use of its own
        v.uses[:] = [u for u in v.uses if u[0] is not tmp.return_op]
    return tmp.returns


def _parse_block(lines, i, env, block, counter):
    """Ops of one block, from line `i` up to (and including) the line that closes it; returns
    the index after that line. `env` maps names to Values (a region sees its parents' names)."""

    def lookup(tok):
        name, _, idx = tok.partition("#")
        v = env[name]
        return v[int(idx)] if isinstance(v, list) else v

    while i < len(lines):
        ln = lines[i].strip()
        i += 1
        if not ln or ln.startswith("//"):
            continue
        if ln.startswith("}"):
            break
        m = re.match(r"(?:(%[\w.$-]+)(?::(\d+))?\s*=\s*)?\"?([\w.]+)\"?\s*(.*)", ln, re.S)
        res_name, res_count, name, rest = m.group(1), m.group(2), m.group(3), m.group(4)
        if name in ("return", "func.return", "stablehlo.return"):
            block.returns = [lookup(t[1:]) for t in re.findall(r"%[\w.$#-]+", rest.split(" : ")[0])]
            block.return_op = Op("func.return" if block.owner is None else "stablehlo.return", block.returns, {}, "")
            for k, v in enumerate(block.returns):
                v.uses.append((block.return_op, k))                # a use like any other
            continue
        if name == "stablehlo.while":
            i = _parse_while(lines, i, ln, res_name, res_count, rest, env, block, counter, lookup)
            continue
        if name == "reducer" and not res_name:
            # the region of the reduce printed on the line before (its multi-result form):
            # swallowed, and that op stays opaque
            depth = ln.count("{") - ln.count("}")
            while depth > 0 and i < len(lines):
                depth += lines[i].count("{") - lines[i].count("}")
                i += 1
            if block.ops:
                block.ops[-1].opaque = True
            continue
        if name in ("func.call", "call", "stablehlo.composite") and len(counter) > 1:
            # `call @f(%a, %b)`; `stablehlo.composite "name" %a, %b {..., decomposition = @f}`
            composite = name == "stablehlo.composite"
            callee = re.search(r"decomposition\s*=\s*@([\w.$-]+)" if composite else r"@([\w.$-]+)", rest)
            target = counter[1].get(callee.group(1)) if callee else None
            if target is not None:
                inside = rest.split("{")[0] if composite else rest[rest.index("(") + 1: rest.index(")")]
                outs = _inline_call(lines, target, [lookup(t[1:]) for t in re.findall(r"%[\w.$#-]+", inside)], block, counter)
                if res_name:
                    env[res_name[1:]] = list(outs) if res_count else outs[0]
                continue
        # any other op with regions: swallow lines until its braces balance, keep it opaque
        body = ln
        if ln.endswith("{") or ln.endswith("({"):
            depth = ln.count("{") - ln.count("}")
            while depth > 0 and i < len(lines):
                nxt = lines[i]
                i += 1
                depth += nxt.count("{") - nxt.count("}")
                body += "\n" + nxt
            rest = body[body.index(name) + len(name):].lstrip('"').lstrip()
        opaque = "\n" in body
        parts = _top_level_split(rest, " : ")
        pre, sig_text = (" : ".join(parts[:-1]), parts[-1]) if len(parts) > 1 else (rest, "")
        operand_text = pre if not opaque else pre.split("\n")[0]
        operands = [lookup(t[1:]) for t in re.findall(r"%[\w.$#-]+", operand_text)]
        types = [parse_type(t) for t in re.findall(r"tensor<[^<>]*>", sig_text.split("\n")[-1] if opaque else sig_text)]
        if "->" in sig_text:
            n_res = int(res_count) if res_count else 1
            result_types = types[-n_res:] if n_res else []
        elif name == "stablehlo.select" and len(types) == 2:
            result_types = [types[1]]
        else:
            result_types = types[-1:] if res_name else []
        op = Op(name, operands, {}, pre, opaque)
        _register(op, res_name, res_count, result_types, env, block, counter)
        _attrs(op)
    return i


def _register(op, res_name, res_count, result_types, env, block, counter):
    op.position = counter[0]
    counter[0] += 1
    for k, v in enumerate(op.operands):
        v.uses.append((op, k))
    if res_name:
        res = [Value(res_name[1:] + (f"#{k}" if res_count else ""), t, op, k) for k, t in enumerate(result_types)]
        op.results = res
        env[res_name[1:]] = res if res_count else res[0]
    block.ops.append(op)


def _parse_while(lines, i, ln, res_name, res_count, rest, env, block, counter, lookup):
    """`%r:N = stablehlo.while(%iterArg = %init, ...) : types  cond { ... } do { ... }`."""
    head = ln
    while not re.search(r"\bcond\s*\{", head) and i < len(lines):
        head += " " + lines[i].strip()                             # `cond {` may sit on the next line
        i += 1
    inside = head[head.index("(") + 1:]
    depth, end = 1, 0
    for end, c in enumerate(inside):
        depth += c == "("
        depth -= c == ")"
        if depth == 0:
            break
    pairs = [p.split("=") for p in _top_level_split(inside[:end], ",") if p.strip()]
    names = [a.strip()[1:] for a, _ in pairs]
    inits = [lookup(b.strip()[1:]) for _, b in pairs]
    types = [parse_type(t) for t in re.findall(r"tensor<[^<>]*>", inside[end:].split("cond")[0])]
    op = Op("stablehlo.while", inits, {}, "")
    _register(op, res_name, res_count if res_count else None, types if res_name else [], env, block, counter)
    if res_name and not res_count:                                 # a single carried value
        env[res_name[1:]] = op.results[0]
    for _ in range(2):                                             # cond, then body
        region = Block(op)
        renv = dict(env)
        for k, (nm, t) in enumerate(zip(names, types)):
            v = Value(nm, t, None, k, region)
            region.args.append(v)
            renv[nm] = v
        i = _parse_block(lines, i, renv, region, counter)
        op.regions.append(region)
    return i


def _attrs(op):
    """Typed attributes of the ops the recognizer and the evaluator look at."""
    t, a = op.text, op.attrs
    n = op.name
    if n == "stablehlo.broadcast_in_dim":
        a["dims"] = _attr(t, "dims", _attr(t, "broadcast_dimensions", []))
    elif n == "stablehlo.transpose":
        a["dims"] = _attr(t, "dims", _attr(t, "permutation", []))
    elif n == "stablehlo.dot_general":
        a["batching"] = _pair(t, "batching_dims")
        a["contracting"] = _pair(t, "contracting_dims")
        if not re.search(r"batching_dims\s*=\s*\[", t) and "lhs_batching_dimensions" in t:   # generic form
            a["batching"] = (_attr(t, "lhs_batching_dimensions", []), _attr(t, "rhs_batching_dimensions", []))
            a["contracting"] = (_attr(t, "lhs_contracting_dimensions", []), _attr(t, "rhs_contracting_dimensions", []))
    elif n == "stablehlo.concatenate":
        a["dim"] = _attr(t, "dim", _attr(t, "dimension", 0))
    elif n == "stablehlo.iota":
        a["dim"] = _attr(t, "dim", _attr(t, "iota_dimension", 0))
    elif n == "stablehlo.slice":
        m = re.search(r"\[([^\]]*)\]\s*$", t.strip())
        a["slices"] = [tuple(int(x) for x in s.split(":")) for s in m.group(1).split(",")] if m else []
    elif n == "stablehlo.compare":
        a["direction"] = re.search(r"\b(EQ|NE|LT|LE|GT|GE)\b", t).group(1)
    elif n == "stablehlo.reduce":
        m = re.search(r"applies\s+([\w.]+)\s+across\s+dimensions\s*=\s*(\[[^\]]*\])", t)
        if m:                                               # the one-line form of a plain reduction
            a["applies"], a["dims"] = m.group(1), _int_list(m.group(2))
    elif n == "chlo.top_k":
        a["k"] = _attr(t, "k", 1)
    elif n == "stablehlo.gather":
        for key in ("offset_dims", "collapsed_slice_dims", "start_index_map", "slice_sizes", "operand_batching_dims"):
            a[key] = _attr(t, key, [])
        a["index_vector_dim"] = _attr(t, "index_vector_dim", 0)


# ---------------------------------------------------------------------------------------
# literal evaluation
# ---------------------------------------------------------------------------------------


def _binary(fn):
    return lambda op, x, y: fn(x, y)


def _convert(op, x):
    dt = op.results[0].type.dtype
    if dt == torch.bool:
        return x != 0
    if x.dtype.is_floating_point and not dt.is_floating_point:
        return torch.trunc(x).to(dt)          # round toward zero
    return x.to(dt)


def _broadcast(op, x):
    shape = op.results[0].type.shape
    dims = op.attrs["dims"]
    order = sorted(range(len(dims)), key=lambda i: dims[i])       # operand axes in result order
    if order != list(range(len(dims))):
        x = x.permute(*order)
    view = [1] * len(shape)
    for i in order:
        view[dims[i]] = x.shape[order.index(i)]
    return x.reshape(view).expand(shape)


def _dot(op, x, y):
    (lb, rb), (lc, rc) = op.attrs["batching"], op.attrs["contracting"]
    lf = [d for d in range(x.dim()) if d not in lb and d not in lc]
    rf = [d for d in range(y.dim()) if d not in rb and d not in rc]
    bs = [x.shape[d] for d in lb]
    xm = x.permute(*lb, *lf, *lc).reshape(*bs, -1, _prod(x.shape[d] for d in lc))
    ym = y.permute(*rb, *rf, *rc).reshape(*bs, -1, _prod(y.shape[d] for d in rc))
    dt = op.results[0].type.dtype
    acc = torch.matmul(xm.to(torch.float32), ym.to(torch.float32).transpose(-1, -2)) if dt.is_floating_point \
        else torch.matmul(xm.to(torch.int64), ym.to(torch.int64).transpose(-1, -2))
    out_shape = bs + [x.shape[d] for d in lf] + [y.shape[d] for d in rf]
    return acc.reshape(out_shape).to(dt)       # float32 accumulation, one rounding on output


def _gather(op, operand, indices):
    """The `jnp.take(table, idx, axis=0)` form: whole slices of the operand picked by one
    index (collapsed_slice_dims = [0], start_index_map = [0])."""
    a = op.attrs
    if a["collapsed_slice_dims"] != [0] or a["start_index_map"] != [0] or a.get("operand_batching_dims"):
        raise NotImplementedError("gather: only row takes are evaluated")
    if a["slice_sizes"][1:] != list(operand.shape[1:]):
        raise NotImplementedError("gather: partial slices")
    ivd = a["index_vector_dim"]
    idx = indices.select(ivd, 0) if ivd < indices.dim() else indices
    idx = idx.to(torch.int64).clamp(0, operand.shape[0] - 1)
    out = operand[idx]
    return out.reshape(op.results[0].type.shape)


_REDUCERS = {"stablehlo.add": lambda x, d: x.sum(dim=d), "stablehlo.maximum": lambda x, d: x.amax(dim=d),
             "stablehlo.minimum": lambda x, d: x.amin(dim=d), "stablehlo.multiply": lambda x, d: x.prod(dim=d)}
_COMBINE = {"stablehlo.add": torch.add, "stablehlo.maximum": torch.maximum, "stablehlo.minimum": torch.minimum,
            "stablehlo.multiply": torch.mul}


def _reduce(op, x, init):
    kind = op.attrs.get("applies")
    if kind not in _REDUCERS:
        raise NotImplementedError("reduce: only the one-line add / max / min / multiply forms are evaluated")
    dt = op.results[0].type.dtype
    wide = x.to(torch.float32) if dt.is_floating_point else x
    out = _REDUCERS[kind](wide, tuple(op.attrs["dims"]))
    return _COMBINE[kind](out, init.to(out.dtype)).to(dt)


def _top_k(op, x):
    """Largest k along the last axis, descending; ties keep the lower index first (stable)."""
    order = torch.sort(x, dim=-1, descending=True, stable=True)
    k = op.attrs["k"]
    return [order.values[..., :k].contiguous(), order.indices[..., :k].to(op.results[1].type.dtype).contiguous()]


def _prod(xs):
    p = 1
    for x in xs:
        p *= x
    return p


def _shift(fn):
    def run(op, x, y):
        bits = torch.iinfo(x.dtype).bits
        ok = (y >= 0) & (y < bits)
        return torch.where(ok, fn(x, y.clamp(0, bits - 1)), torch.zeros_like(x))
    return run


def _srl(x, y):
    if x.dtype == torch.uint8:
        return x >> y
    bits = torch.iinfo(x.dtype).bits
    mask = (1 << bits) - 1
    return ((x.to(torch.int64) & mask) >> y.to(torch.int64)).to(x.dtype)


_CMP = {"EQ": torch.eq, "NE": torch.ne, "LT": torch.lt, "LE": torch.le, "GT": torch.gt, "GE": torch.ge}

EVAL = {
    "stablehlo.add": _binary(torch.add), "stablehlo.subtract": _binary(torch.sub),
    "stablehlo.multiply": _binary(torch.mul),
    "stablehlo.divide": lambda op, x, y: x / y if x.dtype.is_floating_point else torch.div(x, y, rounding_mode="trunc"),
    "stablehlo.maximum": _binary(torch.maximum), "stablehlo.minimum": _binary(torch.minimum),
    "stablehlo.clamp": lambda op, lo, x, hi: torch.minimum(torch.maximum(x, lo), hi),
    "stablehlo.and": _binary(torch.bitwise_and), "stablehlo.or": _binary(torch.bitwise_or),
    "stablehlo.xor": _binary(torch.bitwise_xor),
    "stablehlo.shift_left": _shift(lambda x, y: x << y),
    "stablehlo.shift_right_logical": _shift(_srl),
    "stablehlo.shift_right_arithmetic": lambda op, x, y: x >> y.clamp(0, torch.iinfo(x.dtype).bits - 1),
    "stablehlo.negate": lambda op, x: -x, "stablehlo.abs": lambda op, x: x.abs(),
    "stablehlo.exponential": lambda op, x: torch.exp(x), "stablehlo.rsqrt": lambda op, x: torch.rsqrt(x),
    "stablehlo.logistic": lambda op, x: torch.sigmoid(x),
    "stablehlo.sqrt": lambda op, x: torch.sqrt(x), "stablehlo.tanh": lambda op, x: torch.tanh(x),
    "stablehlo.log": lambda op, x: torch.log(x),
    "stablehlo.power": _binary(torch.pow),
    "stablehlo.convert": _convert,
    "stablehlo.bitcast_convert": lambda op, x: x.contiguous().view(op.results[0].type.dtype).reshape(op.results[0].type.shape),
    "stablehlo.reshape": lambda op, x: x.reshape(op.results[0].type.shape),
    "stablehlo.transpose": lambda op, x: x.permute(*op.attrs["dims"]),
    "stablehlo.broadcast_in_dim": _broadcast,
    "stablehlo.concatenate": lambda op, *xs: torch.cat(xs, dim=op.attrs["dim"]),
    "stablehlo.slice": lambda op, x: x[tuple(slice(*s) for s in op.attrs["slices"])],
    "stablehlo.compare": lambda op, x, y: _CMP[op.attrs["direction"]](x, y),
    "stablehlo.select": lambda op, p, x, y: torch.where(p, x, y),
    "stablehlo.dot_general": _dot,
    "stablehlo.reduce": lambda op, x, init: _reduce(op, x, init),
    "stablehlo.gather": _gather,
}


def eval_op(op, ins, device=None):
    """One op on concrete tensors; returns the list of its results."""
    if op.opaque:
        raise NotImplementedError(f"{op.name} has regions: not evaluated here")
    if op.name == "stablehlo.constant":
        return [_dense(op.text, op.results[0].type).to(device)]
    if op.name == "stablehlo.iota":
        t = op.results[0].type
        view = [1] * len(t.shape)
        view[op.attrs["dim"]] = t.shape[op.attrs["dim"]]
        return [torch.arange(t.shape[op.attrs["dim"]], device=device).reshape(view).expand(t.shape).to(t.dtype)]
    if op.name == "chlo.top_k":
        return _top_k(op, *ins)
    fn = EVAL.get(op.name)
    if fn is None:
        raise NotImplementedError(f"{op.name} is not evaluated here")
    out = fn(op, *ins)
    return [out]


def evaluate_value(value, env):
    """`value` on concrete buffers: `env` maps Values (the function's arguments at least) to
    tensors and memoizes every intermediate. Iterative (subtrees can be deep). An argument of a
    while region that the loop hands on unchanged evaluates to the loop's initial operand."""
    stack = [value]
    device = next((t.device for t in env.values() if isinstance(t, torch.Tensor)), None)
    while stack:
        v = stack[-1]
        if v in env:
            stack.pop()
            continue
        if v.op is None:
            init = invariant_init(v)
            if init is None:
                raise KeyError(f"argument %{v.name} has no buffer")
            if init not in env:
                stack.append(init)
                continue
            env[v] = env[init]
            stack.pop()
            continue
        if v.op.name == "stablehlo.while":
            raise NotImplementedError("a while result is not evaluated as a subtree")
        missing = [o for o in v.op.operands if o not in env]
        if missing:
            stack.extend(missing)
            continue
        outs = eval_op(v.op, [env[o] for o in v.op.operands], device)
        for r, t in zip(v.op.results, outs):
            env[r] = t
        stack.pop()
    return env[value]


def run_block(block, env, hook=None, device=None):
    """The ops of `block` in order on the buffers in `env` (updated in place). `hook(op, env)`
    may take an op over (it returns True when it did: a fused root or a skipped op); while loops
    run their regions through the same hook."""
    for op in block.ops:
        if hook is not None and hook(op, env):
            continue
        if op.name == "stablehlo.while":
            cond, body = op.regions
            carries = [env[o] for o in op.operands]
            for _ in range(1 << 20):
                for a, t in zip(cond.args, carries):
                    env[a] = t
                run_block(cond, env, hook, device)
                if not bool(env[cond.returns[0]]):
                    break
                for a, t in zip(body.args, carries):
                    env[a] = t
                run_block(body, env, hook, device)
                carries = [env[r] for r in body.returns]
            for r, t in zip(op.results, carries):
                env[r] = t
            continue
        outs = eval_op(op, [env[o] for o in op.operands], device)
        for r, t in zip(op.results, outs):
            env[r] = t


def evaluate(fn: Func, args):
    """The whole function, literally."""
    env = dict(zip(fn.args, args))
    run_block(fn, env, None, args[0].device if args else None)
    return [env[v] for v in fn.returns]
