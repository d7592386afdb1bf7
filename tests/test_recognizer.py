"""The quantized-matmul recognizer on hand-written StableHLO in jax's print syntax: structural
analysis, rejections, pruning, the pack prologue against the oracle's packer and the build
cache. CPU only (the fused op itself is exercised in tests/test_gpu_recognizer.py)."""

import numpy as np
import torch

from metaljax_b200 import hlo, qmm, recognizer
from oracle import qmm_oracle as O

from programs import (DONATED, LHS_QUANT, MXFP4, PER_CHANNEL, RMS_NORM, SHARED_WEIGHT, SUB_CHANNEL, WHILE_LOOP,
                      mxfp4_inputs, sub_channel_inputs, while_loop_inputs)


def test_parser_round_trip():
    fn = hlo.parse(SUB_CHANNEL)
    assert [a.type.shape for a in fn.args] == [(5, 256), (16, 256), (16, 4), (16, 4)]
    assert fn.ops[-1].name == "stablehlo.dot_general"
    assert fn.ops[-1].attrs["contracting"] == ([1], [1])
    x, codes, scales, zeros = sub_channel_inputs(seed=0)
    got = hlo.evaluate(fn, [x, codes, scales, zeros])[0]
    w = (codes.float() - zeros.float().repeat_interleave(64, 1)) * scales.float().repeat_interleave(64, 1)
    want = (x.float() @ w.T)
    assert torch.allclose(got.float(), want, rtol=2e-2, atol=2e-2)


def test_analyze_sub_channel():
    it = recognizer.Interpreter(SUB_CHANNEL)
    st = recognizer.analyze(it)
    assert len(st.matches) == 1 and st.active
    m = st.matches[0]
    assert (m.B, m.M, m.K, m.N) == (1, 5, 256, 16) and not m.swapped and m.mode == "affine"
    assert m.zero is not None and m.sub_range is None            # float subtraction
    assert m.arg_indices == (1, 2, 3)
    # everything between the arguments and the dot is skipped; the dot is the root
    skipped = {o.name for o in it.func.ops if id(o) in st.skip}
    assert "stablehlo.multiply" in skipped and "stablehlo.subtract" in skipped
    assert it.func.ops[-1].name == "stablehlo.dot_general" and id(it.func.ops[-1]) in st.roots
    assert recognizer.analyze(it) is st                          # once per program


def test_analyze_other_forms():
    m = recognizer.analyze(recognizer.Interpreter(PER_CHANNEL)).matches
    assert len(m) == 1 and m[0].recip and m[0].root.name == "stablehlo.divide" and m[0].bcast_dims == [0]
    m = recognizer.analyze(recognizer.Interpreter(MXFP4)).matches
    assert len(m) == 1 and m[0].mode == "mxfp4" and (m[0].M, m[0].K, m[0].N) == (3, 64, 8)
    m = recognizer.analyze(recognizer.Interpreter(LHS_QUANT)).matches
    assert len(m) == 1 and m[0].swapped and (m[0].M, m[0].K, m[0].N) == (5, 256, 16)


def test_rejections_and_pruning():
    # a donated weight buffer may be reused by the callee: never packed
    assert recognizer.analyze(recognizer.Interpreter(DONATED)).matches == []
    # x * broadcast(rsqrt(...)) has one scale per row, not per 32: not MXFP4
    assert recognizer.analyze(recognizer.Interpreter(RMS_NORM)).matches == []
    # the dequantized weight is also returned: materialized anyway, so the dot stays literal
    assert recognizer.analyze(recognizer.Interpreter(SHARED_WEIGHT)).matches == []


def test_prologue_packs_like_the_oracle():
    it = recognizer.Interpreter(SUB_CHANNEL)
    x, codes, scales, zeros = sub_channel_inputs(seed=1)
    args = [x, codes, scales, zeros]
    assert recognizer.prologue(it, args) is False
    m = it._qmm.matches[0]
    assert (m.gs, m.bits, m.slot, m.nvals) == (64, 4, 0, 3)
    w, s, b = it._qmm.values
    want_w, want_s, want_b = O.pack_exact(codes.numpy().astype(np.int64), scales.float().numpy(),
                                          zeros.float().numpy(), 4)
    np.testing.assert_array_equal(w.view(torch.int32).numpy().view(np.uint32), want_w)
    np.testing.assert_array_equal(s.float().numpy(), want_s.astype(np.float32))
    np.testing.assert_array_equal(b.float().numpy(), want_b.astype(np.float32))
    # same buffers again: the match's own pack; a second program over the same buffers: the
    # build cache; new buffers: a fresh pack
    packs0 = qmm.stats()["packs"]
    recognizer.prologue(it, args)
    it2 = recognizer.Interpreter(SUB_CHANNEL)
    recognizer.prologue(it2, args)
    assert qmm.stats()["packs"] == packs0 and it2._qmm.values[0] is w
    recognizer.prologue(it2, [x, codes.clone(), scales, zeros])
    assert qmm.stats()["packs"] == packs0 + 1


def test_prologue_rejects_values():
    it = recognizer.Interpreter(SUB_CHANNEL)
    x, codes, scales, zeros = sub_channel_inputs(seed=2)
    scales = scales.clone()
    bad = scales.float().repeat_interleave(64, 1)
    del bad
    codes = codes.clone()
    codes[0, 0] = 100                                            # spans more than... still 8 bits
    codes[0, 1] = -100
    zeros = zeros.clone()
    zeros[0, 0] = 0.5                                            # a non-integer zero point
    assert recognizer.prologue(it, [x, codes, scales, zeros]) is True
    assert it._qmm.matches[0].disabled and not it._qmm.active
    assert "zero points" in it.rejections[0][1]


def test_mxfp4_prologue():
    it = recognizer.Interpreter(MXFP4)
    x, nib, sbytes = mxfp4_inputs(seed=3)
    recognizer.prologue(it, [x, nib, sbytes])
    m = it._qmm.matches[0]
    assert not m.disabled and (m.gs, m.bits, m.mode, m.nvals) == (32, 4, "mxfp4", 2)
    w, s = it._qmm.values
    np.testing.assert_array_equal(w.view(torch.int32).numpy().view(np.uint32),
                                  O.pack_codes(nib.numpy().astype(np.uint8), 4))
    np.testing.assert_array_equal(s.numpy(), sbytes.numpy())


def test_weights_carried_through_a_loop():
    """A while loop's closed-over weights are loop carries the body returns unchanged: the
    recognizer follows them out to @main's arguments and fuses the dot inside the body."""
    it = recognizer.Interpreter(WHILE_LOOP)
    fn = it.func
    loop = next(o for o in fn.ops if o.name == "stablehlo.while")
    assert len(loop.regions) == 2 and len(loop.regions[1].args) == 5
    assert hlo.invariant_init(loop.regions[1].args[1]) is fn.args[1]
    assert hlo.invariant_init(loop.regions[1].args[4]) is None          # the activations change
    st = recognizer.analyze(it)
    assert len(st.matches) == 1
    m = st.matches[0]
    assert m.arg_indices == (1, 2, 3) and (m.M, m.K, m.N) == (5, 256, 256)
    assert m.root.name == "stablehlo.dot_general" and m.lhs is loop.regions[1].args[4]
    # literal evaluation of the loop, and the pack built from @main's buffers
    args = while_loop_inputs(seed=4)
    lit = hlo.evaluate(fn, args)[0]
    x, codes, scales, zeros = args
    w = ((codes.float() - zeros.float().repeat_interleave(64, 1)) * scales.float().repeat_interleave(64, 1))
    want = x.float()
    for _ in range(3):
        want = (want.to(torch.bfloat16).float() @ w.to(torch.bfloat16).float().T)
    assert torch.allclose(lit.float(), want.to(torch.bfloat16).float(), rtol=5e-2, atol=5e-2 * float(want.abs().max()))
    assert recognizer.prologue(it, args) is False and not m.disabled and (m.gs, m.bits) == (64, 4)


def test_block_cost_bytes_and_captures():
    """What a tracing host asks of the recognizer (the reference's ops/control.py:251-283,
    317-401, 700-725): an absorbed op costs nothing, a fused root 2 units; loops are unrolled;
    the packed arrays travel with a body's captures."""
    it = recognizer.Interpreter(WHILE_LOOP)
    fn = it.func
    loop = next(o for o in fn.ops if o.name == "stablehlo.while")
    body = loop.regions[1]
    assert recognizer.static_trip(loop) == 3
    # body: 7 reconstruction ops absorbed, the dot = 2 units, the counter's add = 1
    assert recognizer.block_cost(it, body) == 3
    # @main: three constants, the while itself, three bodies
    assert recognizer.block_cost(it, fn) == 3 + 1 + 3 * 3
    lit = recognizer.Interpreter(WHILE_LOOP)
    lit._qmm = qmm.State()                                       # a program with no rewrite: every op counts
    assert recognizer.block_cost(lit, lit.func.ops[3].regions[1]) == 9
    # bytes: the body materializes the dot's result (5x256 bf16), one activation copy, the counter
    assert recognizer.block_bytes(it, body) == 5 * 256 * 2 + 5 * 256 * 2 + 4
    literal_body = recognizer.block_bytes(lit, lit.func.ops[3].regions[1])
    assert literal_body > 7 * 256 * 256 * 2 // 2                 # the dequantize chain at full weight size
    whole = recognizer.block_bytes(it, fn)
    assert whole == 3 * 4 + (4 + 256 * 256 + 2 * 256 * 4 * 2 + 5 * 256 * 2) + 3 * recognizer.block_bytes(it, body)
    # captures: free values of the body in first-use order, then the packed arrays
    free = recognizer.free_values(body)
    assert [v.name for v in free] == [fn.ops[2].results[0].name]           # only the constant 1
    args = while_loop_inputs(seed=4)
    recognizer.prologue(it, args)
    env = {fn.ops[2].results[0]: torch.tensor(1, dtype=torch.int32)}
    caps = recognizer.captures(it, env, free)
    assert caps[0] is env[free[0]] and len(caps) == 1 + len(qmm.values(it)) and len(qmm.values(it)) == 3
    assert all(a is b for a, b in zip(caps[1:], qmm.values(it)))


def test_captures_stand_in_for_an_absorbed_value():
    """A reconstruction op hoisted out of the loop is skipped in the enclosing block, so it has
    no buffer; the body's capture list keeps its arity with a stand-in."""
    it = recognizer.Interpreter(SUB_CHANNEL)
    st = recognizer.analyze(it)
    absorbed = next(o for o in it.func.ops if id(o) in st.skip)
    caps = recognizer.captures(it, {}, [absorbed.results[0]])
    assert caps[0].numel() == 1 and caps[0].dtype == torch.uint8
    live = it.func.ops[-1].results[0]                            # not absorbed and not in env: an error, as before
    try:
        recognizer.captures(it, {}, [live])
    except KeyError:
        pass
    else:
        raise AssertionError("a missing live capture must raise")


def test_unknown_trip_count_is_pessimistic():
    text = WHILE_LOOP.replace("%1 = stablehlo.compare LT, %iterArg, %c_0, SIGNED", "%1 = stablehlo.compare NE, %iterArg, %c_0, SIGNED")
    it = recognizer.Interpreter(text)
    loop = next(o for o in it.func.ops if o.name == "stablehlo.while")
    assert recognizer.static_trip(loop) is None
    assert recognizer.block_cost(it, it.func) == 3 + 1 + 1024 * recognizer.block_cost(it, loop.regions[1])


def test_real_jax_lowering_recognizes_nothing():
    """The one program text in the reference's tree that jax itself printed (a shrunk qwen3
    prefill, bf16 weights, a scan over layers, private callees): it parses, and an ordinary
    float graph matches nothing -- no quantized dot, no expert block. Read from the reference
    checkout where that exists; the file is not redistributed."""
    import os
    import pytest
    beside = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
    path = os.path.join(os.environ.get("METALJAX_REFERENCE", beside), "tests", "data", "qwen3_prefill_shrunk.mlir")
    if not os.path.exists(path):
        pytest.skip("no reference checkout on this machine")
    it = recognizer.Interpreter(open(path).read())
    fn = it.func
    names = [o.name for o in fn.walk()]
    assert fn.name == "main" and len(fn.args) > 8
    # the private callees (dynamic_index_in_dim, the layer body, silu, argmax, ...) are inlined
    assert names.count("stablehlo.while") == 1 and names.count("stablehlo.dot_general") == 15 and "func.call" not in names
    loop = next(o for o in fn.ops if o.name == "stablehlo.while")
    assert len(loop.regions) == 2 and recognizer.static_trip(loop) == 8          # one trip per layer
    st = recognizer.analyze(it)
    assert st.matches == [] and not st.roots and not st.skip
    # with nothing absorbed the cost walk charges every op: 8 unrolled bodies dominate
    body_cost = recognizer.block_cost(it, loop.regions[1])
    assert body_cost >= len(loop.regions[1].ops)
    assert recognizer.block_cost(it, fn) >= 8 * body_cost


def _packs_equal(a, b):
    xa, xb = a.arrays(), b.arrays()
    return (a.gs, a.bits, a.mode, len(xa)) == (b.gs, b.bits, b.mode, len(xb)) and all(
        p.dtype == q.dtype and p.shape == q.shape and torch.equal(p, q) for p, q in zip(xa, xb))


def _build_both(text, args, block_elems, monkeypatch):
    """The pack of every match from row blocks of `block_elems` weight elements and from one
    whole evaluation; sharing off so that each build keeps its own arrays."""
    out = []
    for elems in (block_elems, 1 << 40):
        monkeypatch.setattr(recognizer, "_BLOCK_ELEMS", elems)
        monkeypatch.setattr(qmm, "_SHARED", {})
        recognizer._BUILD_CACHE.clear()
        qmm.reset_stats()
        it = recognizer.Interpreter(text)
        recognizer.prologue(it, args)
        ms = [m for m in recognizer.analyze(it).matches]
        assert ms and not any(m.disabled for m in ms), it.rejections
        out.append(([m.packs[0] for m in ms], dict(qmm.stats())))
    return out


def test_row_blocked_build_equals_whole(monkeypatch):
    """Packing from blocks of rows (the reference's `_Source`, src/metaljax/qmm.py:1360-1631)
    takes the same decisions and gives the same arrays as packing from the whole maps."""
    from programs import moe_inputs, moe_program, per_channel_inputs, sub_channel_inputs_at, sub_channel_program
    cases = [
        (sub_channel_program(4, 256, 96, gs=64), sub_channel_inputs_at(4, 256, 96, gs=64, seed=3), 256 * 10),
        (MXFP4, mxfp4_inputs(seed=2), 64 * 3),
        (WHILE_LOOP, while_loop_inputs(seed=5), 256 * 100),
        (PER_CHANNEL, per_channel_inputs(seed=7), 0),
        (moe_program(t=6, d=64, e=4, f=64, gs=32, k=2), moe_inputs(t=6, d=64, e=4, f=64, gs=32, seed=1), 64 * 64),
    ]
    for text, args, elems in cases:
        if not elems:                                            # too small a weight to cut: sized below
            w = next(a for a in args if a.dtype == torch.int8)
            elems = w.shape[-1] * max(w.shape[0] // 3, 1)
        (blocked, bstats), (whole, wstats) = _build_both(text, args, elems, monkeypatch)
        if text is PER_CHANNEL:                                   # stored [K, N]: the leading axis is not the row axis
            assert not bstats.get("blocked")
        else:
            assert bstats.get("blocked", 0) == len(blocked) and not bstats.get("unblocked"), bstats
        assert not wstats.get("blocked")
        assert len(blocked) == len(whole) and all(_packs_equal(a, b) for a, b in zip(blocked, whole))


def test_row_blocked_build_rejects_like_whole(monkeypatch):
    """A bad value in the LAST block is still found: codes off the integer grid reject."""
    args = mxfp4_inputs(seed=2)
    bad = args[1].clone()
    monkeypatch.setattr(recognizer, "_BLOCK_ELEMS", 64 * 3)
    recognizer._BUILD_CACHE.clear()
    it = recognizer.Interpreter(MXFP4)
    scales = args[2].clone()
    scales[-1, -1] = 255                                          # E8M0 byte 255 decodes to NaN in the table: not a power of two
    recognizer.prologue(it, [args[0], bad, scales])
    assert recognizer.analyze(it).matches[0].disabled and it.rejections


def test_share_aliases_equal_packs(monkeypatch):
    """Two chains that reconstruct the same weight from different buffers hold one packed copy
    (content-addressed: equal arrays, not equal graphs; src/metaljax/qmm.py:1652-1704)."""
    monkeypatch.setattr(qmm, "_SHARED", {})
    recognizer._BUILD_CACHE.clear()
    qmm.reset_stats()
    args = sub_channel_inputs(seed=6)
    it1, it2 = recognizer.Interpreter(SUB_CHANNEL), recognizer.Interpreter(SUB_CHANNEL)
    recognizer.prologue(it1, args)
    copy = [a.clone() for a in args]                               # other buffers, same contents
    recognizer.prologue(it2, copy)
    p1, p2 = recognizer.analyze(it1).matches[0].packs[0], recognizer.analyze(it2).matches[0].packs[0]
    assert p1 is not p2 and p1.w is p2.w and p1.scales is p2.scales and p1.biases is p2.biases
    assert qmm.stats().get("shared") == 1
    other = [a.clone() for a in args]
    other[1][0, 0] = (other[1][0, 0] + 1) if int(other[1][0, 0]) < 7 else (other[1][0, 0] - 1)        # one code differs
    it3 = recognizer.Interpreter(SUB_CHANNEL)
    recognizer.prologue(it3, other)
    p3 = recognizer.analyze(it3).matches[0].packs[0]
    assert p3.w is not p1.w and not torch.equal(p3.w, p1.w) and qmm.stats().get("shared") == 1


def test_outlined_helpers_are_inlined():
    """jax outlines helpers as private functions; the dequantization chain inside one is matched
    through the call, and the packed weight is the one of the flat program."""
    from programs import OUTLINED
    it = recognizer.Interpreter(OUTLINED)
    assert [o.name for o in it.func.ops].count("stablehlo.dot_general") == 1
    assert not any(o.name in ("call", "func.call") for o in it.func.walk())
    st = recognizer.analyze(it)
    assert len(st.matches) == 1 and st.matches[0].arg_indices == (1, 2, 3) and st.matches[0].mode == "affine"
    args = sub_channel_inputs(seed=3)
    flat = recognizer.Interpreter(SUB_CHANNEL)
    assert torch.equal(hlo.evaluate(it.func, args)[0], (hlo.evaluate(flat.func, args)[0].float() * 2).to(torch.bfloat16))
    recognizer._BUILD_CACHE.clear()
    recognizer.prologue(it, args)
    recognizer.prologue(flat, args)
    a, b = st.matches[0].packs[0], recognizer.analyze(flat).matches[0].packs[0]
    assert all(torch.equal(x, y) for x, y in zip(a.arrays(), b.arrays()))


def test_composite_decomposition_is_inlined():
    from programs import OUTLINED
    text = OUTLINED.replace("%0 = call @dequantize(%arg1, %arg2, %arg3) :",
                            '%0 = stablehlo.composite "my.dequantize" %arg1, %arg2, %arg3 {composite_attributes = {group = 64 : i64}, decomposition = @dequantize} :')
    it = recognizer.Interpreter(text)
    assert not any(o.name == "stablehlo.composite" for o in it.func.walk())
    assert len(recognizer.analyze(it).matches) == 1
