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
