"""The mixture-of-experts recognizer on a dense SwiGLU expert layer in jax's StableHLO syntax:
the router proof, its numeric verification on synthetic logits, the planned block, and the
rejections. CPU only (the gathered block itself runs in tests/test_gpu_recognizer.py)."""

import torch

from metaljax_b200 import hlo, moe_recognizer, recognizer

from programs import moe_inputs, moe_program


def test_router_is_proved_and_verified():
    it = recognizer.Interpreter(moe_program())
    st = recognizer.analyze(it)
    assert len(st.matches) == 3 and all(m.absorbed for m in st.matches)
    assert len(st.moe) == 1
    b = st.moe[0]
    r = b.router
    assert (r.T, r.K, r.E, r.t_axis, r.e_axis) == (6, 2, 4, 0, 1)
    assert r.top_k.name == "chlo.top_k" and r.indices is r.top_k.results[1]
    assert moe_recognizer.verify_router(r)
    # the root is the block; the three projections are no longer roots of their own
    assert [type(v).__name__ for v in st.roots.values()] == ["ExpertBlock"]
    assert (b.gate.nshape, b.up.nshape, b.down.bshape) == ([4, 64], [4, 64], [4])
    # what stays: only the router's own outputs and what they are computed from
    kept = [o.name for o in it.func.ops if id(o) not in st.skip and id(o) not in st.roots]
    assert "chlo.top_k" in kept and "stablehlo.dot_general" not in kept and "stablehlo.compare" not in kept


def test_prologue_packs_the_experts_and_keeps_the_block():
    it = recognizer.Interpreter(moe_program())
    args = moe_inputs(seed=1)
    assert recognizer.prologue(it, args) is False
    st = it._qmm
    assert st.moe[0].verified and not st.moe[0].disabled
    assert all((m.gs, m.bits, m.disabled) == (32, 4, False) for m in st.matches)
    w, s, b = moe_recognizer._expert_pack(it, st.moe[0].gate, 4)
    assert tuple(w.shape) == (4, 64, 8) and tuple(s.shape) == (4, 64, 2) and tuple(b.shape) == (4, 64, 2)
    # the literal program (every expert for every token) is what the block must reproduce
    out = hlo.evaluate(it.func, args)[0]
    assert tuple(out.shape) == (6, 64) and float(out.float().abs().max()) > 0


def test_a_router_that_is_not_top_k_is_rejected():
    text = moe_program()
    # (1) the outer sum over the token axis instead of the expert axis
    wrong_axis = text.replace("across dimensions = [0] : (tensor<4x6x64xbf16>", "across dimensions = [1] : (tensor<4x6x64xbf16>") \
                     .replace("-> tensor<6x64xbf16>\n    return %34 : tensor<6x64xbf16>", "-> tensor<4x64xbf16>\n    return %34 : tensor<4x64xbf16>") \
                     .replace("-> (tensor<6x64xbf16>) {", "-> (tensor<4x64xbf16>) {")
    st = recognizer.analyze(recognizer.Interpreter(wrong_axis))
    assert st.moe == [] and len(st.roots) == 3                     # the three dots are fused on their own
    # (2) a one-hot compared for inequality selects everything but the top-k
    st = recognizer.analyze(recognizer.Interpreter(text.replace("stablehlo.compare EQ, %6, %5", "stablehlo.compare NE, %6, %5")))
    assert st.moe == []
    # (3) verification fails closed when the structure was misread: force a wrong axis reading
    it = recognizer.Interpreter(text)
    st = recognizer.analyze(it)
    st.moe[0].router.t_axis, st.moe[0].router.e_axis = 1, 0
    assert recognizer.prologue(it, moe_inputs(seed=2)) is True
    assert st.moe[0].disabled and len(st.roots) == 3 and not any(m.absorbed for m in st.matches)


def test_literal_evaluation_of_the_layer_matches_einsum():
    """The front end's literal evaluator is the ground truth of the fused-vs-literal gates, so
    it is pinned here against a direct einsum formulation (including the transposing
    broadcast_in_dim of the routing matrix)."""
    args = moe_inputs(seed=6)
    x, logits, cg, sg, cu, su, cd, sd = args
    got = hlo.evaluate(hlo.parse(moe_program()), args)[0].float()
    wg, wu, wd = (c.float() * s.float().repeat_interleave(32, -1) for c, s in ((cg, sg), (cu, su), (cd, sd)))
    v, i = torch.topk(logits, 2)
    S = torch.zeros(6, 4).scatter_add_(1, i, torch.softmax(v, -1))
    g, u = torch.einsum("td,efd->tef", x.float(), wg), torch.einsum("td,efd->tef", x.float(), wu)
    y = torch.einsum("tef,edf->etd", torch.nn.functional.silu(g) * u, wd)
    want = (y * S.T[:, :, None]).sum(0)
    assert (got - want).abs().max() <= 3e-2 * want.abs().max()
