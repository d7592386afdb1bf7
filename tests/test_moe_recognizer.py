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


def test_router_verification_forces_ties_and_counts_nonzeros():
    """A hand-rolled router that keeps every logit >= the k-th largest agrees with top-k until two
    logits tie at the k-th place: then it routes a token to K + 1 experts. The reference's
    verification rounds its later draws to halves exactly to provoke that
    (src/metaljax/moe.py:1128-1131) and counts the nonzeros per token (`:1144-1152`); a
    verification on the first, continuous draw alone would have accepted this router."""
    from metaljax_b200 import hlo
    from metaljax_b200 import moe_recognizer as M
    text = """
module @threshold_router {
  func.func public @main(%arg0: tensor<64x8xf32>) -> (tensor<64x8xf32>) {
    %0:2 = chlo.top_k(%arg0, k = 2) : tensor<64x8xf32> -> (tensor<64x2xf32>, tensor<64x2xi32>)
    %1 = stablehlo.slice %0#0 [0:64, 1:2] : (tensor<64x2xf32>) -> tensor<64x1xf32>
    %2 = stablehlo.reshape %1 : (tensor<64x1xf32>) -> tensor<64xf32>
    %3 = stablehlo.broadcast_in_dim %2, dims = [0] : (tensor<64xf32>) -> tensor<64x8xf32>
    %4 = stablehlo.compare GE, %arg0, %3 : (tensor<64x8xf32>, tensor<64x8xf32>) -> tensor<64x8xi1>
    %cst = stablehlo.constant dense<0.000000e+00> : tensor<64x8xf32>
    %5 = stablehlo.select %4, %arg0, %cst : tensor<64x8xi1>, tensor<64x8xf32>
    return %5 : tensor<64x8xf32>
  }
}
"""
    fn = hlo.parse(text)
    ops = {o.name: o for o in fn.walk()}
    r = M.Router()
    r.top_k = ops["chlo.top_k"]
    r.indices, r.weights = r.top_k.results[1], r.top_k.results[0]
    r.S = ops["stablehlo.select"].results[0]
    r.T, r.K, r.E, r.t_axis, r.e_axis = 64, 2, 8, 0, 1
    before = M.STATS["verified"]
    assert M.verify_router(r, draws=1)                  # continuous logits: no ties, looks like top-2
    assert not M.verify_router(r, draws=3)              # halves: ties at the second place give it away
    assert M.STATS["verified"] == before + 1


def test_float_expert_block_is_planned_on_the_float_grouped_product():
    """Unquantized (bf16) experts: the same router proof and region, the three projections read
    their weights straight from the arguments and are planned onto the float grouped product
    (the reference's `mx.gather_mm` branch, src/metaljax/moe.py:1324-1336)."""
    from programs import moe_program_float
    it = recognizer.Interpreter(moe_program_float(t=6, d=64, e=4, f=64, k=2))
    st = recognizer.analyze(it)
    assert st.matches == [] and len(st.moe) == 1 and st.active
    b = st.moe[0]
    assert (b.gate.mode, b.up.mode, b.down.mode) == ("float", "float", "float")
    assert b.gate.nshape == [4, 64] and b.gate.K == 64 and b.down.bshape == [4] and (b.down.N, b.down.K) == (64, 64)
    assert b.gate.arg_indices == (2,) and b.up.arg_indices == (3,) and b.down.arg_indices == (4,)
    names = [o.name for o in it.func.ops if id(o) in st.skip]
    assert names.count("stablehlo.dot_general") == 3 and "stablehlo.logistic" in names
    assert "chlo.top_k" not in names                              # the router's own outputs stay
    # float32 experts keep their literal dots (the fused product takes the activations' 16-bit type)
    f32 = moe_program_float(t=6, d=64, e=4, f=64, k=2).replace("%arg2: tensor<4x64x64xbf16>", "%arg2: tensor<4x64x64xf32>")
    f32 = f32.replace("(tensor<6x64xbf16>, tensor<4x64x64xbf16>) -> tensor<6x4x64xbf16>\n    %21", "(tensor<6x64xbf16>, tensor<4x64x64xf32>) -> tensor<6x4x64xbf16>\n    %21")
    assert recognizer.analyze(recognizer.Interpreter(f32)).moe == []
