"""The general pair-space planner (the reference's `_Planner`, src/metaljax/moe.py:450-810) on
expert regions that are NOT the SwiGLU shape: what is planned, what stays dense, what is rejected,
and -- on CPU, with the grouped product stood in for by a per-expert torch matmul on the
dequantized weights -- that running the plan over the routed pairs reproduces the literal dense
program. The same regions run through the real kernels in tests/test_gpu_recognizer.py."""

import numpy as np
import torch

from metaljax_b200 import hlo, moe_recognizer, pair_plan, recognizer
from oracle import qmm_oracle as O

from helpers import to_numpy
from programs import (moe_glu_bias_inputs, moe_gelu_quant_inputs, moe_program, moe_program_glu_bias,
                      moe_program_gelu_quant)


def _torch_ragged(rows, w, sizes, match):
    """Per-expert matmul in float32 on dense weights, rounded to the rows' type."""
    if isinstance(w, tuple):
        packed, scales, biases = (to_numpy(a) for a in w)
        dense = torch.from_numpy(O.dequantize(packed, scales, biases, group_size=match.gs, bits=match.bits,
                                              mode=match.mode).astype(np.float32))
    else:
        dense = w.float()
    out = torch.zeros((rows.shape[0], dense.shape[1]), dtype=torch.float32)
    r0 = 0
    for e, n in enumerate(sizes.tolist()):
        out[r0:r0 + n] = rows[r0:r0 + n].float() @ dense[e].T
        r0 += n
    return out.to(rows.dtype)


def _run_region(text, args):
    it = recognizer.Interpreter(text)
    want = hlo.evaluate(it.func, args)[0]
    recognizer.prologue(it, args)
    st = it._qmm
    assert len(st.moe) == 1 and isinstance(st.moe[0], moe_recognizer.ExpertRegion)
    b = st.moe[0]
    assert b.verified and not b.disabled
    env = dict(zip(it.func.args, args))
    idx = hlo.evaluate_value(b.router.indices, env).to(torch.int64)
    wts = hlo.evaluate_value(b.router.weights, env)
    got = moe_recognizer._emit_region(it, b, env, idx, wts, ragged=_torch_ragged)
    return it, st, b, got, want


def test_gated_region_with_biases_clamps_and_strided_slices():
    it, st, b, got, want = _run_region(moe_program_glu_bias(), moe_glu_bias_inputs(seed=3))
    assert [m.mode for m in b.dots] == ["float", "float"] and st.matches == []
    kinds = [n.kind for n in b.planner.order]
    assert kinds.count("dot") == 2 and "const" in kinds and "view" in kinds and "elem" in kinds
    # outside values: the tokens (token axis only), the two biases (expert axis only), scalar constants
    axes = sorted(("e" if n.ea is not None else "") + ("t" if n.ta is not None else "")
                  for n in b.planner.order if n.kind == "ext" and n.paired)
    assert axes == ["e", "e", "t"]
    skipped = [o.name for o in it.func.ops if id(o) in st.skip]
    assert skipped.count("stablehlo.dot_general") == 2 and "stablehlo.clamp" in skipped and "stablehlo.slice" in skipped
    assert "chlo.top_k" not in skipped
    assert tuple(got.shape) == tuple(want.shape) and got.dtype == want.dtype
    err = (got.float() - want.float()).abs().max().item()
    assert err <= 2e-2 * want.float().abs().max().item(), err


def test_quantized_gelu_region_with_a_per_expert_gain():
    it, st, b, got, want = _run_region(moe_program_gelu_quant(), moe_gelu_quant_inputs(seed=4))
    assert len(st.matches) == 2 and all(m.absorbed for m in st.matches)
    assert [type(v).__name__ for v in st.roots.values()] == ["ExpertRegion"]
    assert sorted(m.mode for m in b.dots) == ["affine", "affine"]
    err = (got.float() - want.float()).abs().max().item()
    assert err <= 2e-2 * want.float().abs().max().item(), err
    # every dense [E, T, ...] op of the region is gone, the gain's broadcast included
    assert all(o.results[0].type.shape[:1] != (4,) or id(o) in st.skip or o.results[0].type.shape == (4,)
               for o in it.func.ops if o.results and len(o.results[0].type.shape) == 3)


def test_the_swiglu_shape_keeps_its_fused_block():
    st = recognizer.analyze(recognizer.Interpreter(moe_program()))
    assert type(st.moe[0]) is moe_recognizer.ExpertBlock


def test_what_pair_space_does_not_model_stays_dense():
    text = moe_program_glu_bias()
    # a reduction inside the region (softmax-like normalisation over the features) is not modelled
    bad = text.replace("%25 = stablehlo.logistic %24 : tensor<6x4x64xbf16>",
                       "%25 = stablehlo.cosine %24 : tensor<6x4x64xbf16>")
    st = recognizer.analyze(recognizer.Interpreter(bad))
    assert st is None or st.moe == []
    # a slice that cuts the expert axis
    bad = text.replace("[0:6, 0:4, 0:128:2]", "[0:6, 0:4:1, 1:128:2]").replace("[0:6, 0:4, 1:128:2]", "[0:6, 1:4, 1:128:2]")
    try:
        st = recognizer.analyze(recognizer.Interpreter(bad))
    except Exception:                                  # the edited text no longer type-checks: also not planned
        st = None
    assert st is None or st.moe == []


def test_weighted_sum_matches_the_dense_form():
    g = torch.Generator().manual_seed(0)
    T, K, E, W = 5, 2, 4, 16
    logits = torch.randn((T, E), generator=g)
    wts, idx = torch.topk(torch.softmax(logits, -1), K, dim=-1)
    from metaljax_b200 import moe
    order, tok, sizes = moe.sort_pairs(idx, E)
    y = torch.randn((T * K, W), generator=g)
    got = pair_plan.weighted_sum(y, order, wts, T, K, torch.float32)
    want = torch.zeros((T, W))
    for r in range(T * K):
        p = int(order[r])
        want[p // K] += wts[p // K, p % K] * y[r]
    assert torch.allclose(got, want, atol=1e-6)


import pytest  # noqa: E402


@pytest.mark.parametrize("t,d,e,f,k", [(1, 64, 4, 64, 2), (1, 64, 8, 128, 4), (3, 128, 4, 64, 1), (7, 64, 8, 64, 3), (2, 64, 4, 192, 2)])
def test_regions_at_other_sizes_one_token_and_one_choice_included(t, d, e, f, k):
    """A single token (every decode step: the token axis is a unit axis, which a broadcast must
    not be mistaken for), a single choice per token, more experts than tokens."""
    for text, args in ((moe_program_glu_bias(t, d, e, f, k), moe_glu_bias_inputs(t, d, e, f, seed=t)),
                       (moe_program_gelu_quant(t, d, e, f, 32, k), moe_gelu_quant_inputs(t, d, e, f, 32, seed=t))):
        it, st, b, got, want = _run_region(text, args)
        assert (b.T, b.K, b.E) == (t, k, e)
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 2e-2 * max(want.float().abs().max().item(), 1e-6), (t, d, e, f, k, err)
