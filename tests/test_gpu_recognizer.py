"""The recognizer end to end on the GPU: a program executed with its dequantize-and-dot chain
fused into one quantized matmul against the same program executed literally and against the
exact float32 answer, with the reference's gate (tests/test_qmm.py:261-282): the fused result
must be within 1e-2 of the exact answer's largest magnitude and no worse than 1.5x the literal
chain's own error."""

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _exact(fn, args):
    """The program in float64 on the host: every float tensor widened, integer ones as they are."""
    from metaljax_b200 import hlo
    wide = [a.double().cpu() if a.dtype.is_floating_point else a.cpu() for a in args]
    f = hlo.parse(fn) if isinstance(fn, str) else fn
    values = list(f.args)
    for o in f.walk():
        values += o.results
        for region in o.regions:
            values += region.args
    for v in values:
        if v.type.el in hlo.FLOAT_ELS:
            v.type = hlo.TensorType(v.type.shape, "f64")
    return hlo.evaluate(f, wide)[0]


def _gate(text, args, expect_fused=1):
    from metaljax_b200 import _lib, recognizer
    it = recognizer.Interpreter(text)
    fused = it.execute(args)[0]
    literal = it.execute(args, fused=False)[0]
    assert it.fused_calls == expect_fused, it.rejections
    exact = _exact(text, args)
    scale = exact.abs().max().item()
    err_f = (fused.double().cpu() - exact).abs().max().item() / scale
    err_l = (literal.double().cpu() - exact).abs().max().item() / scale
    assert fused.shape == literal.shape and fused.dtype == literal.dtype
    assert err_f <= 1e-2, err_f
    assert err_f <= 1.5 * err_l + 1e-6, (err_f, err_l)
    assert _lib.poll_status() == 0
    return it


def test_sub_channel_rhs_and_lhs():
    from programs import LHS_QUANT, SUB_CHANNEL, sub_channel_inputs
    args = sub_channel_inputs(seed=5, device=DEV)
    _gate(SUB_CHANNEL, args)
    _gate(LHS_QUANT, args)


def test_per_channel_and_mxfp4():
    from programs import MXFP4, PER_CHANNEL, mxfp4_inputs, per_channel_inputs
    _gate(PER_CHANNEL, per_channel_inputs(seed=6, device=DEV))
    it = _gate(MXFP4, mxfp4_inputs(seed=7, device=DEV))
    assert it._qmm.matches[0].mode == "mxfp4"


@pytest.mark.parametrize("m,k,n,gs", [(1, 512, 256, 64), (64, 512, 384, 128), (300, 1024, 256, 32)])
def test_sub_channel_sizes(m, k, n, gs):
    from programs import sub_channel_inputs_at, sub_channel_program
    it = _gate(sub_channel_program(m, k, n, gs), sub_channel_inputs_at(m, k, n, gs, seed=m, device=DEV))
    assert it._qmm.matches[0].gs >= gs


def test_rejected_program_runs_literally():
    from metaljax_b200 import recognizer
    from programs import SHARED_WEIGHT, sub_channel_inputs
    it = recognizer.Interpreter(SHARED_WEIGHT)
    out = it.execute(sub_channel_inputs(seed=8, device=DEV))
    assert it.fused_calls == 0 and len(out) == 2


def test_loop_with_carried_weights_fuses_every_iteration():
    from programs import WHILE_LOOP, while_loop_inputs
    it = _gate(WHILE_LOOP, while_loop_inputs(seed=9, device=DEV), expect_fused=3)
    assert it._qmm.matches[0].arg_indices == (1, 2, 3)


def test_dense_moe_layer_becomes_the_gathered_block():
    """Every expert for every token, nulled by a top-2 router, against the gathered block: same
    result within the reference's gate (the gathered sum has K terms, the dense one E)."""
    from programs import moe_inputs, moe_program
    for t, d, e, f in ((6, 64, 4, 64), (40, 128, 8, 256)):
        it = _gate(moe_program(t, d, e, f), moe_inputs(t, d, e, f, seed=t, device=DEV))
        st = it._qmm
        assert len(st.moe) == 1 and st.moe[0].verified and all(m.absorbed for m in st.matches)


def test_dense_float_moe_layer_becomes_the_gathered_block():
    """The same layer with unquantized bf16 experts: planned onto the float grouped product
    (`qmm_ragged_mm`), same gate; the expert weights are laid out once per set of buffers."""
    from metaljax_b200 import moe
    from programs import moe_float_inputs, moe_program_float
    for t, d, e, f in ((6, 64, 4, 64), (40, 128, 8, 256)):
        moe.reset_stats()
        args = moe_float_inputs(t, d, e, f, seed=t, device=DEV)
        it = _gate(moe_program_float(t, d, e, f), args)
        st = it._qmm
        assert st.matches == [] and len(st.moe) == 1 and st.moe[0].verified and st.moe[0].gate.mode == "float"
        assert moe.stats()["ragged_dot"] == 3
        first = st.moe[0].gate.packs[0].w
        it.execute(args)
        assert st.moe[0].gate.packs[0].w is first                  # not rebuilt for the same buffers


def test_general_expert_regions_run_over_the_routed_pairs():
    """Expert regions that are not the SwiGLU shape, planned node by node in pair space
    (`pair_plan`): a gpt-oss-like float block (one interleaved gate/up projection, per-expert
    biases, clamps, strided slices) on `qmm_ragged_mm`, and quantized experts with a tanh-GELU and
    a per-expert gain on `qmm_ragged_dot`. Same gate as every fused program."""
    from metaljax_b200 import moe, moe_recognizer
    from programs import moe_glu_bias_inputs, moe_gelu_quant_inputs, moe_program_glu_bias, moe_program_gelu_quant
    for t, d, e, f in ((6, 64, 4, 64), (48, 128, 8, 192), (1, 64, 4, 64)):
        moe.reset_stats()
        it = _gate(moe_program_glu_bias(t, d, e, f), moe_glu_bias_inputs(t, d, e, f, seed=t, device=DEV))
        st = it._qmm
        assert isinstance(st.moe[0], moe_recognizer.ExpertRegion) and st.moe[0].verified
        assert moe.stats()["ragged_dot"] == 2                       # one grouped product per dot of the region
        moe.reset_stats()
        it = _gate(moe_program_gelu_quant(t, d, e, f), moe_gelu_quant_inputs(t, d, e, f, seed=t + 1, device=DEV))
        st = it._qmm
        assert isinstance(st.moe[0], moe_recognizer.ExpertRegion) and len(st.matches) == 2
        assert moe.stats()["ragged_dot"] == 2


def test_expert_stack_packs_in_row_blocks_within_a_memory_bound():
    """A [32, 5760, 2880] MXFP4 expert weight (the shape the reference's pack-transient notes
    measure, notes/qmm-pack-transient-2026-08.md:100-109): its reconstruction chain evaluated
    whole holds tens of GB; evaluated one block of rows at a time the transient stays a small
    multiple of one block, and the pack is the same."""
    from metaljax_b200 import _lib, qmm, recognizer
    from programs import mxfp4_expert_inputs, mxfp4_expert_program
    e, m, k, n = 32, 4, 2880, 5760
    args = mxfp4_expert_inputs(e, m, k, n, seed=11, device=DEV)
    it = recognizer.Interpreter(mxfp4_expert_program(e, m, k, n))
    qmm.reset_stats()
    recognizer._BUILD_CACHE.clear()
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    recognizer.prologue(it, args)
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated() - base
    mt = recognizer.analyze(it).matches[0]
    assert not mt.disabled and qmm.stats()["blocked"] == 1, it.rejections
    pk = mt.packs[0]
    packed_bytes = sum(a.numel() * a.element_size() for a in pk.arrays())
    assert packed_bytes == e * n * k // 2 + e * n * k // 32
    # the whole chain would hold > 16 bytes per weight element (8.5 GB here) before the packer's own
    # 64-bit temporaries; a block is 1/32 of that
    assert peak < packed_bytes + (3 << 30), peak
    for ex in (0, 17, e - 1):                                    # the pack itself, expert by expert
        assert torch.equal(pk.w[ex], qmm.pack_codes(args[1][ex], 4))
        assert torch.equal(pk.scales[ex], args[2][ex])
    out = it.execute(args)[0]
    assert it.fused_calls == 1 and _lib.poll_status() == 0
    table = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0] + [-0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], device=DEV, dtype=torch.float64)
    ex = e - 1
    w = table[args[1][ex].long()] * torch.exp2(args[2][ex].double() - 127).repeat_interleave(32, dim=1)
    want = args[0][ex].double() @ w.T
    err = (out[ex].double() - want).abs().max().item() / want.abs().max().item()
    assert err <= 1e-2, err
