"""The Llama-shaped decode step (the fused linears' caller at decode time) on one GPU: its
logits against the same step in float32 torch on the dequantized weights, eagerly and
replayed from a CUDA graph, and the three glue kernels against their formulas."""

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _small():
    from metaljax_b200 import llama
    return llama.Shape(layers=2, d_model=256, heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=1000, ctx=48)


@pytest.mark.parametrize("batch", [1, 3, 9])
def test_decode_step_matches_float_reference(batch):
    from metaljax_b200 import _lib, llama
    shape = _small()
    fw = llama.random_full_weights(shape, batch, DEV, seed=batch)
    step = llama.DecodeStep(shape, batch, DEV, full_weights=fw)
    tokens = torch.arange(batch, device=DEV) * 7 % shape.vocab
    step.tokens.copy_(tokens)
    nxt = step.step().clone()
    got = step.logits()
    want = llama.reference_logits(fw, shape, tokens, batch)
    err = (got - want).abs().max().item() / want.abs().max().item()
    assert err <= 3e-2, err                       # a chain of bf16 hand-offs, two layers deep
    # the chosen token is the reference's, unless the reference's top two are within the error
    top2 = want.topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 2 * 3e-2 * want.abs().max()
    assert torch.equal(nxt[clear], want.argmax(-1)[clear])
    # the same step replayed from a CUDA graph
    step.capture()
    step.replay()
    torch.cuda.synchronize()
    assert torch.equal(step.next_tokens, nxt)
    assert _lib.poll_status() == 0


def test_glue_kernels():
    from metaljax_b200 import llama
    g = torch.Generator(device=DEV).manual_seed(0)
    rows, dim = 5, 384
    x = torch.randn((rows, dim), generator=g, device=DEV).to(torch.bfloat16)
    r = torch.randn((rows, dim), generator=g, device=DEV).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(dim, generator=g, device=DEV)).to(torch.bfloat16)
    out, res = torch.empty_like(x), r.clone()
    llama.add_rmsnorm(x, w, out, residual=res, eps=1e-5)
    h = (x.float() + r.float()).to(torch.bfloat16)
    assert torch.equal(res, h)
    want = h.float() * torch.rsqrt((h.float() ** 2).mean(-1, keepdim=True) + 1e-5) * w.float()
    assert (out.float() - want).abs().max() <= 2e-2 * want.abs().max()
    gu = torch.randn((rows, 2 * 512), generator=g, device=DEV).to(torch.bfloat16)
    act = torch.empty((rows, 512), device=DEV, dtype=torch.bfloat16)
    llama.silu_mul(gu, act)
    gate, up = gu[:, :512].float(), gu[:, 512:].float()
    want = gate / (1 + torch.exp(-gate)) * up
    assert (act.float() - want).abs().max() <= 1e-2 * want.abs().max()
    # rotary + cache append
    b, heads, kvh, hd, ctx, pos = 2, 4, 2, 64, 16, 9
    qkv = torch.randn((b, (heads + 2 * kvh) * hd), generator=g, device=DEV).to(torch.bfloat16)
    q = torch.empty((b, heads, 1, hd), device=DEV, dtype=torch.bfloat16)
    kc = torch.zeros((b, kvh, ctx, hd), device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    llama.rope_kv(qkv, q, kc, vc, heads, kvh, hd, pos, 10000.0)
    j = torch.arange(hd // 2, device=DEV, dtype=torch.float32)
    ang = pos * 10000.0 ** (-2.0 * j / hd)
    c, s = torch.cos(ang), torch.sin(ang)

    def rot(t):
        lo, hi = t[..., : hd // 2].float(), t[..., hd // 2:].float()
        return torch.cat([lo * c - hi * s, hi * c + lo * s], dim=-1)

    x3 = qkv.view(b, heads + 2 * kvh, hd)
    assert (q[:, :, 0].float() - rot(x3[:, :heads])).abs().max() <= 3e-2
    assert (kc[:, :, pos].float() - rot(x3[:, heads:heads + kvh])).abs().max() <= 3e-2
    assert torch.equal(vc[:, :, pos], x3[:, heads + kvh:])
    assert kc[:, :, :pos].abs().max() == 0 and kc[:, :, pos + 1:].abs().max() == 0


def test_single_row_step_fused_against_unfused(monkeypatch):
    """Batch 1 takes the fused step (norms, SwiGLU and exchanges inside the linears' kernels);
    with QMM_DECODE_FUSED=0 the same weights go through the separate glue kernels. Both against
    the float reference, and against each other."""
    from metaljax_b200 import _lib, llama
    shape = llama.Shape(layers=3, d_model=512, heads=8, kv_heads=4, head_dim=64, ffn=1024, vocab=2000, ctx=40)
    fw = llama.random_full_weights(shape, 1, DEV, seed=11)
    tokens = torch.tensor([17], device=DEV)
    want = llama.reference_logits(fw, shape, tokens, 1)
    outs = {}
    for fused in ("1", "0"):
        monkeypatch.setenv("QMM_DECODE_FUSED", fused)
        step = llama.DecodeStep(shape, 1, DEV, full_weights=fw)
        assert step.fused == (fused == "1")
        step.tokens.copy_(tokens)
        step.step()
        outs[fused] = step.logits().clone()
        err = (outs[fused] - want).abs().max().item() / want.abs().max().item()
        assert err <= 3e-2, (fused, err)
        step.capture()
        for _ in range(3):
            step.replay()
        torch.cuda.synchronize()
        assert torch.equal(step.logits(), outs[fused])
    assert (outs["1"] - outs["0"]).abs().max().item() <= 2e-2 * want.abs().max().item()
    assert _lib.poll_status() == 0


def test_multi_row_step_with_the_one_kernel_attention(monkeypatch):
    """Above one row the step's attention is the library's rotary + append + attention kernel;
    QMM_DECODE_ATTENTION=sdpa swaps in the rotary kernel and torch's attention. Same logits as
    the float reference, the same rows appended to the cache."""
    from metaljax_b200 import _lib, llama
    shape, batch = _small(), 5
    fw = llama.random_full_weights(shape, batch, DEV, seed=21)
    tokens = torch.arange(batch, device=DEV) * 5 % shape.vocab
    want = llama.reference_logits(fw, shape, tokens, batch)
    caches = {}
    for which in ("sdpa", "own"):
        monkeypatch.setenv("QMM_DECODE_ATTENTION", which)
        step = llama.DecodeStep(shape, batch, DEV, full_weights=fw)
        assert step.own_attention == (which == "own")
        step.tokens.copy_(tokens)
        step.step()
        err = (step.logits() - want).abs().max().item() / want.abs().max().item()
        assert err <= 3e-2, (which, err)
        caches[which] = (step.k_cache.clone(), step.v_cache.clone())
    for own, ref in zip(caches["own"], caches["sdpa"]):
        assert torch.equal(own[0], ref[0])                       # the first layer appends the same bits
        assert (own.float() - ref.float()).abs().max().item() <= 3e-2 * ref.float().abs().max().item()   # deeper ones follow the logits
    assert _lib.poll_status() == 0


def test_decode_linear_prologues_and_self_exchange():
    """`qmm_decode_linear` against the unfused sequence: SwiGLU prologue bit for bit (the same
    bf16 row reaches the same kernel), add + RMS-norm within a bf16 rounding of the row; and the
    exchange protocol on one GPU as a world of one: a linear pushes its row, as stamped units, into
    its own gather slot, the next one reads the row from the slot as it arrives, over several steps."""
    import ctypes
    from metaljax_b200 import _lib, llama, qmm
    g = torch.Generator(device=DEV).manual_seed(5)
    d, f = 512, 1024

    def lin(n, k):
        return llama._Linear(n, k, DEV, g, 64, "normal")

    up, down, nxt = lin(2 * f, d), lin(d, f), lin(384, d)
    x = torch.randn((1, d), generator=g, device=DEV).to(torch.bfloat16)
    res = torch.randn((1, d), generator=g, device=DEV).to(torch.bfloat16)
    wn = (1 + 0.1 * torch.randn(d, generator=g, device=DEV)).to(torch.bfloat16)
    lib = _lib.lib()
    stream = _lib.stream_ptr(x)

    def call(linear, xin, y, ex=None, **kw):
        fz = _lib.DecodeFusion()
        fz.prologue = kw.get("prologue", 0)
        fz.wait_slot, fz.wait_site = kw.get("wait", (-1, 0))
        fz.push_slot, fz.push_site = kw.get("push", (-1, 0))
        for name in ("residual_in", "residual_out", "norm_weight"):
            t = kw.get(name)
            setattr(fz, name, None if t is None else t.data_ptr())
        fz.eps = 1e-5
        p = linear.problem(xin, y)
        _lib.check(lib.qmm_decode_linear(ctypes.byref(p), ctypes.byref(fz), None if ex is None else ctypes.byref(ex), stream))

    # unfused: h = x + res; normed; gate_up; act; down
    normed, h = torch.empty_like(x), res.clone()
    llama.add_rmsnorm(x, wn, normed, residual=h, eps=1e-5)
    gu_ref = torch.empty((1, 2 * f), device=DEV, dtype=torch.bfloat16)
    up(normed, gu_ref)
    act = torch.empty((1, f), device=DEV, dtype=torch.bfloat16)
    llama.silu_mul(gu_ref, act)
    dn_ref = torch.empty((1, d), device=DEV, dtype=torch.bfloat16)
    down(act, dn_ref)
    # fused, plain buffers
    gu, dn, h2 = torch.empty_like(gu_ref), torch.empty_like(dn_ref), torch.empty_like(x)
    call(up, x, gu, prologue=1, residual_in=res, residual_out=h2, norm_weight=wn)
    assert torch.equal(h2, h)
    assert (gu.float() - gu_ref.float()).abs().max() <= 2e-2 * gu_ref.float().abs().max()
    call(down, gu_ref, dn, prologue=2)
    assert torch.equal(dn, dn_ref)
    # the same chain through a gather slot of a world of one, three steps in a row
    slot_bytes = 2 * f * 4                               # a stamped row: 4 bytes per value
    area = torch.zeros((2 * slot_bytes,), device=DEV, dtype=torch.uint8)
    state = torch.zeros((8,), device=DEV, dtype=torch.int32)
    ex = _lib.Exchange()
    bufs = (ctypes.c_void_p * 1)(area.data_ptr())
    ex.peer_bufs = ctypes.cast(bufs, ctypes.POINTER(ctypes.c_void_p))
    ex.epoch, ex.slot_bytes, ex.rank, ex.world = state.data_ptr(), slot_bytes, 0, 1
    out = torch.empty((1, 384), device=DEV, dtype=torch.bfloat16)
    want = torch.empty_like(out)
    h3 = torch.empty_like(x)
    nxt_in = torch.empty_like(x)
    llama.add_rmsnorm(dn_ref, wn, nxt_in, residual=h.clone(), eps=1e-5)
    nxt(nxt_in, want)
    for step in range(3):
        _lib.check(lib.qmm_decode_step_begin(ctypes.byref(ex), stream))
        call(up, x, None, ex, prologue=1, residual_in=res, residual_out=h2, norm_weight=wn, push=(0, 0))
        call(down, None, None, ex, prologue=2, wait=(0, 0), push=(1, 1))
        call(nxt, None, out, ex, prologue=1, wait=(1, 1), residual_in=h2, residual_out=h3, norm_weight=wn)
        torch.cuda.synchronize()
        assert int(state[0]) == step + 1
        units = area.view(torch.int32)                    # {pair, stamp} units: every stamp of a row is the exchange's
        assert bool((units[1: 2 * f: 2] == (((step + 1) << 10) | 1)).all())
        assert bool((units[slot_bytes // 4 + 1: slot_bytes // 4 + d: 2] == (((step + 1) << 10) | 2)).all())
        assert (out.float() - want.float()).abs().max() <= 3e-2 * want.float().abs().max()
    assert _lib.poll_status() == 0


@pytest.mark.parametrize("batch,heads,kvh,hd,ctx,pos", [
    (1, 8, 2, 128, 2048, 2047), (1, 4, 4, 64, 48, 47), (3, 4, 2, 64, 300, 150), (2, 8, 1, 128, 1000, 0),
    (64, 4, 1, 128, 2048, 2047), (5, 16, 2, 64, 513, 512), (1, 32, 8, 128, 2048, 1000),
    (7, 8, 8, 128, 700, 640), (2, 2, 1, 64, 130, 64),
    (64, 32, 8, 128, 2048, 2047),                         # one layer of the batch-64 step: 537 MB of cache
])
@pytest.mark.parametrize("kernel", ["simt", "mma"])
def test_decode_attention_against_rope_and_sdpa(batch, heads, kvh, hd, ctx, pos, kernel, monkeypatch):
    """The one-kernel rotary + append + attention against the rotary kernel followed by torch's
    scaled_dot_product_attention over positions 0..pos, cache contents included -- both of its
    forms: the latency kernel of short slices and the streaming tensor-core kernel of long ones."""
    import torch.nn.functional as F
    from metaljax_b200 import _lib, llama
    monkeypatch.setenv("QMM_ATTN_KERNEL", kernel)
    g = torch.Generator(device=DEV).manual_seed(batch * 100 + heads)
    qkv = torch.randn((batch, (heads + 2 * kvh) * hd), generator=g, device=DEV).to(torch.bfloat16)
    kc = (torch.randn((batch, kvh, ctx, hd), generator=g, device=DEV) * 0.5).to(torch.bfloat16)
    vc = (torch.randn((batch, kvh, ctx, hd), generator=g, device=DEV) * 0.5).to(torch.bfloat16)
    kc2, vc2 = kc.clone(), vc.clone()
    q = torch.empty((batch, heads, 1, hd), device=DEV, dtype=torch.bfloat16)
    llama.rope_kv(qkv, q, kc, vc, heads, kvh, hd, pos, 500000.0)
    want = F.scaled_dot_product_attention(q.float(), kc[:, :, : pos + 1].float(), vc[:, :, : pos + 1].float(), enable_gqa=True)
    want = want.reshape(batch, heads * hd)
    nbytes = _lib.lib().qmm_decode_attention_scratch_bytes(batch, heads, kvh, hd, ctx)
    scratch = torch.zeros((nbytes,), device=DEV, dtype=torch.uint8)
    out = torch.empty((batch, heads * hd), device=DEV, dtype=torch.bfloat16)
    for _ in range(2):                                   # the scratch counters reset themselves
        out.zero_()
        llama.decode_attention(qkv, kc2, vc2, out, scratch, heads, kvh, hd, pos, 500000.0)
        assert (out.float() - want).abs().max().item() <= 2e-2 * max(want.abs().max().item(), 1e-3)
    assert torch.equal(kc2, kc) and torch.equal(vc2, vc)     # the same append
    assert _lib.poll_status() == 0


def test_decode_linear_swiglu_epilogue():
    """Gate and up rows interleaved in one weight, SwiGLU applied where the tile is finished:
    bit for bit the separate SwiGLU of the stored bf16 outputs, written plainly and / or pushed as
    stamped units; the down projection that follows reads either."""
    import ctypes
    from metaljax_b200 import _lib, llama
    g = torch.Generator(device=DEV).manual_seed(9)
    d, f = 512, 1088                                     # 2 f = 2176 rows = 68 tiles of 32: a ragged last wave
    gate_up, down = llama._Linear(2 * f, d, DEV, g, 64, "normal"), llama._Linear(d, f, DEV, g, 64, "normal")
    x = torch.randn((1, d), generator=g, device=DEV).to(torch.bfloat16)
    lib, stream = _lib.lib(), _lib.stream_ptr(x)
    # reference: [gate | up] halves, stored as bf16, then the glue kernel
    gu = torch.empty((1, 2 * f), device=DEV, dtype=torch.bfloat16)
    gate_up(x, gu)
    act_ref = torch.empty((1, f), device=DEV, dtype=torch.bfloat16)
    llama.silu_mul(gu, act_ref)
    dn_ref = torch.empty((1, d), device=DEV, dtype=torch.bfloat16)
    down(act_ref, dn_ref)
    # the interleaved layout of the same weight
    idx = torch.stack([torch.arange(f, device=DEV), torch.arange(f, device=DEV) + f], dim=1).reshape(-1)
    inter = llama._Linear(2 * f, d, DEV, g, 64, "normal",
                          pack=(gate_up.w.view(torch.int32)[idx].view(torch.uint32), gate_up.s[idx], gate_up.b[idx]))

    def call(linear, xin, y, ex=None, wait=(-1, 0), push=(-1, 0), swiglu_out=None, swiglu=False):
        fz = _lib.DecodeFusion()
        fz.wait_slot, fz.wait_site = wait
        fz.push_slot, fz.push_site = push
        fz.epilogue = 1 if swiglu else 0
        fz.epilogue_out = None if swiglu_out is None else swiglu_out.data_ptr()
        p = linear.problem(xin, y)
        _lib.check(lib.qmm_decode_linear(ctypes.byref(p), ctypes.byref(fz), None if ex is None else ctypes.byref(ex), stream))

    act, y_all = torch.zeros_like(act_ref), torch.empty_like(gu)
    call(inter, x, y_all, swiglu=True, swiglu_out=act)
    assert torch.equal(y_all.reshape(f, 2).t().reshape(1, 2 * f), gu)          # the plain outputs, de-interleaved
    assert torch.equal(act, act_ref)
    # pushed through a world of one and consumed by the down projection
    slot_bytes = 2 * f * 4
    area = torch.zeros((2 * slot_bytes,), device=DEV, dtype=torch.uint8)
    state = torch.zeros((8,), device=DEV, dtype=torch.int32)
    ex = _lib.Exchange()
    bufs = (ctypes.c_void_p * 1)(area.data_ptr())
    ex.peer_bufs = ctypes.cast(bufs, ctypes.POINTER(ctypes.c_void_p))
    ex.epoch, ex.slot_bytes, ex.rank, ex.world = state.data_ptr(), slot_bytes, 0, 1
    for step in range(2):
        _lib.check(lib.qmm_decode_step_begin(ctypes.byref(ex), stream))
        dn = torch.zeros_like(dn_ref)
        call(inter, x, None, ex=ex, push=(0, 0), swiglu=True)
        call(down, None, dn, ex=ex, wait=(0, 0))
        assert torch.equal(dn, dn_ref)
    assert _lib.poll_status() == 0
    with pytest.raises(_lib.QmmError):
        call(inter, x, y_all, swiglu=True)                                      # nowhere to put the values


@pytest.mark.parametrize("rows,n,stride", [(1, 128256, 128256), (64, 128256, 128256), (3, 1001, 1008), (2, 7, 16), (5, 16032, 16032)])
def test_decode_argmax_kernel(rows, n, stride):
    """The largest logit of every row and its index (ties: the smallest index), offset added."""
    import ctypes
    from metaljax_b200 import _lib
    g = torch.Generator(device=DEV).manual_seed(rows + n)
    logits = torch.randn((rows, stride), generator=g, device=DEV).to(torch.bfloat16)
    logits[:, n:] = 100.0                                  # beyond n: must not be looked at
    if n > 10:
        logits[0, 5] = logits[0, n - 1] = 50.0             # a tie: the smaller index wins
    lib = _lib.lib()
    scratch = torch.zeros((lib.qmm_decode_argmax_scratch_bytes(rows),), device=DEV, dtype=torch.uint8)
    val = torch.empty((rows,), device=DEV, dtype=torch.float32)
    idx = torch.empty((rows,), device=DEV, dtype=torch.int64)
    for _ in range(2):                                     # (the counters return to zero between calls)
        _lib.check(lib.qmm_decode_argmax(logits.data_ptr(), rows, n, stride, 1000, val.data_ptr(), idx.data_ptr(),
                                         scratch.data_ptr(), scratch.numel(), _lib.stream_ptr(logits)))
        ref = logits[:, :n].float()
        want_val = ref.max(dim=-1).values
        assert torch.equal(val, want_val)
        first = (ref == want_val[:, None]).float().argmax(dim=-1)
        assert torch.equal(idx, first + 1000)
