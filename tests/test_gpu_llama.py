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
