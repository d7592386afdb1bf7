"""Packs straight from stored formats: Hugging Face MXFP4 `_blocks` / `_scales` and the keras
int4 `Dense` kernel (two output columns per byte, groups along the input rows) against the
oracle's dequantizer. CPU only."""

import numpy as np
import pytest
import torch

from metaljax_b200 import qmm
from oracle import qmm_oracle as O

_E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], np.float32)


def test_hf_mxfp4_blocks_are_the_packed_stream():
    g = torch.Generator().manual_seed(0)
    e, n, k = 3, 8, 128
    blocks = torch.randint(0, 256, (e, n, k // 32, 16), generator=g, dtype=torch.uint8)
    scales = torch.randint(100, 140, (e, n, k // 32), generator=g, dtype=torch.uint8)
    w, s = qmm.from_hf_mxfp4(blocks, scales)
    assert w.dtype == torch.uint32 and tuple(w.shape) == (e, n, k // 8) and s is not None
    assert w.untyped_storage().data_ptr() == blocks.untyped_storage().data_ptr()          # a view, no copy
    # the reference's reading of the bytes: low nibble = element 2j, high nibble = element 2j + 1
    codes = torch.stack([blocks & 15, blocks >> 4], dim=-1).reshape(e, n, k).numpy()
    want = _E2M1[codes] * np.exp2(scales.numpy().astype(np.float32) - 127).repeat(32, axis=-1)
    for ex in range(e):
        got = O.dequantize(w[ex].numpy(), s[ex].numpy(), None, 32, 4, mode="mxfp4")
        assert np.array_equal(got, want[ex])
    with pytest.raises(ValueError):
        qmm.from_hf_mxfp4(blocks, torch.zeros_like(scales))                                # byte 0 is not a usable scale
    with pytest.raises(ValueError):
        qmm.from_hf_mxfp4(blocks[..., :8], scales)


def _keras_case(k, n, groups, seed, interleave=False):
    g = torch.Generator().manual_seed(seed)
    wq = torch.randint(-8, 8, (k, n), generator=g, dtype=torch.int8)
    padded = torch.cat([wq, torch.zeros((k, n % 2), dtype=torch.int8)], dim=1).to(torch.int16)
    packed = ((padded[:, 0::2] & 15) | ((padded[:, 1::2] & 15) << 4)).to(torch.uint8).view(torch.int8)
    scale = (torch.rand((groups, n), generator=g) * 0.02 + 0.01).to(torch.bfloat16)
    zero = torch.randint(-2, 3, (groups, n), generator=g).to(torch.bfloat16)
    g_idx = torch.arange(k) // (k // groups)
    if interleave:                                        # act-order style: row i belongs to group i % groups
        g_idx = torch.arange(k) % groups
    return wq, packed, scale, zero, g_idx


@pytest.mark.parametrize("k,n,groups,interleave", [(256, 10, 4, False), (128, 7, 4, False), (256, 6, 4, True)])
def test_keras_int4_kernel(k, n, groups, interleave):
    wq, packed, scale, zero, g_idx = _keras_case(k, n, groups, seed=k + n, interleave=interleave)
    assert torch.equal(qmm.unpack_keras_int4(packed, n), wq)
    pk = qmm.from_keras_int4(packed, scale, zero, g_idx if interleave else None, columns=n)
    assert pk.bits == 4 and tuple(pk.w.shape) == (n, k // 8) and (pk.perm is not None) == interleave
    # what the layer computes: w[k, n] = (code - zero[g(k), n]) * scale[g(k), n]
    want = ((wq.float() - zero.float()[g_idx]) * scale.float()[g_idx]).t().numpy()            # [N, K]
    got = O.dequantize(pk.w.numpy(), pk.scales.float().numpy(), pk.biases.float().numpy(), pk.gs, pk.bits)
    if pk.perm is not None:                               # packed columns are K in permuted order
        want = want[:, pk.perm.numpy()]
    assert np.allclose(got, want, rtol=0, atol=1e-6 * np.abs(want).max() + 1e-9)


def test_keras_int4_rejects_what_the_prologue_rejects():
    wq, packed, scale, zero, g_idx = _keras_case(256, 6, 4, seed=1)
    bad = zero.clone()
    bad[0, 0] = 0.5                                       # a zero point that is not an integer
    with pytest.raises(qmm._Reject):
        qmm.from_keras_int4(packed, scale, bad, columns=6)
    with pytest.raises(qmm._Reject):
        qmm.from_keras_int4(packed, scale[:3], zero[:3], columns=6)                          # 3 groups do not divide 256
