"""The entry point that allocates nothing (`qmm_quantized_matmul_static`) against the ordinary
one, through the C ABI, twice in a row on the same stream; and its refusal of a product whose
partial results do not fit the static block. Collected last on purpose: it is an extra of the
library, not part of the reference's boundary."""

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _problem(m, k, n, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    x = torch.randn((m, k), generator=g, device=DEV).to(torch.bfloat16)
    w = torch.randint(-(1 << 31), (1 << 31) - 1, (n, k // 8), generator=g, device=DEV,
                      dtype=torch.int64).to(torch.int32).view(torch.uint32)
    s = (torch.rand((n, k // 64), generator=g, device=DEV) * 0.018 + 0.002).to(torch.bfloat16)
    b = (-8.0 * s.float()).to(torch.bfloat16)
    return x, w, s, b


def _call(fn, x, w, s, b, y):
    from metaljax_b200 import _lib
    v = _lib.Views()
    return fn(v(x), v(w), v(s), v(b), v(y), 1, 64, 4, 0, _lib.stream_ptr(x))


def test_static_entry_matches_the_ordinary_one_twice():
    """Same bits as the ordinary entry point, within the parity gate of the oracle, and -- the
    property it exists for -- no device-memory allocation by the library during the call, while
    the ordinary entry point allocates the split product's scratch every time."""
    import numpy as np
    from helpers import to_numpy
    from metaljax_b200 import _lib
    from oracle import clib
    from oracle import qmm_oracle as O
    lib = _lib.lib()
    assert _lib.poll_status() == 0          # (the device's status word exists from here on)
    for call in range(2):                                         # two calls in a row
        for m, k, n in ((64, 4096, 1024), (40, 2048, 512), (300, 1024, 256)):
            x, w, s, b = _problem(m, k, n, seed=10 * call + m)
            want = torch.empty((m, n), device=DEV, dtype=torch.bfloat16)
            got = torch.full((m, n), float("nan"), device=DEV, dtype=torch.bfloat16)
            with _lib.force_route("gemm_tc"):
                a0 = _lib.alloc_count()
                _lib.check(_call(lib.qmm_quantized_matmul, x, w, s, b, want))
                assert _lib.alloc_count() - a0 == 1, (m, k, n)   # every one of these shapes shares K among CTAs
            a0 = _lib.alloc_count()
            _lib.check(_call(lib.qmm_quantized_matmul_static, x, w, s, b, got))
            assert _lib.alloc_count() == a0, "the static entry point allocated"
            torch.cuda.synchronize()
            assert torch.equal(got, want), (call, m, k, n)
            exact = clib.qmm(to_numpy(x), to_numpy(w), to_numpy(s), to_numpy(b), m, k, n, 64, 4,
                             out_f32=True).astype(np.float64)
            assert O.rel_err(to_numpy(got).astype(np.float32), exact) <= 1e-2
    assert _lib.poll_status_static() == 0                          # no bounded wait ran out


def test_static_entry_refuses_what_does_not_fit():
    from metaljax_b200 import _lib
    lib = _lib.lib()
    # one token tile x 16 feature tiles -> 8 splits of 256 x 2048 float32 = 16 MiB > 8 MiB
    x, w, s, b = _problem(256, 4096, 2048, seed=5)
    y = torch.zeros((256, 2048), device=DEV, dtype=torch.bfloat16)
    rc = _call(lib.qmm_quantized_matmul_static, x, w, s, b, y)
    assert rc == 10, rc                                            # QMM_ERR_TOO_LARGE
    msg = lib.qmm_last_error().decode()
    assert "scratch" in msg and "static block" in msg, msg
    torch.cuda.synchronize()
    assert float(y.abs().max()) == 0.0                             # nothing was launched
    # float32 activations are not the tensor-core kernel's: refused as unsupported
    xf = x.float()
    rc = _call(lib.qmm_quantized_matmul_static, xf, w, s, b, torch.zeros((256, 2048), device=DEV))
    assert rc == 7, rc                                             # QMM_ERR_UNSUPPORTED
