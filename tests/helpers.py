"""Shared generators for the parity tests: seeded synthetic inputs with the shapes and value
distributions of the benchmark configurations, in numpy (for the oracle) and torch (for the
CUDA path) from the same draws."""

import hashlib

import ml_dtypes
import numpy as np
import torch

BF16 = ml_dtypes.bfloat16
NP2TORCH = {np.dtype(np.float32): torch.float32, np.dtype(np.float16): torch.float16,
            np.dtype(BF16): torch.bfloat16}


def digest(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def np_dtype(name):
    return {"bf16": BF16, "f16": np.float16, "f32": np.float32}[name]


def to_torch(a: np.ndarray, device="cpu") -> torch.Tensor:
    """numpy -> torch without changing a bit (bf16 through its uint16 pattern)."""
    a = np.ascontiguousarray(a)
    if a.dtype == np.dtype(BF16):
        t = torch.from_numpy(a.view(np.uint16).copy()).view(torch.bfloat16)
    elif a.dtype == np.uint32:
        t = torch.from_numpy(a.view(np.int32).copy()).view(torch.uint32)
    else:
        t = torch.from_numpy(a.copy())
    return t.to(device)


def to_numpy(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(BF16)
    if t.dtype == torch.uint32:
        return t.view(torch.int32).numpy().view(np.uint32)
    return t.numpy()


def affine_case(rng, n, k, gs, bits, table="bf16", lead=(), scale_lo=0.005, scale_hi=0.02):
    """Codes uniform over the full range, scales ~ U(lo, hi) in the table dtype,
    bias = -mid*scale (exact in the table dtype): the benchmark's affine convention."""
    from oracle import qmm_oracle as O
    shape = tuple(lead) + (n, k)
    codes = rng.integers(0, 1 << bits, size=shape).astype(np.uint8)
    tdt = np_dtype(table)
    scales = rng.uniform(scale_lo, scale_hi, size=tuple(lead) + (n, k // gs)).astype(tdt)
    biases = (-(float(1 << (bits - 1))) * scales.astype(np.float32)).astype(tdt)
    return codes, O.pack_codes(codes, bits), scales, biases


def mxfp4_case(rng, n, k, lead=(), exp_lo=119, exp_hi=128):
    """All 16 codes uniform, E8M0 exponents uniform in [exp_lo-127, exp_hi-128]."""
    from oracle import qmm_oracle as O
    shape = tuple(lead) + (n, k)
    codes = rng.integers(0, 16, size=shape).astype(np.uint8)
    sb = rng.integers(exp_lo, exp_hi, size=tuple(lead) + (n, k // 32)).astype(np.uint8)
    return codes, O.pack_codes(codes, 4), sb


def activations(rng, shape, dtype="bf16", scale=1.0):
    return (rng.standard_normal(shape) * scale).astype(np.float32).astype(np_dtype(dtype))
