"""StableHLO programs in jax's print syntax for the recognizer tests, with matching inputs.
They restate, op for op, the chains of the reference's own tests: keras' sub-channel and
per-channel int4 Dense (tests/test_qmm.py:179-205) and the MXFP4 weight built from a table
gather and a per-32 scale (tests/test_qmm_mxfp4.py:282-299)."""

import numpy as np
import torch

_SUB = """
module @jit_dense_sub {{
  func.func public @main(%arg0: tensor<5x256xbf16>, %arg1: tensor<16x256xi8>{donor}, %arg2: tensor<16x4xbf16>, %arg3: tensor<16x4xbf16>) -> ({results}) {{
    %0 = stablehlo.convert %arg1 : (tensor<16x256xi8>) -> tensor<16x256xbf16>
    %1 = stablehlo.broadcast_in_dim %arg3, dims = [0, 1] : (tensor<16x4xbf16>) -> tensor<16x4x64xbf16>
    %2 = stablehlo.reshape %1 : (tensor<16x4x64xbf16>) -> tensor<16x256xbf16>
    %3 = stablehlo.subtract %0, %2 : tensor<16x256xbf16>
    %4 = stablehlo.broadcast_in_dim %arg2, dims = [0, 1] : (tensor<16x4xbf16>) -> tensor<16x4x64xbf16>
    %5 = stablehlo.reshape %4 : (tensor<16x4x64xbf16>) -> tensor<16x256xbf16>
    %6 = stablehlo.multiply %3, %5 : tensor<16x256xbf16>
    {dot}
    return {ret} : {results}
  }}
}}
"""
_DOT_RHS = "%7 = stablehlo.dot_general %arg0, %6, contracting_dims = [1] x [1] : (tensor<5x256xbf16>, tensor<16x256xbf16>) -> tensor<5x16xbf16>"
_DOT_LHS = "%7 = stablehlo.dot_general %6, %arg0, contracting_dims = [1] x [1] : (tensor<16x256xbf16>, tensor<5x256xbf16>) -> tensor<16x5xbf16>"

SUB_CHANNEL = _SUB.format(donor="", dot=_DOT_RHS, ret="%7", results="tensor<5x16xbf16>")
DONATED = _SUB.format(donor=" {jax.buffer_donor = true}", dot=_DOT_RHS, ret="%7", results="tensor<5x16xbf16>")
LHS_QUANT = _SUB.format(donor="", dot=_DOT_LHS, ret="%7", results="tensor<16x5xbf16>")
SHARED_WEIGHT = _SUB.format(donor="", dot=_DOT_RHS, ret="%7, %6", results="tensor<5x16xbf16>, tensor<16x256xbf16>")

# The same layer as jax prints it when the dequantization sits in a helper: private functions
# called from @main (`call` and `func.call` both occur in jax's output).
OUTLINED = """
module @jit_dense_outlined {
  func.func public @main(%arg0: tensor<5x256xbf16>, %arg1: tensor<16x256xi8>, %arg2: tensor<16x4xbf16>, %arg3: tensor<16x4xbf16>) -> (tensor<5x16xbf16>) {
    %0 = call @dequantize(%arg1, %arg2, %arg3) : (tensor<16x256xi8>, tensor<16x4xbf16>, tensor<16x4xbf16>) -> tensor<16x256xbf16>
    %1 = stablehlo.dot_general %arg0, %0, contracting_dims = [1] x [1] : (tensor<5x256xbf16>, tensor<16x256xbf16>) -> tensor<5x16xbf16>
    %2 = func.call @twice(%1) : (tensor<5x16xbf16>) -> tensor<5x16xbf16>
    return %2 : tensor<5x16xbf16>
  }
  func.func private @dequantize(%arg0: tensor<16x256xi8>, %arg1: tensor<16x4xbf16>, %arg2: tensor<16x4xbf16>) -> tensor<16x256xbf16> {
    %0 = stablehlo.convert %arg0 : (tensor<16x256xi8>) -> tensor<16x256xbf16>
    %1 = stablehlo.broadcast_in_dim %arg2, dims = [0, 1] : (tensor<16x4xbf16>) -> tensor<16x4x64xbf16>
    %2 = stablehlo.reshape %1 : (tensor<16x4x64xbf16>) -> tensor<16x256xbf16>
    %3 = stablehlo.subtract %0, %2 : tensor<16x256xbf16>
    %4 = stablehlo.broadcast_in_dim %arg1, dims = [0, 1] : (tensor<16x4xbf16>) -> tensor<16x4x64xbf16>
    %5 = stablehlo.reshape %4 : (tensor<16x4x64xbf16>) -> tensor<16x256xbf16>
    %6 = stablehlo.multiply %3, %5 : tensor<16x256xbf16>
    return %6 : tensor<16x256xbf16>
  }
  func.func private @twice(%arg0: tensor<5x16xbf16>) -> tensor<5x16xbf16> {
    %0 = stablehlo.add %arg0, %arg0 : tensor<5x16xbf16>
    return %0 : tensor<5x16xbf16>
  }
}
"""

PER_CHANNEL = """
module @jit_dense_perchannel {
  func.func public @main(%arg0: tensor<5x128xbf16>, %arg1: tensor<128x16xi8>, %arg2: tensor<16xbf16>) -> (tensor<5x16xbf16>) {
    %0 = stablehlo.convert %arg1 : (tensor<128x16xi8>) -> tensor<128x16xbf16>
    %1 = stablehlo.dot_general %arg0, %0, contracting_dims = [1] x [0] : (tensor<5x128xbf16>, tensor<128x16xbf16>) -> tensor<5x16xbf16>
    %2 = stablehlo.broadcast_in_dim %arg2, dims = [1] : (tensor<16xbf16>) -> tensor<5x16xbf16>
    %3 = stablehlo.divide %1, %2 : tensor<5x16xbf16>
    return %3 : tensor<5x16xbf16>
  }
}
"""

_E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
_VTABLE = ", ".join(f"{v:.6e}" for v in _E2M1 + [-v for v in _E2M1])
_STABLE = ", ".join(f"{2.0 ** (b - 127):.9e}" if 0 < b < 255 else "0.000000e+00" for b in range(256))

MXFP4 = f"""
module @jit_dense_mxfp4 {{
  func.func public @main(%arg0: tensor<3x64xbf16>, %arg1: tensor<8x64xui8>, %arg2: tensor<8x2xui8>) -> (tensor<3x8xbf16>) {{
    %cst = stablehlo.constant dense<[{_VTABLE}]> : tensor<16xbf16>
    %cst_0 = stablehlo.constant dense<[{_STABLE}]> : tensor<256xf32>
    %0 = stablehlo.convert %arg1 : (tensor<8x64xui8>) -> tensor<8x64xi32>
    %1 = stablehlo.reshape %0 : (tensor<8x64xi32>) -> tensor<8x64x1xi32>
    %2 = "stablehlo.gather"(%cst, %1) <{{dimension_numbers = #stablehlo.gather<collapsed_slice_dims = [0], start_index_map = [0], index_vector_dim = 2>, indices_are_sorted = false, slice_sizes = array<i64: 1>}}> : (tensor<16xbf16>, tensor<8x64x1xi32>) -> tensor<8x64xbf16>
    %3 = stablehlo.convert %arg2 : (tensor<8x2xui8>) -> tensor<8x2xi32>
    %4 = stablehlo.reshape %3 : (tensor<8x2xi32>) -> tensor<8x2x1xi32>
    %5 = "stablehlo.gather"(%cst_0, %4) <{{dimension_numbers = #stablehlo.gather<collapsed_slice_dims = [0], start_index_map = [0], index_vector_dim = 2>, indices_are_sorted = false, slice_sizes = array<i64: 1>}}> : (tensor<256xf32>, tensor<8x2x1xi32>) -> tensor<8x2xf32>
    %6 = stablehlo.convert %5 : (tensor<8x2xf32>) -> tensor<8x2xbf16>
    %7 = stablehlo.reshape %2 : (tensor<8x64xbf16>) -> tensor<8x2x32xbf16>
    %8 = stablehlo.broadcast_in_dim %6, dims = [0, 1] : (tensor<8x2xbf16>) -> tensor<8x2x32xbf16>
    %9 = stablehlo.multiply %7, %8 : tensor<8x2x32xbf16>
    %10 = stablehlo.reshape %9 : (tensor<8x2x32xbf16>) -> tensor<8x64xbf16>
    %11 = stablehlo.dot_general %arg0, %10, contracting_dims = [1] x [1] : (tensor<3x64xbf16>, tensor<8x64xbf16>) -> tensor<3x8xbf16>
    return %11 : tensor<3x8xbf16>
  }}
}}
"""

def mxfp4_expert_program(e, m, k, n):
    """The MXFP4 chain of `MXFP4` over a stack of `e` expert weights `[e, n, k]` (one code per
    byte, one E8M0 byte per 32), contracted with `[e, m, k]` activations expert by expert."""
    g = k // 32
    return f"""
module @jit_expert_mxfp4 {{
  func.func public @main(%arg0: tensor<{e}x{m}x{k}xbf16>, %arg1: tensor<{e}x{n}x{k}xui8>, %arg2: tensor<{e}x{n}x{g}xui8>) -> (tensor<{e}x{m}x{n}xbf16>) {{
    %cst = stablehlo.constant dense<[{_VTABLE}]> : tensor<16xbf16>
    %cst_0 = stablehlo.constant dense<[{_STABLE}]> : tensor<256xf32>
    %0 = stablehlo.convert %arg1 : (tensor<{e}x{n}x{k}xui8>) -> tensor<{e}x{n}x{k}xi32>
    %1 = stablehlo.reshape %0 : (tensor<{e}x{n}x{k}xi32>) -> tensor<{e}x{n}x{k}x1xi32>
    %2 = "stablehlo.gather"(%cst, %1) <{{dimension_numbers = #stablehlo.gather<collapsed_slice_dims = [0], start_index_map = [0], index_vector_dim = 3>, indices_are_sorted = false, slice_sizes = array<i64: 1>}}> : (tensor<16xbf16>, tensor<{e}x{n}x{k}x1xi32>) -> tensor<{e}x{n}x{k}xbf16>
    %3 = stablehlo.convert %arg2 : (tensor<{e}x{n}x{g}xui8>) -> tensor<{e}x{n}x{g}xi32>
    %4 = stablehlo.reshape %3 : (tensor<{e}x{n}x{g}xi32>) -> tensor<{e}x{n}x{g}x1xi32>
    %5 = "stablehlo.gather"(%cst_0, %4) <{{dimension_numbers = #stablehlo.gather<collapsed_slice_dims = [0], start_index_map = [0], index_vector_dim = 3>, indices_are_sorted = false, slice_sizes = array<i64: 1>}}> : (tensor<256xf32>, tensor<{e}x{n}x{g}x1xi32>) -> tensor<{e}x{n}x{g}xf32>
    %6 = stablehlo.convert %5 : (tensor<{e}x{n}x{g}xf32>) -> tensor<{e}x{n}x{g}xbf16>
    %7 = stablehlo.reshape %2 : (tensor<{e}x{n}x{k}xbf16>) -> tensor<{e}x{n}x{g}x32xbf16>
    %8 = stablehlo.broadcast_in_dim %6, dims = [0, 1, 2] : (tensor<{e}x{n}x{g}xbf16>) -> tensor<{e}x{n}x{g}x32xbf16>
    %9 = stablehlo.multiply %7, %8 : tensor<{e}x{n}x{g}x32xbf16>
    %10 = stablehlo.reshape %9 : (tensor<{e}x{n}x{g}x32xbf16>) -> tensor<{e}x{n}x{k}xbf16>
    %11 = stablehlo.dot_general %arg0, %10, batching_dims = [0] x [0], contracting_dims = [2] x [2] : (tensor<{e}x{m}x{k}xbf16>, tensor<{e}x{n}x{k}xbf16>) -> tensor<{e}x{m}x{n}xbf16>
    return %11 : tensor<{e}x{m}x{n}xbf16>
  }}
}}
"""


def mxfp4_expert_inputs(e, m, k, n, seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((e, m, k), generator=g).to(torch.bfloat16).to(device)
    codes = torch.randint(0, 16, (e, n, k), generator=g, dtype=torch.uint8).to(device)
    scales = torch.randint(118, 126, (e, n, k // 32), generator=g, dtype=torch.uint8).to(device)
    return [x, codes, scales]


RMS_NORM = """
module @jit_embed_norm_dot {
  func.func public @main(%arg0: tensor<3x64xf32>, %arg1: tensor<4x1xi32>, %arg2: tensor<100x64xf32>, %arg3: tensor<4xf32>) -> (tensor<3x4xf32>) {
    %0 = "stablehlo.gather"(%arg2, %arg1) <{dimension_numbers = #stablehlo.gather<offset_dims = [1], collapsed_slice_dims = [0], start_index_map = [0], index_vector_dim = 1>, indices_are_sorted = false, slice_sizes = array<i64: 1, 64>}> : (tensor<100x64xf32>, tensor<4x1xi32>) -> tensor<4x64xf32>
    %1 = stablehlo.rsqrt %arg3 : tensor<4xf32>
    %2 = stablehlo.broadcast_in_dim %1, dims = [0] : (tensor<4xf32>) -> tensor<4x64xf32>
    %3 = stablehlo.multiply %0, %2 : tensor<4x64xf32>
    %4 = stablehlo.dot_general %arg0, %3, contracting_dims = [1] x [1] : (tensor<3x64xf32>, tensor<4x64xf32>) -> tensor<3x4xf32>
    return %4 : tensor<3x4xf32>
  }
}
"""


def sub_channel_inputs(seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((5, 256), generator=g).to(torch.bfloat16)
    codes = torch.randint(-8, 8, (16, 256), generator=g, dtype=torch.int8)
    scales = (torch.rand((16, 4), generator=g) * 0.02 + 0.002).to(torch.bfloat16)
    zeros = torch.randint(-3, 4, (16, 4), generator=g).to(torch.bfloat16)
    return [t.to(device) for t in (x, codes, scales, zeros)]


def per_channel_inputs(seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((5, 128), generator=g).to(torch.bfloat16)
    codes = torch.randint(-8, 8, (128, 16), generator=g, dtype=torch.int8)
    scale = (torch.rand((16,), generator=g) * 40 + 10).to(torch.bfloat16)
    return [t.to(device) for t in (x, codes, scale)]


def mxfp4_inputs(seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((3, 64), generator=g).to(torch.bfloat16)
    nib = torch.randint(0, 16, (8, 64), generator=g, dtype=torch.uint8)
    sbytes = torch.randint(119, 128, (8, 2), generator=g, dtype=torch.uint8)
    return [t.to(device) for t in (x, nib, sbytes)]


def sub_channel_program(m, k, n, gs=64, el="bf16"):
    """The sub-channel chain at any size (quantized operand on the right)."""
    g = k // gs
    return f"""
module @jit_dense_sub {{
  func.func public @main(%arg0: tensor<{m}x{k}x{el}>, %arg1: tensor<{n}x{k}xi8>, %arg2: tensor<{n}x{g}x{el}>, %arg3: tensor<{n}x{g}x{el}>) -> (tensor<{m}x{n}x{el}>) {{
    %0 = stablehlo.convert %arg1 : (tensor<{n}x{k}xi8>) -> tensor<{n}x{k}x{el}>
    %1 = stablehlo.broadcast_in_dim %arg3, dims = [0, 1] : (tensor<{n}x{g}x{el}>) -> tensor<{n}x{g}x{gs}x{el}>
    %2 = stablehlo.reshape %1 : (tensor<{n}x{g}x{gs}x{el}>) -> tensor<{n}x{k}x{el}>
    %3 = stablehlo.subtract %0, %2 : tensor<{n}x{k}x{el}>
    %4 = stablehlo.broadcast_in_dim %arg2, dims = [0, 1] : (tensor<{n}x{g}x{el}>) -> tensor<{n}x{g}x{gs}x{el}>
    %5 = stablehlo.reshape %4 : (tensor<{n}x{g}x{gs}x{el}>) -> tensor<{n}x{k}x{el}>
    %6 = stablehlo.multiply %3, %5 : tensor<{n}x{k}x{el}>
    %7 = stablehlo.dot_general %arg0, %6, contracting_dims = [1] x [1] : (tensor<{m}x{k}x{el}>, tensor<{n}x{k}x{el}>) -> tensor<{m}x{n}x{el}>
    return %7 : tensor<{m}x{n}x{el}>
  }}
}}
"""


def sub_channel_inputs_at(m, k, n, gs=64, seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((m, k), generator=g).to(torch.bfloat16)
    codes = torch.randint(-8, 8, (n, k), generator=g, dtype=torch.int8)
    scales = (torch.rand((n, k // gs), generator=g) * 0.02 + 0.002).to(torch.bfloat16)
    zeros = torch.randint(-3, 4, (n, k // gs), generator=g).to(torch.bfloat16)
    return [t.to(device) for t in (x, codes, scales, zeros)]


# A decode-style loop: three iterations of y <- dot(y_prev-shaped activations, W) with the
# quantized weight's parts closed over. jax lowers closed-over arrays as loop carries that the
# body returns unchanged, so inside the body they are block arguments (%iterArg_*), not @main's.
WHILE_LOOP = """
module @jit_decode_loop {
  func.func public @main(%arg0: tensor<5x256xbf16>, %arg1: tensor<256x256xi8>, %arg2: tensor<256x4xbf16>, %arg3: tensor<256x4xbf16>) -> (tensor<5x256xbf16>) {
    %c = stablehlo.constant dense<0> : tensor<i32>
    %c_0 = stablehlo.constant dense<3> : tensor<i32>
    %c_1 = stablehlo.constant dense<1> : tensor<i32>
    %0:5 = stablehlo.while(%iterArg = %c, %iterArg_2 = %arg1, %iterArg_3 = %arg2, %iterArg_4 = %arg3, %iterArg_5 = %arg0) : tensor<i32>, tensor<256x256xi8>, tensor<256x4xbf16>, tensor<256x4xbf16>, tensor<5x256xbf16>
     cond {
      %1 = stablehlo.compare LT, %iterArg, %c_0, SIGNED : (tensor<i32>, tensor<i32>) -> tensor<i1>
      stablehlo.return %1 : tensor<i1>
    } do {
      %1 = stablehlo.convert %iterArg_2 : (tensor<256x256xi8>) -> tensor<256x256xbf16>
      %2 = stablehlo.broadcast_in_dim %iterArg_4, dims = [0, 1] : (tensor<256x4xbf16>) -> tensor<256x4x64xbf16>
      %3 = stablehlo.reshape %2 : (tensor<256x4x64xbf16>) -> tensor<256x256xbf16>
      %4 = stablehlo.subtract %1, %3 : tensor<256x256xbf16>
      %5 = stablehlo.broadcast_in_dim %iterArg_3, dims = [0, 1] : (tensor<256x4xbf16>) -> tensor<256x4x64xbf16>
      %6 = stablehlo.reshape %5 : (tensor<256x4x64xbf16>) -> tensor<256x256xbf16>
      %7 = stablehlo.multiply %4, %6 : tensor<256x256xbf16>
      %8 = stablehlo.dot_general %iterArg_5, %7, contracting_dims = [1] x [1] : (tensor<5x256xbf16>, tensor<256x256xbf16>) -> tensor<5x256xbf16>
      %9 = stablehlo.add %iterArg, %c_1 : tensor<i32>
      stablehlo.return %9, %iterArg_2, %iterArg_3, %iterArg_4, %8 : tensor<i32>, tensor<256x256xi8>, tensor<256x4xbf16>, tensor<256x4xbf16>, tensor<5x256xbf16>
    }
    return %0#4 : tensor<5x256xbf16>
  }
}
"""


def while_loop_inputs(seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((5, 256), generator=g).to(torch.bfloat16)
    codes = torch.randint(-8, 8, (256, 256), generator=g, dtype=torch.int8)
    scales = (torch.rand((256, 4), generator=g) * 0.01 + 0.004).to(torch.bfloat16)
    zeros = torch.randint(-2, 3, (256, 4), generator=g).to(torch.bfloat16)
    return [t.to(device) for t in (x, codes, scales, zeros)]


def moe_program(t=6, d=64, e=4, f=64, gs=32, k=2):
    """A dense SwiGLU mixture-of-experts layer as jax.numpy code lowers it: every expert runs
    for every token, a top-k router's one-hot weights null the unselected ones
    (the reference's tests/test_moe.py:60-81 writes the same layer in jax)."""
    dg, fg = d // gs, f // gs
    return f"""
module @jit_moe {{
  func.func public @main(%arg0: tensor<{t}x{d}xbf16>, %arg1: tensor<{t}x{e}xf32>, %arg2: tensor<{e}x{f}x{d}xi8>, %arg3: tensor<{e}x{f}x{dg}xbf16>, %arg4: tensor<{e}x{f}x{d}xi8>, %arg5: tensor<{e}x{f}x{dg}xbf16>, %arg6: tensor<{e}x{d}x{f}xi8>, %arg7: tensor<{e}x{d}x{fg}xbf16>) -> (tensor<{t}x{d}xbf16>) {{
    %cst = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %cst_0 = stablehlo.constant dense<0.000000e+00> : tensor<bf16>
    %0:2 = chlo.top_k(%arg1, k = {k}) : tensor<{t}x{e}xf32> -> (tensor<{t}x{k}xf32>, tensor<{t}x{k}xi32>)
    %1 = stablehlo.exponential %0#0 : tensor<{t}x{k}xf32>
    %2 = stablehlo.reduce(%1 init: %cst) applies stablehlo.add across dimensions = [1] : (tensor<{t}x{k}xf32>, tensor<f32>) -> tensor<{t}xf32>
    %3 = stablehlo.broadcast_in_dim %2, dims = [0] : (tensor<{t}xf32>) -> tensor<{t}x{k}xf32>
    %4 = stablehlo.divide %1, %3 : tensor<{t}x{k}xf32>
    %5 = stablehlo.iota dim = 2 : tensor<{t}x{k}x{e}xi32>
    %6 = stablehlo.broadcast_in_dim %0#1, dims = [0, 1] : (tensor<{t}x{k}xi32>) -> tensor<{t}x{k}x{e}xi32>
    %7 = stablehlo.compare EQ, %6, %5, SIGNED : (tensor<{t}x{k}x{e}xi32>, tensor<{t}x{k}x{e}xi32>) -> tensor<{t}x{k}x{e}xi1>
    %8 = stablehlo.convert %7 : (tensor<{t}x{k}x{e}xi1>) -> tensor<{t}x{k}x{e}xf32>
    %9 = stablehlo.broadcast_in_dim %4, dims = [0, 1] : (tensor<{t}x{k}xf32>) -> tensor<{t}x{k}x{e}xf32>
    %10 = stablehlo.multiply %8, %9 : tensor<{t}x{k}x{e}xf32>
    %11 = stablehlo.reduce(%10 init: %cst) applies stablehlo.add across dimensions = [1] : (tensor<{t}x{k}x{e}xf32>, tensor<f32>) -> tensor<{t}x{e}xf32>
    %12 = stablehlo.convert %arg2 : (tensor<{e}x{f}x{d}xi8>) -> tensor<{e}x{f}x{d}xbf16>
    %13 = stablehlo.broadcast_in_dim %arg3, dims = [0, 1, 2] : (tensor<{e}x{f}x{dg}xbf16>) -> tensor<{e}x{f}x{dg}x{gs}xbf16>
    %14 = stablehlo.reshape %13 : (tensor<{e}x{f}x{dg}x{gs}xbf16>) -> tensor<{e}x{f}x{d}xbf16>
    %15 = stablehlo.multiply %12, %14 : tensor<{e}x{f}x{d}xbf16>
    %16 = stablehlo.dot_general %arg0, %15, contracting_dims = [1] x [2] : (tensor<{t}x{d}xbf16>, tensor<{e}x{f}x{d}xbf16>) -> tensor<{t}x{e}x{f}xbf16>
    %17 = stablehlo.convert %arg4 : (tensor<{e}x{f}x{d}xi8>) -> tensor<{e}x{f}x{d}xbf16>
    %18 = stablehlo.broadcast_in_dim %arg5, dims = [0, 1, 2] : (tensor<{e}x{f}x{dg}xbf16>) -> tensor<{e}x{f}x{dg}x{gs}xbf16>
    %19 = stablehlo.reshape %18 : (tensor<{e}x{f}x{dg}x{gs}xbf16>) -> tensor<{e}x{f}x{d}xbf16>
    %20 = stablehlo.multiply %17, %19 : tensor<{e}x{f}x{d}xbf16>
    %21 = stablehlo.dot_general %arg0, %20, contracting_dims = [1] x [2] : (tensor<{t}x{d}xbf16>, tensor<{e}x{f}x{d}xbf16>) -> tensor<{t}x{e}x{f}xbf16>
    %22 = stablehlo.logistic %16 : tensor<{t}x{e}x{f}xbf16>
    %23 = stablehlo.multiply %16, %22 : tensor<{t}x{e}x{f}xbf16>
    %24 = stablehlo.multiply %23, %21 : tensor<{t}x{e}x{f}xbf16>
    %25 = stablehlo.transpose %24, dims = [1, 0, 2] : (tensor<{t}x{e}x{f}xbf16>) -> tensor<{e}x{t}x{f}xbf16>
    %26 = stablehlo.convert %arg6 : (tensor<{e}x{d}x{f}xi8>) -> tensor<{e}x{d}x{f}xbf16>
    %27 = stablehlo.broadcast_in_dim %arg7, dims = [0, 1, 2] : (tensor<{e}x{d}x{fg}xbf16>) -> tensor<{e}x{d}x{fg}x{gs}xbf16>
    %28 = stablehlo.reshape %27 : (tensor<{e}x{d}x{fg}x{gs}xbf16>) -> tensor<{e}x{d}x{f}xbf16>
    %29 = stablehlo.multiply %26, %28 : tensor<{e}x{d}x{f}xbf16>
    %30 = stablehlo.dot_general %25, %29, batching_dims = [0] x [0], contracting_dims = [2] x [2] : (tensor<{e}x{t}x{f}xbf16>, tensor<{e}x{d}x{f}xbf16>) -> tensor<{e}x{t}x{d}xbf16>
    %31 = stablehlo.convert %11 : (tensor<{t}x{e}xf32>) -> tensor<{t}x{e}xbf16>
    %32 = stablehlo.broadcast_in_dim %31, dims = [1, 0] : (tensor<{t}x{e}xbf16>) -> tensor<{e}x{t}x{d}xbf16>
    %33 = stablehlo.multiply %30, %32 : tensor<{e}x{t}x{d}xbf16>
    %34 = stablehlo.reduce(%33 init: %cst_0) applies stablehlo.add across dimensions = [0] : (tensor<{e}x{t}x{d}xbf16>, tensor<bf16>) -> tensor<{t}x{d}xbf16>
    return %34 : tensor<{t}x{d}xbf16>
  }}
}}
"""


def moe_program_float(t=6, d=64, e=4, f=64, k=2):
    """The same dense SwiGLU mixture-of-experts layer with FLOAT (bf16) expert weights: nothing
    to dequantize, the three dots read their weights straight from the arguments."""
    return f"""
module @jit_moe_float {{
  func.func public @main(%arg0: tensor<{t}x{d}xbf16>, %arg1: tensor<{t}x{e}xf32>, %arg2: tensor<{e}x{f}x{d}xbf16>, %arg3: tensor<{e}x{f}x{d}xbf16>, %arg4: tensor<{e}x{d}x{f}xbf16>) -> (tensor<{t}x{d}xbf16>) {{
    %cst = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %cst_0 = stablehlo.constant dense<0.000000e+00> : tensor<bf16>
    %0:2 = chlo.top_k(%arg1, k = {k}) : tensor<{t}x{e}xf32> -> (tensor<{t}x{k}xf32>, tensor<{t}x{k}xi32>)
    %1 = stablehlo.exponential %0#0 : tensor<{t}x{k}xf32>
    %2 = stablehlo.reduce(%1 init: %cst) applies stablehlo.add across dimensions = [1] : (tensor<{t}x{k}xf32>, tensor<f32>) -> tensor<{t}xf32>
    %3 = stablehlo.broadcast_in_dim %2, dims = [0] : (tensor<{t}xf32>) -> tensor<{t}x{k}xf32>
    %4 = stablehlo.divide %1, %3 : tensor<{t}x{k}xf32>
    %5 = stablehlo.iota dim = 2 : tensor<{t}x{k}x{e}xi32>
    %6 = stablehlo.broadcast_in_dim %0#1, dims = [0, 1] : (tensor<{t}x{k}xi32>) -> tensor<{t}x{k}x{e}xi32>
    %7 = stablehlo.compare EQ, %6, %5, SIGNED : (tensor<{t}x{k}x{e}xi32>, tensor<{t}x{k}x{e}xi32>) -> tensor<{t}x{k}x{e}xi1>
    %8 = stablehlo.convert %7 : (tensor<{t}x{k}x{e}xi1>) -> tensor<{t}x{k}x{e}xf32>
    %9 = stablehlo.broadcast_in_dim %4, dims = [0, 1] : (tensor<{t}x{k}xf32>) -> tensor<{t}x{k}x{e}xf32>
    %10 = stablehlo.multiply %8, %9 : tensor<{t}x{k}x{e}xf32>
    %11 = stablehlo.reduce(%10 init: %cst) applies stablehlo.add across dimensions = [1] : (tensor<{t}x{k}x{e}xf32>, tensor<f32>) -> tensor<{t}x{e}xf32>
    %16 = stablehlo.dot_general %arg0, %arg2, contracting_dims = [1] x [2] : (tensor<{t}x{d}xbf16>, tensor<{e}x{f}x{d}xbf16>) -> tensor<{t}x{e}x{f}xbf16>
    %21 = stablehlo.dot_general %arg0, %arg3, contracting_dims = [1] x [2] : (tensor<{t}x{d}xbf16>, tensor<{e}x{f}x{d}xbf16>) -> tensor<{t}x{e}x{f}xbf16>
    %22 = stablehlo.logistic %16 : tensor<{t}x{e}x{f}xbf16>
    %23 = stablehlo.multiply %16, %22 : tensor<{t}x{e}x{f}xbf16>
    %24 = stablehlo.multiply %23, %21 : tensor<{t}x{e}x{f}xbf16>
    %25 = stablehlo.transpose %24, dims = [1, 0, 2] : (tensor<{t}x{e}x{f}xbf16>) -> tensor<{e}x{t}x{f}xbf16>
    %30 = stablehlo.dot_general %25, %arg4, batching_dims = [0] x [0], contracting_dims = [2] x [2] : (tensor<{e}x{t}x{f}xbf16>, tensor<{e}x{d}x{f}xbf16>) -> tensor<{e}x{t}x{d}xbf16>
    %31 = stablehlo.convert %11 : (tensor<{t}x{e}xf32>) -> tensor<{t}x{e}xbf16>
    %32 = stablehlo.broadcast_in_dim %31, dims = [1, 0] : (tensor<{t}x{e}xbf16>) -> tensor<{e}x{t}x{d}xbf16>
    %33 = stablehlo.multiply %30, %32 : tensor<{e}x{t}x{d}xbf16>
    %34 = stablehlo.reduce(%33 init: %cst_0) applies stablehlo.add across dimensions = [0] : (tensor<{e}x{t}x{d}xbf16>, tensor<bf16>) -> tensor<{t}x{d}xbf16>
    return %34 : tensor<{t}x{d}xbf16>
  }}
}}
"""


def moe_float_inputs(t=6, d=64, e=4, f=64, seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn((t, d), generator=g) * 0.5).to(torch.bfloat16)
    logits = torch.randn((t, e), generator=g)
    w1 = (torch.randn((e, f, d), generator=g) * 0.1).to(torch.bfloat16)
    w3 = (torch.randn((e, f, d), generator=g) * 0.1).to(torch.bfloat16)
    w2 = (torch.randn((e, d, f), generator=g) * 0.1).to(torch.bfloat16)
    return [a.to(device) for a in (x, logits, w1, w3, w2)]


def moe_inputs(t=6, d=64, e=4, f=64, gs=32, seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn((t, d), generator=g) * 0.5).to(torch.bfloat16)
    logits = torch.randn((t, e), generator=g)

    def pack(n, kk):
        codes = torch.randint(-8, 8, (e, n, kk), generator=g, dtype=torch.int8)
        scales = (torch.rand((e, n, kk // gs), generator=g) * 0.02 + 0.01).to(torch.bfloat16)
        return codes, scales

    cg, sg = pack(f, d)
    cu, su = pack(f, d)
    cd, sd = pack(d, f)
    return [a.to(device) for a in (x, logits, cg, sg, cu, su, cd, sd)]


_ROUTER = """    %cst = stablehlo.constant dense<0.000000e+00> : tensor<f32>
    %cst_0 = stablehlo.constant dense<0.000000e+00> : tensor<bf16>
    %0:2 = chlo.top_k(%arg1, k = {k}) : tensor<{t}x{e}xf32> -> (tensor<{t}x{k}xf32>, tensor<{t}x{k}xi32>)
    %1 = stablehlo.exponential %0#0 : tensor<{t}x{k}xf32>
    %2 = stablehlo.reduce(%1 init: %cst) applies stablehlo.add across dimensions = [1] : (tensor<{t}x{k}xf32>, tensor<f32>) -> tensor<{t}xf32>
    %3 = stablehlo.broadcast_in_dim %2, dims = [0] : (tensor<{t}xf32>) -> tensor<{t}x{k}xf32>
    %4 = stablehlo.divide %1, %3 : tensor<{t}x{k}xf32>
    %5 = stablehlo.iota dim = 2 : tensor<{t}x{k}x{e}xi32>
    %6 = stablehlo.broadcast_in_dim %0#1, dims = [0, 1] : (tensor<{t}x{k}xi32>) -> tensor<{t}x{k}x{e}xi32>
    %7 = stablehlo.compare EQ, %6, %5, SIGNED : (tensor<{t}x{k}x{e}xi32>, tensor<{t}x{k}x{e}xi32>) -> tensor<{t}x{k}x{e}xi1>
    %8 = stablehlo.convert %7 : (tensor<{t}x{k}x{e}xi1>) -> tensor<{t}x{k}x{e}xf32>
    %9 = stablehlo.broadcast_in_dim %4, dims = [0, 1] : (tensor<{t}x{k}xf32>) -> tensor<{t}x{k}x{e}xf32>
    %10 = stablehlo.multiply %8, %9 : tensor<{t}x{k}x{e}xf32>
    %11 = stablehlo.reduce(%10 init: %cst) applies stablehlo.add across dimensions = [1] : (tensor<{t}x{k}x{e}xf32>, tensor<f32>) -> tensor<{t}x{e}xf32>
"""


def moe_program_glu_bias(t=6, d=64, e=4, f=64, k=2):
    """A dense expert layer of the gpt-oss kind, float (bf16) weights: ONE gate/up projection with
    interleaved output features and a per-expert bias, `gate` clamped from above and `up` clamped
    both ways, `(up + 1) * gate * logistic(1.702 * gate)`, a down projection with a per-expert
    bias. Nothing of the SwiGLU shape: strided slices, clamps, scalar constants and biases that
    have the expert axis but no token axis sit between the two dots."""
    f2 = 2 * f
    return f"""
module @jit_moe_glu {{
  func.func public @main(%arg0: tensor<{t}x{d}xbf16>, %arg1: tensor<{t}x{e}xf32>, %arg2: tensor<{e}x{f2}x{d}xbf16>, %arg3: tensor<{e}x{f2}xbf16>, %arg4: tensor<{e}x{d}x{f}xbf16>, %arg5: tensor<{e}x{d}xbf16>) -> (tensor<{t}x{d}xbf16>) {{
{_ROUTER.format(t=t, e=e, k=k)}    %lim = stablehlo.constant dense<7.000000e+00> : tensor<bf16>
    %nlim = stablehlo.constant dense<-7.000000e+00> : tensor<bf16>
    %alpha = stablehlo.constant dense<1.703130e+00> : tensor<{t}x{e}x{f}xbf16>
    %one = stablehlo.constant dense<1.000000e+00> : tensor<bf16>
    %16 = stablehlo.dot_general %arg0, %arg2, contracting_dims = [1] x [2] : (tensor<{t}x{d}xbf16>, tensor<{e}x{f2}x{d}xbf16>) -> tensor<{t}x{e}x{f2}xbf16>
    %17 = stablehlo.broadcast_in_dim %arg3, dims = [1, 2] : (tensor<{e}x{f2}xbf16>) -> tensor<{t}x{e}x{f2}xbf16>
    %18 = stablehlo.add %16, %17 : tensor<{t}x{e}x{f2}xbf16>
    %19 = stablehlo.slice %18 [0:{t}, 0:{e}, 0:{f2}:2] : (tensor<{t}x{e}x{f2}xbf16>) -> tensor<{t}x{e}x{f}xbf16>
    %20 = stablehlo.slice %18 [0:{t}, 0:{e}, 1:{f2}:2] : (tensor<{t}x{e}x{f2}xbf16>) -> tensor<{t}x{e}x{f}xbf16>
    %21 = stablehlo.broadcast_in_dim %lim, dims = [] : (tensor<bf16>) -> tensor<{t}x{e}x{f}xbf16>
    %22 = stablehlo.minimum %19, %21 : tensor<{t}x{e}x{f}xbf16>
    %23 = stablehlo.clamp %nlim, %20, %lim : (tensor<bf16>, tensor<{t}x{e}x{f}xbf16>, tensor<bf16>) -> tensor<{t}x{e}x{f}xbf16>
    %24 = stablehlo.multiply %22, %alpha : tensor<{t}x{e}x{f}xbf16>
    %25 = stablehlo.logistic %24 : tensor<{t}x{e}x{f}xbf16>
    %26 = stablehlo.multiply %22, %25 : tensor<{t}x{e}x{f}xbf16>
    %27 = stablehlo.broadcast_in_dim %one, dims = [] : (tensor<bf16>) -> tensor<{t}x{e}x{f}xbf16>
    %28 = stablehlo.add %23, %27 : tensor<{t}x{e}x{f}xbf16>
    %29 = stablehlo.multiply %28, %26 : tensor<{t}x{e}x{f}xbf16>
    %30 = stablehlo.transpose %29, dims = [1, 0, 2] : (tensor<{t}x{e}x{f}xbf16>) -> tensor<{e}x{t}x{f}xbf16>
    %31 = stablehlo.dot_general %30, %arg4, batching_dims = [0] x [0], contracting_dims = [2] x [2] : (tensor<{e}x{t}x{f}xbf16>, tensor<{e}x{d}x{f}xbf16>) -> tensor<{e}x{t}x{d}xbf16>
    %32 = stablehlo.broadcast_in_dim %arg5, dims = [0, 2] : (tensor<{e}x{d}xbf16>) -> tensor<{e}x{t}x{d}xbf16>
    %33 = stablehlo.add %31, %32 : tensor<{e}x{t}x{d}xbf16>
    %34 = stablehlo.convert %11 : (tensor<{t}x{e}xf32>) -> tensor<{t}x{e}xbf16>
    %35 = stablehlo.broadcast_in_dim %34, dims = [1, 0] : (tensor<{t}x{e}xbf16>) -> tensor<{e}x{t}x{d}xbf16>
    %36 = stablehlo.multiply %33, %35 : tensor<{e}x{t}x{d}xbf16>
    %37 = stablehlo.reduce(%36 init: %cst_0) applies stablehlo.add across dimensions = [0] : (tensor<{e}x{t}x{d}xbf16>, tensor<bf16>) -> tensor<{t}x{d}xbf16>
    return %37 : tensor<{t}x{d}xbf16>
  }}
}}
"""


def moe_glu_bias_inputs(t=6, d=64, e=4, f=64, seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn((t, d), generator=g) * 0.5).to(torch.bfloat16)
    logits = torch.randn((t, e), generator=g)
    w1 = (torch.randn((e, 2 * f, d), generator=g) * 0.1).to(torch.bfloat16)
    b1 = (torch.randn((e, 2 * f), generator=g) * 0.1).to(torch.bfloat16)
    w2 = (torch.randn((e, d, f), generator=g) * 0.1).to(torch.bfloat16)
    b2 = (torch.randn((e, d), generator=g) * 0.1).to(torch.bfloat16)
    return [a.to(device) for a in (x, logits, w1, b1, w2, b2)]


def moe_program_gelu_quant(t=6, d=64, e=4, f=64, gs=32, k=2):
    """Quantized experts (int8 codes, group scales) with a two-dot tanh-GELU feed-forward per
    expert and a per-expert output scale: `down(gelu(up(x))) * gain[e]`. Not the SwiGLU shape."""
    dg, fg = d // gs, f // gs
    return f"""
module @jit_moe_gelu {{
  func.func public @main(%arg0: tensor<{t}x{d}xbf16>, %arg1: tensor<{t}x{e}xf32>, %arg2: tensor<{e}x{f}x{d}xi8>, %arg3: tensor<{e}x{f}x{dg}xbf16>, %arg4: tensor<{e}x{d}x{f}xi8>, %arg5: tensor<{e}x{d}x{fg}xbf16>, %arg6: tensor<{e}xbf16>) -> (tensor<{t}x{d}xbf16>) {{
{_ROUTER.format(t=t, e=e, k=k)}    %half = stablehlo.constant dense<5.000000e-01> : tensor<bf16>
    %c1 = stablehlo.constant dense<4.467770e-02> : tensor<bf16>
    %c2 = stablehlo.constant dense<7.968750e-01> : tensor<bf16>
    %one = stablehlo.constant dense<1.000000e+00> : tensor<bf16>
    %12 = stablehlo.convert %arg2 : (tensor<{e}x{f}x{d}xi8>) -> tensor<{e}x{f}x{d}xbf16>
    %13 = stablehlo.broadcast_in_dim %arg3, dims = [0, 1, 2] : (tensor<{e}x{f}x{dg}xbf16>) -> tensor<{e}x{f}x{dg}x{gs}xbf16>
    %14 = stablehlo.reshape %13 : (tensor<{e}x{f}x{dg}x{gs}xbf16>) -> tensor<{e}x{f}x{d}xbf16>
    %15 = stablehlo.multiply %12, %14 : tensor<{e}x{f}x{d}xbf16>
    %16 = stablehlo.dot_general %arg0, %15, contracting_dims = [1] x [2] : (tensor<{t}x{d}xbf16>, tensor<{e}x{f}x{d}xbf16>) -> tensor<{t}x{e}x{f}xbf16>
    %h = stablehlo.broadcast_in_dim %half, dims = [] : (tensor<bf16>) -> tensor<{t}x{e}x{f}xbf16>
    %k1 = stablehlo.broadcast_in_dim %c1, dims = [] : (tensor<bf16>) -> tensor<{t}x{e}x{f}xbf16>
    %k2 = stablehlo.broadcast_in_dim %c2, dims = [] : (tensor<bf16>) -> tensor<{t}x{e}x{f}xbf16>
    %o = stablehlo.broadcast_in_dim %one, dims = [] : (tensor<bf16>) -> tensor<{t}x{e}x{f}xbf16>
    %17 = stablehlo.multiply %16, %16 : tensor<{t}x{e}x{f}xbf16>
    %18 = stablehlo.multiply %17, %16 : tensor<{t}x{e}x{f}xbf16>
    %19 = stablehlo.multiply %18, %k1 : tensor<{t}x{e}x{f}xbf16>
    %20 = stablehlo.add %16, %19 : tensor<{t}x{e}x{f}xbf16>
    %21 = stablehlo.multiply %20, %k2 : tensor<{t}x{e}x{f}xbf16>
    %22 = stablehlo.tanh %21 : tensor<{t}x{e}x{f}xbf16>
    %23 = stablehlo.add %22, %o : tensor<{t}x{e}x{f}xbf16>
    %24 = stablehlo.multiply %16, %h : tensor<{t}x{e}x{f}xbf16>
    %25 = stablehlo.multiply %24, %23 : tensor<{t}x{e}x{f}xbf16>
    %26 = stablehlo.transpose %25, dims = [1, 0, 2] : (tensor<{t}x{e}x{f}xbf16>) -> tensor<{e}x{t}x{f}xbf16>
    %27 = stablehlo.convert %arg4 : (tensor<{e}x{d}x{f}xi8>) -> tensor<{e}x{d}x{f}xbf16>
    %28 = stablehlo.broadcast_in_dim %arg5, dims = [0, 1, 2] : (tensor<{e}x{d}x{fg}xbf16>) -> tensor<{e}x{d}x{fg}x{gs}xbf16>
    %29 = stablehlo.reshape %28 : (tensor<{e}x{d}x{fg}x{gs}xbf16>) -> tensor<{e}x{d}x{f}xbf16>
    %30 = stablehlo.multiply %27, %29 : tensor<{e}x{d}x{f}xbf16>
    %31 = stablehlo.dot_general %26, %30, batching_dims = [0] x [0], contracting_dims = [2] x [2] : (tensor<{e}x{t}x{f}xbf16>, tensor<{e}x{d}x{f}xbf16>) -> tensor<{e}x{t}x{d}xbf16>
    %32 = stablehlo.broadcast_in_dim %arg6, dims = [0] : (tensor<{e}xbf16>) -> tensor<{e}x{t}x{d}xbf16>
    %33 = stablehlo.multiply %31, %32 : tensor<{e}x{t}x{d}xbf16>
    %34 = stablehlo.convert %11 : (tensor<{t}x{e}xf32>) -> tensor<{t}x{e}xbf16>
    %35 = stablehlo.broadcast_in_dim %34, dims = [1, 0] : (tensor<{t}x{e}xbf16>) -> tensor<{e}x{t}x{d}xbf16>
    %36 = stablehlo.multiply %33, %35 : tensor<{e}x{t}x{d}xbf16>
    %37 = stablehlo.reduce(%36 init: %cst_0) applies stablehlo.add across dimensions = [0] : (tensor<{e}x{t}x{d}xbf16>, tensor<bf16>) -> tensor<{t}x{d}xbf16>
    return %37 : tensor<{t}x{d}xbf16>
  }}
}}
"""


def moe_gelu_quant_inputs(t=6, d=64, e=4, f=64, gs=32, seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn((t, d), generator=g) * 0.5).to(torch.bfloat16)
    logits = torch.randn((t, e), generator=g)
    cu = torch.randint(-8, 8, (e, f, d), generator=g, dtype=torch.int8)
    su = (torch.rand((e, f, d // gs), generator=g) * 0.02 + 0.01).to(torch.bfloat16)
    cd = torch.randint(-8, 8, (e, d, f), generator=g, dtype=torch.int8)
    sd = (torch.rand((e, d, f // gs), generator=g) * 0.02 + 0.01).to(torch.bfloat16)
    gain = (torch.rand((e,), generator=g) + 0.5).to(torch.bfloat16)
    return [a.to(device) for a in (x, logits, cu, su, cd, sd, gain)]
