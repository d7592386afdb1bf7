"""B200-native fused dequantize-and-matmul behind metaljax's recognizer interface.

`metaljax_b200.qmm` mirrors the reference's `metaljax.qmm` (pack primitives, `Match` /
`State`, `emit`), `metaljax_b200.moe` its expert-gather `emit`; both end in calls into
`libqmm.so` (hand-written CUDA for sm_100a, C ABI in `include/qmm.h`) through ctypes with
tensors passed as DLPack views. There is no CPU fallback: without the library, or
without a CUDA device, the fused ops raise.
"""

__version__ = "0.1.0"
