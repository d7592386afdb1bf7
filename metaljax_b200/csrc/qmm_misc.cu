// Element-wise helpers around the fused op: full dequantization of a packed weight (the
// reference pins its packed layout with mx.dequantize, tests/test_qmm.py:121 and
// tests/test_qmm_mxfp4.py:192) and the packer itself (src/metaljax/qmm.py:206-232).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "qmm_internal.h"

namespace qmm {
namespace {

__device__ __forceinline__ float table_at(const void* p, int dtype, int64_t i) {
  if (dtype == QMM_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  if (dtype == QMM_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  return reinterpret_cast<const float*>(p)[i];
}

__device__ __forceinline__ float e2m1_value(uint32_t code) {
  // magnitude bits (e1 e0 m) -> 0, .5, 1, 1.5, 2, 3, 4, 6
  const uint32_t m3 = code & 7u;
  const float mag = m3 < 2u ? 0.5f * static_cast<float>(m3)
                            : __uint_as_float(((m3 >> 1) + 126u) << 23 | (m3 & 1u) << 22);
  return (code & 8u) ? -mag : mag;
}

// One thread per packed word; a word never straddles a group (groups are >= 32 elements).
__global__ void dequantize_kernel(const uint32_t* __restrict__ w, const void* __restrict__ scales,
                                  const void* __restrict__ biases, int table_dtype,
                                  void* __restrict__ out, int out_dtype, int64_t total_words,
                                  int64_t words_per_row, int64_t K, int group_size, int bits,
                                  int mode) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int epw = 32 / bits;
  const int64_t groups = K / group_size;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total_words;
       i += stride) {
    const int64_t row = i / words_per_row, wi = i % words_per_row;
    const int64_t k0 = wi * epw;
    const int64_t t = row * groups + k0 / group_size;
    const uint32_t word = w[i];
    float s, b = 0.0f;
    if (mode == QMM_MODE_MXFP4) {
      const uint32_t e8 = reinterpret_cast<const uint8_t*>(scales)[t];
      s = __uint_as_float(e8 ? (e8 << 23) : 0x00400000u);
    } else {
      s = table_at(scales, table_dtype, t);
      b = table_at(biases, table_dtype, t);
    }
    for (int e = 0; e < epw; ++e) {
      const uint32_t code = (word >> (e * bits)) & ((1u << bits) - 1u);
      const float v = (mode == QMM_MODE_MXFP4) ? e2m1_value(code) * s
                                               : fmaf(s, static_cast<float>(code), b);
      const int64_t o = row * K + k0 + e;
      if (out_dtype == QMM_BF16) reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(v);
      else if (out_dtype == QMM_F16) reinterpret_cast<__half*>(out)[o] = __float2half_rn(v);
      else reinterpret_cast<float*>(out)[o] = v;
    }
  }
}

// One thread per output word: gathers 32/bits codes (one byte each) and masks them.
__global__ void pack_codes_kernel(const uint8_t* __restrict__ codes, uint32_t* __restrict__ out,
                                  int64_t total_words, int bits) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int epw = 32 / bits;
  const uint32_t mask = (1u << bits) - 1u;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total_words;
       i += stride) {
    uint32_t word = 0;
    if (epw == 8) {
      const uint2 v = *reinterpret_cast<const uint2*>(codes + i * 8);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        word |= ((v.x >> (8 * e)) & mask) << (4 * e);
        word |= ((v.y >> (8 * e)) & mask) << (4 * (e + 4));
      }
    } else {
      word = *reinterpret_cast<const uint32_t*>(codes + i * 4);
    }
    out[i] = word;
  }
}

int grid_for(int64_t n, int block) {
  int64_t g = (n + block - 1) / block;
  const int64_t cap = 148 * 16;
  return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

int launch_dequantize(const uint32_t* w, const void* scales, const void* biases, int table_dtype,
                      void* out, int out_dtype, int64_t rows, int64_t K, int group_size, int bits,
                      int mode, cudaStream_t stream) {
  const int64_t words_per_row = K * bits / 32;
  const int64_t total = rows * words_per_row;
  if (total == 0) return QMM_OK;
  dequantize_kernel<<<grid_for(total, 256), 256, 0, stream>>>(
      w, scales, biases, table_dtype, out, out_dtype, total, words_per_row, K, group_size, bits,
      mode);
  count_launch();
  return check_launch("dequantize_kernel");
}

int launch_pack_codes(const uint8_t* codes, uint32_t* out, int64_t rows, int64_t K, int bits,
                      cudaStream_t stream) {
  const int64_t total = rows * (K * bits / 32);
  if (total == 0) return QMM_OK;
  pack_codes_kernel<<<grid_for(total, 256), 256, 0, stream>>>(codes, out, total, bits);
  count_launch();
  return check_launch("pack_codes_kernel");
}

}  // namespace qmm
