// The element-wise steps between the grouped products of a gathered expert block
// (eterevsky/metaljax src/metaljax/moe.py:1425-1461): the SwiGLU of the gate and up products, and
// the routed sum -- every token's K expert outputs times their routing weights, added in float32.
// Both are plain HBM-bound passes; they exist so that the block does not make three extra
// round trips through pair-sized float32 temporaries.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <type_traits>

#include "qmm_internal.h"

namespace qmm {
namespace {

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      f[2 * i] = __uint_as_float(u[i] << 16);
      f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    } else {
      const float2 h = __half22float2(*reinterpret_cast<const __half2*>(&u[i]));
      f[2 * i] = h.x;
      f[2 * i + 1] = h.y;
    }
  }
}

template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint32_t u[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      const __nv_bfloat162 v = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      u[i] = *reinterpret_cast<const uint32_t*>(&v);
    } else {
      const __half2 v = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      u[i] = *reinterpret_cast<const uint32_t*>(&v);
    }
  }
  return make_uint4(u[0], u[1], u[2], u[3]);
}

// out = silu(gate) * up, the product rounded as the two-step form rounds it: silu to T, then
// the product to T.
template <typename T>
__global__ void silu_mul_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up, uint4* __restrict__ out,
                                int64_t pieces) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < pieces; i += stride) {
    float g[8], u[8];
    unpack8<T>(__ldcs(gate + i), g);
    unpack8<T>(__ldcs(up + i), u);
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] = g[k] / (1.0f + __expf(-g[k]));
    unpack8<T>(pack8<T>(g), g);
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] *= u[k];
    out[i] = pack8<T>(g);
  }
}

// out[t] = sum_k weights[t, k] * rows[row_of_pair[t * K + k]] in float32 (products rounded, then
// added in k order, as separate multiply and add steps do), cast to T.
template <typename T>
__global__ void routed_sum_kernel(const uint4* __restrict__ rows, const int64_t* __restrict__ row_of_pair,
                                  const float* __restrict__ weights, uint4* __restrict__ out, int64_t tokens, int k,
                                  int64_t pieces, int64_t total_rows, int* status) {
  for (int64_t t = blockIdx.x; t < tokens; t += gridDim.x) {
    for (int64_t pc = threadIdx.x; pc < pieces; pc += blockDim.x) {
      float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
      for (int j = 0; j < k; ++j) {
        int64_t r = row_of_pair[t * k + j];
        if (r < 0 || r >= total_rows) {                  // never followed: reported and clamped
          if (pc == 0) atomicCAS(status, 0, QMM_DEVICE_BAD_INDEX);
          r = r < 0 ? 0 : total_rows - 1;
        }
        const float w = weights[t * k + j];
        float v[8];
        unpack8<T>(__ldcs(rows + r * pieces + pc), v);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = __fadd_rn(acc[e], __fmul_rn(v[e], w));
      }
      out[t * pieces + pc] = pack8<T>(acc);
    }
  }
}

}  // namespace
}  // namespace qmm

using namespace qmm;

extern "C" int qmm_moe_silu_mul(const void* gate, const void* up, void* out, int64_t elements, int dtype, void* stream) {
  if (elements < 0 || elements % 8) return fail(QMM_ERR_SHAPE, "moe_silu_mul: element count must be a multiple of 8");
  if (elements == 0) return QMM_OK;                     // (an expert-parallel rank that was sent no rows: empty arrays have no address)
  if (!gate || !up || !out) return fail(QMM_ERR_NULL, "moe_silu_mul: null pointer");
  if (dtype != QMM_BF16 && dtype != QMM_F16) return fail(QMM_ERR_DTYPE, "moe_silu_mul: bf16 or f16");
  if ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(out)) & 15)
    return fail(QMM_ERR_LAYOUT, "moe_silu_mul: pointers must be 16-byte aligned");
  if (elements == 0) return QMM_OK;
  const int64_t pieces = elements / 8;
  int64_t blocks = (pieces + 255) / 256;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == QMM_BF16)
    silu_mul_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        static_cast<const uint4*>(gate), static_cast<const uint4*>(up), static_cast<uint4*>(out), pieces);
  else
    silu_mul_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        static_cast<const uint4*>(gate), static_cast<const uint4*>(up), static_cast<uint4*>(out), pieces);
  count_launch();
  return check_launch("moe silu_mul_kernel");
}

extern "C" int qmm_moe_routed_sum(const void* rows, const int64_t* row_of_pair, const float* weights, void* out,
                                  int64_t tokens, int k, int64_t width, int64_t total_rows, int dtype, void* stream) {
  if (tokens < 0 || k < 1 || width < 8 || width % 8 || total_rows < (tokens ? 1 : 0))
    return fail(QMM_ERR_SHAPE, "moe_routed_sum: width must be a positive multiple of 8, k >= 1");
  if (tokens == 0) return QMM_OK;
  if (!rows || !row_of_pair || !weights || !out) return fail(QMM_ERR_NULL, "moe_routed_sum: null pointer");
  if (dtype != QMM_BF16 && dtype != QMM_F16) return fail(QMM_ERR_DTYPE, "moe_routed_sum: bf16 or f16");
  if ((reinterpret_cast<uintptr_t>(rows) | reinterpret_cast<uintptr_t>(out)) & 15)
    return fail(QMM_ERR_LAYOUT, "moe_routed_sum: pointers must be 16-byte aligned");
  if (tokens == 0) return QMM_OK;
  int* status = device_status_word();
  if (!status) return fail(QMM_ERR_CUDA, "could not allocate the device status word");
  const int64_t pieces = width / 8;
  int64_t blocks = tokens;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  const int threads = pieces >= 256 ? 256 : (pieces >= 128 ? 128 : 64);
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == QMM_BF16)
    routed_sum_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), threads, 0, st>>>(
        static_cast<const uint4*>(rows), row_of_pair, weights, static_cast<uint4*>(out), tokens, k, pieces, total_rows, status);
  else
    routed_sum_kernel<__half><<<static_cast<unsigned>(blocks), threads, 0, st>>>(
        static_cast<const uint4*>(rows), row_of_pair, weights, static_cast<uint4*>(out), tokens, k, pieces, total_rows, status);
  count_launch();
  return check_launch("moe routed_sum_kernel");
}
