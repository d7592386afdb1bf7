// General SIMT kernel of the fused dequantize-and-matmul: every mode, every element type,
// dense / gathered / ragged. It is the route for float32 activations and for shapes the
// specialised kernels decline, and the in-library cross-check for them.
//
// Computation (MLX's quantized_matmul with transpose=True, as the reference calls it at
// src/metaljax/qmm.py:2491): y[m, n] = sum_k x[m, k] * deq(w)[n, k]. Within one
// quantization group the affine dequant is linear in the code, so a lane accumulates
// sum x*q and sum x over its 16-byte chunk (always inside one group, since groups are
// >= 32 elements) and applies `scale` and `bias` once per chunk:
//     sum_k x_k (s q_k + b) = s * sum x_k q_k + b * sum x_k.
// All accumulation is float32.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "qmm_internal.h"

namespace qmm {
namespace {

constexpr int kWarps = 4;  // warps per block
constexpr int kRows = 2;   // weight rows per warp

enum { kAff4 = 0, kAff8 = 1, kMx4 = 2 };

struct SimtParams {
  const void* x;
  const uint32_t* w;
  const void* scales;
  const void* biases;
  void* y;
  const int32_t* lhs_idx;
  const int32_t* rhs_idx;
  const int32_t* group_sizes;
  int64_t M, K, N, batch;
  int64_t x_batch_stride, y_batch_stride, w_batch_rows;
  int64_t num_weights, x_batches;   // gather: valid ranges of rhs_idx / lhs_idx (x_batches 0 = unknown)
  int* status;
  int group_size, table_dtype, y_dtype;
};

__device__ __forceinline__ float load_table(const void* p, int dtype, int64_t i) {
  if (dtype == QMM_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  if (dtype == QMM_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  return reinterpret_cast<const float*>(p)[i];
}

__device__ __forceinline__ void store_y(void* p, int dtype, int64_t i, float v) {
  if (dtype == QMM_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else if (dtype == QMM_F16) reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
  else reinterpret_cast<float*>(p)[i] = v;
}

// E elements of x starting at `p` (16-byte aligned for E == 8, 8-byte for E == 4) as floats.
template <typename XT, int E>
__device__ __forceinline__ void load_x(const XT* p, float (&out)[E]) {
  if constexpr (sizeof(XT) == 4) {
#pragma unroll
    for (int i = 0; i < E; i += 4) {
      float4 v = __ldg(reinterpret_cast<const float4*>(p) + i / 4);
      out[i] = v.x; out[i + 1] = v.y; out[i + 2] = v.z; out[i + 3] = v.w;
    }
  } else {
    uint32_t u[E / 2];
    if constexpr (E == 8) {
      uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
      u[0] = v.x; u[1] = v.y; u[2] = v.z; u[3] = v.w;
    } else {
      uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
      u[0] = v.x; u[1] = v.y;
    }
#pragma unroll
    for (int i = 0; i < E / 2; ++i) {
      if constexpr (std::is_same<XT, __nv_bfloat16>::value) {
        out[2 * i] = __uint_as_float(u[i] << 16);
        out[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
      } else {
        float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u[i]));
        out[2 * i] = f.x; out[2 * i + 1] = f.y;
      }
    }
  }
}

// The EPW code values of one packed word, as floats (integers for affine, E2M1 values for
// MXFP4). Element e of the word sits at bits [e*bits, (e+1)*bits).
template <int QK>
__device__ __forceinline__ void decode_word(uint32_t word, float (&q)[QK == kAff8 ? 4 : 8]) {
  if constexpr (QK == kAff4) {
#pragma unroll
    for (int e = 0; e < 8; ++e)  // 2^23 + nibble, then the exact subtraction
      q[e] = __uint_as_float(0x4B000000u | ((word >> (4 * e)) & 0xFu)) - 8388608.0f;
  } else if constexpr (QK == kAff8) {
#pragma unroll
    for (int e = 0; e < 4; ++e)
      q[e] = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7650 + e)) - 8388608.0f;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {  // byte j holds elements 2j (low nibble) and 2j+1
      uint32_t h2;
      uint16_t byte = static_cast<uint16_t>((word >> (8 * j)) & 0xFFu);
      asm("{ .reg .b8 t; cvt.u8.u16 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(h2) : "h"(byte));
      float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
      q[2 * j] = f.x; q[2 * j + 1] = f.y;
    }
  }
}

template <int QK, typename XT, int MT>
__global__ void __launch_bounds__(kWarps * 32)
qmm_simt_kernel(const SimtParams p) {
  constexpr int BITS = (QK == kAff8) ? 8 : 4;
  constexpr int EPW = 32 / BITS;  // elements per packed word
  constexpr int EPC = EPW * 4;    // elements per 16-byte chunk
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t n0 = (static_cast<int64_t>(blockIdx.x) * kWarps + warp) * kRows;
  if (n0 >= p.N) return;
  const int64_t words = p.K * BITS / 32;
  const int64_t groups = p.K / p.group_size;
  const int64_t nchunks = p.K / EPC;
  const int64_t nseg = p.group_sizes ? p.batch + 1 : p.batch;

  for (int64_t seg = blockIdx.y; seg < nseg; seg += gridDim.y) {
    int64_t m_count, x_off, y_off, wb;
    if (p.group_sizes) {
      int64_t lo = 0;
      const int64_t upto = seg < p.batch ? seg : p.batch;
      for (int64_t g = 0; g < upto; ++g) lo += p.group_sizes[g];
      if (lo > p.M) lo = p.M;
      if (seg == p.batch) {  // rows past the last group are zero
        for (int64_t m = lo + lane; m < p.M; m += 32)
          for (int r = 0; r < kRows; ++r)
            if (n0 + r < p.N) store_y(p.y, p.y_dtype, m * p.N + n0 + r, 0.0f);
        continue;
      }
      m_count = p.group_sizes[seg];
      if (lo + m_count > p.M) m_count = p.M - lo;
      x_off = lo * p.K; y_off = lo * p.N; wb = seg;
    } else if (p.lhs_idx) {
      m_count = p.M;
      int64_t li = p.lhs_idx[seg], ri = p.rhs_idx[seg];
      if (ri < 0 || ri >= p.num_weights || li < 0 || (p.x_batches > 0 && li >= p.x_batches)) {
        if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, QMM_DEVICE_BAD_INDEX);
        if (ri < 0 || ri >= p.num_weights) ri = 0;
        if (li < 0 || (p.x_batches > 0 && li >= p.x_batches)) li = 0;
      }
      x_off = li * p.x_batch_stride;
      y_off = seg * p.y_batch_stride;
      wb = ri;
    } else {
      m_count = p.M;
      x_off = seg * p.x_batch_stride;
      y_off = seg * p.y_batch_stride;
      wb = p.w_batch_rows ? seg : 0;
    }
    const XT* xs = reinterpret_cast<const XT*>(p.x) + x_off;
    int64_t rows[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r)
      rows[r] = wb * p.N + (n0 + r < p.N ? n0 + r : p.N - 1);

    for (int64_t m0 = 0; m0 < m_count; m0 += MT) {
      float acc[MT][kRows];
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int r = 0; r < kRows; ++r) acc[m][r] = 0.0f;

#pragma unroll 2
      for (int64_t c = lane; c < nchunks; c += 32) {
        uint32_t wv[kRows][4];
        float s[kRows], b[kRows];
        const int64_t g = (c * EPC) / p.group_size;
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
          uint4 v = __ldg(reinterpret_cast<const uint4*>(p.w + rows[r] * words) + c);
          wv[r][0] = v.x; wv[r][1] = v.y; wv[r][2] = v.z; wv[r][3] = v.w;
          if constexpr (QK == kMx4) {
            const uint32_t e8 = reinterpret_cast<const uint8_t*>(p.scales)[rows[r] * groups + g];
            // 2^(e8-127); byte 0 is the subnormal 2^-127
            s[r] = __uint_as_float(e8 ? (e8 << 23) : 0x00400000u);
            b[r] = 0.0f;
          } else {
            s[r] = load_table(p.scales, p.table_dtype, rows[r] * groups + g);
            b[r] = load_table(p.biases, p.table_dtype, rows[r] * groups + g);
          }
        }
        float accq[MT][kRows], sx[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          sx[m] = 0.0f;
#pragma unroll
          for (int r = 0; r < kRows; ++r) accq[m][r] = 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float q[kRows][EPW];
#pragma unroll
          for (int r = 0; r < kRows; ++r) decode_word<QK>(wv[r][j], q[r]);
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            const int64_t mm = (m0 + m < m_count) ? m0 + m : m_count - 1;
            float xf[EPW];
            load_x<XT, EPW>(xs + mm * p.K + c * EPC + j * EPW, xf);
#pragma unroll
            for (int e = 0; e < EPW; ++e) {
              if constexpr (QK != kMx4) sx[m] += xf[e];
#pragma unroll
              for (int r = 0; r < kRows; ++r) accq[m][r] = fmaf(xf[e], q[r][e], accq[m][r]);
            }
          }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
          for (int r = 0; r < kRows; ++r)
            acc[m][r] += s[r] * accq[m][r] + b[r] * sx[m];
      }

#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
          float v = acc[m][r];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if (lane == 0 && m0 + m < m_count && n0 + r < p.N)
            store_y(p.y, p.y_dtype, y_off + (m0 + m) * p.N + n0 + r, v);
        }
    }
  }
}

template <int QK, typename XT>
int launch_mt(const SimtParams& sp, int mt, dim3 grid, cudaStream_t stream) {
  dim3 block(kWarps * 32);
  if (mt >= 4) qmm_simt_kernel<QK, XT, 4><<<grid, block, 0, stream>>>(sp);
  else if (mt >= 2) qmm_simt_kernel<QK, XT, 2><<<grid, block, 0, stream>>>(sp);
  else qmm_simt_kernel<QK, XT, 1><<<grid, block, 0, stream>>>(sp);
  count_launch();
  return check_launch("qmm_simt_kernel");
}

template <int QK>
int launch_x(const SimtParams& sp, int x_dtype, int mt, dim3 grid, cudaStream_t stream) {
  switch (x_dtype) {
    case QMM_BF16: return launch_mt<QK, __nv_bfloat16>(sp, mt, grid, stream);
    case QMM_F16: return launch_mt<QK, __half>(sp, mt, grid, stream);
    case QMM_F32: return launch_mt<QK, float>(sp, mt, grid, stream);
  }
  return fail(QMM_ERR_DTYPE, "simt: activation dtype %d", x_dtype);
}

}  // namespace

int launch_simt(const qmm_problem& p, cudaStream_t stream) {
  SimtParams sp;
  sp.x = p.x; sp.w = p.w; sp.scales = p.scales; sp.biases = p.biases; sp.y = p.y;
  sp.lhs_idx = p.lhs_idx; sp.rhs_idx = p.rhs_idx; sp.group_sizes = p.group_sizes;
  sp.M = p.M; sp.K = p.K; sp.N = p.N; sp.batch = p.batch;
  sp.x_batch_stride = p.x_batch_stride; sp.y_batch_stride = p.y_batch_stride;
  sp.w_batch_rows = (p.group_sizes || p.rhs_idx) ? p.N : p.w_batch_stride;
  sp.num_weights = p.num_weights > 0 ? p.num_weights : 1;
  sp.x_batches = p.x_batches;
  sp.status = p.lhs_idx ? device_status_word() : nullptr;
  sp.group_size = p.group_size; sp.table_dtype = p.table_dtype; sp.y_dtype = p.y_dtype;
  if (p.M == 0 || p.N == 0 || p.batch == 0) return QMM_OK;

  const int64_t nseg = p.group_sizes ? p.batch + 1 : p.batch;
  dim3 grid(static_cast<unsigned>((p.N + kWarps * kRows - 1) / (kWarps * kRows)),
            static_cast<unsigned>(nseg < 65535 ? nseg : 65535));
  // Rows of x handled per pass over the weight; ragged segments have their own counts.
  const int mt = p.group_sizes ? 4 : (p.M >= 4 ? 4 : (p.M >= 2 ? 2 : 1));
  if (p.mode == QMM_MODE_MXFP4) return launch_x<kMx4>(sp, p.x_dtype, mt, grid, stream);
  if (p.bits == 8) return launch_x<kAff8>(sp, p.x_dtype, mt, grid, stream);
  return launch_x<kAff4>(sp, p.x_dtype, mt, grid, stream);
}

}  // namespace qmm
