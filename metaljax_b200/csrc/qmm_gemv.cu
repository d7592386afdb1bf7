// Decode kernel of the fused dequantize-and-matmul: up to 16 activation rows against a
// streamed packed weight (M <= 16 of `y = x . deq(w)^T`, src/metaljax/qmm.py:2491).
//
// HBM-bound: every packed weight byte is read exactly once, straight from global memory
// into registers, and never dequantized element by element. A CTA owns 16 weight rows; its
// 8 warps split K. Per 32-wide K step a lane holds one packed word (two for 8-bit) of rows
// g and g+8 and turns it into the A fragments of two m16n8k16 MMAs with a magic-number OR:
// the 16-bit pattern 0x4300|q is the bf16 number 128+q (0x6400|q is the f16 number 1024+q),
// so the tensor core accumulates  sum (C + q_k) x_k  exactly in float32. All 16 K slots of
// such an MMA lie inside one 32-element span, hence inside one quantization group, so the
// group's scale and bias are applied to the accumulators once per group:
//     y += s * sum (C + q) x  +  (b - C s) * sum x ,
// with  sum x  taken from one more MMA whose A fragment is all ones. The activations are
// staged once per CTA in shared memory in the MMA's element type (for 4-bit codes with the
// pair order the magic-number extraction produces), tokens beyond M being zero fragments.
// MXFP4 converts code pairs with cvt.e2m1x2 to f16 and scales per 32-group by 2^(e8-127).
//
// The K split is reduced across the CTA's warps in shared memory; there is no global
// scratch and no atomics, and the summation order is fixed.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "qmm_internal.h"

namespace qmm {
namespace {

constexpr int kWarps = 8;
constexpr int kRowsPerCta = 16;
constexpr int kXPad = 32;        // elements of padding per staged activation row (64 bytes)

enum { kAff4 = 0, kAff8 = 1, kMx4 = 2 };

struct GemvParams {
  const void* x;
  const uint32_t* w;
  const void* scales;
  const void* biases;
  void* y;
  const int32_t* lhs_idx;
  const int32_t* rhs_idx;
  int64_t M, K, N, batch;
  int64_t x_batch_stride, y_batch_stride, w_batch_rows;
  int group_size, table_dtype, y_dtype, x_dtype;
  int kc;  // K elements staged per pass
};

template <typename AT>
struct MmaOps;

template <>
struct MmaOps<__nv_bfloat16> {
  static constexpr uint32_t kMagic = 0x43004300u;
  static constexpr float kMagicValue = 128.0f;
  static constexpr uint32_t kOnes = 0x3F803F80u;
  static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};

template <>
struct MmaOps<__half> {
  static constexpr uint32_t kMagic = 0x64006400u;
  static constexpr float kMagicValue = 1024.0f;
  static constexpr uint32_t kOnes = 0x3C003C00u;
  static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};

__device__ __forceinline__ float gv_table(const void* p, int dtype, int64_t i) {
  if (dtype == QMM_BF16) return __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16*>(p) + i));
  if (dtype == QMM_F16) return __half2float(__ldg(reinterpret_cast<const __half*>(p) + i));
  return __ldg(reinterpret_cast<const float*>(p) + i);
}

__device__ __forceinline__ void gv_store(void* p, int dtype, int64_t i, float v) {
  if (dtype == QMM_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else if (dtype == QMM_F16) reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
  else reinterpret_cast<float*>(p)[i] = v;
}

// Two activations as one 32-bit pair of the MMA's element type (f16 saturates instead of
// overflowing to infinity when the source is bf16).
template <typename AT>
__device__ __forceinline__ uint32_t pack_pair(float a, float b) {
  if constexpr (std::is_same<AT, __nv_bfloat16>::value) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    a = fminf(fmaxf(a, -65504.0f), 65504.0f);
    b = fminf(fmaxf(b, -65504.0f), 65504.0f);
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// Eight consecutive activations starting at a 16-byte aligned address, as floats.
template <typename XT>
__device__ __forceinline__ void load8(const XT* p, float (&f)[8]) {
  const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (std::is_same<XT, __nv_bfloat16>::value) {
      f[2 * i] = __uint_as_float(u[i] << 16);
      f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    } else {
      const float2 h = __half22float2(*reinterpret_cast<const __half2*>(&u[i]));
      f[2 * i] = h.x; f[2 * i + 1] = h.y;
    }
  }
}

// What one warp requests from global memory ahead of a run of MMAs: the packed words of
// rows g and g+8 for up to kSteps K steps, and the group tables that go with them.
template <int QK, int SPG>
struct BatchShape {
  static constexpr int kWpl = (QK == kAff8) ? 2 : 1;                       // words per lane per step
  static constexpr int kMaxSteps = (QK == kAff8) ? 8 : 16;
  static constexpr int kMaxGroups = (QK == kMx4) ? 16 : 8;
  static constexpr int kGroups = (kMaxSteps / SPG < kMaxGroups) ? kMaxSteps / SPG : kMaxGroups;
  static constexpr int kSteps = kGroups * SPG;
};

// QK: quantization kind. XT: activation type in memory. NT: token halves (1: M <= 8,
// 2: M <= 16). SPG: 32-wide K steps per quantization group (1, 2, 4).
template <int QK, typename XT, int NT, int SPG>
__global__ void __launch_bounds__(kWarps * 32, 2)
qmm_gemv_kernel(const GemvParams p) {
  // MMA element type: 4-bit affine codes fit bf16's 7 mantissa bits; 8-bit codes and the
  // E2M1 conversion need f16.
  using AT = typename std::conditional<QK == kAff4, XT, __half>::type;
  using Ops = MmaOps<AT>;
  using BS = BatchShape<QK, SPG>;
  constexpr int BITS = (QK == kAff8) ? 8 : 4;
  constexpr int WPL = BS::kWpl;

  extern __shared__ __align__(16) uint8_t gv_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int xrow = p.kc + kXPad;                  // staged row stride in elements
  AT* xs = reinterpret_cast<AT*>(gv_smem);
  float* red = reinterpret_cast<float*>(gv_smem + static_cast<size_t>(p.M) * xrow * sizeof(AT));

  const int64_t seg = blockIdx.y;
  int64_t x_off, wb;
  if (p.lhs_idx) {
    x_off = static_cast<int64_t>(p.lhs_idx[seg]) * p.x_batch_stride;
    wb = p.rhs_idx[seg];
  } else {
    x_off = seg * p.x_batch_stride;
    wb = p.w_batch_rows ? seg : 0;
  }
  const int64_t y_off = seg * p.y_batch_stride;
  const XT* xg = reinterpret_cast<const XT*>(p.x) + x_off;

  const int64_t n0 = static_cast<int64_t>(blockIdx.x) * kRowsPerCta;
  const int64_t words = p.K * BITS / 32;
  const int64_t groups = p.K / (32 * SPG);
  const int64_t r0 = wb * p.N + (n0 + g < p.N ? n0 + g : p.N - 1);
  const int64_t r1 = wb * p.N + (n0 + g + 8 < p.N ? n0 + g + 8 : p.N - 1);
  const uint32_t* w0 = p.w + r0 * words;
  const uint32_t* w1 = p.w + r1 * words;

  uint32_t wr[BS::kSteps][2][WPL];
  float sc[BS::kGroups][2], bi[BS::kGroups][2];

  // Requests groups [gfirst, gfirst+ng) (absolute group indices) of this lane's two rows.
  auto load_batch = [&](int64_t gfirst, int ng) {
#pragma unroll
    for (int q = 0; q < BS::kGroups; ++q) {
      if (q < ng) {
#pragma unroll
        for (int s = 0; s < SPG; ++s) {
          const int64_t wi = ((gfirst + q) * SPG + s) * (4 * WPL) + t * WPL;
          if constexpr (WPL == 2) {
            const uint2 a = __ldg(reinterpret_cast<const uint2*>(w0 + wi));
            const uint2 b = __ldg(reinterpret_cast<const uint2*>(w1 + wi));
            wr[q * SPG + s][0][0] = a.x; wr[q * SPG + s][0][1] = a.y;
            wr[q * SPG + s][1][0] = b.x; wr[q * SPG + s][1][1] = b.y;
          } else {
            wr[q * SPG + s][0][0] = __ldg(w0 + wi);
            wr[q * SPG + s][1][0] = __ldg(w1 + wi);
          }
        }
        const int64_t gi = gfirst + q;
        if constexpr (QK == kMx4) {
          const uint32_t e0 = __ldg(reinterpret_cast<const uint8_t*>(p.scales) + r0 * groups + gi);
          const uint32_t e1 = __ldg(reinterpret_cast<const uint8_t*>(p.scales) + r1 * groups + gi);
          sc[q][0] = __uint_as_float(e0 ? (e0 << 23) : 0x00400000u);
          sc[q][1] = __uint_as_float(e1 ? (e1 << 23) : 0x00400000u);
          bi[q][0] = bi[q][1] = 0.0f;
        } else {
          sc[q][0] = gv_table(p.scales, p.table_dtype, r0 * groups + gi);
          sc[q][1] = gv_table(p.scales, p.table_dtype, r1 * groups + gi);
          bi[q][0] = gv_table(p.biases, p.table_dtype, r0 * groups + gi);
          bi[q][1] = gv_table(p.biases, p.table_dtype, r1 * groups + gi);
        }
      }
    }
  };

  float yacc[NT][4];
#pragma unroll
  for (int h = 0; h < NT; ++h)
#pragma unroll
    for (int i = 0; i < 4; ++i) yacc[h][i] = 0.0f;

  for (int64_t kbase = 0; kbase < p.K; kbase += p.kc) {
    const int kc = static_cast<int>(p.K - kbase < p.kc ? p.K - kbase : p.kc);   // multiple of 32
    // this warp's share of the chunk's groups, as indices within the chunk
    const int cgroups = kc / (32 * SPG);
    const int glo = cgroups * warp / kWarps, ghi = cgroups * (warp + 1) / kWarps;
    const int64_t gbase = kbase / (32 * SPG);
    // The first batch's weights are requested before the activations are staged, so the
    // two global-memory latencies overlap.
    int ng = (ghi - glo < BS::kGroups) ? ghi - glo : BS::kGroups;
    if (ng > 0) load_batch(gbase + glo, ng);

    __syncthreads();
    for (int idx = threadIdx.x; idx < static_cast<int>(p.M) * (kc / 8); idx += blockDim.x) {
      const int m = idx / (kc / 8), ch = idx % (kc / 8);
      float f[8];
      load8<XT>(xg + static_cast<int64_t>(m) * p.K + kbase + ch * 8, f);
      uint4 o;
      if constexpr (QK == kAff4) {  // pair order (0,4)(1,5)(2,6)(3,7): what one LOP3 extracts
        o.x = pack_pair<AT>(f[0], f[4]); o.y = pack_pair<AT>(f[1], f[5]);
        o.z = pack_pair<AT>(f[2], f[6]); o.w = pack_pair<AT>(f[3], f[7]);
      } else {
        o.x = pack_pair<AT>(f[0], f[1]); o.y = pack_pair<AT>(f[2], f[3]);
        o.z = pack_pair<AT>(f[4], f[5]); o.w = pack_pair<AT>(f[6], f[7]);
      }
      *reinterpret_cast<uint4*>(xs + static_cast<size_t>(m) * xrow + ch * 8) = o;
    }
    __syncthreads();

    for (int gb = glo; gb < ghi; gb += BS::kGroups) {
      if (gb != glo) {
        ng = (ghi - gb < BS::kGroups) ? ghi - gb : BS::kGroups;
        load_batch(gbase + gb, ng);
      }
#pragma unroll
      for (int q = 0; q < BS::kGroups; ++q) {
        if (q < ng) {
          float acc[NT][4], ones[NT][4];
#pragma unroll
          for (int h = 0; h < NT; ++h)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[h][i] = ones[h][i] = 0.0f;
#pragma unroll
          for (int s = 0; s < SPG; ++s) {
            const int kloc = ((gb + q) * SPG + s) * 32 + t * 8;     // within the staged chunk
            uint32_t a[2][4];
            if constexpr (QK == kAff4) {
              const uint32_t u0 = wr[q * SPG + s][0][0], u1 = wr[q * SPG + s][1][0];
              a[0][0] = (u0 & 0x000F000Fu) | Ops::kMagic;         a[0][1] = (u1 & 0x000F000Fu) | Ops::kMagic;
              a[0][2] = ((u0 >> 4) & 0x000F000Fu) | Ops::kMagic;  a[0][3] = ((u1 >> 4) & 0x000F000Fu) | Ops::kMagic;
              a[1][0] = ((u0 >> 8) & 0x000F000Fu) | Ops::kMagic;  a[1][1] = ((u1 >> 8) & 0x000F000Fu) | Ops::kMagic;
              a[1][2] = ((u0 >> 12) & 0x000F000Fu) | Ops::kMagic; a[1][3] = ((u1 >> 12) & 0x000F000Fu) | Ops::kMagic;
            } else if constexpr (QK == kAff8) {
#pragma unroll
              for (int j = 0; j < 2; ++j) {   // word j: bytes (0,1) and (2,3) under the f16 magic
                a[j][0] = __byte_perm(wr[q * SPG + s][0][j], 0x64646464u, 0x4140);
                a[j][1] = __byte_perm(wr[q * SPG + s][1][j], 0x64646464u, 0x4140);
                a[j][2] = __byte_perm(wr[q * SPG + s][0][j], 0x64646464u, 0x4342);
                a[j][3] = __byte_perm(wr[q * SPG + s][1][j], 0x64646464u, 0x4342);
              }
            } else {
#pragma unroll
              for (int r = 0; r < 2; ++r) {
                const uint32_t u = wr[q * SPG + s][r][0];
#pragma unroll
                for (int bb = 0; bb < 4; ++bb) {  // byte bb -> elements (2bb, 2bb+1)
                  uint32_t h2;
                  const uint16_t byte = static_cast<uint16_t>((u >> (8 * bb)) & 0xFFu);
                  asm("{ .reg .b8 t; cvt.u8.u16 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(h2) : "h"(byte));
                  a[bb >> 1][(bb & 1) * 2 + r] = h2;
                }
              }
            }
            const uint32_t one4[4] = {Ops::kOnes, Ops::kOnes, Ops::kOnes, Ops::kOnes};
#pragma unroll
            for (int h = 0; h < NT; ++h) {
              uint4 xv = make_uint4(0u, 0u, 0u, 0u);
              if (h * 8 + g < p.M)
                xv = *reinterpret_cast<const uint4*>(xs + static_cast<size_t>(h * 8 + g) * xrow + kloc);
              Ops::mma(acc[h], a[0], xv.x, xv.y);
              Ops::mma(acc[h], a[1], xv.z, xv.w);
              if constexpr (QK != kMx4) {
                Ops::mma(ones[h], one4, xv.x, xv.y);
                Ops::mma(ones[h], one4, xv.z, xv.w);
              }
            }
          }
          // fold the group: rows g (c0, c1) and g+8 (c2, c3), tokens 2t and 2t+1
          const float s0 = sc[q][0], s1 = sc[q][1];
          const float b0 = bi[q][0] - Ops::kMagicValue * s0, b1 = bi[q][1] - Ops::kMagicValue * s1;
#pragma unroll
          for (int h = 0; h < NT; ++h) {
            if constexpr (QK == kMx4) {
              yacc[h][0] = fmaf(s0, acc[h][0], yacc[h][0]);
              yacc[h][1] = fmaf(s0, acc[h][1], yacc[h][1]);
              yacc[h][2] = fmaf(s1, acc[h][2], yacc[h][2]);
              yacc[h][3] = fmaf(s1, acc[h][3], yacc[h][3]);
            } else {
              yacc[h][0] = fmaf(s0, acc[h][0], fmaf(b0, ones[h][0], yacc[h][0]));
              yacc[h][1] = fmaf(s0, acc[h][1], fmaf(b0, ones[h][1], yacc[h][1]));
              yacc[h][2] = fmaf(s1, acc[h][2], fmaf(b1, ones[h][0], yacc[h][2]));
              yacc[h][3] = fmaf(s1, acc[h][3], fmaf(b1, ones[h][1], yacc[h][3]));
            }
          }
        }
      }
    }
  }

  // ---- reduce the K split across warps (fixed order) and store ----
  __syncthreads();
#pragma unroll
  for (int h = 0; h < NT; ++h)
#pragma unroll
    for (int i = 0; i < 4; ++i) red[(warp * NT * 4 + h * 4 + i) * 32 + lane] = yacc[h][i];
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int h = 0; h < NT; ++h)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float v = 0.0f;
#pragma unroll
        for (int wv = 0; wv < kWarps; ++wv) v += red[(wv * NT * 4 + h * 4 + i) * 32 + lane];
        const int64_t row = n0 + g + (i >> 1) * 8;
        const int64_t tok = h * 8 + 2 * t + (i & 1);
        if (row < p.N && tok < p.M) gv_store(p.y, p.y_dtype, y_off + tok * p.N + row, v);
      }
  }
}

template <int QK, typename XT, int NT, int SPG>
int launch_kernel(const GemvParams& gp, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(gp.M) * (gp.kc + kXPad) * 2 +
                      static_cast<size_t>(kWarps) * 2 * 4 * 32 * sizeof(float);
  dim3 grid(static_cast<unsigned>((gp.N + kRowsPerCta - 1) / kRowsPerCta), static_cast<unsigned>(gp.batch));
  auto kernel = qmm_gemv_kernel<QK, XT, NT, SPG>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured = true;
  }
  kernel<<<grid, kWarps * 32, smem, stream>>>(gp);
  count_launch();
  return check_launch("qmm_gemv_kernel");
}

template <int QK, typename XT, int NT>
int launch_spg(const GemvParams& gp, cudaStream_t stream) {
  if constexpr (QK == kMx4) {
    return launch_kernel<QK, XT, NT, 1>(gp, stream);
  } else {
    if (gp.group_size == 32) return launch_kernel<QK, XT, NT, 1>(gp, stream);
    if (gp.group_size == 64) return launch_kernel<QK, XT, NT, 2>(gp, stream);
    return launch_kernel<QK, XT, NT, 4>(gp, stream);
  }
}

template <int QK>
int launch_xt(const GemvParams& gp, cudaStream_t stream) {
  if (gp.x_dtype == QMM_BF16)
    return gp.M <= 8 ? launch_spg<QK, __nv_bfloat16, 1>(gp, stream) : launch_spg<QK, __nv_bfloat16, 2>(gp, stream);
  return gp.M <= 8 ? launch_spg<QK, __half, 1>(gp, stream) : launch_spg<QK, __half, 2>(gp, stream);
}

}  // namespace

bool gemv_supports(const qmm_problem& p) {
  if (p.x_dtype != QMM_BF16 && p.x_dtype != QMM_F16) return false;
  if (p.group_sizes) return false;                 // ragged rows go to the tensor-core kernel
  if (p.M < 1 || p.M > 16) return false;
  if (p.batch > 65535) return false;
  if (p.K % 32) return false;
  return true;
}

int launch_gemv(const qmm_problem& p, cudaStream_t stream) {
  GemvParams gp;
  gp.x = p.x; gp.w = p.w; gp.scales = p.scales; gp.biases = p.biases; gp.y = p.y;
  gp.lhs_idx = p.lhs_idx; gp.rhs_idx = p.rhs_idx;
  gp.M = p.M; gp.K = p.K; gp.N = p.N; gp.batch = p.batch;
  gp.x_batch_stride = p.x_batch_stride; gp.y_batch_stride = p.y_batch_stride;
  gp.w_batch_rows = p.rhs_idx ? p.N : p.w_batch_stride;
  gp.group_size = p.group_size; gp.table_dtype = p.table_dtype; gp.y_dtype = p.y_dtype;
  gp.x_dtype = p.x_dtype;
  // K elements staged per pass: the staged activations stay under ~64 KiB per CTA.
  int kc = p.M <= 8 ? 4096 : 2048;
  if (p.K < kc) kc = static_cast<int>(p.K);
  gp.kc = kc;
  if (p.mode == QMM_MODE_MXFP4) return launch_xt<kMx4>(gp, stream);
  if (p.bits == 8) return launch_xt<kAff8>(gp, stream);
  return launch_xt<kAff4>(gp, stream);
}

}  // namespace qmm
