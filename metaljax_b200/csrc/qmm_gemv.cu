// Decode kernel of the fused dequantize-and-matmul: up to 16 activation rows against a
// streamed packed weight (M <= 16 of `y = x . deq(w)^T`, src/metaljax/qmm.py:2491).
//
// HBM-bound: every packed weight byte is read exactly once and never dequantized element by
// element. A CTA owns 16 weight rows and its 8 warps split K. The packed rows arrive by TMA in
// boxes of 16 rows x 128 bytes (128-byte swizzle, so that the fragment reads below are free
// of bank conflicts); every warp feeds its own ring of boxes from its own mbarriers, and the
// first boxes are requested before anything else happens in the kernel.
//
// Per 32-wide K step a lane reads one packed word (two for 8-bit) of rows g and g+8 and turns
// it into the A fragments of two m16n8k16 MMAs with a magic-number OR: the 16-bit pattern
// 0x4300|q is the bf16 number 128+q (0x6400|q is the f16 number 1024+q), so the tensor core
// accumulates  sum (C + q_k) x_k  exactly in float32. All 16 K slots of such an MMA lie
// inside one 32-element span, hence inside one quantization group, so the group's scale and
// bias are applied to the accumulators once per group:
//     y += s * sum (C + q) x  +  (b - C s) * sum x ,
// with  sum x  taken from one more MMA whose A fragment is all ones. The activations are
// staged in shared memory in the MMA's element type (for 4-bit codes in the pair order the
// magic-number extraction produces), tokens beyond M being zero fragments, next to the
// tile's slice of the scale table and of the folded bias table  b - C s.
// MXFP4 places each code's magnitude bits at the f16 exponent/mantissa boundary (the E2M1
// value times 2^-14, exactly) and scales the accumulators per 32-group by 2^(e8-127+14).
//
// CTAs are persistent: a CTA walks 16-row tiles with a grid stride, keeps the staged
// activations for all of them, requests the next tile's tables
// while it computes the current one, and its warps' TMA rings run ahead across tile
// boundaries. The K split is reduced across the CTA's warps in shared memory; there is no
// global scratch and no atomics, and the summation order is fixed. Waits on the TMA barriers
// are bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "qmm_internal.h"
#include "qmm_ptx.cuh"

namespace qmm {
namespace {

using namespace ptx;

constexpr int kWarps = 8;
constexpr int kRowsPerCta = 16;
constexpr int kXPad = 32;           // elements of padding per staged activation row (64 bytes)
constexpr int kBoxBytes = 128;      // bytes of one weight row in a TMA box
constexpr int kBoxSmem = kRowsPerCta * kBoxBytes;   // 2 KiB
constexpr int kMaxRing = 4;         // boxes a warp keeps in flight

enum { kAff4 = 0, kAff8 = 1, kMx4 = 2 };

struct GemvParams {
  const void* x;
  const void* scales;
  const void* biases;
  void* y;
  const int32_t* lhs_idx;
  const int32_t* rhs_idx;
  int* status;
  int64_t M, K, N, batch;
  int64_t x_batch_stride, y_batch_stride, w_batch_rows;
  int group_size, table_dtype, y_dtype;
  int kc;     // K elements staged per pass (a multiple of the box width)
  int ring;   // boxes per warp ring (1..kMaxRing)
  int tiles;  // 16-row tiles per weight matrix
};

template <typename AT>
struct MmaOps;

template <>
struct MmaOps<__nv_bfloat16> {
  static constexpr uint32_t kMagic = 0x43004300u;
  static constexpr float kMagicValue = 128.0f;
  static constexpr uint32_t kOnes = 0x3F803F80u;
  // d = a * b + c (m16n8k16, float32 accumulate)
  static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                             const float (&c)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
  }
};

template <>
struct MmaOps<__half> {
  static constexpr uint32_t kMagic = 0x64006400u;
  static constexpr float kMagicValue = 1024.0f;
  static constexpr uint32_t kOnes = 0x3C003C00u;
  // d = a * b + c (m16n8k16, float32 accumulate)
  static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                             const float (&c)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
  }
};

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

// Walks one warp's boxes in the order they are consumed: tile by tile (grid stride), inside a
// tile chunk by chunk (a chunk is what the CTA stages of x at a time), and inside a chunk the
// warp's contiguous share of its boxes.
struct BoxCursor {
  int tile, chunk, j, hi;
};

template <int BOXK>
__device__ __forceinline__ void cursor_seek(BoxCursor& c, int ntiles, int tstride, int nchunks, int warp,
                                            int K, int kc) {
  while (c.tile < ntiles) {
    while (c.chunk < nchunks) {
      const int left = K - c.chunk * kc;                    // 32-bit on purpose: no 64-bit division
      const int nb = ((left < kc ? left : kc) + BOXK - 1) / BOXK;
      c.j = nb * warp / kWarps;
      c.hi = nb * (warp + 1) / kWarps;
      if (c.j < c.hi) return;
      ++c.chunk;
    }
    c.tile += tstride;
    c.chunk = 0;
  }
}

template <int BOXK>
__device__ __forceinline__ void cursor_next(BoxCursor& c, int ntiles, int tstride, int nchunks, int warp,
                                            int K, int kc) {
  if (++c.j < c.hi) return;
  ++c.chunk;
  cursor_seek<BOXK>(c, ntiles, tstride, nchunks, warp, K, kc);
}

// QK: quantization kind. XT: activation type in memory. NT: token halves (1: M <= 8,
// 2: M <= 16). SPG: 32-wide K steps per quantization group (1, 2, 4).
template <int QK, typename XT, int NT, int SPG>
__global__ void __launch_bounds__(kWarps * 32, 2)
qmm_gemv_kernel(const __grid_constant__ CUtensorMap w_map, const GemvParams p) {
  // MMA element type: 4-bit affine codes fit bf16's 7 mantissa bits; 8-bit codes and the
  // E2M1 bit placement need f16.
  using AT = typename std::conditional<QK == kAff4, XT, __half>::type;
  using Ops = MmaOps<AT>;
  constexpr int BITS = (QK == kAff8) ? 8 : 4;
  constexpr int kBoxK = kBoxBytes * 8 / BITS;      // K elements per box: 256 or 128
  constexpr int kStepsPerBox = kBoxK / 32;         // 8 or 4
  constexpr int kGroupK = 32 * SPG;
  constexpr int kTU = 4;                           // table loads per thread kept in flight

  extern __shared__ uint8_t gv_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gv_smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int ring = p.ring;
  const int xrow = p.kc + kXPad;                   // staged row stride in elements
  const int tgroups = p.kc / kGroupK;              // groups staged per pass
  const int trow = tgroups + 1;                    // table row stride in float2 (odd: no conflicts)

  uint8_t* wring = smem + warp * ring * kBoxSmem;                                    // this warp's boxes
  AT* xs = reinterpret_cast<AT*>(smem + kWarps * ring * kBoxSmem);
  float2* tbl = reinterpret_cast<float2*>(reinterpret_cast<uint8_t*>(xs) + static_cast<size_t>(p.M) * xrow * sizeof(AT));
  float* red = reinterpret_cast<float*>(tbl + 2 * kRowsPerCta * trow);   // two buffers
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + 2 * kWarps * NT * 4 * 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + kWarps * kMaxRing);
  uint64_t* full = bars + warp * kMaxRing;

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
  const int64_t groups = p.K / kGroupK;
  const int nchunks = static_cast<int>((p.K + p.kc - 1) / p.kc);
  const int boxes_per_chunk = p.kc / kBoxK;
  const int ntiles = p.tiles, tstride = gridDim.x;
  const int tsize = (p.table_dtype == QMM_F32) ? 4 : 2;

  // Each warp owns its barriers: it initializes them itself and nobody else touches them.
  if (lane == 0) {
    for (int i = 0; i < kMaxRing; ++i) mbar_init(&full[i], 1);
    if (warp == 0) *abort_flag = 0;
    mbar_init_fence();
  }
  __syncwarp();

  // ---- request this warp's first boxes before anything else ----
  BoxCursor issue = {static_cast<int>(blockIdx.x), 0, 0, 0};
  cursor_seek<kBoxK>(issue, ntiles, tstride, nchunks, warp, static_cast<int>(p.K), p.kc);
  int issued = 0;
  auto issue_box = [&]() {   // lane 0 only
    const int slot = issued % ring;
    mbar_expect_tx(&full[slot], kBoxSmem);
    tma_load_2d(&w_map, wring + slot * kBoxSmem, &full[slot],
                (issue.chunk * boxes_per_chunk + issue.j) * kBoxBytes,
                static_cast<int>(wb * p.N) + issue.tile * kRowsPerCta);
    ++issued;
    cursor_next<kBoxK>(issue, ntiles, tstride, nchunks, warp, static_cast<int>(p.K), p.kc);
  };
  if (lane == 0)
    while (issued < ring && issue.tile < ntiles) issue_box();

  // ---- staging helpers ----
  // Activations of one chunk. Items are (token, 8-element piece). When the MMA's element type
  // is the activations' own, a piece is only re-paired with byte permutes; otherwise it is
  // converted through float32.
  auto stage_x = [&](int64_t kbase, int kc, int kfill) {
    constexpr int kXU = 4;
    const int pieces = kfill / 8;
    const int pieces_pad = (pieces + 31) & ~31;
    const float inv_pad = 1.0f / static_cast<float>(pieces_pad);
    const int items = static_cast<int>(p.M) * pieces_pad;
    for (int e0 = threadIdx.x; e0 < items; e0 += blockDim.x * kXU) {
      uint4 raw[kXU];
      int mm[kXU], pc[kXU];
#pragma unroll
      for (int u = 0; u < kXU; ++u) {
        const int e = e0 + u * blockDim.x;
        mm[u] = __float2int_rz((static_cast<float>(e) + 0.5f) * inv_pad);
        pc[u] = e - mm[u] * pieces_pad;
        raw[u] = make_uint4(0u, 0u, 0u, 0u);
        if (e < items && pc[u] * 8 < kc)
          raw[u] = __ldg(reinterpret_cast<const uint4*>(xg + static_cast<int64_t>(mm[u]) * p.K + kbase + pc[u] * 8));
      }
#pragma unroll
      for (int u = 0; u < kXU; ++u) {
        if (e0 + u * static_cast<int>(blockDim.x) - lane < items) {     // whole warps only
          uint4 o;
          if constexpr (std::is_same<AT, XT>::value) {
            if constexpr (QK == kAff4) {  // pair order (0,4)(1,5)(2,6)(3,7): what one LOP3 extracts
              o.x = __byte_perm(raw[u].x, raw[u].z, 0x5410); o.y = __byte_perm(raw[u].x, raw[u].z, 0x7632);
              o.z = __byte_perm(raw[u].y, raw[u].w, 0x5410); o.w = __byte_perm(raw[u].y, raw[u].w, 0x7632);
            } else {
              o = raw[u];
            }
          } else {                        // bf16 activations, f16 MMA
            const uint32_t r4[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
            uint32_t c4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
              c4[i] = pack_pair<AT>(__uint_as_float(r4[i] << 16), __uint_as_float(r4[i] & 0xffff0000u));
            o = make_uint4(c4[0], c4[1], c4[2], c4[3]);
          }
          if (pc[u] < pieces) *reinterpret_cast<uint4*>(xs + mm[u] * xrow + pc[u] * 8) = o;
        }
      }
    }
  };

  // Tables of one tile's 16 rows for one chunk: thread (r, c) of a 16 x 16 arrangement takes
  // groups c, c+16, ... of row r. `load` requests kTU of them, `store` converts and writes
  // (scale, bias - C*scale) pairs; the two halves can be separated by other work.
  const int tr = threadIdx.x >> 4, tc = threadIdx.x & 15;
  auto table_load = [&](int tile, int64_t kbase, int cgroups, int g0, uint32_t (&rs)[kTU], uint32_t (&rb)[kTU]) {
    const int64_t n0 = static_cast<int64_t>(tile) * kRowsPerCta;
    const int64_t row = wb * p.N + (n0 + tr < p.N ? n0 + tr : p.N - 1);
    const int64_t ti0 = row * groups + kbase / kGroupK;
#pragma unroll
    for (int u = 0; u < kTU; ++u) {
      const int gi = g0 + 16 * u;
      rs[u] = rb[u] = 0u;
      if (gi < cgroups) {
        if constexpr (QK == kMx4) {
          rs[u] = __ldg(reinterpret_cast<const uint8_t*>(p.scales) + ti0 + gi);
        } else {
          rs[u] = table_raw(p.scales, tsize, ti0 + gi);
          rb[u] = table_raw(p.biases, tsize, ti0 + gi);
        }
      }
    }
  };
  auto table_store = [&](float2* dst, int cgroups, int g0, const uint32_t (&rs)[kTU], const uint32_t (&rb)[kTU]) {
#pragma unroll
    for (int u = 0; u < kTU; ++u) {
      const int gi = g0 + 16 * u;
      if (gi < cgroups) {
        if constexpr (QK == kMx4) {
          dst[tr * trow + gi] = make_float2(__uint_as_float(rs[u] ? (rs[u] << 23) : 0x00400000u), 0.0f);
        } else {
          const float sv = table_value(rs[u], p.table_dtype);
          dst[tr * trow + gi] = make_float2(sv, table_value(rb[u], p.table_dtype) - Ops::kMagicValue * sv);
        }
      }
    }
  };
  auto stage_tables = [&](float2* dst, int tile, int64_t kbase, int cgroups) {
    for (int g0 = tc; g0 < cgroups; g0 += 16 * kTU) {
      uint32_t rs[kTU], rb[kTU];
      table_load(tile, kbase, cgroups, g0, rs, rb);
      table_store(dst, cgroups, g0, rs, rb);
    }
  };

  // With a single chunk the activations are staged once and the next tile's tables are
  // requested while the current tile is computed (one batch of kTU loads per thread).
  const bool resident = nchunks == 1 && tgroups <= 16 * kTU;
  int consumed = 0, tbuf = 0, rbuf = 0;
  bool ok = true, first = true;
  for (int tile = blockIdx.x; tile < ntiles; tile += tstride) {
    const int64_t n0 = static_cast<int64_t>(tile) * kRowsPerCta;
    float yacc[NT][4];
#pragma unroll
    for (int h = 0; h < NT; ++h)
#pragma unroll
      for (int i = 0; i < 4; ++i) yacc[h][i] = 0.0f;

    for (int chunk = 0; chunk < nchunks; ++chunk) {
      const int64_t kbase = static_cast<int64_t>(chunk) * p.kc;
      const int kc = static_cast<int>(p.K - kbase < p.kc ? p.K - kbase : p.kc);     // multiple of 32
      const int nb = (kc + kBoxK - 1) / kBoxK;
      const int kfill = nb * kBoxK;                                                 // zero-padded extent
      const int cgroups = kc / kGroupK;
      if (!resident || first) {
        __syncthreads();                       // everyone is done with the previous contents
        if (nchunks > 1 || first) stage_x(kbase, kc, kfill);
        stage_tables(tbl + tbuf * kRowsPerCta * trow, tile, kbase, cgroups);
        __syncthreads();
        first = false;
      }
      const float2* tcur = tbl + tbuf * kRowsPerCta * trow;
      uint32_t prs[kTU], prb[kTU];
      const bool prefetch = resident && tile + tstride < ntiles;
      if (prefetch) table_load(tile + tstride, 0, cgroups, tc, prs, prb);

      // ---- this warp's boxes of the chunk ----
      const int jlo = nb * warp / kWarps, jhi = nb * (warp + 1) / kWarps;
      for (int j = jlo; j < jhi && ok; ++j, ++consumed) {
        const int slot = consumed % ring;
        if (!(ok = mbar_wait(&full[slot], (consumed / ring) & 1, abort_flag, 11))) break;
        const uint8_t* box = wring + slot * kBoxSmem;
        const uint8_t* row0 = box + g * kBoxBytes;
        const uint8_t* row1 = box + (g + 8) * kBoxBytes;
#pragma unroll
        for (int q = 0; q < kStepsPerBox / SPG; ++q) {          // groups of this box
          const int gi = (j * kBoxK) / kGroupK + q;             // group index within the chunk
          if (gi < cgroups) {
            float acc[NT][4], ones[NT][4];
#pragma unroll
            for (int s = 0; s < SPG; ++s) {
              const int ks = q * SPG + s;                         // K step within the box
              const int kloc = j * kBoxK + ks * 32 + t * 8;       // within the staged chunk
              uint32_t a[2][4];
              if constexpr (QK == kAff8) {
                // 32 bytes per row and step: lane t takes bytes [8t, 8t+8) of them
                const int off = (((ks * 2 + (t >> 1)) ^ (g & 7)) << 4) + (t & 1) * 8;
                const uint2 u0 = *reinterpret_cast<const uint2*>(row0 + off);
                const uint2 u1 = *reinterpret_cast<const uint2*>(row1 + off);
                a[0][0] = __byte_perm(u0.x, 0x64646464u, 0x4140); a[0][1] = __byte_perm(u1.x, 0x64646464u, 0x4140);
                a[0][2] = __byte_perm(u0.x, 0x64646464u, 0x4342); a[0][3] = __byte_perm(u1.x, 0x64646464u, 0x4342);
                a[1][0] = __byte_perm(u0.y, 0x64646464u, 0x4140); a[1][1] = __byte_perm(u1.y, 0x64646464u, 0x4140);
                a[1][2] = __byte_perm(u0.y, 0x64646464u, 0x4342); a[1][3] = __byte_perm(u1.y, 0x64646464u, 0x4342);
              } else {
                // 16 bytes per row and step: lane t takes word t
                const int off = ((ks ^ (g & 7)) << 4) + t * 4;
                const uint32_t u0 = *reinterpret_cast<const uint32_t*>(row0 + off);
                const uint32_t u1 = *reinterpret_cast<const uint32_t*>(row1 + off);
                if constexpr (QK == kAff4) {
                  a[0][0] = (u0 & 0x000F000Fu) | Ops::kMagic;         a[0][1] = (u1 & 0x000F000Fu) | Ops::kMagic;
                  a[0][2] = ((u0 >> 4) & 0x000F000Fu) | Ops::kMagic;  a[0][3] = ((u1 >> 4) & 0x000F000Fu) | Ops::kMagic;
                  a[1][0] = ((u0 >> 8) & 0x000F000Fu) | Ops::kMagic;  a[1][1] = ((u1 >> 8) & 0x000F000Fu) | Ops::kMagic;
                  a[1][2] = ((u0 >> 12) & 0x000F000Fu) | Ops::kMagic; a[1][3] = ((u1 >> 12) & 0x000F000Fu) | Ops::kMagic;
                } else {
                  // The three magnitude bits of an E2M1 code at f16's exponent/mantissa boundary
                  // are the code's value times 2^-14 (code 1 = 0.5 lands on a subnormal); the
                  // sign bit goes to bit 15. The 2^14 is restored in the fold.
#pragma unroll
                  for (int r = 0; r < 2; ++r) {
                    const uint32_t u = r ? u1 : u0;
                    const uint32_t uh = u >> 4;
#pragma unroll
                    for (int bb = 0; bb < 4; ++bb) {  // byte bb -> elements (2bb, 2bb+1)
                      const uint32_t tt = __byte_perm(u, uh, bb | ((4 + bb) << 8));
                      a[bb >> 1][(bb & 1) * 2 + r] = ((tt << 9) & 0x0E000E00u) | ((tt << 12) & 0x80008000u);
                    }
                  }
                }
              }
              const float zero4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
              const uint32_t one4[4] = {Ops::kOnes, Ops::kOnes, Ops::kOnes, Ops::kOnes};
#pragma unroll
              for (int h = 0; h < NT; ++h) {
                uint4 xv = make_uint4(0u, 0u, 0u, 0u);
                if (h * 8 + g < p.M) xv = *reinterpret_cast<const uint4*>(xs + (h * 8 + g) * xrow + kloc);
                if (s == 0) Ops::mma(acc[h], a[0], xv.x, xv.y, zero4);
                else Ops::mma(acc[h], a[0], xv.x, xv.y, acc[h]);
                Ops::mma(acc[h], a[1], xv.z, xv.w, acc[h]);
                if constexpr (QK != kMx4) {   // sum of x over the group: A = all ones
                  if (s == 0) Ops::mma(ones[h], one4, xv.x, xv.y, zero4);
                  else Ops::mma(ones[h], one4, xv.x, xv.y, ones[h]);
                  Ops::mma(ones[h], one4, xv.z, xv.w, ones[h]);
                }
              }
            }
            // fold the group: rows g (c0, c1) and g+8 (c2, c3), tokens 2t and 2t+1
            const float2 sb0 = tcur[g * trow + gi], sb1 = tcur[(g + 8) * trow + gi];
#pragma unroll
            for (int h = 0; h < NT; ++h) {
              if constexpr (QK == kMx4) {
                yacc[h][0] = fmaf(sb0.x, acc[h][0] * 16384.0f, yacc[h][0]);
                yacc[h][1] = fmaf(sb0.x, acc[h][1] * 16384.0f, yacc[h][1]);
                yacc[h][2] = fmaf(sb1.x, acc[h][2] * 16384.0f, yacc[h][2]);
                yacc[h][3] = fmaf(sb1.x, acc[h][3] * 16384.0f, yacc[h][3]);
              } else {
                yacc[h][0] = fmaf(sb0.x, acc[h][0], fmaf(sb0.y, ones[h][0], yacc[h][0]));
                yacc[h][1] = fmaf(sb0.x, acc[h][1], fmaf(sb0.y, ones[h][1], yacc[h][1]));
                yacc[h][2] = fmaf(sb1.x, acc[h][2], fmaf(sb1.y, ones[h][0], yacc[h][2]));
                yacc[h][3] = fmaf(sb1.x, acc[h][3], fmaf(sb1.y, ones[h][1], yacc[h][3]));
              }
            }
          }
        }
        // the slot is free again: refill it with the next box this warp will need
        __syncwarp();
        if (lane == 0 && issue.tile < ntiles) {
          fence_proxy_async();
          issue_box();
        }
      }
      if (prefetch) table_store(tbl + (tbuf ^ 1) * kRowsPerCta * trow, cgroups, tc, prs, prb);
      if (resident) tbuf ^= 1;
    }

    // ---- reduce the K split across warps (fixed order) and store this tile ----
    float* rcur = red + rbuf * kWarps * NT * 4 * 32;
#pragma unroll
    for (int h = 0; h < NT; ++h)
#pragma unroll
      for (int i = 0; i < 4; ++i) rcur[(warp * NT * 4 + h * 4 + i) * 32 + lane] = yacc[h][i];
    __syncthreads();
    if (*abort_flag) {
      if (threadIdx.x == 0) atomicCAS(p.status, 0, *abort_flag);
      return;
    }
    if (warp == 0) {
#pragma unroll
      for (int h = 0; h < NT; ++h)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float v = 0.0f;
#pragma unroll
          for (int wv = 0; wv < kWarps; ++wv) v += rcur[(wv * NT * 4 + h * 4 + i) * 32 + lane];
          const int64_t row = n0 + g + (i >> 1) * 8;
          const int64_t tok = h * 8 + 2 * t + (i & 1);
          if (row < p.N && tok < p.M) gv_store(p.y, p.y_dtype, y_off + tok * p.N + row, v);
        }
    }
    rbuf ^= 1;
  }
}

template <int QK, typename XT, int NT, int SPG>
int launch_kernel(const CUtensorMap& wm, const GemvParams& gp, cudaStream_t stream) {
  const int tgroups = gp.kc / (32 * SPG);
  const size_t smem = 1024 + static_cast<size_t>(kWarps) * gp.ring * kBoxSmem +
                      static_cast<size_t>(gp.M) * (gp.kc + kXPad) * 2 +
                      static_cast<size_t>(2) * kRowsPerCta * (tgroups + 1) * sizeof(float2) +
                      static_cast<size_t>(2) * kWarps * NT * 4 * 32 * sizeof(float) +
                      static_cast<size_t>(kWarps) * kMaxRing * sizeof(uint64_t) + 16;
  // Persistent CTAs: two per SM share the machine's segments; a CTA walks tiles with a grid stride.
  int64_t per_seg = (2LL * device_sm_count() + gp.batch - 1) / gp.batch;
  if (per_seg < 1) per_seg = 1;
  if (per_seg > gp.tiles) per_seg = gp.tiles;
  dim3 grid(static_cast<unsigned>(per_seg), static_cast<unsigned>(gp.batch));
  auto kernel = qmm_gemv_kernel<QK, XT, NT, SPG>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured = true;
  }
  kernel<<<grid, kWarps * 32, smem, stream>>>(wm, gp);
  count_launch();
  return check_launch("qmm_gemv_kernel");
}

template <int QK, typename XT, int NT>
int launch_spg(const CUtensorMap& wm, const GemvParams& gp, cudaStream_t stream) {
  if constexpr (QK == kMx4) {
    return launch_kernel<QK, XT, NT, 1>(wm, gp, stream);
  } else {
    if (gp.group_size == 32) return launch_kernel<QK, XT, NT, 1>(wm, gp, stream);
    if (gp.group_size == 64) return launch_kernel<QK, XT, NT, 2>(wm, gp, stream);
    return launch_kernel<QK, XT, NT, 4>(wm, gp, stream);
  }
}

template <int QK>
int launch_xt(const CUtensorMap& wm, const GemvParams& gp, int x_dtype, cudaStream_t stream) {
  if (x_dtype == QMM_BF16)
    return gp.M <= 8 ? launch_spg<QK, __nv_bfloat16, 1>(wm, gp, stream) : launch_spg<QK, __nv_bfloat16, 2>(wm, gp, stream);
  return gp.M <= 8 ? launch_spg<QK, __half, 1>(wm, gp, stream) : launch_spg<QK, __half, 2>(wm, gp, stream);
}

}  // namespace

bool gemv_supports(const qmm_problem& p) {
  if (p.x_dtype != QMM_BF16 && p.x_dtype != QMM_F16) return false;
  if (p.group_sizes) return false;                 // ragged rows go to the tensor-core kernel
  if (p.M < 1 || p.M > 16) return false;
  if (p.batch > 65535) return false;
  if (p.K % 32 || p.K >= (1LL << 30)) return false;
  const int64_t nw = p.num_weights > 0 ? p.num_weights : (p.w_batch_stride ? p.batch : 1);
  if (nw * p.N >= (1LL << 31)) return false;        // TMA row coordinates are 32-bit
  return true;
}

int launch_gemv(const qmm_problem& p, cudaStream_t stream) {
  GemvParams gp;
  gp.x = p.x; gp.scales = p.scales; gp.biases = p.biases; gp.y = p.y;
  gp.lhs_idx = p.lhs_idx; gp.rhs_idx = p.rhs_idx;
  gp.status = device_status_word();
  if (!gp.status) return fail(QMM_ERR_CUDA, "could not allocate the device status word");
  gp.M = p.M; gp.K = p.K; gp.N = p.N; gp.batch = p.batch;
  gp.x_batch_stride = p.x_batch_stride; gp.y_batch_stride = p.y_batch_stride;
  gp.w_batch_rows = p.rhs_idx ? p.N : p.w_batch_stride;
  gp.group_size = p.group_size; gp.table_dtype = p.table_dtype; gp.y_dtype = p.y_dtype;
  gp.tiles = static_cast<int>((p.N + kRowsPerCta - 1) / kRowsPerCta);
  const int bits = (p.mode == QMM_MODE_AFFINE && p.bits == 8) ? 8 : 4;
  const int boxk = kBoxBytes * 8 / bits;
  // K elements staged per pass: the staged activations stay under ~64 KiB per CTA, and a
  // pass is a whole number of boxes.
  int kc = static_cast<int>(65536 / (2 * p.M) / boxk * boxk);
  const int64_t kround = (p.K + boxk - 1) / boxk * boxk;
  if (kround < kc) kc = static_cast<int>(kround);
  gp.kc = kc;
  // Ring depth: two tiles' worth of a warp's boxes, up to kMaxRing, so that a warp's requests
  // run ahead across tile boundaries.
  const int64_t boxes = (p.K + boxk - 1) / boxk;
  int64_t per_warp = 2 * ((boxes + kWarps - 1) / kWarps);
  gp.ring = static_cast<int>(per_warp < 1 ? 1 : (per_warp > kMaxRing ? kMaxRing : per_warp));

  // The packed weight as a 2-D byte tensor [rows, K*bits/8] over every weight matrix behind
  // `w`; a box that reaches past the last row is zero-filled by the TMA unit.
  const uint64_t row_bytes = static_cast<uint64_t>(p.K) * bits / 8;
  const uint64_t nw = p.num_weights > 0 ? p.num_weights : (p.w_batch_stride ? p.batch : 1);
  const uint64_t rows = static_cast<uint64_t>(p.N) * nw;
  CUtensorMap wm;
  int rc = tensor_map_2d(&wm, QMM_U8, p.w, row_bytes, rows, row_bytes, kBoxBytes, kRowsPerCta, 1);
  if (rc) return rc;
  if (p.mode == QMM_MODE_MXFP4) return launch_xt<kMx4>(wm, gp, p.x_dtype, stream);
  if (p.bits == 8) return launch_xt<kAff8>(wm, gp, p.x_dtype, stream);
  return launch_xt<kAff4>(wm, gp, p.x_dtype, stream);
}

}  // namespace qmm
