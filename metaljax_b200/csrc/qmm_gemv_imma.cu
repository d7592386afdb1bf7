// Single-row decode kernel of the fused dequantize-and-matmul (M = 1 of `y = x . deq(w)^T`,
// src/metaljax/qmm.py:2491): the packed weight is streamed once and meets the activation row
// on the integer tensor-core path, so that a packed word costs four instructions instead of
// the dozen a floating-point dequantization needs.
//
// Arithmetic. The activation row is rewritten once per CTA as a 24-bit fixed-point number per
// element, relative to the row's largest magnitude (x_k = X_k * 2^(e-148), |X_k| <= 2^22, the
// resolution a float32 accumulator has relative to its largest term), and X_k is split into
// three signed base-256 digits  X_k = d0 + 256 d1 + 65536 d2,  d in [-128, 127].  The digit
// planes are the A operand (16 rows x 32 K, s8) of `mma.sync.m16n8k32.s32.s8.u8`; eight weight
// rows are the B operand (32 K x 8, u8): a packed 4-bit word becomes two B registers with
// `w & 0x0F0F0F0F` and `(w >> 4) & 0x0F0F0F0F`, an 8-bit word is a B register as it stands, an
// E2M1 word goes through two byte-permute lookups (16 + 2*value, the 16 is taken out again
// through the accumulator's start value). The integer sums are exact.
//
// The 16 A rows carry (group slot, digit) pairs: row 3s+d of an MMA holds digit plane d with
// every K position outside quantization group slot s zeroed, so ONE chain of MMAs over a box of
// 256 codes leaves the four groups' sums  sum_k q_k d_k  in separate accumulator rows, and the
// per-group scale is applied once per box: y += scale[n, g] * sum. The accumulators start at
// the float32 magic 2^23 + 2^22, which makes `int -> float` one subtraction. The bias term
// sum_g bias[n, g] * sum_{k in g} x_k  is added when a tile of rows is finished.
//
// Data movement. A CTA owns 8R consecutive weight rows at a time (R = 1, 2, 4) and its 8 warps
// split K by 128-byte columns; packed rows arrive by TMA in boxes of 8R rows x 128 bytes
// (128-byte swizzle: the 16-byte fragment reads are conflict free), every warp with its own
// ring of boxes and one mbarrier per slot. Lane 0 of a warp requests the first boxes before
// anything else happens in the kernel and refills a slot as soon as the warp has consumed it.
// Scale pairs are read straight from global memory (L1/L2) at the start of a box and used at
// its end. The K split is reduced in shared memory in fixed order; no global scratch, no
// atomics, every wait bounded.
//
// The kernel is launched with programmatic stream serialization: it lets its successor start
// at once, and itself touches only the packed weight and its tables before
// `griddepcontrol.wait` (of the kernels that release their successors early -- this library's
// decode kernels -- none writes a weight); the activations are read, and y is written, after it.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <type_traits>

#include "qmm_internal.h"
#include "qmm_ptx.cuh"

namespace qmm {
namespace {

using namespace ptx;

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kBoxBytes = 128;                 // bytes of one weight row in a box
constexpr int kMaxRing = 8;                    // boxes a warp keeps in flight, at most
constexpr uint32_t kMagicBits = 0x4B400000u;   // float32 2^23 + 2^22
constexpr float kMagicValue = 12582912.0f;
constexpr int kXCache = 4;                     // 8-element pieces of x a thread keeps in registers

enum { kAff4 = 0, kAff8 = 1, kMx4 = 2 };

struct ImmaParams {
  const void* x;
  const void* scales;
  const void* biases;
  void* y;
  int* status;
  int K, N;
  int groups;         // K / group_size
  int group_size, table_dtype, y_dtype;
  int ntiles;         // tiles of 8R rows
  int nchunks;        // boxes per row: ceil(K * bits / 8 / 128)
  int ring;           // boxes per warp in flight (1..kMaxRing)
  int part_stride;    // bytes between the digit planes of the staged activations
};

// d = a * b + c: 16 x 32 (s8) times 32 x 8 (u8), int32 accumulate.
__device__ __forceinline__ void imma(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, const int (&c)[4]) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}

// Generic byte permute: each selector nibble picks one of the eight bytes of {a, b}; with its
// bit 3 set it yields the sign bit of that byte replicated over the byte instead.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

__device__ __forceinline__ uint32_t ldg_u32(const void* p) { return __ldg(static_cast<const uint32_t*>(p)); }
__device__ __forceinline__ uint32_t ldg_u16(const void* p) { return __ldg(static_cast<const uint16_t*>(p)); }
__device__ __forceinline__ uint32_t ldg_u8(const void* p) { return __ldg(static_cast<const uint8_t*>(p)); }

template <typename XT>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
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

// Largest 15-bit magnitude pattern among the eight 16-bit floats of `v` (for both bf16 and f16
// the patterns order like the magnitudes).
__device__ __forceinline__ uint32_t max_mag16(const uint4& v, uint32_t m) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m = max(m, u[i] & 0x7fffu);
    m = max(m, (u[i] >> 16) & 0x7fffu);
  }
  return m;
}

// Sum over the 8 lanes that share `lane & 3` of NV values per lane, leaving value number
// (bits 4, 3, 2 of the lane, as far as NV reaches) in v[0]: each step sends half of what is
// left to the partner lane and adds what the partner sent.
template <int NV>
__device__ __forceinline__ void reduce_over_g(float (&v)[NV], int lane) {
  int n = NV;
#pragma unroll
  for (int stage = 0; stage < 3; ++stage) {
    const int mask = 16 >> stage;
    const bool up = (lane & mask) != 0;
    if (n > 1) {
      n >>= 1;
#pragma unroll
      for (int i = 0; i < NV / 2; ++i) {
        if (i < n) {
          const float send = up ? v[i] : v[i + n];
          const float keep = up ? v[i + n] : v[i];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
        }
      }
    } else {
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], mask);
    }
  }
}

// QK: quantization kind. XT: activation type in memory. R: 8-row blocks per tile.
template <int QK, typename XT, int R>
__global__ void __launch_bounds__(kThreads, 2)
qmm_gemv_imma_kernel(const __grid_constant__ CUtensorMap w_map, const ImmaParams p) {
  constexpr int BITS = (QK == kAff8) ? 8 : 4;
  constexpr int kBoxCodes = kBoxBytes * 8 / BITS;    // 256 or 128 codes per row and box
  constexpr int kSpanBytes = 16 * 8 / BITS;          // staged activation bytes per 16 weight bytes: 32 or 16
  constexpr int kSteps = 16 * 8 / BITS / 8;          // MMAs per 16 weight bytes: 4 or 2
  constexpr int kTileRows = 8 * R;
  constexpr int kBoxSmem = kTileRows * kBoxBytes;
  constexpr bool kNatural = (QK != kAff4);           // order of the staged activations inside 8 codes

  extern __shared__ uint8_t imma_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(imma_smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ring = p.ring;
  const int kpad = p.nchunks * kBoxCodes;            // staged bytes per digit plane

  uint8_t* xs = smem + kWarps * ring * kBoxSmem;     // three digit planes, p.part_stride apart (+0, +16, +64)
  float* xsum = reinterpret_cast<float*>(xs + 3 * p.part_stride);       // [groups] sums of x (int32 [groups][4] for MXFP4)
  const int xsum_words = (QK == kMx4) ? 4 * ((p.groups + 7) & ~7) : ((p.groups + 7) & ~7);
  float* red = xsum + xsum_words;                    // [2][kWarps][kTileRows]
  uint64_t* full_all = reinterpret_cast<uint64_t*>(red + 2 * kWarps * kTileRows);
  uint32_t* zeros = reinterpret_cast<uint32_t*>(full_all + kWarps * kMaxRing);   // 32 zero bytes
  uint32_t* amax_w = zeros + 8;                      // [kWarps]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(amax_w + kWarps);

  // ---- barriers, then this warp's first boxes: before anything else ----
  uint64_t* full = full_all + warp * kMaxRing;
  uint8_t* wring = smem + warp * ring * kBoxSmem;
  const int ntiles = p.ntiles, nchunks = p.nchunks, tstride = gridDim.x;
  int itile = blockIdx.x, ichunk = warp, issued = 0, islot = 0;       // lane 0: the next box to request
  auto issue_box = [&]() {
    mbar_expect_tx(&full[islot], kBoxSmem);
    tma_load_2d(&w_map, wring + islot * kBoxSmem, &full[islot], ichunk * kBoxBytes, itile * kTileRows);
    ++issued;
    if (++islot == ring) islot = 0;
    ichunk += kWarps;
    if (ichunk >= nchunks) { ichunk = warp; itile += tstride; }
  };
  if (lane == 0) {
    if (warp == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&w_map)) : "memory");
      *abort_flag = 0;
    }
    for (int i = 0; i < ring; ++i) mbar_init(&full[i], 1);
    mbar_init_fence();
    if (warp < nchunks)
      while (issued < ring && itile < ntiles) issue_box();
  }
  if (threadIdx.x < 8) zeros[threadIdx.x] = 0u;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __syncwarp();

  // ---- lane constants ----
  const int g = lane >> 2, t = lane & 3;
  const int rho = (g >> 1) | ((g & 1) << 2);         // box row (of 8) behind MMA column g: the two
                                                     // rows a quarter-warp reads lie 4 apart
  const int gpb = kBoxCodes / p.group_size;          // groups per box: 8, 4, 2 or 1
  const bool fold_half = gpb == 8;                   // eight groups: the box is folded in two halves
  const bool valid = g < 6;
  const int sigma0 = 2 * (g / 3);                    // group slot of A row g (row g + 8: sigma0 + 1)
  const int part = valid ? g % 3 : 0;                // digit plane of A rows g and g + 8
  const uint32_t xs_u32 = smem_u32(xs), zero_u32 = smem_u32(zeros);
  const uint32_t part_base = xs_u32 + part * p.part_stride + (part == 1 ? 16 : (part == 2 ? 64 : 0));
  uint32_t woff[2], xa[2][2], xinc[2][2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    woff[h] = smem_u32(wring) + rho * kBoxBytes + ((((4 * h + t) ^ rho) & 7) << 4);
    const int grp = (4 * h + t) * kSpanBytes / p.group_size;     // group of this lane's span within the box
    const int slot = fold_half ? (grp & 3) : grp;
#pragma unroll
    for (int rh = 0; rh < 2; ++rh) {
      const bool act = valid && (sigma0 + rh == slot);
      xa[h][rh] = act ? part_base + (4 * h + t) * kSpanBytes : zero_u32;
      xinc[h][rh] = act ? kBoxCodes : 0;
    }
  }
  // rows of the scale tables this lane folds (tile-relative): columns 2t and 2t + 1 of the MMA
  const int frow0 = t, frow1 = t + 4;
  const int tsize = (QK == kMx4) ? 1 : 2;
  const bool tpair = (p.groups & 1) == 0 && gpb >= 2 && (reinterpret_cast<uintptr_t>(p.scales) & 3) == 0;
  const uint8_t* sc8 = static_cast<const uint8_t*>(p.scales);

  // The (sigma0, sigma0 + 1) scale entries of table row `n` for the fold that starts at group
  // `gb`, as two 16-bit fields of one word. Indices past the end are clamped: the sums they
  // meet are zero.
  auto scale_pair = [&](int trow, int gb) -> uint32_t {
    const int64_t n = trow;
    int g0 = gb + sigma0;
    if (tpair) {
      if (g0 + 1 >= p.groups) g0 = p.groups - 2;
      const uint8_t* at = sc8 + (n * p.groups + g0) * tsize;
      return (QK == kMx4) ? ldg_u16(at) : ldg_u32(at);
    }
    const int g1 = g0 + 1 < p.groups ? g0 + 1 : p.groups - 1;
    if (g0 >= p.groups) g0 = p.groups - 1;
    const uint8_t* tr = sc8 + n * p.groups * tsize;
    if (QK == kMx4) return ldg_u8(tr + g0) | (ldg_u8(tr + g1) << 8);
    return ldg_u16(tr + g0 * 2) | (ldg_u16(tr + g1 * 2) << 16);
  };
  auto scale_lo = [&](uint32_t raw) -> float {
    if (QK == kMx4) return __uint_as_float(max((raw & 0xffu) << 23, 0x00400000u));
    if (p.table_dtype == QMM_BF16) return __uint_as_float(raw << 16);
    return __half2float(__ushort_as_half(static_cast<unsigned short>(raw & 0xffffu)));
  };
  auto scale_hi = [&](uint32_t raw) -> float {
    if (QK == kMx4) return __uint_as_float(max(((raw >> 8) & 0xffu) << 23, 0x00400000u));
    if (p.table_dtype == QMM_BF16) return __uint_as_float(raw & 0xffff0000u);
    return __half2float(__ushort_as_half(static_cast<unsigned short>(raw >> 16)));
  };

  // ---- the activation row: after everything the previous kernel wrote is visible ----
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const XT* xg = static_cast<const XT*>(p.x);
  const int vpieces = p.K / 8, ppieces = kpad / 8;
  const int iters = (ppieces + kThreads - 1) / kThreads;
  uint4 xcache[kXCache];
  uint32_t mag = 0;
#pragma unroll
  for (int i = 0; i < kXCache; ++i) {
    const int pc = threadIdx.x + i * kThreads;
    xcache[i] = make_uint4(0u, 0u, 0u, 0u);
    if (pc < vpieces) xcache[i] = __ldg(reinterpret_cast<const uint4*>(xg + pc * 8));
    mag = max_mag16(xcache[i], mag);
  }
  for (int i = kXCache; i < iters; ++i) {
    const int pc = threadIdx.x + i * kThreads;
    if (pc < vpieces) mag = max_mag16(__ldg(reinterpret_cast<const uint4*>(xg + pc * 8)), mag);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mag = max(mag, __shfl_xor_sync(0xffffffffu, mag, o));
  if (lane == 0) amax_w[warp] = mag;
  __syncthreads();
  mag = 0;
#pragma unroll
  for (int i = 0; i < kWarps; ++i) mag = max(mag, amax_w[i]);
  // exponent field of the largest magnitude as a float32; infinities and NaNs poison the row
  uint32_t ebits;
  bool nonfinite;
  if constexpr (std::is_same<XT, __nv_bfloat16>::value) {
    ebits = mag >> 7;
    nonfinite = mag >= 0x7f80u;
  } else {
    ebits = (__float_as_uint(__half2float(__ushort_as_half(static_cast<unsigned short>(mag)))) >> 23) & 0xffu;
    nonfinite = mag >= 0x7c00u;
  }
  if (ebits < 23u || nonfinite) ebits = 23u;   // (magnitudes below 2^-104 lose digits: far below anything real)
  const float to_fixed = __uint_as_float((275u - ebits) << 23);      // 2^(148 - e): |x| * this <= 2^22
  const float from_fixed = __uint_as_float((ebits - 21u) << 23);     // 2^(e - 148)
  {
    const int lanes_per_group = (QK == kMx4 ? 32 : p.group_size) / 8;
    for (int i = 0; i < iters; ++i) {
      const int pc = threadIdx.x + i * kThreads;
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if (i < kXCache) {
#pragma unroll
        for (int c = 0; c < kXCache; ++c)
          if (c == i) raw = xcache[c];
      } else if (pc < vpieces) {
        raw = __ldg(reinterpret_cast<const uint4*>(xg + pc * 8));
      }
      float f[8];
      unpack8<XT>(raw, f);
      uint32_t d[8], tsum = 0;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const uint32_t tb = __float_as_uint(fmaf(nonfinite ? 0.0f : f[e], to_fixed, kMagicValue));   // magic + X
        tsum += tb;
        d[e] = (tb + (0x00808080u - kMagicBits)) ^ 0x00808080u;       // bytes 0..2: the three digits
      }
      const int xsum_i = static_cast<int>(tsum - 8u * kMagicBits);    // sum of the piece's X
      uint32_t lo[3], hi[3];
#pragma unroll
      for (int q = 0; q < 3; ++q) {
        if constexpr (kNatural) {     // codes 0..3 | 4..7
          lo[q] = __byte_perm(__byte_perm(d[0], d[1], q | ((4 + q) << 4)), __byte_perm(d[2], d[3], q | ((4 + q) << 4)), 0x5410);
          hi[q] = __byte_perm(__byte_perm(d[4], d[5], q | ((4 + q) << 4)), __byte_perm(d[6], d[7], q | ((4 + q) << 4)), 0x5410);
        } else {                      // codes 0, 2, 4, 6 | 1, 3, 5, 7: what the two nibble masks extract
          lo[q] = __byte_perm(__byte_perm(d[0], d[2], q | ((4 + q) << 4)), __byte_perm(d[4], d[6], q | ((4 + q) << 4)), 0x5410);
          hi[q] = __byte_perm(__byte_perm(d[1], d[3], q | ((4 + q) << 4)), __byte_perm(d[5], d[7], q | ((4 + q) << 4)), 0x5410);
        }
      }
      if (pc < ppieces) {
        *reinterpret_cast<uint2*>(xs + pc * 8) = make_uint2(lo[0], hi[0]);
        *reinterpret_cast<uint2*>(xs + p.part_stride + 16 + pc * 8) = make_uint2(lo[1], hi[1]);
        *reinterpret_cast<uint2*>(xs + 2 * p.part_stride + 64 + pc * 8) = make_uint2(lo[2], hi[2]);
      }
      if constexpr (QK == kMx4) {
        // per group and digit plane: the sum of the digits (what the +16 of every code met)
        int ds[3];
#pragma unroll
        for (int q = 0; q < 3; ++q) ds[q] = __dp4a(static_cast<int>(lo[q]), 0x01010101, __dp4a(static_cast<int>(hi[q]), 0x01010101, 0));
#pragma unroll
        for (int o = 1; o < 4; o <<= 1)
#pragma unroll
          for (int q = 0; q < 3; ++q) ds[q] += __shfl_xor_sync(0xffffffffu, ds[q], o);
        const int grp = pc >> 2;
        if ((lane & 3) == 0 && grp < p.groups) {
          int* dst = reinterpret_cast<int*>(xsum) + grp * 4;
          dst[0] = ds[0]; dst[1] = ds[1]; dst[2] = ds[2]; dst[3] = 0;
        }
      } else {
        int s = xsum_i;
        for (int o = 1; o < lanes_per_group; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const int grp = pc / lanes_per_group;
        if ((lane & (lanes_per_group - 1)) == 0 && grp < p.groups) xsum[grp] = static_cast<float>(s) * from_fixed;
      }
    }
  }
  __syncthreads();                   // the staged activations, their sums and the zeros are in place

  // what one unit of an accumulator is worth for this lane's digit plane
  const float pscale = valid ? __uint_as_float((ebits - 21u + 8u * part - (QK == kMx4 ? 1u : 0u)) << 23) : 0.0f;
  uint32_t nib = 0x0F0F0F0Fu;
  asm volatile("" : "+r"(nib));      // keep the mask in a register: one LOP3 per use
  const int magic4[4] = {static_cast<int>(kMagicBits), static_cast<int>(kMagicBits), static_cast<int>(kMagicBits),
                         static_cast<int>(kMagicBits)};

  int cslot = 0, rbuf = 0;
  uint32_t cphase = 0;
  bool ok = true;
  for (int tile = blockIdx.x; tile < ntiles; tile += tstride) {
    const int64_t n0 = static_cast<int64_t>(tile) * kTileRows;
    float yacc[R][2];
#pragma unroll
    for (int rb = 0; rb < R; ++rb) yacc[rb][0] = yacc[rb][1] = 0.0f;
    int nrow[R][2];                  // table rows of this lane's two MMA columns, clamped to the last row
#pragma unroll
    for (int rb = 0; rb < R; ++rb) {
      nrow[rb][0] = min(tile * kTileRows + rb * 8 + frow0, p.N - 1);
      nrow[rb][1] = min(tile * kTileRows + rb * 8 + frow1, p.N - 1);
    }

    for (int c = warp; c < nchunks && ok; c += kWarps) {
      // scale pairs of the box's (first) fold: requested now, used after the MMAs
      uint32_t sraw[R][2];
      const int gb0 = c * gpb;
#pragma unroll
      for (int rb = 0; rb < R; ++rb) {
        sraw[rb][0] = scale_pair(nrow[rb][0], gb0);
        sraw[rb][1] = scale_pair(nrow[rb][1], gb0);
      }
      if (!(ok = mbar_wait(&full[cslot], cphase, abort_flag, 21))) break;
      const uint32_t boxoff = cslot * kBoxSmem;
      if (++cslot == ring) { cslot = 0; cphase ^= 1u; }
      int acc[R][4];
      bool fresh = true;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        // this lane's 16 bytes of every row block, and the digit bytes they meet
        uint32_t wv[R][4];
#pragma unroll
        for (int rb = 0; rb < R; ++rb) {
          uint4 v;
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                       : "r"(woff[h] + boxoff + rb * 8 * kBoxBytes));
          wv[rb][0] = v.x; wv[rb][1] = v.y; wv[rb][2] = v.z; wv[rb][3] = v.w;
        }
        uint32_t xv[2][2 * kSteps];      // [row half][step: (k-slots 0..15, k-slots 16..31)]
#pragma unroll
        for (int rh = 0; rh < 2; ++rh) {
          const uint32_t a = xa[h][rh] + c * xinc[h][rh];
#pragma unroll
          for (int q = 0; q < kSpanBytes / 16; ++q) {
            const uint4 v = (q == 0) ? lds128<0>(a) : lds128<16>(a);
            xv[rh][4 * q] = v.x; xv[rh][4 * q + 1] = v.y; xv[rh][4 * q + 2] = v.z; xv[rh][4 * q + 3] = v.w;
          }
        }
        int cinit[4] = {magic4[0], magic4[1], magic4[2], magic4[3]};
        if constexpr (QK == kMx4) {
          if (fresh) {
            // every code was given as 16 + 2*value: start at magic - 16 * (sum of the digits)
            const int gbase = c * gpb + (fold_half ? 4 * h : 0) + sigma0;
            const int* xi = reinterpret_cast<const int*>(xsum);   // (groups past the end of K met only zeros)
            const int s0 = gbase < p.groups ? xi[gbase * 4 + part] : 0;
            const int s1 = gbase + 1 < p.groups ? xi[(gbase + 1) * 4 + part] : 0;
            cinit[0] = cinit[1] = static_cast<int>(kMagicBits) - 16 * s0;
            cinit[2] = cinit[3] = static_cast<int>(kMagicBits) - 16 * s1;
          }
        }
#pragma unroll
        for (int j = 0; j < kSteps; ++j) {
          const uint32_t a[4] = {xv[0][2 * j], xv[1][2 * j], xv[0][2 * j + 1], xv[1][2 * j + 1]};
#pragma unroll
          for (int rb = 0; rb < R; ++rb) {
            uint32_t b0, b1;
            if constexpr (QK == kAff4) {
              const uint32_t w = wv[rb][j];
              b0 = w & nib;
              b1 = (w >> 4) & nib;
            } else if constexpr (QK == kAff8) {
              b0 = wv[rb][2 * j];
              b1 = wv[rb][2 * j + 1];
            } else {
              // E2M1 code -> 16 + 2*value by two 8-entry byte lookups: codes 0..7 find 16 + m in the
              // first table and (selector bit 3 set = "replicate the sign bit of a positive byte")
              // zero in the second; codes 8..15, with bit 3 flipped, the other way round.
              const uint32_t w = wv[rb][j], wn = w ^ 0x88888888u;
              b0 = prmt(0x13121110u, 0x1C181614u, w) | prmt(0x0D0E0F10u, 0x04080A0Cu, wn);
              b1 = prmt(0x13121110u, 0x1C181614u, w >> 16) | prmt(0x0D0E0F10u, 0x04080A0Cu, wn >> 16);
            }
            if (fresh && j == 0) imma(acc[rb], a, b0, b1, cinit);
            else imma(acc[rb], a, b0, b1, acc[rb]);
          }
        }
        fresh = false;
        if (h == 1 || fold_half) {
          // fold: accumulator rows g (c0, c1) and g + 8 (c2, c3) hold group slots sigma0 and
          // sigma0 + 1 of MMA columns 2t and 2t + 1, i.e. tile rows 8 rb + t and 8 rb + t + 4
#pragma unroll
          for (int rb = 0; rb < R; ++rb) {
            const float f0 = __int_as_float(acc[rb][0]) - kMagicValue, f1 = __int_as_float(acc[rb][1]) - kMagicValue;
            const float f2 = __int_as_float(acc[rb][2]) - kMagicValue, f3 = __int_as_float(acc[rb][3]) - kMagicValue;
            yacc[rb][0] = fmaf(f0, scale_lo(sraw[rb][0]), fmaf(f2, scale_hi(sraw[rb][0]), yacc[rb][0]));
            yacc[rb][1] = fmaf(f1, scale_lo(sraw[rb][1]), fmaf(f3, scale_hi(sraw[rb][1]), yacc[rb][1]));
          }
          fresh = true;
          if (h == 0) {              // eight groups per box: the second half has its own scales
#pragma unroll
            for (int rb = 0; rb < R; ++rb) {
              sraw[rb][0] = scale_pair(nrow[rb][0], gb0 + 4);
              sraw[rb][1] = scale_pair(nrow[rb][1], gb0 + 4);
            }
          }
        }
      }
      // the slot is free again: every read of it has been consumed by an MMA issued above
      __syncwarp();
      if (lane == 0 && itile < ntiles) issue_box();
    }

    // ---- this warp's share of K, for its lanes' digit planes and slots: scale, add up ----
    float v[2 * R];
#pragma unroll
    for (int rb = 0; rb < R; ++rb) {
      v[2 * rb] = yacc[rb][0] * pscale;
      v[2 * rb + 1] = yacc[rb][1] * pscale;
    }
    reduce_over_g<2 * R>(v, lane);
    {
      // value number `idx` of 2R: (row block, column parity) -> tile row 8 rb + t + 4 j
      constexpr int kBitsUsed = (2 * R >= 8) ? 3 : ((2 * R >= 4) ? 2 : 1);
      const int idx = (lane >> (5 - kBitsUsed)) & (2 * R - 1);
      const bool writer = kBitsUsed == 3 || (kBitsUsed == 2 && (lane & 4) == 0) || (kBitsUsed == 1 && (lane & 12) == 0);
      if (writer) red[(rbuf * kWarps + warp) * kTileRows + (idx >> 1) * 8 + t + 4 * (idx & 1)] = v[0];
    }
    __syncthreads();
    if (*abort_flag) {
      if (threadIdx.x == 0) atomicCAS(p.status, 0, *abort_flag);
      return;
    }
    // ---- rows x 8 threads: the warps' shares (fixed order) plus the bias term ----
    if (threadIdx.x < kTileRows * 8) {
      const int row = threadIdx.x >> 3, slice = threadIdx.x & 7;
      const int64_t n = n0 + row;
      const int64_t nn = n < p.N ? n : p.N - 1;
      float s = red[(rbuf * kWarps + slice) * kTileRows + row];
      if constexpr (QK != kMx4) {
        const bool bf = p.table_dtype == QMM_BF16;
        const uint8_t* brow = static_cast<const uint8_t*>(p.biases) + nn * p.groups * 2;
        if ((p.groups & 7) == 0 && (reinterpret_cast<uintptr_t>(p.biases) & 15) == 0) {
          for (int o = slice; o < p.groups / 8; o += 8) {
            const uint4 bv = __ldg(reinterpret_cast<const uint4*>(brow) + o);
            float bf8[8];
            if (bf) unpack8<__nv_bfloat16>(bv, bf8);
            else unpack8<__half>(bv, bf8);
            const float4 x0 = *reinterpret_cast<const float4*>(xsum + o * 8);
            const float4 x1 = *reinterpret_cast<const float4*>(xsum + o * 8 + 4);
            s = fmaf(bf8[0], x0.x, s); s = fmaf(bf8[1], x0.y, s); s = fmaf(bf8[2], x0.z, s); s = fmaf(bf8[3], x0.w, s);
            s = fmaf(bf8[4], x1.x, s); s = fmaf(bf8[5], x1.y, s); s = fmaf(bf8[6], x1.z, s); s = fmaf(bf8[7], x1.w, s);
          }
        } else {
          for (int gi = slice; gi < p.groups; gi += 8) {
            const uint32_t raw = ldg_u16(brow + gi * 2);
            const float bvf = bf ? __uint_as_float(raw << 16) : __half2float(__ushort_as_half(static_cast<unsigned short>(raw)));
            s = fmaf(bvf, xsum[gi], s);
          }
        }
      }
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      if (nonfinite) s = __uint_as_float(0x7fc00000u);
      if (slice == 0 && n < p.N) {
        if (p.y_dtype == QMM_BF16) static_cast<__nv_bfloat16*>(p.y)[n] = __float2bfloat16_rn(s);
        else if (p.y_dtype == QMM_F16) static_cast<__half*>(p.y)[n] = __float2half_rn(s);
        else static_cast<float*>(p.y)[n] = s;
      }
    }
    rbuf ^= 1;
  }
}

struct ImmaPlan {
  int r;            // row blocks per tile
  int ring;
  int grid;
  size_t smem;
};

size_t imma_smem(int r, int ring, int part_stride, int groups, bool mx) {
  const size_t xsum_words = mx ? 4 * static_cast<size_t>((groups + 7) & ~7) : static_cast<size_t>((groups + 7) & ~7);
  return 1024 + static_cast<size_t>(kWarps) * ring * r * 8 * kBoxBytes + 3 * static_cast<size_t>(part_stride) +
         xsum_words * 4 + static_cast<size_t>(2) * kWarps * 8 * r * 4 + static_cast<size_t>(kWarps) * kMaxRing * 8 +
         32 + kWarps * 4 + 16;
}

int env_int(const char* name, int fallback) {
  const char* e = getenv(name);
  return (e && *e) ? atoi(e) : fallback;
}

template <int QK, typename XT, int R>
int launch_r(const CUtensorMap& wm, const ImmaParams& ip, const ImmaPlan& plan, cudaStream_t stream) {
  auto kernel = qmm_gemv_imma_kernel<QK, XT, R>;
  static bool configured[kMaxDevices] = {};
  const int dev = current_device();
  if (dev < 0) return fail(QMM_ERR_DEVICE, "no current CUDA device");
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(plan.grid));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = plan.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, wm, ip);
  if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "qmm_gemv_imma_kernel launch: %s", cudaGetErrorString(e));
  count_launch();
  return check_launch("qmm_gemv_imma_kernel");
}

template <int QK, typename XT>
int launch_qx(const CUtensorMap& wm, const ImmaParams& ip, const ImmaPlan& plan, cudaStream_t stream) {
  if (plan.r == 4) return launch_r<QK, XT, 4>(wm, ip, plan, stream);
  if (plan.r == 2) return launch_r<QK, XT, 2>(wm, ip, plan, stream);
  return launch_r<QK, XT, 1>(wm, ip, plan, stream);
}

// Tile height, ring depth and grid for one problem, or r = 0 when the activations do not fit.
ImmaPlan make_plan(const qmm_problem& p, int nchunks, int part_stride, int groups, bool mx) {
  const int sms = device_sm_count();
  ImmaPlan best = {0, 0, 0, 0};
  const int force_r = env_int("QMM_IMMA_R", 0), force_ring = env_int("QMM_IMMA_RING", 0);
  double best_cost = 0;
  for (int r = 4; r >= 1; r >>= 1) {
    if (force_r && r != force_r) continue;
    const int64_t tiles = (p.N + 8 * r - 1) / (8 * r);
    // two CTAs per SM when they fit (the successor's CTAs can then become resident early)
    int ring = force_ring ? force_ring : (r == 4 ? 2 : (r == 2 ? 4 : 8));
    const int per_warp = (nchunks + kWarps - 1) / kWarps;
    size_t smem = imma_smem(r, ring, part_stride, groups, mx);
    while (!force_ring && ring > 1 && smem > 110 * 1024) smem = imma_smem(r, --ring, part_stride, groups, mx);
    if (smem > 220 * 1024) continue;
    const int ctas_per_sm = smem <= 110 * 1024 ? 2 : 1;
    int64_t grid = static_cast<int64_t>(sms) * ctas_per_sm;
    if (grid > tiles) grid = tiles;
    // cost: row blocks the busiest SM streams, plus a fixed charge per tile (reduce and bias)
    const int64_t tiles_per_cta = (tiles + grid - 1) / grid;
    const int64_t ctas_on_sm = (grid + sms - 1) / sms;
    const double cost = static_cast<double>(tiles_per_cta * ctas_on_sm) * (r * per_warp + 1.5);
    if (!best.r || cost < best_cost * 0.98) {
      best = {r, ring, static_cast<int>(grid), smem};
      best_cost = cost;
    }
  }
  return best;
}

}  // namespace

bool gemv_imma_supports(const qmm_problem& p) {
  static const bool enabled = env_int("QMM_GEMV_IMMA", 1) != 0;
  if (!enabled) return false;
  if (p.M != 1 || p.batch != 1 || p.lhs_idx || p.rhs_idx || p.group_sizes) return false;
  if (p.x_dtype != QMM_BF16 && p.x_dtype != QMM_F16) return false;
  const bool mx = p.mode == QMM_MODE_MXFP4;
  if (!mx && p.table_dtype != QMM_BF16 && p.table_dtype != QMM_F16) return false;   // float32 tables: the other kernel
  if (p.K % 32 || p.K < 32 || p.K > (1 << 20) || p.N < 1 || p.N >= (1LL << 31)) return false;
  const int bits = (!mx && p.bits == 8) ? 8 : 4;
  const int boxcodes = kBoxBytes * 8 / bits;
  const int nchunks = static_cast<int>((p.K + boxcodes - 1) / boxcodes);
  const int part_stride = ((nchunks * boxcodes + 127) & ~127) + 128;
  const int groups = static_cast<int>(p.K / (mx ? 32 : p.group_size));
  return imma_smem(1, 1, part_stride, groups, mx) <= 220 * 1024;
}

int launch_gemv_imma(const qmm_problem& p, cudaStream_t stream) {
  const bool mx = p.mode == QMM_MODE_MXFP4;
  const int bits = (!mx && p.bits == 8) ? 8 : 4;
  const int boxcodes = kBoxBytes * 8 / bits;
  ImmaParams ip;
  ip.x = p.x; ip.scales = p.scales; ip.biases = p.biases; ip.y = p.y;
  ip.status = device_status_word();
  if (!ip.status) return fail(QMM_ERR_CUDA, "could not allocate the device status word");
  ip.K = static_cast<int>(p.K); ip.N = static_cast<int>(p.N);
  ip.group_size = mx ? 32 : p.group_size;
  ip.groups = ip.K / ip.group_size;
  ip.table_dtype = p.table_dtype; ip.y_dtype = p.y_dtype;
  ip.nchunks = (ip.K + boxcodes - 1) / boxcodes;
  ip.part_stride = ((ip.nchunks * boxcodes + 127) & ~127) + 128;
  const ImmaPlan plan = make_plan(p, ip.nchunks, ip.part_stride, ip.groups, mx);
  if (!plan.r) return fail(QMM_ERR_UNSUPPORTED, "single-row decode kernel: the activations do not fit shared memory");
  ip.ring = plan.ring;
  ip.ntiles = static_cast<int>((p.N + 8 * plan.r - 1) / (8 * plan.r));

  // The packed weight as a 2-D byte tensor [N, K*bits/8]; a box that reaches past the last row
  // or past the end of a row is zero-filled by the TMA unit.
  const uint64_t row_bytes = static_cast<uint64_t>(p.K) * bits / 8;
  CUtensorMap wm;
  int rc = tensor_map_2d(&wm, QMM_U8, p.w, row_bytes, static_cast<uint64_t>(p.N), row_bytes, kBoxBytes, 8 * plan.r, 1);
  if (rc) return rc;
  const bool bf = p.x_dtype == QMM_BF16;
  if (mx) return bf ? launch_qx<kMx4, __nv_bfloat16>(wm, ip, plan, stream) : launch_qx<kMx4, __half>(wm, ip, plan, stream);
  if (bits == 8) return bf ? launch_qx<kAff8, __nv_bfloat16>(wm, ip, plan, stream) : launch_qx<kAff8, __half>(wm, ip, plan, stream);
  return bf ? launch_qx<kAff4, __nv_bfloat16>(wm, ip, plan, stream) : launch_qx<kAff4, __half>(wm, ip, plan, stream);
}

}  // namespace qmm
