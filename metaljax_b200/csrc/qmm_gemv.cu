// Decode kernel of the fused dequantize-and-matmul: up to 16 activation rows against a
// streamed packed weight (M <= 16 of `y = x . deq(w)^T`, src/metaljax/qmm.py:2491).
//
// HBM-bound: every packed weight byte is read exactly once and never dequantized element by
// element. A CTA owns 16 weight rows at a time and its 8 warps split K. The packed
// rows arrive by TMA in boxes of 16 rows x 128 bytes (128-byte swizzle, so that the fragment
// reads below are free of bank conflicts). Every warp has its own ring of boxes with one
// mbarrier per slot; its lane 0 requests the first boxes before anything else happens in the
// kernel and refills a slot as soon as the warp has consumed it, running ahead across tile
// boundaries.
//
// Per 32-wide K step a lane reads one packed word (two for 8-bit) of rows g and g+8 and turns
// it into the A fragments of two m16n8k16 MMAs with a magic-number OR: the 16-bit pattern
// 0x4300|q is the bf16 number 128+q (0x6400|q is the f16 number 1024+q), so the tensor core
// accumulates  sum (C + q_k) x_k  exactly in float32. All 16 K slots of such an MMA lie
// inside one 32-element span, hence inside one quantization group, so the group's scale and
// bias are applied to the accumulators once per group:
//     y += s * sum (C + q) x  +  (b - C s) * sum x .
// The activations are staged once in shared memory in the MMA's element type (for 4-bit
// codes in the pair order the magic-number extraction produces), tokens beyond M being zero
// fragments; each warp then takes  sum x  of its groups from MMAs whose A fragment is all
// ones and keeps them in shared memory for all the tiles it will process. The tile's
// (s, b - C s) pairs are staged next to them as float32, those of the next tile being
// requested while the current tile is computed.
// MXFP4 places each code's magnitude bits at the f16 exponent/mantissa boundary (the E2M1
// value times 2^-14, exactly) and scales the accumulators per 32-group by 2^(e8-127+14).
//
// CTAs are persistent (grid stride over 16-row tiles). The K split is reduced across the
// consumer warps in shared memory; there is no global scratch and no atomics, and the
// summation order is fixed. Every wait on an mbarrier is bounded.
//
// The kernel is launched with programmatic stream serialization: it lets the next kernel in
// the stream start early, and itself touches only the weights (which no earlier kernel of
// the stream produces) before `griddepcontrol.wait`; the activations are read and the
// output is written after it.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdio>
#include <cstdlib>
#include <type_traits>

#include "qmm_internal.h"
#include "qmm_ptx.cuh"

namespace qmm {
namespace {

using namespace ptx;

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kConsumerThreads = kThreads;
#ifndef QMM_GEMV_TRACING
#define QMM_GEMV_TRACING 0          // development builds: per-phase cycle counts (costs registers)
#endif
constexpr int kRowsPerCta = 16;
constexpr int kXPad = 32;           // elements of padding per staged activation row (64 bytes)
constexpr int kBoxBytes = 128;      // bytes of one weight row in a TMA box
constexpr int kBoxSmem = kRowsPerCta * kBoxBytes;   // 2 KiB
constexpr int kMaxRing = 4;         // boxes a warp keeps in flight
constexpr int kSmemBudget = 112 * 1024;      // two CTAs per SM
constexpr int kSmemBudgetOne = 220 * 1024;   // one CTA per SM

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
  int64_t num_weights, x_batches;   // gather: valid ranges of rhs_idx / lhs_idx (x_batches 0 = unknown)
  int group_size, table_dtype, y_dtype;
  int kc;          // K elements per pass: the tile's tables are staged pass by pass (a multiple
                   // of the box width)
  int xk;          // K elements of the activations held in shared memory: all of K (rounded up
                   // to boxes) when that fits, else kc
  int ring_shift;  // log2 of the boxes per warp ring (0..2)
  int xshift;      // log2 of the 8-element pieces per staged row, rounded up to a power of two
  int tiles;       // 16-row tiles per weight matrix
  int nchunks;     // staging passes over K: ceil(K / kc)
  int tiles_per_cta;   // most tiles any CTA walks: ceil(tiles / grid)
  int grid;        // CTAs per weight matrix
  long long* trace;   // development aid: cycles per phase of consumer warp 0 of every CTA, or NULL
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

// Walks one warp's boxes in the order they are consumed: pass by pass over K (a pass is what
// the CTA stages of the tables at a time), inside a pass tile by tile (grid stride), and
// inside a tile the warp's contiguous share of the pass's boxes. Done when chunk == nchunks.
struct BoxCursor {
  int chunk, tile, j, lo, hi;
};

// Positions the cursor on the first box of pass c.chunk (or of the next pass in which this
// warp has boxes) of tile `tile0`.
template <int BOXK>
__device__ __forceinline__ void cursor_seek(BoxCursor& c, int tile0, int nchunks, int warp, int K, int kc) {
  for (; c.chunk < nchunks; ++c.chunk) {
    const int left = K - c.chunk * kc;                    // 32-bit on purpose: no 64-bit division
    const int nb = ((left < kc ? left : kc) + BOXK - 1) / BOXK;
    c.lo = nb * warp / kWarps;
    c.hi = nb * (warp + 1) / kWarps;
    if (c.lo < c.hi) break;
  }
  c.tile = tile0;
  c.j = c.lo;
}

__device__ __forceinline__ void consumer_barrier() { __syncthreads(); }

// (a & b) | c as one LOP3 with all three operands in registers: left to itself the compiler
// may keep the two constants as immediates and spend two instructions.
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// Compile-time loop: f(integral_constant<int, 0>) ... f(integral_constant<int, N-1>).
template <int N, int I = 0, typename F>
__device__ __forceinline__ void static_for(F&& f) {
  if constexpr (I < N) {
    f(std::integral_constant<int, I>{});
    static_for<N, I + 1>(f);
  }
}

// QK: quantization kind. XT: activation type in memory. NT: token halves (1: M <= 8,
// 2: M <= 16). SPG: 32-wide K steps per quantization group (1, 2, 4).
template <int QK, typename XT, int NT, int SPG>
__global__ void __launch_bounds__(kThreads, 2)
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
  constexpr int kSumTok = 8 * NT;                  // tokens per row of the sum-of-x table

  extern __shared__ uint8_t gv_smem_raw[];
  const long long tr_entry = (QMM_GEMV_TRACING && p.trace) ? clock64() : 0;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gv_smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ring = 1 << p.ring_shift, rmask = ring - 1;
  const int nchunks = p.nchunks;
  const int xrow = p.xk + kXPad;                   // staged row stride in elements
  const bool xres = p.xk > p.kc || p.nchunks == 1;  // the activations of all of K are staged once
  const int tgroups = p.kc / kGroupK;              // groups staged per pass
  const int trow = tgroups + 1;                    // table row stride in entries (odd: no conflicts)
  const int tsize = (p.table_dtype == QMM_F32) ? 4 : 2;
  constexpr int tent = (QK == kMx4) ? 1 : 2;             // 32-bit words per table entry

  AT* xs = reinterpret_cast<AT*>(smem + kWarps * ring * kBoxSmem);
  float* sumx = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(xs) + static_cast<size_t>(p.M) * xrow * sizeof(AT));
  uint32_t* tbl = reinterpret_cast<uint32_t*>(sumx + (QK == kMx4 ? 0 : (p.xk / kGroupK) * kSumTok));
  float* red = reinterpret_cast<float*>(tbl + 2 * kRowsPerCta * trow * tent);   // two buffers
  float* accs = red + 2 * kWarps * NT * 4 * 32;     // per local tile, warp 0's partial sums between passes
  uint64_t* full_all = reinterpret_cast<uint64_t*>(accs + (nchunks > 1 ? p.tiles_per_cta * NT * 4 * 32 : 0));
  uint8_t* zeros = reinterpret_cast<uint8_t*>(full_all + kWarps * kMaxRing);      // 512 zero bytes: the
                                                                                  // "activations" of tokens >= M
  volatile int* abort_flag = reinterpret_cast<volatile int*>(zeros + 512);

  const int64_t seg = blockIdx.y;
  int64_t x_off, wb;
  if (p.lhs_idx) {
    // (this launch is serialized in the ordinary way, see launch_kernel: the indices are final)
    int64_t li = p.lhs_idx[seg], ri = p.rhs_idx[seg];
    if (ri < 0 || ri >= p.num_weights || li < 0 || (p.x_batches > 0 && li >= p.x_batches)) {
      if (threadIdx.x == 0) atomicCAS(p.status, 0, QMM_DEVICE_BAD_INDEX);
      if (ri < 0 || ri >= p.num_weights) ri = 0;
      if (li < 0 || (p.x_batches > 0 && li >= p.x_batches)) li = 0;
    }
    x_off = li * p.x_batch_stride;
    wb = ri;
  } else {
    x_off = seg * p.x_batch_stride;
    wb = p.w_batch_rows ? seg : 0;
  }
  const int boxes_per_chunk = p.kc / kBoxK;
  const int ntiles = p.tiles, tstride = gridDim.x;
  const int64_t groups = p.K / kGroupK;

  // Tables of one tile's 16 rows for one chunk: thread (r, c) of a 16 x 16 arrangement takes
  // the four consecutive groups 4c .. 4c+3 (+ 64 per batch) of row r. `load` requests them
  // (one 8-byte load per table when the tables are 16-bit and suitably aligned), `store`
  // converts and writes (scale, bias - C*scale) pairs; the two halves can be separated by
  // other work. Every load is unconditional: a group index past the end is clamped and its
  // entry is zeroed when stored, which makes that group's fold a no-op.
  const int tr = threadIdx.x >> 4, tc = threadIdx.x & 15;
  const bool tvec = QK != kMx4 && tsize == 2 && (groups & 3) == 0 &&
                    ((reinterpret_cast<uintptr_t>(p.scales) | reinterpret_cast<uintptr_t>(p.biases)) & 7) == 0;
  auto table_load = [&](int tile, int64_t kbase, int cgroups, int g0, uint32_t (&rs)[kTU], uint32_t (&rb)[kTU]) {
    const int64_t n0 = static_cast<int64_t>(tile) * kRowsPerCta;
    const int64_t row = wb * p.N + (n0 + tr < p.N ? n0 + tr : p.N - 1);
    const int64_t ti0 = row * groups + kbase / kGroupK;
    if constexpr (QK == kMx4) {
#pragma unroll
      for (int u = 0; u < kTU; ++u) {
        const int gi = g0 + u;
        rs[u] = __ldg(reinterpret_cast<const uint8_t*>(p.scales) + ti0 + (gi < cgroups ? gi : cgroups - 1));
        rb[u] = 0u;
      }
    } else if (tvec && ((kbase / kGroupK) & 3) == 0 && (cgroups & 3) == 0) {
      const int64_t i = ti0 + (g0 < cgroups ? g0 : 0);
      const uint2 vs = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(p.scales) + i));
      const uint2 vb = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(p.biases) + i));
      rs[0] = vs.x; rs[1] = vs.y; rb[0] = vb.x; rb[1] = vb.y;     // unpacked when stored: nothing here
      rs[2] = rs[3] = rb[2] = rb[3] = 0u;                         // may depend on the loaded values
    } else if (tsize == 2) {
#pragma unroll
      for (int u = 0; u < kTU; ++u) {
        const int gi = g0 + u;
        const int64_t i = ti0 + (gi < cgroups ? gi : cgroups - 1);
        rs[u] = table_raw(p.scales, false, i);
        rb[u] = table_raw(p.biases, false, i);
      }
    } else {
#pragma unroll
      for (int u = 0; u < kTU; ++u) {
        const int gi = g0 + u;
        const int64_t i = ti0 + (gi < cgroups ? gi : cgroups - 1);
        rs[u] = table_raw(p.scales, true, i);
        rb[u] = table_raw(p.biases, true, i);
      }
    }
  };
  // The first tile's tables are requested before anything else: their DRAM latency then runs
  // under the whole prologue.
  const int tg0 = tc * kTU;                                // this thread's first group of a batch
  uint32_t frs[kTU], frb[kTU];
  table_load(static_cast<int>(blockIdx.x), 0, static_cast<int>((p.K < p.kc ? p.K : p.kc) / kGroupK), tg0, frs, frb);


  // Each warp owns its barriers: it initializes them itself and nobody else touches them. The
  // block of zeros and the abort flag are first needed after the staging barrier further down.
  if (lane == 0) {
    if (warp == 0) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&w_map)) : "memory");
    for (int i = 0; i < kMaxRing; ++i) mbar_init(&full_all[warp * kMaxRing + i], 1);
    if (warp == 0) *abort_flag = 0;
    mbar_init_fence();
  }
  if (threadIdx.x < 128) reinterpret_cast<uint32_t*>(zeros)[threadIdx.x] = 0u;
  // The next kernel of the stream may start; whatever it reads of ours it reads after its own
  // griddepcontrol.wait, that is after this grid has completed.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __syncwarp();

  const bool tracing = QMM_GEMV_TRACING && p.trace != nullptr;
  long long tr_t[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const long long tr_c0 = tr_entry;

  const int g = lane >> 2, t = lane & 3;
  uint8_t* wring = smem + warp * ring * kBoxSmem;
  uint64_t* full = full_all + warp * kMaxRing;

  // ---- lane 0 requests this warp's first boxes before anything else ----
  BoxCursor issue = {0, 0, 0, 0, 0};
  int issued = 0;
  const int row_base = static_cast<int>(wb * p.N);
  auto issue_box = [&]() {   // lane 0 only; issue.chunk < nchunks
    const int slot = issued & rmask;
    mbar_expect_tx(&full[slot], kBoxSmem);
    tma_load_2d(&w_map, wring + slot * kBoxSmem, &full[slot], (issue.chunk * boxes_per_chunk + issue.j) * kBoxBytes,
                row_base + issue.tile * kRowsPerCta);
    ++issued;
    if (++issue.j >= issue.hi) {
      issue.j = issue.lo;
      issue.tile += tstride;
      if (issue.tile >= ntiles) {
        ++issue.chunk;
        cursor_seek<kBoxK>(issue, static_cast<int>(blockIdx.x), nchunks, warp, static_cast<int>(p.K), p.kc);
      }
    }
  };
  if (lane == 0) {
    cursor_seek<kBoxK>(issue, static_cast<int>(blockIdx.x), nchunks, warp, static_cast<int>(p.K), p.kc);
    while (issued < ring && issue.chunk < nchunks) issue_box();
  }
  const int64_t y_off = seg * p.y_batch_stride;
  const XT* xg = reinterpret_cast<const XT*>(p.x) + x_off;

  // The two constants of the magic-number extraction, pinned in registers (see and_or).
  uint32_t nib_mask = 0x000F000Fu, magic = Ops::kMagic;
  asm volatile("" : "+r"(nib_mask), "+r"(magic));

  // Per-thread shared addresses for the main loop.
  constexpr int kGroupsPerBox = kStepsPerBox / SPG;
  constexpr int kStepBytes = 4 * BITS;              // bytes of one row in a 32-wide K step
  const uint32_t wthread = smem_u32(wring) + g * kBoxBytes +
                           (QK == kAff8 ? ((((t >> 1) ^ (g & 7)) << 4) + (t & 1) * 8) : (((g & 7) << 4) + t * 4));
  const uint32_t zero_u32 = smem_u32(zeros);
  const uint32_t sumx_u32 = smem_u32(sumx);
  uint32_t xthread[NT];
  bool xvalid[NT];
#pragma unroll
  for (int h = 0; h < NT; ++h) {
    xvalid[h] = h * 8 + g < p.M;
    xthread[h] = smem_u32(xs) + ((h * 8 + g) * xrow + t * 8) * 2;
  }

  // Activations of one chunk. Items are (token, 8-element piece) with the pieces per token
  // padded to a power of two. When the MMA's element type is the activations' own, a piece is
  // only re-paired with byte permutes; otherwise it is converted through float32.
  auto stage_x = [&](int64_t kbase, int kc, int kfill) {
    constexpr int kXU = 8;      // pieces a thread has in flight: 4 leaves the staging of 16 rows four round trips
                                // long (a layer's linears at 16 rows: 114 -> 103 µs with 8; 16 spills)
    const int pieces = kfill >> 3;
    const int pmask = (1 << p.xshift) - 1;
    const int items = static_cast<int>(p.M) << p.xshift;
    for (int e0 = threadIdx.x; e0 < items; e0 += kConsumerThreads * kXU) {
      uint4 raw[kXU];
#pragma unroll
      for (int u = 0; u < kXU; ++u) {
        const int e = e0 + u * kConsumerThreads;
        const int mm = e >> p.xshift, pc = e & pmask;
        raw[u] = make_uint4(0u, 0u, 0u, 0u);
        if (e < items && pc * 8 < kc)
          raw[u] = __ldg(reinterpret_cast<const uint4*>(xg + static_cast<int64_t>(mm) * p.K + kbase + pc * 8));
      }
#pragma unroll
      for (int u = 0; u < kXU; ++u) {
        const int e = e0 + u * kConsumerThreads;
        const int mm = e >> p.xshift, pc = e & pmask;
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
        if (e < items && pc < pieces) *reinterpret_cast<uint4*>(xs + mm * xrow + pc * 8) = o;
      }
    }
  };

  auto table_store = [&](uint32_t* dst, int64_t kbase, int cgroups, int g0, uint32_t (&rs)[kTU], uint32_t (&rb)[kTU]) {
    if (QK != kMx4 && tvec && ((kbase / kGroupK) & 3) == 0 && (cgroups & 3) == 0) {   // as in table_load
      rs[3] = rs[1] >> 16; rs[2] = rs[1] & 0xffffu; rs[1] = rs[0] >> 16; rs[0] &= 0xffffu;
      rb[3] = rb[1] >> 16; rb[2] = rb[1] & 0xffffu; rb[1] = rb[0] >> 16; rb[0] &= 0xffffu;
    }
#pragma unroll
    for (int u = 0; u < kTU; ++u) {
      const int gi = g0 + u;
      if (gi < tgroups) {
        if constexpr (QK == kMx4) {
          dst[tr * trow + gi] = gi >= cgroups ? 0u : (rs[u] ? (rs[u] << 23) : 0x00400000u);   // 2^(e8 - 127)
        } else {
          const float sv = table_value(rs[u], p.table_dtype);
          const float bv = table_value(rb[u], p.table_dtype) - Ops::kMagicValue * sv;
          *reinterpret_cast<float2*>(dst + (tr * trow + gi) * 2) = gi >= cgroups ? make_float2(0.0f, 0.0f) : make_float2(sv, bv);
        }
      }
    }
  };

  // When the activations of all of K fit (xres), they and the sums of x are staged once, the
  // tables are staged pass by pass, and the tables of the next pass (of this tile or of the
  // CTA's next tile) are requested while the current pass is computed. Otherwise every pass
  // restages its slice of the activations, the sums and the tables.
  const int nbatch = (tgroups + 16 * kTU - 1) / (16 * kTU);
  int consumed = 0, tbuf = 0, rbuf = 0;
  bool ok = true, first = true;
  if (tracing) tr_t[1] = clock64() - tr_entry;        // prologue

  // sums of x over this warp's groups of one pass (A = all ones); every row of the result is
  // the same, the lanes of row 0 keep it. `xoff` is the pass's first K element in `xs`.
  auto sum_x = [&](int xoff, int jlo, int jhi) {
    if constexpr (QK != kMx4) {
      if (p.M <= 2) {
        // One or two tokens: plain float32 sums, four lanes per (token, group), instead of
        // MMAs that would be seven-eighths empty.
        constexpr int kPer = kGroupK / 4;                      // elements per lane: 8, 16 or 32
        const int ng = (jhi - jlo) * kGroupsPerBox;
        const int g_first = xoff / kGroupK + jlo * kGroupsPerBox;
        const int items = static_cast<int>(p.M) * ng;
        const int quad = lane >> 2, ql = lane & 3;
        for (int it0 = 0; it0 < items; it0 += 8) {
          const int item = it0 + quad;
          const int m = item >= ng ? 1 : 0;
          const int gi = g_first + (item - m * ng);
          float acc = 0.0f;
          if (item < items) {
            const AT* src = xs + m * xrow + gi * kGroupK + ql * kPer;
#pragma unroll
            for (int c = 0; c < kPer / 8; ++c) {
              const uint4 v = *reinterpret_cast<const uint4*>(src + c * 8);
              const uint32_t u4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                if constexpr (std::is_same<AT, __nv_bfloat16>::value) {
                  acc += __uint_as_float(u4[i] << 16) + __uint_as_float(u4[i] & 0xffff0000u);
                } else {
                  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u4[i]));
                  acc += f.x + f.y;
                }
              }
            }
          }
          acc += __shfl_xor_sync(0xffffffffu, acc, 1);
          acc += __shfl_xor_sync(0xffffffffu, acc, 2);
          if (item < items && ql == 0) sumx[gi * kSumTok + m] = acc;
        }
        return;
      }
      const uint32_t one4[4] = {Ops::kOnes, Ops::kOnes, Ops::kOnes, Ops::kOnes};
      for (int j = jlo; j < jhi; ++j) {
#pragma unroll
        for (int q = 0; q < kGroupsPerBox; ++q) {
          const int gi = xoff / kGroupK + j * kGroupsPerBox + q;     // zero-padded x past K: those sums are 0
#pragma unroll
          for (int h = 0; h < NT; ++h) {
            float o0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, o1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int s = 0; s < SPG; ++s) {
              uint4 xv = make_uint4(0u, 0u, 0u, 0u);
              if (h * 8 + g < p.M) xv = *reinterpret_cast<const uint4*>(xs + (h * 8 + g) * xrow + (gi * SPG + s) * 32 + t * 8);
              Ops::mma(o0, one4, xv.x, xv.y, o0);
              Ops::mma(o1, one4, xv.z, xv.w, o1);
            }
            if (g == 0)
              *reinterpret_cast<float2*>(sumx + gi * kSumTok + h * 8 + 2 * t) = make_float2(o0[0] + o1[0], o0[1] + o1[1]);
          }
        }
      }
    }
  };
  auto pass_extent = [&](int chunk, int& kc, int& nb) {
    const int left = static_cast<int>(p.K) - chunk * p.kc;
    kc = left < p.kc ? left : p.kc;                   // multiple of 32
    nb = (kc + kBoxK - 1) / kBoxK;
  };

  for (int chunk = 0; chunk < nchunks; ++chunk) {
    const int64_t kbase = static_cast<int64_t>(chunk) * p.kc;
    int kc, nb;
    pass_extent(chunk, kc, nb);
    const int cgroups = kc / kGroupK;
    const int jlo = nb * warp / kWarps, jhi = nb * (warp + 1) / kWarps;
    const int xoff = xres ? static_cast<int>(kbase) : 0;        // this pass's first K element in xs
    if (first) {
      // ---- the CTA's first unit: its tables were requested at kernel entry ----
      const long long ts0 = tracing ? clock64() : 0;
      asm volatile("griddepcontrol.wait;" ::: "memory");
      if (xres) stage_x(0, static_cast<int>(p.K), p.xk);
      else stage_x(kbase, kc, nb * kBoxK);
      table_store(tbl, kbase, cgroups, tg0, frs, frb);       // requested at kernel entry
      for (int g0 = tg0 + 16 * kTU; g0 < tgroups; g0 += 16 * kTU) {
        table_load(static_cast<int>(blockIdx.x), kbase, cgroups, g0, frs, frb);
        table_store(tbl, kbase, cgroups, g0, frs, frb);
      }
      consumer_barrier();                                    // activations and tables are staged
      if (tracing) tr_t[3] += clock64() - ts0;
      const long long tp0 = tracing ? clock64() : 0;
      if (xres) {                                            // every pass's sums, once
        for (int c = 0; c < nchunks; ++c) {
          int ckc, cnb;
          pass_extent(c, ckc, cnb);
          sum_x(c * p.kc, cnb * warp / kWarps, cnb * (warp + 1) / kWarps);
        }
      } else {
        sum_x(0, jlo, jhi);
      }
      __syncwarp();                                          // a warp reads only its own sums
      first = false;
      if (tracing) tr_t[6] += clock64() - tp0;
    } else if (!xres) {
      // ---- a later pass of activations that do not fit: restage this pass's slice. Everyone
      // is past the previous unit's barrier, so nobody reads the old slice any more; the
      // pass's first tables were requested during the previous unit. ----
      stage_x(kbase, kc, nb * kBoxK);
      consumer_barrier();
      sum_x(0, jlo, jhi);
      __syncwarp();
    }

    int tl = 0;                                             // index of the tile among this CTA's tiles
    for (int tile = blockIdx.x; tile < ntiles; tile += tstride, ++tl) {
      const int64_t n0 = static_cast<int64_t>(tile) * kRowsPerCta;
      float yacc[NT][4];
#pragma unroll
      for (int h = 0; h < NT; ++h)
#pragma unroll
        for (int i = 0; i < 4; ++i) yacc[h][i] = 0.0f;
      const uint32_t* tcur = tbl + tbuf * kRowsPerCta * trow * tent;
      uint32_t* tnext = tbl + (tbuf ^ 1) * kRowsPerCta * trow * tent;
      // the unit after this one: the pass's next tile, or the first tile of the next pass
      const bool last_tile = tile + tstride >= ntiles;
      const int ptile = last_tile ? static_cast<int>(blockIdx.x) : tile + tstride;
      const int pchunk = last_tile ? chunk + 1 : chunk;
      int pkc, pnb;
      pass_extent(pchunk, pkc, pnb);
      const int64_t pkbase = static_cast<int64_t>(pchunk) * p.kc;
      const int pgroups = pkc / kGroupK;
      uint32_t prs[kTU], prb[kTU];
      int pb = pchunk < nchunks ? 0 : nbatch + 1;
      auto prefetch_step = [&]() {
        if (pb > 0) table_store(tnext, pkbase, pgroups, tg0 + 16 * kTU * (pb - 1), prs, prb);
        if (pb < nbatch) table_load(ptile, pkbase, pgroups, tg0 + 16 * kTU * pb, prs, prb);
        ++pb;
      };

      // ---- this warp's boxes of the chunk ----
      // All shared-memory reads of the loop below go through 32-bit shared addresses that
      // are fixed per thread, plus compile-time offsets.
      const uint32_t tcur_u32 = smem_u32(tcur);
      for (int j = jlo; j < jhi && ok; ++j, ++consumed) {
        const long long tq0 = tracing ? clock64() : 0;
        if (pb < nbatch) prefetch_step();                 // the last store waits for the tile's end
        const long long tq1 = tracing ? clock64() : 0;
        const int slot = consumed & rmask;
        if (!(ok = mbar_wait(&full[slot], (consumed >> p.ring_shift) & 1, abort_flag, 11))) break;
        const long long tq2 = tracing ? clock64() : 0;
        if (tracing) { tr_t[7] += tq1 - tq0; tr_t[0] += tq2 - tq1; }
        // Row g of the box, with the swizzle term of K step 0 folded in: K step ks of the box
        // is at this address XOR ks * kStepBytes (the box is 2 KiB aligned, so bits 4..6 of the
        // address are exactly the swizzle term); row g + 8 is 1 KiB further.
        const uint32_t wrow = wthread + slot * kBoxSmem;
        uint32_t xbox[NT];
#pragma unroll
        for (int h = 0; h < NT; ++h) xbox[h] = xvalid[h] ? xthread[h] + (xoff + j * kBoxK) * 2 : zero_u32;
        const uint32_t tb0 = tcur_u32 + (g * trow + j * kGroupsPerBox) * 4 * tent;
        const uint32_t tb1 = tb0 + 8 * trow * 4 * tent;
        const uint32_t sxb = sumx_u32 + ((xoff / kGroupK + j * kGroupsPerBox) * kSumTok + 2 * t) * 4;
        static_for<kGroupsPerBox>([&](auto qc) {               // groups of this box
          constexpr int q = decltype(qc)::value;
          float acc[NT][4];
          static_for<SPG>([&](auto sc) {
            constexpr int s = decltype(sc)::value;
            constexpr int ks = q * SPG + s;                       // K step within the box
            const uint32_t waddr = wrow ^ (ks * kStepBytes);
            uint32_t a[2][4];
            if constexpr (QK == kAff8) {
              // 32 bytes per row and step: lane t takes bytes [8t, 8t+8) of them
              const uint2 u0 = lds64<0>(waddr);
              const uint2 u1 = lds64<8 * kBoxBytes>(waddr);
              a[0][0] = __byte_perm(u0.x, 0x64646464u, 0x4140); a[0][1] = __byte_perm(u1.x, 0x64646464u, 0x4140);
              a[0][2] = __byte_perm(u0.x, 0x64646464u, 0x4342); a[0][3] = __byte_perm(u1.x, 0x64646464u, 0x4342);
              a[1][0] = __byte_perm(u0.y, 0x64646464u, 0x4140); a[1][1] = __byte_perm(u1.y, 0x64646464u, 0x4140);
              a[1][2] = __byte_perm(u0.y, 0x64646464u, 0x4342); a[1][3] = __byte_perm(u1.y, 0x64646464u, 0x4342);
            } else {
              // 16 bytes per row and step: lane t takes word t
              const uint32_t u0 = lds32<0>(waddr);
              const uint32_t u1 = lds32<8 * kBoxBytes>(waddr);
              if constexpr (QK == kAff4) {
                a[0][0] = and_or(u0, nib_mask, magic);       a[0][1] = and_or(u1, nib_mask, magic);
                a[0][2] = and_or(u0 >> 4, nib_mask, magic);  a[0][3] = and_or(u1 >> 4, nib_mask, magic);
                a[1][0] = and_or(u0 >> 8, nib_mask, magic);  a[1][1] = and_or(u1 >> 8, nib_mask, magic);
                a[1][2] = and_or(u0 >> 12, nib_mask, magic); a[1][3] = and_or(u1 >> 12, nib_mask, magic);
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
#pragma unroll
            for (int h = 0; h < NT; ++h) {
              const uint4 xv = lds128<ks * 64>(xbox[h]);
              if (s == 0) Ops::mma(acc[h], a[0], xv.x, xv.y, zero4);
              else Ops::mma(acc[h], a[0], xv.x, xv.y, acc[h]);
              Ops::mma(acc[h], a[1], xv.z, xv.w, acc[h]);
            }
          });
          // fold the group: rows g (c0, c1) and g+8 (c2, c3), tokens 2t and 2t+1
          if constexpr (QK == kMx4) {
            const float s0 = __uint_as_float(lds32<q * 4>(tb0)), s1 = __uint_as_float(lds32<q * 4>(tb1));
#pragma unroll
            for (int h = 0; h < NT; ++h) {
              yacc[h][0] = fmaf(s0, acc[h][0] * 16384.0f, yacc[h][0]);
              yacc[h][1] = fmaf(s0, acc[h][1] * 16384.0f, yacc[h][1]);
              yacc[h][2] = fmaf(s1, acc[h][2] * 16384.0f, yacc[h][2]);
              yacc[h][3] = fmaf(s1, acc[h][3] * 16384.0f, yacc[h][3]);
            }
          } else {
            const uint2 v0 = lds64<q * 8>(tb0), v1 = lds64<q * 8>(tb1);      // (scale, bias - C*scale)
            const float s0 = __uint_as_float(v0.x), b0 = __uint_as_float(v0.y);
            const float s1 = __uint_as_float(v1.x), b1 = __uint_as_float(v1.y);
            static_for<NT>([&](auto hc) {
              constexpr int h = decltype(hc)::value;
              const uint2 sxr = lds64<(q * kSumTok + h * 8) * 4>(sxb);
              const float sx0 = __uint_as_float(sxr.x), sx1 = __uint_as_float(sxr.y);
              yacc[h][0] = fmaf(s0, acc[h][0], fmaf(b0, sx0, yacc[h][0]));
              yacc[h][1] = fmaf(s0, acc[h][1], fmaf(b0, sx1, yacc[h][1]));
              yacc[h][2] = fmaf(s1, acc[h][2], fmaf(b1, sx0, yacc[h][2]));
              yacc[h][3] = fmaf(s1, acc[h][3], fmaf(b1, sx1, yacc[h][3]));
            });
          }
        });
        // the slot is free again: refill it with the next box this warp will need
        __syncwarp();
        // (Every read of the slot has been consumed by an MMA issued before the __syncwarp, so the
        // refill needs no further ordering.)
        if (lane == 0 && issue.chunk < nchunks) issue_box();
        if (tracing) tr_t[4] += clock64() - tq2;
      }
      const long long tq3 = tracing ? clock64() : 0;
      while (pb <= nbatch) prefetch_step();
      if (tracing) tr_t[7] += clock64() - tq3;
      tbuf ^= 1;

      // ---- reduce the K split across warps (fixed order); the pass's partial sums of the
      // tile wait in shared memory for the next pass, the last pass stores the tile ----
      float* rcur = red + rbuf * kWarps * NT * 4 * 32;
#pragma unroll
      for (int h = 0; h < NT; ++h)
#pragma unroll
        for (int i = 0; i < 4; ++i) rcur[(warp * NT * 4 + h * 4 + i) * 32 + lane] = yacc[h][i];
      const long long tb0 = tracing ? clock64() : 0;
      consumer_barrier();                        // also: the next unit's tables are complete
      if (tracing) tr_t[2] += clock64() - tb0;
      if (*abort_flag) {
        if (threadIdx.x == 0) atomicCAS(p.status, 0, *abort_flag);
        return;
      }
      if (warp == 0) {
        float* acc = accs + tl * NT * 4 * 32;
#pragma unroll
        for (int h = 0; h < NT; ++h)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float v = chunk > 0 ? acc[(h * 4 + i) * 32 + lane] : 0.0f;
#pragma unroll
            for (int wv = 0; wv < kWarps; ++wv) v += rcur[(wv * NT * 4 + h * 4 + i) * 32 + lane];
            if (chunk + 1 < nchunks) {
              acc[(h * 4 + i) * 32 + lane] = v;
            } else {
              const int64_t row = n0 + g + (i >> 1) * 8;
              const int64_t tok = h * 8 + 2 * t + (i & 1);
              if (row < p.N && tok < p.M) gv_store(p.y, p.y_dtype, y_off + tok * p.N + row, v);
            }
          }
      }
      rbuf ^= 1;
    }
  }
  if (tracing && threadIdx.x == 32 * 3) {     // warp 3 speaks for the CTA
    for (int i = 0; i < 8; ++i) p.trace[blockIdx.x * 8 + i] = tr_t[i];
    p.trace[blockIdx.x * 8 + 5] = clock64() - tr_c0;
  }
}

// Shared memory one CTA needs: rings, activations of `xk` K elements, their group sums, two
// table buffers of `kc` K elements, two reduce buffers, barriers, the block of zeros.
size_t smem_bytes(const GemvParams& gp, int nt, int group_k, bool mx, int ring) {
  const size_t tgroups = gp.kc / group_k;
  const size_t tent = mx ? 1 : 2;
  return 1024 + static_cast<size_t>(kWarps) * ring * kBoxSmem +
         static_cast<size_t>(gp.M) * (gp.xk + kXPad) * 2 +
         (mx ? 0 : static_cast<size_t>(gp.xk / group_k) * 8 * nt * sizeof(float)) +
         static_cast<size_t>(2) * kRowsPerCta * (tgroups + 1) * tent * sizeof(uint32_t) +
         static_cast<size_t>(2) * kWarps * nt * 4 * 32 * sizeof(float) +
         (gp.nchunks > 1 ? static_cast<size_t>(gp.tiles_per_cta) * nt * 4 * 32 * sizeof(float) : 0) +
         static_cast<size_t>(kWarps) * kMaxRing * sizeof(uint64_t) + 512 + 16;
}

bool use_pdl() {
  static const bool on = [] {
    const char* e = getenv("QMM_GEMV_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

template <int QK, typename XT, int NT, int SPG>
int launch_kernel(const CUtensorMap& wm, const GemvParams& gp, cudaStream_t stream) {
  const size_t smem = smem_bytes(gp, NT, 32 * SPG, QK == kMx4, 1 << gp.ring_shift);
  // Persistent CTAs share the machine's segments; a CTA walks tiles with a grid stride.
  const int64_t per_seg = gp.grid;
  auto kernel = qmm_gemv_kernel<QK, XT, NT, SPG>;
  static bool configured[kMaxDevices] = {};     // the attribute is per device
  const int dev = current_device();
  if (dev < 0) return QMM_ERR_DEVICE;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudgetOne);
    if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(per_seg), static_cast<unsigned>(gp.batch));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // A gather reads its index arrays before `griddepcontrol.wait` (they decide which weight the
  // first boxes come from), and those are usually the previous kernel's output: such a launch
  // is serialized in the ordinary way.
  cfg.numAttrs = (use_pdl() && !gp.lhs_idx) ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, wm, gp);
  if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "qmm_gemv_kernel launch: %s", cudaGetErrorString(e));
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
  if (route_override() != QMM_ROUTE_GEMV_FMMA && gemv_imma_supports(p)) return launch_gemv_imma(p, stream);
  GemvParams gp;
  gp.x = p.x; gp.scales = p.scales; gp.biases = p.biases; gp.y = p.y;
  gp.lhs_idx = p.lhs_idx; gp.rhs_idx = p.rhs_idx;
  gp.status = device_status_word();
  if (!gp.status) return fail(QMM_ERR_CUDA, "could not allocate the device status word");
  gp.M = p.M; gp.K = p.K; gp.N = p.N; gp.batch = p.batch;
  gp.x_batch_stride = p.x_batch_stride; gp.y_batch_stride = p.y_batch_stride;
  gp.w_batch_rows = p.rhs_idx ? p.N : p.w_batch_stride;
  gp.num_weights = p.num_weights > 0 ? p.num_weights : 1;
  gp.x_batches = p.x_batches;
  gp.group_size = p.group_size; gp.table_dtype = p.table_dtype; gp.y_dtype = p.y_dtype;
  gp.tiles = static_cast<int>((p.N + kRowsPerCta - 1) / kRowsPerCta);
  const bool mx = p.mode == QMM_MODE_MXFP4;
  const int bits = (!mx && p.bits == 8) ? 8 : 4;
  const int boxk = kBoxBytes * 8 / bits;
  const int group_k = mx ? 32 : p.group_size;
  const int nt = p.M <= 8 ? 1 : 2;
  // Tables are staged in passes of 64 or 128 groups (one or two batches of table loads).
  // Preference order: (1) the activations of all of K stay in shared memory, two CTAs per SM,
  // ring of 4, then 2, then 1 box per warp, passes of 128 then of 64 groups; (2) the activations are restaged pass by pass, a pass
  // being a multiple of 8 boxes (one per warp), two CTAs per SM; (3) the same with one CTA
  // per SM and its larger shared memory; (4) whatever pass fits.
  const int kround = static_cast<int>((p.K + boxk - 1) / boxk * boxk);
  const int pass_k = 64 * group_k / boxk * boxk;           // group_k >= 32: at least 2048
  const int sms = device_sm_count();
  auto configure = [&](int xk, int kc, int ring_shift, int ctas_per_sm) -> size_t {
    gp.xk = xk; gp.kc = kc; gp.ring_shift = ring_shift;
    gp.nchunks = static_cast<int>((p.K + kc - 1) / kc);
    int64_t grid = (static_cast<int64_t>(ctas_per_sm) * sms + gp.batch - 1) / gp.batch;
    if (grid < 1) grid = 1;
    if (grid > gp.tiles) grid = gp.tiles;
    gp.grid = static_cast<int>(grid);
    gp.tiles_per_cta = static_cast<int>((gp.tiles + grid - 1) / grid);
    return smem_bytes(gp, nt, group_k, mx, 1 << ring_shift);
  };
  bool done = false;
  // (down to a single box per warp: at 8 rows and K = 4096 that keeps the activations resident at
  // two CTAs per SM -- one pass over K instead of two restaged ones, 1301 -> ~940 instructions per
  // warp-tile -- and sixteen warps per SM still cover the box round trip; QMM_GEMV_RING_MIN=1
  // restores the two-box floor)
  static const int ring_min = [] { const char* e = getenv("QMM_GEMV_RING_MIN"); return e ? atoi(e) : 0; }();
  for (int ring_shift = 2; !done && ring_shift >= ring_min; --ring_shift)
    for (int mult = 2; !done && mult >= 1; --mult) {       // passes of 128, then of 64 groups
      const int want = mult * pass_k;
      done = configure(kround, kround < want ? kround : want, ring_shift, 2) <= kSmemBudget;
    }
  const int kc_res = kround < pass_k ? kround : pass_k;
  for (int ctas = 2; !done && ctas >= 1; --ctas) {
    const size_t budget = ctas == 2 ? kSmemBudget : kSmemBudgetOne;
    for (int kc = kc_res / (8 * boxk) * (8 * boxk); !done && kc >= 8 * boxk; kc -= 8 * boxk)
      done = configure(kc, kc, 2, ctas) <= budget || configure(kc, kc, 1, ctas) <= budget ||
             (ring_min == 0 && nt == 1 && configure(kc, kc, 0, ctas) <= budget);     // (up to 8 rows: fewer, longer passes win)
  }
  for (int kc = kc_res; !done && kc >= boxk; kc -= boxk) done = configure(kc, kc, 1, 1) <= kSmemBudgetOne;
  if (!done) return fail(QMM_ERR_UNSUPPORTED, "decode kernel: no staging plan fits shared memory");
#if QMM_GEMV_TRACING
  static long long* trace_buf = nullptr;
  static const bool trace_on = getenv("QMM_GEMV_TRACE") != nullptr;
  if (trace_on && !trace_buf) cudaMalloc(&trace_buf, sizeof(long long) * 8 * 1024);
  if (trace_on) cudaMemsetAsync(trace_buf, 0, sizeof(long long) * 8 * 1024, stream);
  gp.trace = trace_on ? trace_buf : nullptr;
#else
  gp.trace = nullptr;
#endif
  int pieces = gp.xk / 8, xs = 5;
  while ((1 << xs) < pieces) ++xs;
  gp.xshift = xs;

  // The packed weight as a 2-D byte tensor [rows, K*bits/8] over every weight matrix behind
  // `w`; a box that reaches past the last row is zero-filled by the TMA unit.
  const uint64_t row_bytes = static_cast<uint64_t>(p.K) * bits / 8;
  const uint64_t nw = p.num_weights > 0 ? p.num_weights : (p.w_batch_stride ? p.batch : 1);
  const uint64_t rows = static_cast<uint64_t>(p.N) * nw;
  CUtensorMap wm;
  int rc = tensor_map_2d(&wm, QMM_U8, p.w, row_bytes, rows, row_bytes, kBoxBytes, kRowsPerCta, 1);
  if (rc) return rc;
  if (p.mode == QMM_MODE_MXFP4) rc = launch_xt<kMx4>(wm, gp, p.x_dtype, stream);
  else if (p.bits == 8) rc = launch_xt<kAff8>(wm, gp, p.x_dtype, stream);
  else rc = launch_xt<kAff4>(wm, gp, p.x_dtype, stream);
#if QMM_GEMV_TRACING
  if (trace_on && rc == 0) {   // development aid: average cycles per phase over the CTAs
    cudaStreamSynchronize(stream);
    static long long host[8 * 1024];
    int64_t grid = gp.grid > 1024 ? 1024 : gp.grid;
    cudaMemcpy(host, trace_buf, sizeof(long long) * 8 * grid, cudaMemcpyDeviceToHost);
    double avg[8] = {0};
    for (int64_t c = 0; c < grid; ++c)
      for (int i = 0; i < 8; ++i) avg[i] += static_cast<double>(host[c * 8 + i]) / grid;
    fprintf(stderr,
            "qmm_gemv cycles/CTA (warp 3): full-wait %.0f | prologue %.0f | reduce barrier %.0f | staging %.0f | "
            "compute %.0f | sum-x %.0f | total %.0f | table prefetch %.0f | tiles/CTA %.2f\n",
            avg[0], avg[1], avg[2], avg[3], avg[4], avg[6], avg[5], avg[7], static_cast<double>(gp.tiles) / grid);
  }
#endif
  return rc;
}

}  // namespace qmm
