// Prefill kernel of the fused dequantize-and-matmul on the 5th-generation tensor cores.
//
//   y[t, f] = sum_k x[t, k] * deq(w)[f, k]          (transpose=True of the reference's call,
//                                                    src/metaljax/qmm.py:2491)
//
// The WEIGHT is the MMA's A operand and lives in tensor memory: a tile is 128 output
// features (= 128 TMEM lanes) x 64 K-elements, so one dequantizing thread owns one weight
// row, reads its 32 packed bytes (64 for 8-bit) from shared memory, applies its own
// per-group scale and bias in registers, and writes the bf16/f16 result straight to TMEM
// with tcgen05.st -- the dequantized weight never exists in shared or global memory. The
// ACTIVATIONS are the B operand: TMA brings [BT tokens x 64 K] tiles into shared memory in
// the 128-byte-swizzled K-major layout tcgen05.mma reads. The accumulator D[feature, token]
// (float32) sits in TMEM; the epilogue reads it back with tcgen05.ld, casts and stores
// y[token, feature].
//
// Warp roles (18 warps): 0 = TMA producer, 1 = MMA issuer (+ TMEM allocation),
// 2..17 = sixteen dequant/epilogue warps in four teams of four (one warp per TMEM lane
// quarter); the teams take K blocks round-robin.
//
// One persistent CTA per SM walks a list of tiles (segment, token tile, feature tile).
// A segment is a run of x rows that meets one weight matrix: the whole of x for the plain
// op, one batch of a batched weight, or one expert's rows of a ragged (grouped) product,
// in which case the per-expert row offsets are prefix sums of `group_sizes` computed here.
//
// Every wait is bounded: when a barrier does not flip within ~2 s of SM clock the kernel
// records the place in a status word, stops issuing work and drains.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdio>
#include <cstdlib>
#include <type_traits>

#include "qmm_internal.h"

namespace qmm {
namespace {

constexpr int kBF = 128;        // features per tile (MMA M, TMEM lanes)
constexpr int kBK = 64;         // K elements per pipeline stage
// Dequant / epilogue teams of four warps (one per TMEM lane quarter): five for wide token tiles,
// where the dequantization is what the issuer waits for (C2a 965 -> 1009 TFLOP/s, C2b 1106 -> 1199,
// int8 891 -> 991 against four); four for narrow tiles (five lose there: fewer ring slots fit)
// and for float weights (whose 16 KB slots leave room for four).
template <int QK, int BT>
struct Teams {
#ifndef QMM_TC_WIDE_TEAMS
#define QMM_TC_WIDE_TEAMS 5
#endif
  static constexpr int kTeams = (BT <= 64 || QK == 3 /* kFloat */) ? 4 : QMM_TC_WIDE_TEAMS;
  static constexpr int kThreads = (2 + 4 * kTeams) * 32;
};
constexpr int kMaxSegments = 256;
constexpr long long kSpinLimit = 4000000000LL;  // SM clocks (~2 s)
#ifndef QMM_TC_TRACING
#define QMM_TC_TRACING 0        // development builds: cycles per wait site (-DQMM_TC_TRACING=1)
#endif

enum { kAff4 = 0, kAff8 = 1, kMx4 = 2, kFloat = 3 };    // kFloat: the weight holds values of the activation type (nothing to dequantize)

struct TcParams {
  const void* scales;
  const void* biases;
  void* y;
  const int32_t* group_sizes;  // ragged: [segments]; else NULL
  int* status;                 // device status word (0 = ok)
  long long* trace;            // development aid: per-CTA cycles spent in each wait site, or NULL
  int64_t M;                   // rows of x per segment (dense) or total rows (ragged)
  int64_t K, N;
  int64_t segments;            // weight matrices
  int64_t w_seg_rows;          // rows of the packed weight between segments (N, or 0 = shared)
  int group_size, table_dtype, y_dtype;
  int splits;                  // > 1: the K blocks of a tile are divided among `splits` CTAs, each
  float* partial;              // of which writes its float32 partial tile to partial[split][M][N]
  int64_t item0, item_end;     // the work items [item0, item_end) of the persistent walk are this launch's
  int64_t tail_tile0;          // >= 0: this launch splits only the tiles from here on, and partial is
  int64_t tail_tiles;          //       compact: partial[split][tile - tail_tile0][BT][128]
};

// ---- PTX wrappers ---------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait. Returns false (and records `where`) when the barrier never flips or another
// role has already given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int where) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  int spins = 0;
  while (!mbar_try(bar, parity)) {
    if ((++spins & 1023) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kSpinLimit) {
        *abort_flag = where;
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void tma_load_2d(const CUtensorMap* map, void* dst, uint64_t* bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// D[tmem_d] (+)= A[tmem_a] * B[desc_b]; A from tensor memory, B from shared memory.
__device__ __forceinline__ void tc_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0;"
      "  tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p; }" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

#define QMM_R32(a, o) a[o + 0], a[o + 1], a[o + 2], a[o + 3], a[o + 4], a[o + 5], a[o + 6], a[o + 7]
#define QMM_ASM_R(o) "r"(r[o]), "r"(r[o + 1]), "r"(r[o + 2]), "r"(r[o + 3]), "r"(r[o + 4]), "r"(r[o + 5]), "r"(r[o + 6]), "r"(r[o + 7])
#define QMM_ASM_W(o) "=r"(r[o]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3]), "=r"(r[o + 4]), "=r"(r[o + 5]), "=r"(r[o + 6]), "=r"(r[o + 7])

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp owns lane (base + i).
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      QMM_ASM_R(0), QMM_ASM_R(8), QMM_ASM_R(16), QMM_ASM_R(24)
      : "memory");
}

// 32 lanes x 8 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
               QMM_ASM_R(0)
               : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : QMM_ASM_W(0), QMM_ASM_W(8), QMM_ASM_W(16), QMM_ASM_W(24)
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- dequantization of one weight row's K block into 32 packed 16-bit pairs ---------------

template <typename XT>
struct Half2Ops;

template <>
struct Half2Ops<__nv_bfloat16> {
  static constexpr uint32_t kMagic = 0x43004300u;  // (128, 128): 7 mantissa bits hold the code
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ uint32_t sub(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  static __device__ __forceinline__ uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {
    __nv_bfloat162 r = __hfma2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b),
                               *reinterpret_cast<__nv_bfloat162*>(&c));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
};

template <>
struct Half2Ops<__half> {
  static constexpr uint32_t kMagic = 0x64006400u;  // (1024, 1024)
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ uint32_t sub(uint32_t a, uint32_t b) {
    __half2 r = __hsub2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  static __device__ __forceinline__ uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {
    __half2 r = __hfma2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b),
                        *reinterpret_cast<__half2*>(&c));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b) {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
};

// 4-bit affine, NW packed words -> NW*4 pairs. A byte holds elements (2i, 2i+1): PRMT takes
// it from the word (even element in its low nibble) into byte 0 and from the word shifted
// right by four (odd element) into byte 2, one LOP3 keeps the two nibbles under the magic
// exponent (128 + q, or 1024 + q for f16, both exact), an exact subtraction removes the
// magic, and one FMA with (s, s), (b, b) rounds once.
template <typename XT, int NW>
__device__ __forceinline__ void dequant_aff4(const uint32_t (&w)[NW], float s, float b, uint32_t* out) {
  using H = Half2Ops<XT>;
  const uint32_t s2 = H::pack(s, s);
  const uint32_t b2 = H::pack(b, b);
#pragma unroll
  for (int j = 0; j < NW; ++j) {
    const uint32_t hi = w[j] >> 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t t = __byte_perm(w[j], hi, i | ((4 + i) << 8));
      const uint32_t v = (t & 0x000F000Fu) | H::kMagic;
      out[j * 4 + i] = H::fma(H::sub(v, H::kMagic), s2, b2);
    }
  }
}

// 8-bit affine, NW packed words -> NW*2 pairs: float32 FMA per element, rounded to the
// 16-bit type in pairs.
// The same for float32 tables (what the packer emits when a bias is not exactly
// representable in the narrow type): the magic pair is widened to float32, one float32 FMA
// per element with (s, b - C s), one rounding to the pair type.
template <typename XT, int NW>
__device__ __forceinline__ void dequant_aff4_wide(const uint32_t (&w)[NW], float s, float b, uint32_t* out) {
  using H = Half2Ops<XT>;
  const float c = std::is_same<XT, __nv_bfloat16>::value ? 128.0f : 1024.0f;
  const float bc = fmaf(-c, s, b);
#pragma unroll
  for (int j = 0; j < NW; ++j) {
    const uint32_t hi = w[j] >> 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t t = __byte_perm(w[j], hi, i | ((4 + i) << 8));
      const uint32_t v = (t & 0x000F000Fu) | H::kMagic;
      float lo, up;
      if constexpr (std::is_same<XT, __nv_bfloat16>::value) {
        lo = __uint_as_float(v << 16);
        up = __uint_as_float(v & 0xffff0000u);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v));
        lo = f.x; up = f.y;
      }
      out[j * 4 + i] = H::pack(fmaf(s, lo, bc), fmaf(s, up, bc));
    }
  }
}

template <typename XT, int NW>
__device__ __forceinline__ void dequant_aff8(const uint32_t (&w)[NW], float s, float b, uint32_t* out) {
  using H = Half2Ops<XT>;
#pragma unroll
  for (int j = 0; j < NW; ++j) {
    float q[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      q[e] = __uint_as_float(__byte_perm(w[j], 0x4B000000u, 0x7540u + e)) - 8388608.0f;
    out[j * 2] = H::pack(fmaf(s, q[0], b), fmaf(s, q[1], b));
    out[j * 2 + 1] = H::pack(fmaf(s, q[2], b), fmaf(s, q[3], b));
  }
}

// MXFP4, NW packed words of one 32-element group -> NW*4 pairs. The three magnitude bits of a
// code, placed at the 16-bit type's exponent/mantissa boundary, are the E2M1 value scaled by
// 2^-126 (bf16) or 2^-14 (f16), including the subnormal code 1 = 0.5; two exact power-of-two
// multiplies undo that and apply the group's E8M0 scale.
template <typename XT, int NW>
__device__ __forceinline__ void dequant_mx4(const uint32_t (&w)[NW], uint32_t e8, uint32_t* out) {
  using H = Half2Ops<XT>;
  constexpr bool kBf = std::is_same<XT, __nv_bfloat16>::value;
  constexpr int kShift = kBf ? 6 : 9;  // magnitude bit 0 -> top mantissa bit
  const float unbias = kBf ? 8.507059173023462e37f /* 2^126 */ : 16384.0f /* 2^14 */;
  const uint32_t u2 = H::pack(unbias, unbias);
  const float sc = __uint_as_float(e8 ? (e8 << 23) : 0x00400000u);
  const uint32_t s2 = H::pack(sc, sc);
#pragma unroll
  for (int j = 0; j < NW; ++j) {
    const uint32_t hi = w[j] >> 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // byte 0 <- byte i of w (even element in its low nibble), byte 2 <- byte i of w>>4
      const uint32_t t = __byte_perm(w[j], hi, i | ((4 + i) << 8)) & 0x000F000Fu;
      const uint32_t bits = ((t & 0x00070007u) << kShift) | ((t & 0x00080008u) << 12);
      out[j * 4 + i] = H::mul(H::mul(bits, u2), s2);
    }
  }
}

// ---- UMMA descriptors ------------------------------------------------------------------

// K-major operand in the 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);        // start address
  d |= static_cast<uint64_t>(1) << 16;                        // leading byte offset (unused)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                        // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                        // SWIZZLE_128B
  return d;
}

// kind::f16, float32 accumulate, both operands K-major.
__host__ __device__ constexpr uint32_t instr_desc(int fmt /*0 f16, 1 bf16*/, int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(fmt) << 7) | (static_cast<uint32_t>(fmt) << 10) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// ---- shared-memory plan -----------------------------------------------------------------

template <int QK, int BT>
struct Plan {
  static constexpr int kTeams = Teams<QK, BT>::kTeams;
  static constexpr int kThreads = Teams<QK, BT>::kThreads;
  static constexpr int kBits = (QK == kFloat) ? 16 : ((QK == kAff8) ? 8 : 4);
  static constexpr int kWRowBytes = kBK * kBits / 8;          // 32, 64 or (float weights) 128
  static constexpr int kXBytes = BT * kBK * 2;                // one activation stage
  static constexpr int kWBytes = kBF * kWRowBytes;            // one packed-weight stage
  static constexpr int kStageBytes = kXBytes + kWBytes;
  // as many stages as fit next to the barriers and the tile tables (the dequantized-A ring in
  // tensor memory has one 32-column slot per stage)
  static constexpr int kFit = (232448 - 4200 - 2048) / kStageBytes;
  // The depth is a multiple of the number of dequant teams, so that a ring slot is always
  // handled by the same team: a waiter then never lags its barrier by two phases, which a
  // parity wait could not tell from "ready".
  // Narrow token tiles leave most of tensor memory to the A ring and stage little: twelve
  // slots instead of eight cover the per-slot latency chain (TMA, one team's dequantization,
  // MMA, commit) that bounds a CTA's rate at a few dozen rows.
  static constexpr int kACol0 = (BT <= 64) ? 64 : (BT <= 128 ? 128 : 256);   // A ring starts here (D is columns [0, BT))
  static constexpr int kTmemFit = (512 - kACol0) / 32;
  static constexpr int kMost = kFit < kTmemFit ? kFit : kTmemFit;
  // (at most three rounds of the teams: twelve slots for four teams, five for five at 256 tokens)
  static constexpr int kStages = (kMost / kTeams >= 3 ? 3 : (kMost / kTeams >= 2 ? 2 : 1)) * kTeams;
  static_assert(kMost >= kTeams, "one slot per team must fit");
  static constexpr int kBarBytes = 1024;
  static constexpr int kSmem = kStages * kStageBytes + kBarBytes + 1024 /* alignment slack */;
  static constexpr int kDCols = BT;                           // accumulator columns
  static constexpr int kTmemCols = 512;
};

struct TileInfo {
  int split, kb_lo, kb_hi;   // this work item's share of the tile's K blocks
  int seg;
  int64_t tile;      // index in the walk
  int64_t row0;      // first x / y row of this tile
  int rows;          // valid rows in the tile (<= BT)
  int64_t f0;        // first feature
};

// Tile t of the persistent walk -> (segment, token tile, feature tile); feature tiles vary
// fastest inside a token tile so that concurrently running CTAs share the activation tile
// and stream disjoint weight rows.
template <int BT>
__device__ __forceinline__ bool tile_at(int64_t item, const int64_t* seg_tile0, const int64_t* seg_row0,
                                        int nseg, int64_t ftiles, int64_t N, int splits, int num_kb,
                                        TileInfo* out) {
  // work item -> (tile, split): the splits of a tile are adjacent items, so they run together
  int64_t t = item;
  out->split = 0;
  if (splits > 1) {                                   // (the common case divides nothing)
    t = item / splits;
    out->split = static_cast<int>(item - t * splits);
  }
  if (t >= seg_tile0[nseg]) return false;
  out->tile = t;
  out->kb_lo = static_cast<int>(static_cast<int64_t>(out->split) * num_kb / splits);
  out->kb_hi = static_cast<int>(static_cast<int64_t>(out->split + 1) * num_kb / splits);
  int s = 0;
  while (t >= seg_tile0[s + 1]) ++s;
  const int64_t local = t - seg_tile0[s];
  const int64_t tt = local / ftiles, ft = local % ftiles;
  const int64_t rows = seg_row0[s + 1] - seg_row0[s];
  out->seg = s;
  out->row0 = seg_row0[s] + tt * BT;
  const int64_t left = rows - tt * BT;
  out->rows = static_cast<int>(left < BT ? left : BT);
  out->f0 = ft * kBF;
  (void)N;
  return true;
}

// SPLIT: the K blocks of a tile are shared among p.splits CTAs (float32 partial tiles). A
// separate instantiation, so that the unsplit kernel keeps compile-time K bounds.
template <int QK, typename XT, int BT, bool SPLIT>
__global__ void __launch_bounds__((Teams<QK, BT>::kThreads), 1)
qmm_gemm_tc_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map,
                   const TcParams p) {
  using P = Plan<QK, BT>;
  constexpr int kTeams = P::kTeams;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* bar_base = smem + P::kStages * P::kStageBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(bar_base);      // [kStages] TMA landed
  uint64_t* empty = full + P::kStages;                         // [kStages] stage consumed
  uint64_t* a_full = empty + P::kStages;                       // [kStages] dequantized A is in TMEM
  uint64_t* d_full = a_full + P::kStages;                      // accumulator complete
  uint64_t* d_empty = d_full + 1;                              // accumulator drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  __shared__ int64_t seg_tile0[kMaxSegments + 1];
  __shared__ int64_t seg_row0[kMaxSegments + 1];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nseg = static_cast<int>(p.segments);
  const int64_t ftiles = (p.N + kBF - 1) / kBF;
  const int num_kb = static_cast<int>((p.K + kBK - 1) / kBK);

  // Programmatic dependent launch: the grid that follows may be scheduled as soon as every CTA
  // of this one has got here (it touches memory only after its own griddepcontrol.wait). This
  // grid sets itself up, and requests its first weight boxes, while the grid it depends on is
  // still running; what that grid produces -- the activations, the group sizes of a ragged
  // product -- is read only after thread 0's griddepcontrol.wait, and everything this grid
  // writes is downstream of those reads.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    if (p.group_sizes) asm volatile("griddepcontrol.wait;" ::: "memory");
    int64_t tiles = 0, rows = 0;
    for (int s = 0; s < nseg; ++s) {
      seg_tile0[s] = tiles;
      seg_row0[s] = rows;
      int64_t r = p.group_sizes ? p.group_sizes[s] : p.M;
      if (p.group_sizes && rows + r > p.M) r = p.M - rows;
      if (r < 0) r = 0;
      rows += r;
      tiles += ((r + BT - 1) / BT) * ftiles;
    }
    seg_tile0[nseg] = tiles;
    seg_row0[nseg] = rows;
    for (int i = 0; i < P::kStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1 + 4);
    }
    for (int i = 0; i < P::kStages; ++i) mbar_init(&a_full[i], 4);
    mbar_init(d_full, 1);
    mbar_init(d_empty, 4 * kTeams);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(P::kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Waits go through here so that a development build can account the cycles per wait site.
  long long waited[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const bool tracing = QMM_TC_TRACING && p.trace != nullptr;
  long long trace_c0 = 0, trace_n0 = 0;
  if (tracing && threadIdx.x == 0) {
    trace_c0 = clock64();
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(trace_n0));
  }
  auto twait = [&](uint64_t* bar, uint32_t parity, volatile int* flag, int where) -> bool {
    if (!tracing) return mbar_wait(bar, parity, flag, where);
    const long long t0 = clock64();
    const bool r = mbar_wait(bar, parity, flag, where);
    waited[where] += clock64() - t0;
    return r;
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0, early = 0;
      TileInfo ti;
      bool ok = true;
      // The weight boxes of the first tile's first ring (the stages start out free) go out before
      // the wait for the preceding grid; their activation boxes follow it.
      const int64_t first = p.item0 + blockIdx.x;
      if (first < p.item_end && tile_at<BT>(first, seg_tile0, seg_row0, nseg, ftiles, p.N, SPLIT ? p.splits : 1, num_kb, &ti)) {
        const int64_t wrow = ti.seg * p.w_seg_rows + ti.f0;
        for (int kb = ti.kb_lo; kb < ti.kb_hi && early < static_cast<uint32_t>(P::kStages); ++kb, ++early) {
          mbar_expect_tx(&full[early], P::kStageBytes);
          tma_load_2d(&w_map, smem + early * P::kStageBytes + P::kXBytes, &full[early], kb * P::kWRowBytes, static_cast<int>(wrow));
        }
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int64_t t = first; ok && t < p.item_end && tile_at<BT>(t, seg_tile0, seg_row0, nseg, ftiles, p.N, SPLIT ? p.splits : 1, num_kb, &ti);
           t += gridDim.x) {
        const int64_t wrow = ti.seg * p.w_seg_rows + ti.f0;
        for (int kb = ti.kb_lo; kb < ti.kb_hi; ++kb, ++it) {
          const int s = it % P::kStages;
          uint8_t* stage = smem + s * P::kStageBytes;
          if (it < early) {              // armed above, its weight box is on the way
            tma_load_2d(&x_map, stage, &full[s], kb * kBK, static_cast<int>(ti.row0));
            continue;
          }
          const uint32_t ph = (it / P::kStages) & 1;
          if (!(ok = twait(&empty[s], ph ^ 1, abort_flag, 1))) break;
          mbar_expect_tx(&full[s], P::kStageBytes);
          tma_load_2d(&x_map, stage, &full[s], kb * kBK, static_cast<int>(ti.row0));
          tma_load_2d(&w_map, stage + P::kXBytes, &full[s], kb * P::kWRowBytes, static_cast<int>(wrow));
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // The whole warp walks the loop so that stage indices, descriptors and TMEM addresses
    // are warp-uniform values; one lane issues the tensor-core instructions.
    constexpr uint32_t idesc = instr_desc(std::is_same<XT, __nv_bfloat16>::value ? 1 : 0, kBF, BT);
    uint32_t tile_n = 0, ph = 0;
    int s = 0;
    TileInfo ti;
    bool ok = true;
    for (int64_t t = p.item0 + blockIdx.x; ok && t < p.item_end && tile_at<BT>(t, seg_tile0, seg_row0, nseg, ftiles, p.N, SPLIT ? p.splits : 1, num_kb, &ti);
         t += gridDim.x, ++tile_n) {
      if (!(ok = twait(d_empty, (tile_n & 1) ^ 1, abort_flag, 2))) break;
      tc_fence_after();
      for (int kb = ti.kb_lo; kb < ti.kb_hi; ++kb) {
        // The dequantized A of this K block sits in TMEM slot s, the slot of its shared-
        // memory stage. Its writers waited for the stage's TMA barrier themselves, so
        // their barrier also says that the activation tile has landed.
        if (!(ok = twait(&a_full[s], ph, abort_flag, 4))) break;
        const long long tf0 = tracing ? clock64() : 0;
        tc_fence_after();
        const long long ti0 = tracing ? clock64() : 0;
        if (tracing) waited[3] += ti0 - tf0;         // cycles in the fence
        const uint64_t bdesc = smem_desc_sw128(smem_u32(smem + s * P::kStageBytes));
        const uint32_t acol = tmem_base + P::kACol0 + s * 32;
        if (lane == 0) {
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k)
            tc_mma_ts(tmem_base, acol + k * 8, bdesc + static_cast<uint64_t>(k * 2), idesc,
                      (kb > ti.kb_lo || k) ? 1u : 0u);
          tc_commit(&empty[s]);     // frees the stage and its TMEM slot together
        }
        if (tracing) waited[0] += clock64() - ti0;   // cycles spent issuing
        if (++s == P::kStages) { s = 0; ph ^= 1u; }
      }
      if (ok && lane == 0) tc_commit(d_full);
    }
  } else {
    // ---------------- dequant + epilogue warps ----------------
    const int team = (warp - 2) >> 2;            // takes K blocks with it % kTeams == team
    const int quarter = warp & 3;                // TMEM lane quarter this warp may touch
    const int frow = quarter * 32 + lane;        // feature row within the tile
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int64_t groups = p.K / p.group_size;
    uint32_t it = 0, tile_n = 0;
    TileInfo ti;
    bool ok = true;
    for (int64_t t = p.item0 + blockIdx.x; ok && t < p.item_end && tile_at<BT>(t, seg_tile0, seg_row0, nseg, ftiles, p.N, SPLIT ? p.splits : 1, num_kb, &ti);
         t += gridDim.x, ++tile_n) {
      int64_t feat = ti.f0 + frow;
      const bool feat_ok = feat < p.N;
      if (!feat_ok) feat = p.N - 1;
      const int64_t trow = (ti.seg * p.w_seg_rows + feat) * groups;   // row of the scale tables
      // The teams take the tile's K blocks round-robin (block kb belongs to the team whose
      // number is the block's global iteration index modulo kTeams). The per-group constants
      // of a block are requested one of the team's blocks ahead, so their global-memory
      // latency hides behind the previous block's work.
      const int tsize = (p.table_dtype == QMM_F32) ? 4 : 2;
      const bool twide = p.table_dtype == QMM_F32;
      auto fetch_tables = [&](int kbb, float (&fs)[2], float (&fb)[2], uint32_t (&fe)[2]) {
        int64_t gidx[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          int64_t g = (kbb * kBK + h * 32) / p.group_size;
          gidx[h] = trow + (g >= groups ? groups - 1 : g);
          fs[h] = fb[h] = 0.0f;
          fe[h] = 0u;
        }
        if constexpr (QK == kMx4) {
#pragma unroll
          for (int h = 0; h < 2; ++h) fe[h] = __ldg(reinterpret_cast<const uint8_t*>(p.scales) + gidx[h]);
        } else if (twide) {          // raw bits until used; the width is decided outside the loads
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            fs[h] = __uint_as_float(table_raw(p.scales, true, gidx[h]));
            fb[h] = __uint_as_float(table_raw(p.biases, true, gidx[h]));
          }
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            fs[h] = __uint_as_float(table_raw(p.scales, false, gidx[h]));
            fb[h] = __uint_as_float(table_raw(p.biases, false, gidx[h]));
          }
        }
      };
      constexpr int kHalfWords = P::kWRowBytes / 8;                // packed words per 32 elements
      const uint32_t it0 = it;
      int kb = ti.kb_lo + static_cast<int>((static_cast<uint32_t>(team) + kTeams - (it0 % kTeams)) % kTeams);
      const int kb_end = ti.kb_hi;
      float sc[2], bi[2];
      uint32_t e8[2];
      if constexpr (QK == kFloat) { sc[0] = sc[1] = bi[0] = bi[1] = 0.0f; e8[0] = e8[1] = 0u; }
      if (QK != kFloat && kb < kb_end) fetch_tables(kb, sc, bi, e8);
      for (; kb < kb_end; kb += kTeams) {
        it = it0 + static_cast<uint32_t>(kb - ti.kb_lo);
        const int s = it % P::kStages;
        float nsc[2] = {0.0f, 0.0f}, nbi[2] = {0.0f, 0.0f};
        uint32_t ne8[2] = {0u, 0u};
        if (QK != kFloat && kb + kTeams < kb_end) fetch_tables(kb + kTeams, nsc, nbi, ne8);
        if (!(ok = twait(&full[s], (it / P::kStages) & 1, abort_flag, 5))) break;
        const uint8_t* wsm = smem + s * P::kStageBytes + P::kXBytes + frow * P::kWRowBytes;
        uint32_t packed[2][kHalfWords];
#pragma unroll
        for (int i = 0; i < P::kWRowBytes / 16; ++i) {
          // float weights are 128-byte rows in the TMA unit's 128-byte swizzle (chunk i of row r
          // sits at chunk i ^ (r & 7)): the lanes of a quarter-warp then read distinct banks
          const int ci = (QK == kFloat) ? (i ^ (frow & 7)) : i;
          const uint4 v = *reinterpret_cast<const uint4*>(wsm + ci * 16);
          const uint32_t q4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) packed[(i * 4 + e) / kHalfWords][(i * 4 + e) % kHalfWords] = q4[e];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);     // this warp's share of the stage is in registers
        uint32_t out[32];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if constexpr (QK == kFloat) {
#pragma unroll
            for (int j = 0; j < 16; ++j) out[h * 16 + j] = packed[h][j];
          } else if constexpr (QK == kAff4) {
            if (twide)
              dequant_aff4_wide<XT, kHalfWords>(packed[h], sc[h], bi[h], &out[h * 16]);
            else
              dequant_aff4<XT, kHalfWords>(packed[h], table_value(__float_as_uint(sc[h]), p.table_dtype),
                                           table_value(__float_as_uint(bi[h]), p.table_dtype), &out[h * 16]);
          } else if constexpr (QK == kAff8) {
            dequant_aff8<XT, kHalfWords>(packed[h], table_value(__float_as_uint(sc[h]), p.table_dtype),
                                         table_value(__float_as_uint(bi[h]), p.table_dtype), &out[h * 16]);
          } else {
            dequant_mx4<XT, kHalfWords>(packed[h], e8[h], &out[h * 16]);
          }
        }
        // TMEM slot s is free: the TMA for this stage was only issued after the MMAs that
        // read the slot's previous contents had completed (the producer waited for them).
        tc_fence_after();
        const long long ts0 = tracing ? clock64() : 0;
        tmem_st32(tmem_base + lane_addr + P::kACol0 + s * 32, out);
        tmem_wait_st();
        if (tracing) waited[0] += clock64() - ts0;   // cycles in tcgen05.st + wait
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&a_full[s]);
#pragma unroll
        for (int h = 0; h < 2; ++h) { sc[h] = nsc[h]; bi[h] = nbi[h]; e8[h] = ne8[h]; }
      }
      it = it0 + static_cast<uint32_t>(kb_end - ti.kb_lo);
      if (!ok) break;
      // ---- epilogue: the teams drain disjoint 32-column chunks of the accumulator ----
      if (!(ok = twait(d_full, tile_n & 1, abort_flag, 7))) break;
      __syncwarp();      // lanes leave the wait loop one by one; tcgen05.ld needs the whole warp
      tc_fence_after();
#pragma unroll 1
      for (int c0 = team * 32; c0 < BT; c0 += 32 * kTeams) {
        if (c0 >= ti.rows) break;                  // warp-uniform: no valid token rows left
        uint32_t r[32];
        tmem_ld32(tmem_base + lane_addr + c0, r);
        tmem_wait_ld();
        if (SPLIT && p.tail_tile0 >= 0) {          // the last partial wave only: compact partial tiles
          float* part = p.partial + ((static_cast<int64_t>(ti.split) * p.tail_tiles + (ti.tile - p.tail_tile0)) * BT + c0) * kBF + frow;
#pragma unroll
          for (int j = 0; j < 32; ++j) part[j * kBF] = __uint_as_float(r[j]);
        } else if (SPLIT && feat_ok) {             // a share of the tile's K: float32 partial sums
          float* part = p.partial + static_cast<int64_t>(ti.split) * p.M * p.N;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c0 + j < ti.rows) part[(ti.row0 + c0 + j) * p.N + feat] = __uint_as_float(r[j]);
        } else if (feat_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (c0 + j < ti.rows) {
              const int64_t o = (ti.row0 + c0 + j) * p.N + feat;
              const float v = __uint_as_float(r[j]);
              if (p.y_dtype == QMM_BF16) reinterpret_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16_rn(v);
              else if (p.y_dtype == QMM_F16) reinterpret_cast<__half*>(p.y)[o] = __float2half_rn(v);
              else reinterpret_cast<float*>(p.y)[o] = v;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(d_empty);
    }
    // ragged: rows past the last group are zero
    if (p.group_sizes) {
      const int64_t used = seg_row0[nseg];
      const int64_t total = (p.M - used) * p.N;
      const int64_t nth = 128 * kTeams;
      const int64_t tid = static_cast<int64_t>(blockIdx.x) * nth + (threadIdx.x - 64);
      for (int64_t i = tid; i < total; i += static_cast<int64_t>(gridDim.x) * nth) {
        const int64_t o = used * p.N + i;
        if (p.y_dtype == QMM_F32) reinterpret_cast<float*>(p.y)[o] = 0.0f;
        else reinterpret_cast<uint16_t*>(p.y)[o] = 0;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(P::kTmemCols)
                 : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag) atomicCAS(p.status, 0, *abort_flag);
  if (tracing && threadIdx.x == 0) {
    long long n1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(n1));
    p.trace[blockIdx.x * 16 + 14] = clock64() - trace_c0;
    p.trace[blockIdx.x * 16 + 15] = n1 - trace_n0;
  }
  if (tracing && lane == 0 && (warp == 0 || warp == 1 || warp == 2 || warp == 6))
    for (int i = 0; i < 8; ++i)
      if (waited[i]) p.trace[blockIdx.x * 16 + (warp == 1 ? 8 : 0) + i] = waited[i];
}

// ---- host side ---------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

int make_map(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t outer,
             uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(QMM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(QMM_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return QMM_OK;
}

int* status_word() {
  return device_status_word();
}

int sm_count() { return device_sm_count(); }

// Launches with programmatic stream serialization (QMM_TC_PDL=0: plain stream order): the
// kernels of this file wait for the grid before them themselves, as late as they can.
bool tc_pdl() {
  static const bool on = [] {
    const char* e = getenv("QMM_TC_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

template <typename... Params, typename... Args>
void launch_dependent(void (*kernel)(Params...), unsigned grid, unsigned threads, size_t smem, cudaStream_t stream,
                      Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = tc_pdl() ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);      // a failure stays as the last error: check_launch reports it
}

// Sums the float32 partial tiles of a split product in split order and casts to y's type.
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, void* __restrict__ y, int y_dtype,
                                     int64_t total, int splits) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");               // the partial tiles come from the grid before
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x * 4;
  for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < total; i += stride) {
    float4 acc = *reinterpret_cast<const float4*>(partial + i);
    for (int s = 1; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(partial + static_cast<int64_t>(s) * total + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (y_dtype == QMM_BF16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(y) + i) =
          make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    } else if (y_dtype == QMM_F16) {
      __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
      *reinterpret_cast<uint2*>(static_cast<__half*>(y) + i) =
          make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    } else {
      *reinterpret_cast<float4*>(static_cast<float*>(y) + i) = acc;
    }
  }
}

// The same for a split last wave: partial[split][tile][BT][128] -> the tiles' places in y
// (one dense segment; tile t of the walk is token tile t / ftiles, feature tile t % ftiles).
__global__ void splitk_tail_reduce_kernel(const float* __restrict__ partial, void* __restrict__ y, int y_dtype,
                                          int64_t M, int64_t N, int64_t ftiles, int64_t tile0, int64_t tiles,
                                          int bt, int splits) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t per_tile = static_cast<int64_t>(bt) * kBF, total = tiles * per_tile;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t tl = i / per_tile, in = i - tl * per_tile;
    const int64_t r = in / kBF, c = in - r * kBF;
    const int64_t t = tile0 + tl;
    const int64_t row = (t / ftiles) * bt + r, col = (t % ftiles) * kBF + c;
    if (row >= M || col >= N) continue;
    float acc = partial[i];
    for (int s = 1; s < splits; ++s) acc += partial[static_cast<int64_t>(s) * total + i];
    const int64_t o = row * N + col;
    if (y_dtype == QMM_BF16) static_cast<__nv_bfloat16*>(y)[o] = __float2bfloat16_rn(acc);
    else if (y_dtype == QMM_F16) static_cast<__half*>(y)[o] = __float2half_rn(acc);
    else static_cast<float*>(y)[o] = acc;
  }
}

// How many CTAs share one tile's K blocks. A short row run against a narrow weight leaves most
// SMs without a tile while each busy CTA walks all of K alone; dividing K among CTAs fills the
// machine. Only for one dense segment, N a multiple of 4 (the reduce kernel's vectors), and
// never fewer than 8 K blocks per share.
bool tail_split_enabled() {
  static const bool on = [] { const char* e = getenv("QMM_TC_TAIL_SPLIT"); return !(e && *e == '0'); }();
  return on;
}

int choose_splits(const qmm_problem& p, int64_t tiles, int num_kb) {
  if (p.group_sizes || p.batch != 1 || (p.N & 3)) return 1;
  int64_t s = sm_count() / (tiles < 1 ? 1 : tiles);
  if (s > num_kb / 8) s = num_kb / 8;
  if (s > 8) s = 8;
  return s < 2 ? 1 : static_cast<int>(s);
}

template <int QK, typename XT, int BT>
int launch_cfg(const qmm_problem& p, cudaStream_t stream) {
  using P = Plan<QK, BT>;
  const bool ragged = p.group_sizes != nullptr;
  const int64_t x_rows = ragged ? p.M : p.batch * p.M;
  const int64_t w_rows = (p.w_batch_stride ? p.batch : 1) * p.N;
  CUtensorMap xm, wm;
  int rc;
  const CUtensorMapDataType xdt =
      std::is_same<XT, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  if ((rc = make_map(&xm, xdt, p.x, static_cast<uint64_t>(p.K), static_cast<uint64_t>(x_rows),
                     static_cast<uint64_t>(p.K) * 2, kBK, BT, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  const uint64_t wrow_bytes = static_cast<uint64_t>(p.K) * P::kBits / 8;
  if ((rc = make_map(&wm, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.w, wrow_bytes, static_cast<uint64_t>(w_rows),
                     wrow_bytes, P::kWRowBytes, kBF, QK == kFloat ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE)))
    return rc;
  TcParams tp;
  tp.scales = p.scales; tp.biases = p.biases; tp.y = p.y; tp.group_sizes = p.group_sizes;
  tp.status = scratch_override() ? scratch_override()->status : status_word();
#if QMM_TC_TRACING
  static long long* trace_buf = nullptr;
  static const bool trace_on = getenv("QMM_TC_TRACE") != nullptr;
  if (trace_on && !trace_buf) {
    cudaMalloc(&trace_buf, sizeof(long long) * 16 * 1024);
  }
  if (trace_on) cudaMemsetAsync(trace_buf, 0, sizeof(long long) * 16 * 1024, stream);
  tp.trace = trace_on ? trace_buf : nullptr;
#else
  tp.trace = nullptr;
#endif
  if (!tp.status) return fail(QMM_ERR_CUDA, "could not allocate the device status word");
  tp.M = p.M; tp.K = p.K; tp.N = p.N;
  tp.segments = p.batch;
  tp.w_seg_rows = p.w_batch_stride ? p.N : 0;
  tp.group_size = p.group_size; tp.table_dtype = p.table_dtype; tp.y_dtype = p.y_dtype;
  tp.splits = 1;
  tp.partial = nullptr;
  tp.item0 = 0;
  tp.item_end = INT64_MAX;
  tp.tail_tile0 = -1;
  tp.tail_tiles = 0;

  static bool configured[kMaxDevices] = {};     // the attribute is per device
  const int dev = current_device();
  if (dev < 0) return QMM_ERR_DEVICE;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(qmm_gemm_tc_kernel<QK, XT, BT, false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, P::kSmem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(qmm_gemm_tc_kernel<QK, XT, BT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               P::kSmem);
    if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured[dev] = true;
  }
  const int64_t ftiles = (p.N + kBF - 1) / kBF;
  int64_t max_tiles = ragged ? ((p.M + BT - 1) / BT + p.batch) * ftiles
                             : p.batch * ((p.M + BT - 1) / BT) * ftiles;
  // Split products need float32 scratch for the partial tiles: the caller's static block
  // (qmm_quantized_matmul_static) or a stream-ordered allocation that lives until the reduce
  // kernel has run. No scratch, no split.
  const int num_kb = static_cast<int>((p.K + kBK - 1) / kBK);
  int splits = choose_splits(p, max_tiles, num_kb);
  bool scratch_async = false;
  if (splits > 1) {
    const size_t need = static_cast<size_t>(splits) * p.M * p.N * sizeof(float);
    const ScratchBlock* block = scratch_override();
    if (block) {
      if (need > block->bytes)
        return fail(QMM_ERR_TOO_LARGE, "split product needs %zu bytes of scratch, the static block has %zu", need,
                    block->bytes);
      tp.partial = static_cast<float*>(block->ptr);
    } else {
      void* ptr = nullptr;
      if (cudaMallocAsync(&ptr, need, stream) == cudaSuccess) {
        count_alloc();
        tp.partial = static_cast<float*>(ptr);
        scratch_async = true;
      } else {
        cudaGetLastError();
        splits = 1;
      }
    }
  }
  tp.splits = splits;
  int64_t items = max_tiles * splits;
  int grid = sm_count();
  if (items < grid) grid = static_cast<int>(items < 1 ? 1 : items);
  // More tiles than SMs and a last wave that does not fill them: the full waves run unsplit, and
  // the leftover tiles' K blocks are divided among the SMs (compact float32 partial tiles, a small
  // reduce) instead of some CTAs walking all of K while the rest idle.
  if (splits == 1 && !ragged && p.batch == 1 && max_tiles > grid && tail_split_enabled()) {
    const int64_t rem = max_tiles % grid;
    // (only a last wave that fills under half of the SMs: dividing a fuller one was measured and
    // lost more to the short K shares' pipeline fill than the idle SMs cost)
    int64_t s = rem ? grid / rem : 0;
    if (s > num_kb / 8) s = num_kb / 8;
    if (s > 8) s = 8;
    if (rem > 0 && s >= 2) {
      const size_t need = static_cast<size_t>(s) * rem * BT * kBF * sizeof(float);
      const ScratchBlock* block = scratch_override();
      float* part = nullptr;
      bool part_async = false;
      if (block) {
        if (need <= block->bytes) part = static_cast<float*>(block->ptr);
      } else {
        void* ptr = nullptr;
        if (cudaMallocAsync(&ptr, need, stream) == cudaSuccess) {
          count_alloc();
          part = static_cast<float*>(ptr);
          part_async = true;
        } else {
          cudaGetLastError();
        }
      }
      if (part) {
        TcParams head = tp, tail = tp;
        head.item_end = max_tiles - rem;
        launch_dependent(qmm_gemm_tc_kernel<QK, XT, BT, false>, grid, P::kThreads, P::kSmem, stream, xm, wm, head);
        tail.splits = static_cast<int>(s);
        tail.partial = part;
        tail.tail_tile0 = max_tiles - rem;
        tail.tail_tiles = rem;
        tail.item0 = (max_tiles - rem) * s;
        tail.item_end = max_tiles * s;
        const int64_t tail_grid = rem * s < grid ? rem * s : grid;
        launch_dependent(qmm_gemm_tc_kernel<QK, XT, BT, true>, static_cast<unsigned>(tail_grid), P::kThreads, P::kSmem, stream, xm, wm, tail);
        const int64_t total = rem * BT * kBF;
        int64_t blocks = (total + 255) / 256;
        if (blocks > 4 * sm_count()) blocks = 4 * sm_count();
        launch_dependent(splitk_tail_reduce_kernel, static_cast<unsigned>(blocks), 256, 0, stream, part, p.y, p.y_dtype, p.M, p.N,
                         ftiles, max_tiles - rem, rem, BT, static_cast<int>(s));
        count_launch(3);
        if (part_async) cudaFreeAsync(part, stream);
        return check_launch("qmm_gemm_tc_kernel");
      }
    }
  }
  if (splits > 1) launch_dependent(qmm_gemm_tc_kernel<QK, XT, BT, true>, grid, P::kThreads, P::kSmem, stream, xm, wm, tp);
  else launch_dependent(qmm_gemm_tc_kernel<QK, XT, BT, false>, grid, P::kThreads, P::kSmem, stream, xm, wm, tp);
  count_launch();
  if (splits > 1) {
    const int64_t total = p.M * p.N;
    int64_t blocks = (total / 4 + 255) / 256;
    if (blocks > 4 * sm_count()) blocks = 4 * sm_count();
    launch_dependent(splitk_reduce_kernel, static_cast<unsigned>(blocks), 256, 0, stream, tp.partial, p.y, p.y_dtype, total, splits);
    count_launch();
    if (scratch_async) cudaFreeAsync(tp.partial, stream);
  }
#if QMM_TC_TRACING
  if (trace_on) {   // development aid: average cycles per wait site over the CTAs
    cudaStreamSynchronize(stream);
    static long long host[16 * 1024];
    cudaMemcpy(host, trace_buf, sizeof(long long) * 16 * grid, cudaMemcpyDeviceToHost);
    double avg[16] = {0};
    for (int c = 0; c < grid; ++c)
      for (int i = 0; i < 16; ++i) avg[i] += static_cast<double>(host[c * 16 + i]) / grid;
    fprintf(stderr, "qmm_gemm_tc CTA lifetime %.0f cycles, %.1f us -> %.0f MHz\n", avg[14], avg[15] / 1e3,
            avg[14] / (avg[15] / 1e3));
    fprintf(stderr, "qmm_gemm_tc cycles/CTA: producer.empty %.0f | mma.issue %.0f mma.d_empty %.0f mma.fence %.0f mma.a_full %.0f |"
            " dequant.st %.0f dequant.full %.0f dequant.a_empty %.0f dequant.d_full %.0f\n",
            avg[1], avg[8], avg[8 + 2], avg[8 + 3], avg[8 + 4], avg[0], avg[5], avg[6], avg[7]);
  }
#endif
  return check_launch("qmm_gemm_tc_kernel");
}

template <int QK, typename XT>
int launch_bt(const qmm_problem& p, cudaStream_t stream) {
  // Token-tile width: wide tiles amortize the dequantization, narrow ones waste less MMA
  // work on short row runs.
  const int64_t rows = p.group_sizes ? (p.M + p.batch - 1) / (p.batch ? p.batch : 1) : p.M;
  if (rows > 128) return launch_cfg<QK, XT, 256>(p, stream);
  if (rows > 64) return launch_cfg<QK, XT, 128>(p, stream);
  return launch_cfg<QK, XT, 64>(p, stream);
}

template <int QK>
int launch_xt(const qmm_problem& p, cudaStream_t stream) {
  if (p.x_dtype == QMM_BF16) return launch_bt<QK, __nv_bfloat16>(p, stream);
  return launch_bt<QK, __half>(p, stream);
}

}  // namespace

bool gemm_tc_supports(const qmm_problem& p) {
  if (p.x_dtype != QMM_BF16 && p.x_dtype != QMM_F16) return false;
  if (p.lhs_idx || p.rhs_idx) return false;                   // unsorted gathers go elsewhere
  if (p.batch > kMaxSegments) return false;
  if (p.K < kBK || p.K % (p.mode == QMM_MODE_FLOAT ? 8 : 32)) return false;
  if ((p.K * 2) % 16) return false;
  if (!p.group_sizes && p.batch > 1 && p.x_batch_stride != p.M * p.K) return false;
  if (!p.group_sizes && p.batch > 1 && p.y_batch_stride != p.M * p.N) return false;
  if (p.M * (p.group_sizes ? 1 : p.batch) >= (1LL << 31) || p.N * p.batch >= (1LL << 31)) return false;
  return true;
}

int launch_gemm_tc(const qmm_problem& p, cudaStream_t stream) {
  if (p.mode == QMM_MODE_FLOAT) return launch_xt<kFloat>(p, stream);
  if (p.mode == QMM_MODE_MXFP4) return launch_xt<kMx4>(p, stream);
  if (p.bits == 8) return launch_xt<kAff8>(p, stream);
  return launch_xt<kAff4>(p, stream);
}

}  // namespace qmm
