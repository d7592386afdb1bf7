// Single-row decode kernel of the fused dequantize-and-matmul (M = 1 of `y = x . deq(w)^T`,
// src/metaljax/qmm.py:2491): the packed weight is streamed once and meets the activation row
// on the integer tensor-core path, so that a packed word costs four instructions instead of
// the dozen a floating-point dequantization needs.
//
// Arithmetic. The activation row is rewritten once per CTA as a 32-bit fixed-point number per
// element, relative to the row's largest magnitude (x_k = X_k * 2^(e-156), |X_k| <= 2^30: finer
// than the resolution a float32 accumulator has relative to its largest term), and X_k is split
// into four signed base-256 digits  X_k = d0 + 256 d1 + 256^2 d2 + 256^3 d3,  d in [-128, 127].
// The digit planes are the A operand (16 rows x 32 K, s8) of `mma.sync.m16n8k32.s32.s8.u8`;
// eight weight rows are the B operand (32 K x 8, u8): a packed 4-bit word becomes two B
// registers with `w & 0x0F0F0F0F` and `(w >> 4) & 0x0F0F0F0F`, an 8-bit word is a B register as
// it stands, an E2M1 word goes through two byte-permute lookups (16 + 2*value, the 16 is taken
// out again through the accumulator's start value). The integer sums are exact.
//
// The 16 A rows carry (group slot, digit) pairs: rows g and g + 8 of an MMA hold digit planes
// 2(g&1) and 2(g&1)+1 with every K position outside quantization group slot g/2 zeroed, so ONE
// chain of MMAs over a box of 256 codes leaves the four groups' sums  sum_k q_k d_k  in
// separate accumulator rows, and the per-group scale is applied once per box:
// y += scale[n, g] * sum. The two planes of a row pair are staged interleaved, so that one
// 16-byte shared-memory read is a lane's whole A fragment. The accumulators start at the
// float32 magic 2^23 + 2^22, which makes `int -> float` one subtraction. The bias term
// sum_g bias[n, g] * sum_{k in g} x_k  is added when a tile of rows is finished.
//
// Data movement. A CTA owns 8R consecutive weight rows at a time (R = 1, 2, 4) and its warps
// (8, or 16 when the staged row is long) split K by 128-byte columns; packed rows arrive by TMA
// in boxes of 8R rows x 128 bytes (128-byte swizzle: the 16-byte fragment reads are conflict
// free), every warp with its own ring of boxes and one mbarrier per slot. Lane 0 of a warp
// requests the first boxes before anything else happens in the kernel and refills a slot as
// soon as the warp has consumed it. Scales are read straight from global memory (L1/L2) at the
// start of a box and used at its end. The K split is reduced in shared memory in fixed order;
// no global scratch, no atomics, every wait bounded.
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

constexpr int kBoxBytes = 128;                 // bytes of one weight row in a box
constexpr int kMaxRing = 8;                    // boxes a warp keeps in flight, at most
constexpr uint32_t kMagicBits = 0x4B400000u;   // float32 2^23 + 2^22
constexpr float kMagicValue = 12582912.0f;
constexpr int kXCache = 4;                     // 8-element pieces of x a thread keeps in registers
constexpr int kPlaneSkew = 16;                 // bytes by which the second plane pair is offset (banks)

enum { kAff4 = 0, kAff8 = 1, kMx4 = 2 };

struct ImmaParams {
  const void* x;
  const void* scales;
  const void* biases;
  void* y;
  int* status;
  int K, N;
  int groups;         // K / group_size
  int group_size, y_dtype;
  int ntiles;         // tiles of 8R rows
  int nchunks;        // boxes per row: ceil(K * bits / 8 / 128)
  int ring;           // boxes per warp in flight (1..kMaxRing)
  int plane_bytes;    // bytes of one staged plane pair (2 bytes per code, whole boxes, plus padding)
  // ---- what the activation row is made from (decode step fusion; bf16 only) ----
  int prologue;             // kProNone | kProAddNorm | kProSwiglu
  const void* residual_in;  // kProAddNorm: h = x (+ residual_in); the row is rmsnorm(h) * norm_weight
  void* residual_out;       //              CTA 0 stores h here (never the buffer residual_in points to)
  const void* norm_weight;
  float eps;
  int swiglu_width;         // kProSwiglu: x holds blocks of [gate | up], each half this wide
  // ---- exchange over peer memory (none when wait_world == push_world == 0) ----
  // A gathered row travels as 8-byte units {two bf16 values, stamp}: a unit is valid when its
  // stamp is (epoch, site) of the exchange, so data and "it has arrived" cross NVLink in one
  // store and the reader needs no separate flag, fence or counter.
  const uint32_t* epoch;    // this rank's step counter
  int wait_world;           // > 0: x is such a row in this rank's gather slot, stamped (epoch, wait_site)
  int wait_site;
  int push_world;           // > 0: y also goes, stamped (epoch, push_site), to this rank's column block
  int push_site;            //      of every rank's slot
  uint8_t* push_dst[8];
  int epilogue;             // 1: rows alternate gate, up; the pushed values are silu(gate) * up
  void* epilogue_out;       //    ... also written plainly here ([N / 2] bf16) when not NULL
  long long spin_limit;
#if QMM_STEP_TRACING
  unsigned long long* trace;
#endif
};

enum { kProNone = 0, kProAddNorm = 1, kProSwiglu = 2 };

__device__ __forceinline__ uint32_t exchange_seq(uint32_t epoch, int site) { return (epoch << 10) | static_cast<uint32_t>(site + 1); }

// Eight bf16 values of a stamped row (four 8-byte units {pair, stamp}): read until every unit
// carries `stamp` (bounded; a timeout is recorded in *status and whatever is there is returned).
__device__ __noinline__ uint4 ld_stamped8(const uint8_t* p, uint32_t stamp, long long limit, int* status) {
  uint4 a, b;
  long long t0 = 0;
  int spins = 0;
  for (;;) {
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(p) : "memory");
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(p + 16) : "memory");
    if (a.y == stamp && a.w == stamp && b.y == stamp && b.w == stamp) break;
    if (++spins >= 32) {
      if (*reinterpret_cast<volatile int*>(status) != 0) break;            // someone already gave up: do not wait again
      if (t0 == 0) t0 = clock64();
      else if (clock64() - t0 > limit) {
        atomicCAS(status, 0, 100);
        break;
      }
    }
  }
  return make_uint4(a.x, a.z, b.x, b.z);
}

__device__ __forceinline__ uint4 pack8_bf16(const float (&f)[8]) {
  uint32_t u[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    u[i] = *reinterpret_cast<const uint32_t*>(&v);
  }
  return make_uint4(u[0], u[1], u[2], u[3]);
}

// d = a * b + c: 16 x 32 (s8) times 32 x 8 (u8), int32 accumulate.
__device__ __forceinline__ void imma(int (&d)[4], const uint4& a, uint32_t b0, uint32_t b1, const int (&c)[4]) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}

// Generic byte permute: each selector nibble picks one of the eight bytes of {a, b}; with its
// bit 3 set it yields the sign bit of that byte replicated over the byte instead.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

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

// How the activation row is made (a by-value subset of the launch parameters).
struct RowSource {
  const void* x;
  const void* residual_in;
  int* status;
  long long spin_limit;
  int K, prologue, swiglu_width, wait_world;
};

// Where piece pc (8 elements) of the row starts in x: for SwiGLU the gate part (the up part is
// swiglu_width further on).
__device__ __forceinline__ int64_t x_index_of(int prologue, int swiglu_width, int pc) {
  if (prologue != kProSwiglu) return static_cast<int64_t>(pc) * 8;
  const int k = pc * 8, blk = k / swiglu_width;
  return static_cast<int64_t>(blk) * 2 * swiglu_width + (k - blk * swiglu_width);
}

// Piece of the row before its last step, from its parts: the activations themselves,
// silu(gate) * up, or h = x + residual (whose normalisation needs the whole row first).
__device__ __forceinline__ uint4 compose_piece(int prologue, bool has_residual, const uint4& x0, const uint4& x1, const uint4& res) {
  if (prologue == kProSwiglu) {
    float gt[8], up[8];
    unpack8<__nv_bfloat16>(x0, gt);
    unpack8<__nv_bfloat16>(x1, up);
#pragma unroll
    for (int e = 0; e < 8; ++e) gt[e] = gt[e] / (1.0f + __expf(-gt[e])) * up[e];
    return pack8_bf16(gt);
  }
  if (prologue == kProAddNorm && has_residual) {
    float a[8], r[8];
    unpack8<__nv_bfloat16>(x0, a);
    unpack8<__nv_bfloat16>(res, r);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] += r[e];
    return pack8_bf16(a);              // the sum as it is stored: bf16
  }
  return x0;
}

// The same piece read from memory on the spot (rows longer than a thread's registers hold; out
// of line: it runs rarely and the kernel's prologue is paid for by its size).
template <typename XT>
__device__ __noinline__ uint4 load_piece_slow(const RowSource src, int pc, uint32_t wait_stamp) {
  if (pc >= src.K / 8) return make_uint4(0u, 0u, 0u, 0u);
  const int64_t xi = x_index_of(src.prologue, src.swiglu_width, pc);
  const uint8_t* xb = static_cast<const uint8_t*>(src.x);
  uint4 x0, x1 = make_uint4(0u, 0u, 0u, 0u), res = make_uint4(0u, 0u, 0u, 0u);
  if (src.wait_world > 0) {
    x0 = ld_stamped8(xb + xi * 4, wait_stamp, src.spin_limit, src.status);
    if (src.prologue == kProSwiglu) x1 = ld_stamped8(xb + (xi + src.swiglu_width) * 4, wait_stamp, src.spin_limit, src.status);
  } else {
    x0 = __ldcg(reinterpret_cast<const uint4*>(xb + xi * sizeof(XT)));
    if (src.prologue == kProSwiglu) x1 = __ldcg(reinterpret_cast<const uint4*>(xb + (xi + src.swiglu_width) * sizeof(XT)));
  }
  if (src.prologue == kProAddNorm && src.residual_in)
    res = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(src.residual_in) + pc * 8));
  return compose_piece(src.prologue, src.residual_in != nullptr, x0, x1, res);
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

// Bytes 0..3 of four words, transposed: out[q] = (byte q of d0, of d1, of d2, of d3).
__device__ __forceinline__ void transpose4(uint32_t d0, uint32_t d1, uint32_t d2, uint32_t d3, uint32_t (&out)[4]) {
  const uint32_t t0 = __byte_perm(d0, d1, 0x5140), t1 = __byte_perm(d0, d1, 0x7362);
  const uint32_t t2 = __byte_perm(d2, d3, 0x5140), t3 = __byte_perm(d2, d3, 0x7362);
  out[0] = __byte_perm(t0, t2, 0x5410); out[1] = __byte_perm(t0, t2, 0x7632);
  out[2] = __byte_perm(t1, t3, 0x5410); out[3] = __byte_perm(t1, t3, 0x7632);
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

// QK: quantization kind. XT: activation type in memory. R: 8-row blocks per tile. NW: warps.
// FUSED: the decode-step form (a prologue PRO, stamped exchange rows, pushes); the plain product is a
// separate instantiation without any of that code -- a launch runs its prologue once, from a cold
// instruction cache, and pays for every byte of it.
template <int QK, typename XT, int R, int NW, bool FUSED, int PRO>
__global__ void __launch_bounds__(NW * 32, NW == 8 ? 2 : 1)
qmm_gemv_imma_kernel(const __grid_constant__ CUtensorMap w_map, const ImmaParams p) {
  constexpr int pro = PRO;           // how the activation row is made (compile-time: see FUSED)
  const int wait_world = FUSED ? p.wait_world : 0;
  const int push_world = FUSED ? p.push_world : 0;
  constexpr int kThreads = NW * 32;
  constexpr int BITS = (QK == kAff8) ? 8 : 4;
  constexpr int kBoxCodes = kBoxBytes * 8 / BITS;    // 256 or 128 codes per row and box
  constexpr int kSpanCodes = 16 * 8 / BITS;          // codes in a lane's 16 weight bytes: 32 or 16
  constexpr int kSteps = kSpanCodes / 8;             // MMAs per 16 weight bytes: 4 or 2
  constexpr int kTileRows = 8 * R;
  constexpr int kBoxSmem = kTileRows * kBoxBytes;
  constexpr bool kNatural = (QK != kAff4);           // order of the staged activations inside 8 codes
  constexpr int kTS = (QK == kMx4) ? 1 : 2;          // bytes of a scale entry

  extern __shared__ uint8_t imma_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(imma_smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ring = p.ring;

  // two plane pairs of the staged activations: (digits 0, 1) and (digits 2, 3), each 16 bytes per
  // 8 codes = [lo codes of the first digit | of the second | hi codes of the first | of the second]
  uint8_t* xs = smem + NW * ring * kBoxSmem;
  float* xsum = reinterpret_cast<float*>(xs + 2 * p.plane_bytes);       // [groups] sums of x (int32 [groups][4] for MXFP4)
  const int xsum_words = (QK == kMx4) ? 4 * ((p.groups + 7) & ~7) : ((p.groups + 7) & ~7);
  float* red = xsum + xsum_words;                    // [2][NW][kTileRows]
  uint64_t* full_all = reinterpret_cast<uint64_t*>(red + 2 * NW * kTileRows);
  uint32_t* zeros = reinterpret_cast<uint32_t*>(full_all + NW * kMaxRing);   // 64 zero bytes
  uint32_t* amax_w = zeros + 16;                     // [2][NW]: largest magnitude, sum of squares
  volatile int* abort_flag = reinterpret_cast<volatile int*>(amax_w + 2 * NW);
  __nv_bfloat16* ypush = reinterpret_cast<__nv_bfloat16*>(amax_w + 2 * NW + 4);   // [2][kTileRows]: a finished tile on its way to the other ranks

#if QMM_STEP_TRACING
  unsigned long long* const trace = p.trace;
#else
  unsigned long long* const trace = nullptr;
  (void)trace;
#endif
  QMM_TRACE(trace, 0);               // CTA resident
  // ---- barriers, then this warp's first boxes: before anything else ----
  uint64_t* full = full_all + warp * kMaxRing;
  uint8_t* wring = smem + warp * ring * kBoxSmem;
  const int ntiles = p.ntiles, nchunks = p.nchunks, tstride = gridDim.x;
  int itile = blockIdx.x, ichunk = warp, islot = 0;       // lane 0: the next box to request
  auto issue_box = [&]() {
    mbar_expect_tx(&full[islot], kBoxSmem);
    tma_load_2d(&w_map, wring + islot * kBoxSmem, &full[islot], ichunk * kBoxBytes, itile * kTileRows);
    if (++islot == ring) islot = 0;
    ichunk += NW;
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
      for (int i = 0; i < ring && itile < ntiles; ++i) issue_box();
  }
  if (threadIdx.x < 16) zeros[threadIdx.x] = 0u;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __syncwarp();

  // ---- lane constants ----
  const int g = lane >> 2, t = lane & 3;
  const int rho = (g >> 1) | ((g & 1) << 2);         // box row (of 8) behind MMA column g: the two
                                                     // rows a quarter-warp reads lie 4 apart
  const int gpb = kBoxCodes / p.group_size;          // groups per box: 8, 4, 2 or 1
  const bool fold_half = gpb == 8;                   // eight groups: the box is folded in two halves
  const int myslot = g >> 1;                         // group slot of A rows g and g + 8
  const uint32_t plane_base = smem_u32(xs) + (g & 1) * (p.plane_bytes + kPlaneSkew);
  const uint32_t zero_u32 = smem_u32(zeros);
  uint32_t woff[2], xa[2], xinc[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    woff[h] = smem_u32(wring) + rho * kBoxBytes + ((((4 * h + t) ^ rho) & 7) << 4);
    const int grp = (4 * h + t) * kSpanCodes / p.group_size;     // group of this lane's span within the box
    const bool act = myslot == (fold_half ? (grp & 3) : grp);
    xa[h] = act ? plane_base + (4 * h + t) * kSpanCodes * 2 : zero_u32;
    xinc[h] = act ? kBoxCodes * 2 : 0;
  }
  const uint8_t* sc8 = static_cast<const uint8_t*>(p.scales);

  // ---- what does not depend on the previous kernel: requested before the wait ----
  const int vpieces = p.K / 8, ppieces = nchunks * kBoxCodes / 8;
  const int iters = (ppieces + kThreads - 1) / kThreads;
  // (lines of the norm weight, of the first tile's scale rows and of its bias rows into L1: the
  // loads that want them later then cost a cache hit instead of a trip to L2)
  {
    auto prefetch_l1 = [](const void* q) { asm volatile("prefetch.global.L1 [%0];" ::"l"(q)); };
    if (pro == kProAddNorm)
      for (int ln = threadIdx.x; ln * 128 < p.K * 2; ln += kThreads) prefetch_l1(static_cast<const uint8_t*>(p.norm_weight) + ln * 128);
    const int row_bytes = p.groups * kTS, lines_per_row = (row_bytes + 127) / 128;
    const int first_row = blockIdx.x * kTileRows;
    for (int ln = threadIdx.x; ln < kTileRows * lines_per_row; ln += kThreads) {
      const int r = min(first_row + ln / lines_per_row, p.N - 1), o = (ln % lines_per_row) * 128;
      if (static_cast<int>(blockIdx.x) < ntiles && o < row_bytes) {
        prefetch_l1(sc8 + static_cast<int64_t>(r) * row_bytes + o);
        if (QK != kMx4) prefetch_l1(static_cast<const uint8_t*>(p.biases) + static_cast<int64_t>(r) * row_bytes + o);
      }
    }
  }

  // ---- the activation row: after everything the previous kernel wrote is visible ----
  asm volatile("griddepcontrol.wait;" ::: "memory");
  QMM_TRACE(trace, 1);               // predecessor done (or flushed)
  const uint32_t epoch = (wait_world > 0 || push_world > 0) ? *reinterpret_cast<const volatile uint32_t*>(p.epoch) : 0u;
  const uint32_t wait_stamp = exchange_seq(epoch, p.wait_site);
  if (wait_stamp != 0xffffffffu) QMM_TRACE(trace, 8);    // the epoch has arrived
  const bool stamped = wait_world > 0;
  const uint8_t* xbytes = static_cast<const uint8_t*>(p.x);
  // Eight consecutive elements of x starting at element `i` (a multiple of 8): plain memory, or a
  // stamped row of this rank's gather slot that the other ranks are still filling. `request`
  // only reads (both halves of a stamped piece, unchecked); `settle` checks the stamps and falls
  // back to the bounded re-reading loop. All of a thread's requests go out before its first
  // check, so the row costs one trip to memory, not one per piece.
  auto request = [&](int64_t i, uint4& a, uint4& b) {
    if (stamped) {
      // weak loads served by L2 (where the peers' stores land): they pipeline, which the
      // volatile loads of the re-reading loop do not -- those complete one after the other
      const uint8_t* q = xbytes + i * 4;
      asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(q));
      asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(q + 16));
    } else {
      a = __ldcg(reinterpret_cast<const uint4*>(xbytes + i * sizeof(XT)));
    }
  };
  auto settle = [&](int64_t i, const uint4& a, const uint4& b) -> uint4 {
    if (!stamped) return a;
    if (a.y == wait_stamp && a.w == wait_stamp && b.y == wait_stamp && b.w == wait_stamp) return make_uint4(a.x, a.z, b.x, b.z);
    return ld_stamped8(xbytes + i * 4, wait_stamp, p.spin_limit, p.status);
  };
  auto load_piece = [&](int pc) -> uint4 {
    const RowSource src = {p.x, p.residual_in, p.status, p.spin_limit, p.K, pro, p.swiglu_width, wait_world};
    return load_piece_slow<XT>(src, pc, wait_stamp);
  };
  // |f| as an unsigned pattern orders like the magnitude, NaNs above infinity above everything
  auto mag_of = [&](const float (&f)[8], uint32_t m) -> uint32_t {
#pragma unroll
    for (int e = 0; e < 8; ++e) m = max(m, __float_as_uint(f[e]) & 0x7fffffffu);
    return m;
  };
  // Register arrays are only ever indexed by unrolled constants; the loops that do the work stay
  // rolled (this code runs once per CTA from a cold instruction cache: its size is its cost).
  auto pick = [&](const uint4 (&arr)[kXCache], int i) -> uint4 {
    uint4 v = arr[0];
#pragma unroll
    for (int c = 1; c < kXCache; ++c)
      if (c == i) v = arr[c];
    return v;
  };
  uint4 xcache[kXCache];
  uint32_t mag = 0;
  float ss = 0.0f;
  // first pass over the row: its largest magnitude (and the sum of squares of h)
  auto scan_piece = [&](int pc, const uint4& raw, const uint4& nwraw) {
    float f[8];
    unpack8<XT>(raw, f);
    if (pro == kProAddNorm && pc < vpieces) {
      if (blockIdx.x == 0 && p.residual_out) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.residual_out) + pc * 8) = raw;
      float w8[8];
      unpack8<__nv_bfloat16>(nwraw, w8);
#pragma unroll
      for (int e = 0; e < 8; ++e) { ss = fmaf(f[e], f[e], ss); f[e] *= w8[e]; }
    }
    mag = mag_of(f, mag);
  };
  auto norm_piece = [&](int pc) -> uint4 {
    if (pro != kProAddNorm || pc >= vpieces) return make_uint4(0u, 0u, 0u, 0u);
    return __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.norm_weight) + pc * 8));
  };
  {
    // every request of the first kXCache pieces goes out before the first check
    uint4 qa[kXCache], qb[kXCache], ua[kXCache], ub[kXCache];      // (ua doubles as the residual piece: never both)
#pragma unroll
    for (int c = 0; c < kXCache; ++c) {
      const int pc = threadIdx.x + c * kThreads;
      qa[c] = qb[c] = ua[c] = ub[c] = make_uint4(0u, 0u, 0u, 0u);
      if (c < iters && pc < vpieces) {
        const int64_t xi = x_index_of(pro, p.swiglu_width, pc);
        request(xi, qa[c], qb[c]);
        if (pro == kProSwiglu) request(xi + p.swiglu_width, ua[c], ub[c]);
        if (pro == kProAddNorm && p.residual_in)
          ua[c] = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.residual_in) + pc * 8));
      }
    }
    QMM_TRACE(trace, 9);             // requests issued
    for (int i = 0; i < iters; ++i) {
      const int pc = threadIdx.x + i * kThreads;
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if (i < kXCache) {
        if (pc < vpieces) {
          const int64_t xi = x_index_of(pro, p.swiglu_width, pc);
          const uint4 u0 = pick(ua, i);
          const uint4 x0 = settle(xi, pick(qa, i), pick(qb, i));
          uint4 x1 = make_uint4(0u, 0u, 0u, 0u);
          if (pro == kProSwiglu) x1 = settle(xi + p.swiglu_width, u0, pick(ub, i));
          raw = compose_piece(pro, p.residual_in != nullptr, x0, x1, u0);
          if (raw.x != 0x12345677u && i == 0) QMM_TRACE(trace, 10);   // thread 0's first piece settled
        }
#pragma unroll
        for (int c = 0; c < kXCache; ++c)
          if (c == i) xcache[c] = raw;
        scan_piece(pc, raw, norm_piece(pc));
      } else {
        scan_piece(pc, load_piece(pc), norm_piece(pc));
      }
    }
  }
  if (mag != 0xffffffffu) QMM_TRACE(trace, 11);   // thread 0 has scanned its pieces
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mag = max(mag, __shfl_xor_sync(0xffffffffu, mag, o));
    ss += __shfl_xor_sync(0xffffffffu, ss, o);
  }
  if (lane == 0) { amax_w[warp] = mag; amax_w[NW + warp] = __float_as_uint(ss); }
  QMM_TRACE(trace, 12);
  __syncthreads();
  QMM_TRACE(trace, 2);               // the whole row has arrived and been read once
  mag = 0;
  ss = 0.0f;
#pragma unroll
  for (int i = 0; i < NW; ++i) { mag = max(mag, amax_w[i]); ss += __uint_as_float(amax_w[NW + i]); }
  float inv_rms = 1.0f;
  bool nonfinite = mag >= 0x7f800000u;
  if (pro == kProAddNorm) {
    inv_rms = rsqrtf(ss / static_cast<float>(p.K) + p.eps);
    // the row's largest magnitude is at most this (a bf16 rounding above max |h w| / rms)
    const float bound = __uint_as_float(mag) * inv_rms * 1.0079f;
    mag = __float_as_uint(bound);
    nonfinite = nonfinite || mag >= 0x7f800000u;
  }
  // exponent field of the largest magnitude; infinities and NaNs poison the row
  uint32_t ebits = mag >> 23;
  if (ebits < 32u || nonfinite) ebits = 32u;    // (magnitudes below 2^-95 lose digits: far below anything real)
  const float to_fixed = __uint_as_float((283u - ebits) << 23);      // 2^(156 - e): |x| * this <= 2^30
  {
    const int lanes_per_group = p.group_size / 8;
    // second pass: the digits of piece pc into the planes, the per-group sums
    auto stage_piece = [&](int pc, const uint4& raw, const uint4& nwraw) {
      float f[8];
      unpack8<XT>(raw, f);
      if (pro == kProAddNorm && pc < vpieces) {
        float w8[8];
        unpack8<__nv_bfloat16>(nwraw, w8);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = f[e] * inv_rms * w8[e];
        unpack8<__nv_bfloat16>(pack8_bf16(f), f);          // the normalised row as a glue kernel would store it: bf16
      }
      uint32_t d[8];
#pragma unroll
      for (int e = 0; e < 8; ++e)     // X + 0x80808080 has the four digits + 128 as its bytes
        d[e] = (static_cast<uint32_t>(__float2int_rn(nonfinite ? 0.0f : f[e] * to_fixed)) + 0x80808080u) ^ 0x80808080u;
      uint32_t lo[4], hi[4];
      if constexpr (kNatural) {       // codes 0..3 | 4..7
        transpose4(d[0], d[1], d[2], d[3], lo);
        transpose4(d[4], d[5], d[6], d[7], hi);
      } else {                        // codes 0, 2, 4, 6 | 1, 3, 5, 7: what the two nibble masks extract
        transpose4(d[0], d[2], d[4], d[6], lo);
        transpose4(d[1], d[3], d[5], d[7], hi);
      }
      if (pc < ppieces) {
        *reinterpret_cast<uint4*>(xs + pc * 16) = make_uint4(lo[0], lo[1], hi[0], hi[1]);
        *reinterpret_cast<uint4*>(xs + p.plane_bytes + kPlaneSkew + pc * 16) = make_uint4(lo[2], lo[3], hi[2], hi[3]);
      }
      // per digit plane: the sum of the piece's digits
      int ds[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) ds[q] = __dp4a(static_cast<int>(lo[q]), 0x01010101, __dp4a(static_cast<int>(hi[q]), 0x01010101, 0));
      if constexpr (QK == kMx4) {
        // per group and plane, as integers: what the +16 of every code met
#pragma unroll
        for (int o = 1; o < 4; o <<= 1)
#pragma unroll
          for (int q = 0; q < 4; ++q) ds[q] += __shfl_xor_sync(0xffffffffu, ds[q], o);
        const int grp = pc >> 2;
        if ((lane & 3) == 0 && grp < p.groups) *reinterpret_cast<int4*>(reinterpret_cast<int*>(xsum) + grp * 4) = make_int4(ds[0], ds[1], ds[2], ds[3]);
      } else {
        // per group: the sum of x itself, for the bias term (in units of 2^(e-156))
        float sx = fmaf(static_cast<float>(ds[3]), 16777216.0f, fmaf(static_cast<float>(ds[2]), 65536.0f,
                        fmaf(static_cast<float>(ds[1]), 256.0f, static_cast<float>(ds[0]))));
        for (int o = 1; o < lanes_per_group; o <<= 1) sx += __shfl_xor_sync(0xffffffffu, sx, o);
        const int grp = pc / lanes_per_group;
        if ((lane & (lanes_per_group - 1)) == 0 && grp < p.groups) xsum[grp] = sx;
      }
    };
    for (int i = 0; i < iters; ++i) {
      const int pc = threadIdx.x + i * kThreads;
      if (i < kXCache) stage_piece(pc, pick(xcache, i), norm_piece(pc));
      else stage_piece(pc, load_piece(pc), norm_piece(pc));
    }
  }
  QMM_TRACE(trace, 13);              // thread 0 has staged its pieces
  __syncthreads();                   // the staged activations, their sums and the zeros are in place
  QMM_TRACE(trace, 3);               // digits staged

  // what one unit of an accumulator is worth: rows g (digit 2(g&1)) and g + 8 (the next digit)
  const float ps_lo = __uint_as_float((ebits - 29u + 16u * (g & 1) - (QK == kMx4 ? 1u : 0u)) << 23);   // 2^(e - 156 + 8 digit)
  const float ps_hi = ps_lo * 256.0f;
  const float from_fixed = __uint_as_float((ebits - 29u) << 23);
  uint32_t nib = 0x0F0F0F0Fu;
  asm volatile("" : "+r"(nib));      // keep the mask in a register: one LOP3 per use
  const int magic4[4] = {static_cast<int>(kMagicBits), static_cast<int>(kMagicBits), static_cast<int>(kMagicBits),
                         static_cast<int>(kMagicBits)};

  int cslot = 0, rbuf = 0, prev_tile = -1;
  uint32_t cphase = 0;
  bool ok = true;
  // A finished tile goes to every rank as stamped units (this rank's rows are a column block of
  // the row every rank gathers): plain 16-byte peer stores of {pair, stamp, pair, stamp};
  // lane <-> (rank, 8 rows); made by the last warp.
  const uint32_t push_stamp = exchange_seq(epoch, p.push_site);
  const bool pairs = FUSED && p.epilogue == 1;
  const bool tile_out = push_world > 0 || pairs;     // finished tiles pass through shared memory
  auto push_tile = [&](int tl, int buf) {
    const int peer = lane / R, v = lane % R;
    const int n8 = tl * kTileRows + v * 8;
    const bool plain = pairs && peer == 0 && p.epilogue_out != nullptr;
    if ((peer < push_world || plain) && n8 < p.N) {
      const uint4 d = *reinterpret_cast<const uint4*>(ypush + buf * kTileRows + v * 8);
      if (pairs) {
        // rows (2j, 2j + 1) = (gate_j, up_j): four values silu(gate) * up, two stamped units
        float f[8];
        unpack8<__nv_bfloat16>(d, f);
        const __nv_bfloat162 o0 = __floats2bfloat162_rn(f[0] / (1.0f + __expf(-f[0])) * f[1], f[2] / (1.0f + __expf(-f[2])) * f[3]);
        const __nv_bfloat162 o1 = __floats2bfloat162_rn(f[4] / (1.0f + __expf(-f[4])) * f[5], f[6] / (1.0f + __expf(-f[6])) * f[7]);
        const uint32_t u0 = *reinterpret_cast<const uint32_t*>(&o0), u1 = *reinterpret_cast<const uint32_t*>(&o1);
        if (plain) *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.epilogue_out) + n8 / 2) = make_uint2(u0, u1);
        if (peer < push_world)
          *reinterpret_cast<uint4*>(p.push_dst[peer] + static_cast<int64_t>(n8 / 2) * 4) = make_uint4(u0, push_stamp, u1, push_stamp);
      } else {
        uint4* dst = reinterpret_cast<uint4*>(p.push_dst[peer] + static_cast<int64_t>(n8) * 4);
        dst[0] = make_uint4(d.x, push_stamp, d.y, push_stamp);
        dst[1] = make_uint4(d.z, push_stamp, d.w, push_stamp);
      }
    }
  };
  for (int tile = blockIdx.x; tile < ntiles; tile += tstride) {
    float ylo[R][2], yhi[R][2];
    uint32_t rowoff[R][2];           // byte offsets of the scale-table rows behind this lane's two MMA
                                     // columns (tile rows 8 rb + t and 8 rb + t + 4), clamped to the last row
#pragma unroll
    for (int rb = 0; rb < R; ++rb) {
      ylo[rb][0] = ylo[rb][1] = yhi[rb][0] = yhi[rb][1] = 0.0f;
      rowoff[rb][0] = static_cast<uint32_t>(min(tile * kTileRows + rb * 8 + t, p.N - 1)) * static_cast<uint32_t>(p.groups * kTS);
      rowoff[rb][1] = static_cast<uint32_t>(min(tile * kTileRows + rb * 8 + t + 4, p.N - 1)) * static_cast<uint32_t>(p.groups * kTS);
    }
    // this thread's first piece of the tile's bias rows (used when the tile is finished)
    uint4 bias_first = make_uint4(0u, 0u, 0u, 0u);
    const int frow = threadIdx.x / NW, fslice = threadIdx.x % NW;
    const bool bias_vec = QK != kMx4 && (p.groups & 7) == 0 && (reinterpret_cast<uintptr_t>(p.biases) & 15) == 0;
    const uint8_t* brow = nullptr;
    if constexpr (QK != kMx4) {
      brow = static_cast<const uint8_t*>(p.biases) + static_cast<int64_t>(min(tile * kTileRows + frow, p.N - 1)) * p.groups * 2;
      if (bias_vec && frow < kTileRows && fslice < p.groups / 8) bias_first = __ldg(reinterpret_cast<const uint4*>(brow) + fslice);
    }

    for (int c = warp; c < nchunks && ok; c += NW) {
      // this lane's scale entries of the box's (first) fold: requested now, used after the MMAs
      uint32_t sraw[R][2];
      uint32_t goff = static_cast<uint32_t>(min(c * gpb + myslot, p.groups - 1)) * kTS;
#pragma unroll
      for (int rb = 0; rb < R; ++rb)
#pragma unroll
        for (int j = 0; j < 2; ++j)
          sraw[rb][j] = (QK == kMx4) ? __ldg(sc8 + rowoff[rb][j] + goff)
                                     : __ldg(reinterpret_cast<const uint16_t*>(sc8 + rowoff[rb][j] + goff));
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
        const uint32_t xaddr = xa[h] + c * xinc[h];
        uint4 av[kSteps];            // the A fragment of every step: one 16-byte read each
        av[0] = lds128<0>(xaddr);
        av[1] = lds128<16>(xaddr);
        if constexpr (kSteps == 4) {
          av[2] = lds128<32>(xaddr);
          av[3] = lds128<48>(xaddr);
        }
        int cinit[4] = {magic4[0], magic4[1], magic4[2], magic4[3]};
        if constexpr (QK == kMx4) {
          // every code was given as 16 + 2*value: start at magic - 16 * (sum of the digits the
          // row meets); groups past the end of K met only zeros
          const int gi = c * gpb + 4 * h + myslot;
          const int4 xi = gi < p.groups ? *reinterpret_cast<const int4*>(reinterpret_cast<const int*>(xsum) + gi * 4)
                                        : make_int4(0, 0, 0, 0);
          const int s0 = (g & 1) ? xi.z : xi.x, s1 = (g & 1) ? xi.w : xi.y;
          cinit[0] = cinit[1] = static_cast<int>(kMagicBits) - 16 * s0;
          cinit[2] = cinit[3] = static_cast<int>(kMagicBits) - 16 * s1;
        }
#pragma unroll
        for (int j = 0; j < kSteps; ++j) {
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
            if (j == 0 && (h == 0 || QK == kMx4)) {
              imma(acc[rb], av[j], b0, b1, cinit);
            } else if (j == 0) {       // second half of the box: a new chain only if the box folds twice
              if (fresh) imma(acc[rb], av[j], b0, b1, cinit);
              else imma(acc[rb], av[j], b0, b1, acc[rb]);
            } else {
              imma(acc[rb], av[j], b0, b1, acc[rb]);
            }
          }
        }
        fresh = false;
        if (h == 1 || fold_half) {
          // fold: accumulator rows g (c0, c1) and g + 8 (c2, c3) hold this lane's group slot for
          // two digit planes, of MMA columns 2t and 2t + 1, i.e. tile rows 8 rb + t and 8 rb + t + 4
#pragma unroll
          for (int rb = 0; rb < R; ++rb) {
            float s0, s1;
            if constexpr (QK == kMx4) {
              s0 = __uint_as_float(max(sraw[rb][0] << 23, 0x00400000u));
              s1 = __uint_as_float(max(sraw[rb][1] << 23, 0x00400000u));
            } else {
              s0 = __uint_as_float(sraw[rb][0] << 16);
              s1 = __uint_as_float(sraw[rb][1] << 16);
            }
            ylo[rb][0] = fmaf(__int_as_float(acc[rb][0]) - kMagicValue, s0, ylo[rb][0]);
            ylo[rb][1] = fmaf(__int_as_float(acc[rb][1]) - kMagicValue, s1, ylo[rb][1]);
            yhi[rb][0] = fmaf(__int_as_float(acc[rb][2]) - kMagicValue, s0, yhi[rb][0]);
            yhi[rb][1] = fmaf(__int_as_float(acc[rb][3]) - kMagicValue, s1, yhi[rb][1]);
          }
          fresh = true;
          if (h == 0) {              // eight groups per box: the second half has its own scales
            goff = static_cast<uint32_t>(min(c * gpb + 4 + myslot, p.groups - 1)) * kTS;
#pragma unroll
            for (int rb = 0; rb < R; ++rb)
#pragma unroll
              for (int j = 0; j < 2; ++j)
                sraw[rb][j] = (QK == kMx4) ? __ldg(sc8 + rowoff[rb][j] + goff)
                                           : __ldg(reinterpret_cast<const uint16_t*>(sc8 + rowoff[rb][j] + goff));
          }
        }
      }
      // the slot is free again: every read of it has been consumed by an MMA issued above
      __syncwarp();
      if (lane == 0 && itile < ntiles) issue_box();
    }

    if (prev_tile < 0) QMM_TRACE(trace, 7);   // first tile: this warp's K loop done
    // ---- this warp's share of K, for its lanes' digit planes and slots: scale, add up ----
    float v[2 * R];
#pragma unroll
    for (int rb = 0; rb < R; ++rb) {
      v[2 * rb] = fmaf(yhi[rb][0], ps_hi, ylo[rb][0] * ps_lo);
      v[2 * rb + 1] = fmaf(yhi[rb][1], ps_hi, ylo[rb][1] * ps_lo);
    }
    reduce_over_g<2 * R>(v, lane);
    {
      // value number `idx` of 2R: (row block, column parity) -> tile row 8 rb + t + 4 j
      constexpr int kBitsUsed = (2 * R >= 8) ? 3 : ((2 * R >= 4) ? 2 : 1);
      const int idx = (lane >> (5 - kBitsUsed)) & (2 * R - 1);
      const bool writer = kBitsUsed == 3 || (kBitsUsed == 2 && (lane & 4) == 0) || (kBitsUsed == 1 && (lane & 12) == 0);
      if (writer) red[(rbuf * NW + warp) * kTileRows + (idx >> 1) * 8 + t + 4 * (idx & 1)] = v[0];
    }
    __syncthreads();
    if (*abort_flag) {
      if (threadIdx.x == 0) atomicCAS(p.status, 0, *abort_flag);
      return;
    }
    if (tile_out && prev_tile >= 0 && warp == NW - 1) push_tile(prev_tile, rbuf ^ 1);   // (complete since this barrier)
    // ---- rows x NW threads: the warps' shares (fixed order) plus the bias term ----
    if (frow < kTileRows) {
      const int n = tile * kTileRows + frow;
      float s = red[(rbuf * NW + fslice) * kTileRows + frow];
      if constexpr (QK != kMx4) {
        float bsum = 0.0f;
        if (bias_vec) {
          for (int o = fslice; o < p.groups / 8; o += NW) {
            const uint4 bv = o == fslice ? bias_first : __ldg(reinterpret_cast<const uint4*>(brow) + o);
            float b8[8];
            unpack8<__nv_bfloat16>(bv, b8);
            const float4 x0 = *reinterpret_cast<const float4*>(xsum + o * 8);
            const float4 x1 = *reinterpret_cast<const float4*>(xsum + o * 8 + 4);
            bsum = fmaf(b8[0], x0.x, bsum); bsum = fmaf(b8[1], x0.y, bsum); bsum = fmaf(b8[2], x0.z, bsum); bsum = fmaf(b8[3], x0.w, bsum);
            bsum = fmaf(b8[4], x1.x, bsum); bsum = fmaf(b8[5], x1.y, bsum); bsum = fmaf(b8[6], x1.z, bsum); bsum = fmaf(b8[7], x1.w, bsum);
          }
        } else {
          for (int gi = fslice; gi < p.groups; gi += NW)
            bsum = fmaf(__uint_as_float(static_cast<uint32_t>(__ldg(reinterpret_cast<const uint16_t*>(brow) + gi)) << 16), xsum[gi], bsum);
        }
        s = fmaf(bsum, from_fixed, s);
      }
#pragma unroll
      for (int o = 1; o < NW; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (nonfinite) s = __uint_as_float(0x7fc00000u);
      if (fslice == 0) {
        if (p.y && n < p.N) {
          if (p.y_dtype == QMM_BF16) static_cast<__nv_bfloat16*>(p.y)[n] = __float2bfloat16_rn(s);
          else if (p.y_dtype == QMM_F16) static_cast<__half*>(p.y)[n] = __float2half_rn(s);
          else static_cast<float*>(p.y)[n] = s;
        }
        if (tile_out) ypush[rbuf * kTileRows + frow] = __float2bfloat16_rn(s);
      }
    }
    rbuf ^= 1;
    if (prev_tile < 0) QMM_TRACE(trace, 4);   // first tile done
    prev_tile = tile;
  }
  QMM_TRACE(trace, 5);               // all tiles done
  if (tile_out) {
    __syncthreads();                 // the last tile's rows are in shared memory
    if (warp == NW - 1 && prev_tile >= 0) push_tile(prev_tile, rbuf ^ 1);
  }
  QMM_TRACE(trace, 6);
}

struct ImmaPlan {
  int r;            // row blocks per tile
  int nw;           // warps per CTA
  int ring;
  int grid;
  size_t smem;
};

size_t imma_smem(int r, int nw, int ring, int plane_bytes, int groups, bool mx) {
  const size_t xsum_words = mx ? 4 * static_cast<size_t>((groups + 7) & ~7) : static_cast<size_t>((groups + 7) & ~7);
  return 1024 + static_cast<size_t>(nw) * ring * r * 8 * kBoxBytes + 2 * static_cast<size_t>(plane_bytes) +
         xsum_words * 4 + static_cast<size_t>(2) * nw * 8 * r * 4 + static_cast<size_t>(nw) * kMaxRing * 8 +
         64 + nw * 8 + 16 + 2 * 8 * r * 2;
}

int env_int(const char* name, int fallback) {
  const char* e = getenv(name);
  return (e && *e) ? atoi(e) : fallback;
}

template <int QK, typename XT, int R, int NW, bool FUSED, int PRO>
int launch_r(const CUtensorMap& wm, const ImmaParams& ip, const ImmaPlan& plan, cudaStream_t stream) {
  auto kernel = qmm_gemv_imma_kernel<QK, XT, R, NW, FUSED, PRO>;
  static bool configured[kMaxDevices] = {};     // the attribute is per device
  const int dev = current_device();
  if (dev < 0) return QMM_ERR_DEVICE;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
    if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(plan.grid));
  cfg.blockDim = dim3(NW * 32);
  cfg.dynamicSmemBytes = plan.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
#if QMM_STEP_TRACING
  ImmaParams traced = ip;
  traced.trace = next_trace_block(1 + ip.prologue);
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, wm, traced);
#else
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, wm, ip);
#endif
  if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "qmm_gemv_imma_kernel launch: %s", cudaGetErrorString(e));
  count_launch();
  return check_launch("qmm_gemv_imma_kernel");
}

template <int QK, typename XT>
int launch_qx(const CUtensorMap& wm, const ImmaParams& ip, const ImmaPlan& plan, cudaStream_t stream) {
  if (plan.nw == 16) {
    if (plan.r == 4) return launch_r<QK, XT, 4, 16, false, kProNone>(wm, ip, plan, stream);
    if (plan.r == 2) return launch_r<QK, XT, 2, 16, false, kProNone>(wm, ip, plan, stream);
    return launch_r<QK, XT, 1, 16, false, kProNone>(wm, ip, plan, stream);
  }
  if (plan.r == 4) return launch_r<QK, XT, 4, 8, false, kProNone>(wm, ip, plan, stream);
  if (plan.r == 2) return launch_r<QK, XT, 2, 8, false, kProNone>(wm, ip, plan, stream);
  return launch_r<QK, XT, 1, 8, false, kProNone>(wm, ip, plan, stream);
}

// The decode-step forms: 4-bit affine weights, bf16 activations, sixteen warps (one family of
// kernels for every linear of a step, so that consecutive launches find their code cached).
template <int PRO>
int launch_fused(const CUtensorMap& wm, const ImmaParams& ip, const ImmaPlan& plan, cudaStream_t stream) {
  if (plan.nw == 8) {        // (only the tall form: a weight of many tiles per SM)
    if (plan.r == 4) return launch_r<kAff4, __nv_bfloat16, 4, 8, true, PRO>(wm, ip, plan, stream);
  }
  if (plan.r == 4) return launch_r<kAff4, __nv_bfloat16, 4, 16, true, PRO>(wm, ip, plan, stream);
  if (plan.r == 2) return launch_r<kAff4, __nv_bfloat16, 2, 16, true, PRO>(wm, ip, plan, stream);
  return launch_r<kAff4, __nv_bfloat16, 1, 16, true, PRO>(wm, ip, plan, stream);
}

// Tile height, warps per CTA, ring depth and grid for one problem, or r = 0 when the staged
// activations do not fit. A weight of at most one tile per SM is a latency problem: sixteen
// warps per tile (one box each at K = 4096) and the tallest tile that still gives at least half
// the SMs one. A larger weight is a throughput problem: eight warps and two CTAs per SM when
// that leaves every warp 8 KiB of boxes in flight (a tile's fixed costs are then paid by eight
// warps, and the successor's CTAs can become resident early), else sixteen warps in one CTA.
ImmaPlan make_plan(const qmm_problem& p, int nchunks, int plane_bytes, int groups, bool mx, bool fused) {
  const int sms = device_sm_count();
  const int force_r = env_int("QMM_IMMA_R", 0), force_ring = env_int("QMM_IMMA_RING", 0), force_nw = env_int("QMM_IMMA_NW", 0);
  const size_t kTwoPerSm = 113 * 1024;     // an SM has 228 KiB, of which every resident CTA also takes 1 KiB
  const size_t kOnePerSm = 226 * 1024;
  const bool small = (p.N + 31) / 32 <= sms;
  for (int pass = 0; pass < 2; ++pass) {
    // the decode step's linears: sixteen warps, except a weight of at least `big` rows (many
    // tiles per SM), which streams better from two eight-warp CTAs per SM
    static const int big = env_int("QMM_IMMA_FUSED_BIG", 4096);
    const int nw = fused ? ((p.N >= big && pass == 0) ? 8 : 16)
                         : (force_nw ? force_nw : ((pass == 0) == small ? 16 : 8));
    for (int r = 4; r >= 1; r >>= 1) {
      if (force_r && r != force_r) continue;
      if (fused && nw == 8 && r != 4) break;              // (the eight-warp fused form exists for tall tiles only)
      const int64_t tiles = (p.N + 8 * r - 1) / (8 * r);
      if (!force_r && r > 1 && tiles * 2 < sms) continue;
      const size_t budget = nw == 8 ? kTwoPerSm : kOnePerSm;
      int ring = force_ring ? force_ring : 64 / (8 * r);            // 8 KiB in flight per warp
      if (ring > kMaxRing) ring = kMaxRing;
      size_t smem = imma_smem(r, nw, ring, plane_bytes, groups, mx);
      if (pass == 1 || nw == 16)
        while (!force_ring && ring > 2 && smem > budget) smem = imma_smem(r, nw, --ring, plane_bytes, groups, mx);
      if (smem > budget) continue;
      int64_t grid = static_cast<int64_t>(sms) * (nw == 8 ? 2 : 1);
      if (grid > tiles) grid = tiles;
      return {r, nw, ring, static_cast<int>(grid), smem};
    }
  }
  return {0, 0, 0, 0, 0};
}

int plane_bytes_of(int nchunks, int boxcodes) { return ((nchunks * boxcodes * 2 + 127) & ~127) + 128; }

}  // namespace

bool gemv_imma_supports(const qmm_problem& p) {
  static const bool enabled = env_int("QMM_GEMV_IMMA", 1) != 0;
  if (!enabled) return false;
  if (p.M != 1 || p.batch != 1 || p.lhs_idx || p.rhs_idx || p.group_sizes) return false;
  if (p.x_dtype != QMM_BF16 && p.x_dtype != QMM_F16) return false;
  const bool mx = p.mode == QMM_MODE_MXFP4;
  if (!mx && p.table_dtype != QMM_BF16) return false;       // f16 / float32 tables: the other decode kernel
  if (p.K % 32 || p.K < 32 || p.K > (1 << 20) || p.N < 1) return false;
  const int bits = (!mx && p.bits == 8) ? 8 : 4;
  const int boxcodes = kBoxBytes * 8 / bits;
  const int nchunks = static_cast<int>((p.K + boxcodes - 1) / boxcodes);
  const int groups = static_cast<int>(p.K / (mx ? 32 : p.group_size));
  if (p.N * groups * (mx ? 1 : 2) >= (1LL << 31)) return false;        // 32-bit table offsets
  return imma_smem(2, 16, 2, plane_bytes_of(nchunks, boxcodes), groups, mx) <= 226 * 1024;
}

int launch_gemv_imma(const qmm_problem& p, cudaStream_t stream, const DecodeFusion* fusion) {
  const bool mx = p.mode == QMM_MODE_MXFP4;
  const int bits = (!mx && p.bits == 8) ? 8 : 4;
  const int boxcodes = kBoxBytes * 8 / bits;
  ImmaParams ip = {};          // no prologue, no exchange
  if (fusion) {
    if (p.x_dtype != QMM_BF16) return fail(QMM_ERR_DTYPE, "fused decode linears take bf16 activations");
    ip.prologue = fusion->prologue;
    ip.residual_in = fusion->residual_in; ip.residual_out = fusion->residual_out;
    ip.norm_weight = fusion->norm_weight; ip.eps = fusion->eps; ip.swiglu_width = fusion->swiglu_width;
    ip.epoch = fusion->epoch;
    ip.wait_world = fusion->wait_world; ip.wait_site = fusion->wait_site;
    ip.push_world = fusion->push_world; ip.push_site = fusion->push_site;
    for (int r = 0; r < 8; ++r) ip.push_dst[r] = fusion->push_dst[r];
    ip.epilogue = fusion->epilogue;
    ip.epilogue_out = fusion->epilogue_out;
    ip.spin_limit = wait_limit_clocks();
  }
  ip.x = p.x; ip.scales = p.scales; ip.biases = p.biases; ip.y = p.y;
  ip.status = device_status_word();
  if (!ip.status) return fail(QMM_ERR_CUDA, "could not allocate the device status word");
  ip.K = static_cast<int>(p.K); ip.N = static_cast<int>(p.N);
  ip.group_size = mx ? 32 : p.group_size;
  ip.groups = ip.K / ip.group_size;
  ip.y_dtype = p.y_dtype;
  ip.nchunks = (ip.K + boxcodes - 1) / boxcodes;
  ip.plane_bytes = plane_bytes_of(ip.nchunks, boxcodes);
  const ImmaPlan plan = make_plan(p, ip.nchunks, ip.plane_bytes, ip.groups, mx, fusion != nullptr);
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
  if (fusion) {      // the decode step: bf16 activations (checked above), 4-bit affine weights
    if (mx || bits != 4) return fail(QMM_ERR_UNSUPPORTED, "fused decode linears take 4-bit affine weights");
    if (ip.prologue == kProAddNorm) return launch_fused<kProAddNorm>(wm, ip, plan, stream);
    if (ip.prologue == kProSwiglu) return launch_fused<kProSwiglu>(wm, ip, plan, stream);
    return launch_fused<kProNone>(wm, ip, plan, stream);
  }
  if (mx) return bf ? launch_qx<kMx4, __nv_bfloat16>(wm, ip, plan, stream) : launch_qx<kMx4, __half>(wm, ip, plan, stream);
  if (bits == 8) return bf ? launch_qx<kAff8, __nv_bfloat16>(wm, ip, plan, stream) : launch_qx<kAff8, __half>(wm, ip, plan, stream);
  return bf ? launch_qx<kAff4, __nv_bfloat16>(wm, ip, plan, stream) : launch_qx<kAff4, __half>(wm, ip, plan, stream);
}

}  // namespace qmm
