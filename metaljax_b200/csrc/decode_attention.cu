// Attention of one decode position over the key/value cache, with the rotary embedding and the
// cache append folded in, and -- with the weights sharded over GPUs -- the exchange of its
// output row folded into its epilogue. The reference reaches this arithmetic through its generic
// handlers and its fused-attention recognizer (src/metaljax/sdpa.py), which are outside the
// quantized-matmul path; this kernel exists because a decode step is a chain of launches between
// the weight streams, and at a few rows every launch that is not a weight stream is pure latency.
//
// One CTA per (batch row, key/value head, slice of the context): the query heads that share the
// key/value head (grouped-query attention) are rotated once and kept in shared memory; the
// slice is walked in chunks of 128 positions by 512 threads (256 for eight query heads per
// key/value head): scores by four (two) threads per position, each over an interleaved quarter
// (half) of the head dimension, the softmax statistics per chunk, the value sum
// thread-per-(8 dimensions, position subgroup). Every slice writes
// (max, sum, weighted values) to scratch memory the caller provides; the last CTA of a
// (row, head) to finish combines the slices and writes the row. The slice that contains the
// decode position appends the rotated key and the value to the cache; that position is always
// taken from shared memory, never read back.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>

#include "../../include/qmm_decode.h"
#include "qmm_internal.h"

namespace qmm {
namespace {

constexpr int kChunk = 128;                      // positions per chunk

struct AttnParams {
  const __nv_bfloat16* qkv;      // [batch, (heads + 2 kv_heads) * HD]: q heads | k heads | v heads
  __nv_bfloat16* k_cache;        // [batch, kv_heads, ctx, HD]
  __nv_bfloat16* v_cache;
  __nv_bfloat16* out;            // [batch, heads * HD], or NULL
  float* part;                   // scratch: [batch, kv_heads, splits, REP, HD + 4]
  uint32_t* counters;            // scratch: [batch * kv_heads], zero between calls
  int heads, kv_heads, splits;
  int64_t ctx, pos;
  float theta;
  // exchange (push_world == 0: none): the row also goes to every rank's gather slot
  int push_world, push_site;
  uint8_t* push_dst[8];          // every rank's slot + this rank's column block (stamped units: 4 bytes per value)
  int64_t push_row_bytes;        // bytes between batch rows of the gathered matrix
  const uint32_t* epoch;
#if QMM_STEP_TRACING
  unsigned long long* trace;
#endif
};

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(u[i] << 16);
    f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
  }
}

// Largest / sum over the CTA's threads of REP values at once (all threads get the results).
template <int REP, int WARPS, bool MAX>
__device__ __forceinline__ void block_reduce(float (&v)[REP], float (*scratch)[WARPS]) {
#pragma unroll
  for (int h = 0; h < REP; ++h)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, v[h], o);
      v[h] = MAX ? fmaxf(v[h], other) : v[h] + other;
    }
  __syncthreads();
  if ((threadIdx.x & 31) == 0)
#pragma unroll
    for (int h = 0; h < REP; ++h) scratch[h][threadIdx.x >> 5] = v[h];
  __syncthreads();
#pragma unroll
  for (int h = 0; h < REP; ++h) {
    float r = scratch[h][0];
#pragma unroll
    for (int w = 1; w < WARPS; ++w) r = MAX ? fmaxf(r, scratch[h][w]) : r + scratch[h][w];
    v[h] = r;
  }
}

template <int HD, int REP>
__global__ void __launch_bounds__(REP <= 4 ? 512 : 256)
decode_attention_kernel(const AttnParams p) {
  constexpr int kAttnThreads = REP <= 4 ? 512 : 256;
  constexpr int kWarps = kAttnThreads / 32;
  constexpr int kTPP = kAttnThreads / kChunk;       // threads per position in the score phase
#if QMM_STEP_TRACING
  unsigned long long* const trace = p.trace;
#else
  unsigned long long* const trace = nullptr;
  (void)trace;
#endif
  QMM_TRACE(trace, 0);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  constexpr int kPieces = HD / 8;                   // 16-byte pieces per row
  constexpr int kSubs = kAttnThreads / kPieces;     // position subgroups of the value sum
  constexpr int kMine = kPieces / kTPP;             // key pieces per thread in the score phase
  constexpr int kVals = kChunk / kSubs;             // value rows per thread and chunk
  constexpr int kStat = HD + 4;                     // (max, sum) after the values; rows stay 16-byte aligned
  __shared__ __align__(16) float q_s[REP][HD];      // rotated queries, scaled by 1/sqrt(HD)
  __shared__ __align__(16) float knew[HD], vnew[HD];
  __shared__ __align__(16) float prob[REP][kChunk];
  __shared__ __align__(16) float accs[kWarps][REP][HD];
  __shared__ float red4[REP][kWarps];
  __shared__ float wsplit[REP][64];                 // combine: the weight of every slice
  __shared__ float denom[REP];
  __shared__ int is_last;

  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x;
  const int total_heads = p.heads + 2 * p.kv_heads;
  const __nv_bfloat16* row = p.qkv + static_cast<int64_t>(b) * total_heads * HD;
  const int64_t len = p.pos + 1;                                   // positions 0 .. pos
  const int64_t per = (len + p.splits - 1) / p.splits;
  const int64_t lo = split * per, hi = (lo + per < len) ? lo + per : len;
  __nv_bfloat16* kc = p.k_cache + (static_cast<int64_t>(b) * p.kv_heads + kvh) * p.ctx * HD;
  __nv_bfloat16* vc = p.v_cache + (static_cast<int64_t>(b) * p.kv_heads + kvh) * p.ctx * HD;

  // The first chunk's key and value rows are requested before this kernel waits for the one
  // that writes the query row: the cache holds earlier positions only (the decode position's
  // own row is never read back), so the trip to memory runs under the predecessor's tail.
  const int piece = tid % kPieces, sub = tid / kPieces;
  const int spos = tid / kTPP, part = tid % kTPP;    // score phase: position within the chunk, share of its row
  uint4 kr[kMine], vr[kVals];
  auto request_v = [&](int64_t c0) {
    const int chunk_len = static_cast<int>((hi - c0 < kChunk) ? hi - c0 : kChunk);
#pragma unroll
    for (int u = 0; u < kVals; ++u) {
      const int i = sub + u * kSubs;
      vr[u] = make_uint4(0u, 0u, 0u, 0u);
      if (i < chunk_len && c0 + i != p.pos) vr[u] = __ldg(reinterpret_cast<const uint4*>(vc + (c0 + i) * HD) + piece);
    }
  };
  auto request_k = [&](int64_t c0) {
    const int64_t pp = c0 + spos;
#pragma unroll
    for (int u = 0; u < kMine; ++u) {
      kr[u] = make_uint4(0u, 0u, 0u, 0u);
      if (pp < hi && pp != p.pos) kr[u] = __ldg(reinterpret_cast<const uint4*>(kc + pp * HD) + u * kTPP + part);
    }
  };
  if (lo < hi) {
    request_v(lo);
    request_k(lo);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  QMM_TRACE(trace, 1);

  // ---- rotary embedding of this head group's queries and key (rotate-half pairing), the value ----
  constexpr int kHalf = HD / 2;
  const float inv_sqrt = rsqrtf(static_cast<float>(HD));
  for (int i = tid; i < (REP + 1) * kHalf; i += kAttnThreads) {
    const int h = i / kHalf, j = i - h * kHalf;
    const __nv_bfloat16* src = h < REP ? row + (kvh * REP + h) * HD : row + (p.heads + kvh) * HD;
    const float a = __bfloat162float(src[j]), c = __bfloat162float(src[j + kHalf]);
    float sn, cs;
    const float freq = exp2f(-2.0f * static_cast<float>(j) / static_cast<float>(HD) * log2f(p.theta));
    sincosf(static_cast<float>(p.pos) * freq, &sn, &cs);
    const float rlo = bf16_round(a * cs - c * sn), rhi = bf16_round(c * cs + a * sn);
    if (h < REP) {
      q_s[h][j] = rlo * inv_sqrt;
      q_s[h][j + kHalf] = rhi * inv_sqrt;
    } else {
      knew[j] = rlo;
      knew[j + kHalf] = rhi;
    }
  }
  for (int i = tid; i < HD; i += kAttnThreads) vnew[i] = __bfloat162float(row[(p.heads + p.kv_heads + kvh) * HD + i]);
  __syncthreads();
  if (p.pos >= lo && p.pos < hi) {                 // this slice owns the decode position: append
    for (int i = tid; i < HD; i += kAttnThreads) {
      kc[p.pos * HD + i] = __float2bfloat16_rn(knew[i]);
      vc[p.pos * HD + i] = __float2bfloat16_rn(vnew[i]);
    }
  }

  QMM_TRACE(trace, 2);               // queries rotated
  // ---- the slice, in chunks of 128 positions ----
  float m_run[REP], l_run[REP], acc[REP][8];
#pragma unroll
  for (int h = 0; h < REP; ++h) {
    m_run[h] = -INFINITY;
    l_run[h] = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[h][e] = 0.0f;
  }
  for (int64_t c0 = lo; c0 < hi; c0 += kChunk) {
    // scores: kTPP threads <-> position. This thread's share of its key row and its value rows of
    // the chunk are already on their way (the first chunk's since before the wait, a later one's
    // since the registers that hold them were last read)
    const int64_t pp = c0 + spos;
    const int chunk_len = static_cast<int>((hi - c0 < kChunk) ? hi - c0 : kChunk);
    float s[REP];
#pragma unroll
    for (int h = 0; h < REP; ++h) s[h] = 0.0f;
    if (pp < hi) {
#pragma unroll
      for (int u = 0; u < kMine; ++u) {
        const int d8 = u * kTPP + part;
        float kf[8];
        if (pp == p.pos) {
#pragma unroll
          for (int e = 0; e < 8; ++e) kf[e] = knew[d8 * 8 + e];
        } else {
          unpack8(kr[u], kf);
        }
#pragma unroll
        for (int h = 0; h < REP; ++h) {
          const float4 q0 = *reinterpret_cast<const float4*>(&q_s[h][d8 * 8]);
          const float4 q1 = *reinterpret_cast<const float4*>(&q_s[h][d8 * 8 + 4]);
          float sa = q0.x * kf[0], sb = q0.y * kf[1];
          sa = fmaf(q0.z, kf[2], sa); sb = fmaf(q0.w, kf[3], sb);
          sa = fmaf(q1.x, kf[4], sa); sb = fmaf(q1.y, kf[5], sb);
          sa = fmaf(q1.z, kf[6], sa); sb = fmaf(q1.w, kf[7], sb);
          s[h] += sa + sb;
        }
      }
    }
    // the key registers are free: the next chunk's keys travel under the rest of this one
    if (c0 + kChunk < hi) request_k(c0 + kChunk);
    // the position's kTPP shares (adjacent lanes)
#pragma unroll
    for (int h = 0; h < REP; ++h)
#pragma unroll
      for (int o = 1; o < kTPP; o <<= 1) s[h] += __shfl_xor_sync(0xffffffffu, s[h], o);
    if (pp >= hi) {
#pragma unroll
      for (int h = 0; h < REP; ++h) s[h] = -INFINITY;
    }
    // softmax statistics of the chunk, running rescale
    float scale_old[REP], cmax[REP], csum[REP];
#pragma unroll
    for (int h = 0; h < REP; ++h) cmax[h] = s[h];
    block_reduce<REP, kWarps, true>(cmax, red4);
#pragma unroll
    for (int h = 0; h < REP; ++h) {
      const float m_new = fmaxf(m_run[h], cmax[h]);
      const float pr = (pp < hi) ? __expf(s[h] - m_new) : 0.0f;
      csum[h] = part == 0 ? pr : 0.0f;              // one of the position's threads counts it
      if (part == 0) prob[h][spos] = pr;
      scale_old[h] = (m_run[h] == -INFINITY) ? 0.0f : __expf(m_run[h] - m_new);
      m_run[h] = m_new;
    }
    block_reduce<REP, kWarps, false>(csum, red4);     // (its barriers also make prob complete)
#pragma unroll
    for (int h = 0; h < REP; ++h) l_run[h] = l_run[h] * scale_old[h] + csum[h];
    // weighted values: thread <-> (8 dimensions, position subgroup)
#pragma unroll
    for (int h = 0; h < REP; ++h)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[h][e] *= scale_old[h];
#pragma unroll
    for (int u = 0; u < kVals; ++u) {
      const int i = sub + u * kSubs;
      if (i < chunk_len) {
        float vf[8];
        if (c0 + i == p.pos) {
#pragma unroll
          for (int e = 0; e < 8; ++e) vf[e] = vnew[piece * 8 + e];
        } else {
          unpack8(vr[u], vf);
        }
#pragma unroll
        for (int h = 0; h < REP; ++h) {
          const float pr = prob[h][i];
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[h][e] = fmaf(pr, vf[e], acc[h][e]);
        }
      }
    }
    if (c0 + kChunk < hi) request_v(c0 + kChunk);  // ... and its values under its score phase
    __syncthreads();                               // prob may be overwritten
  }

  QMM_TRACE(trace, 3);               // the slice is done
  // ---- this slice's (max, sum, weighted values) to scratch ----
  // the subgroups that share a warp first (lanes piece, piece + kPieces, ...), then the warps
#pragma unroll
  for (int h = 0; h < REP; ++h)
#pragma unroll
    for (int e = 0; e < 8; ++e)
#pragma unroll
      for (int o = kPieces; o < 32; o <<= 1) acc[h][e] += __shfl_xor_sync(0xffffffffu, acc[h][e], o);
  if ((tid & 31) < kPieces) {
#pragma unroll
    for (int h = 0; h < REP; ++h)
#pragma unroll
      for (int e = 0; e < 8; ++e) accs[tid >> 5][h][piece * 8 + e] = acc[h][e];
  }
  __syncthreads();
  float* mine = p.part + ((static_cast<int64_t>(b) * p.kv_heads + kvh) * p.splits + split) * REP * kStat;
  for (int i = tid; i < REP * HD; i += kAttnThreads) {
    const int h = i / HD, d = i - h * HD;
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) v += accs[w][h][d];
    mine[h * kStat + d] = v;
  }
  if (tid < REP) {
    mine[tid * kStat + HD] = m_run[tid];
    mine[tid * kStat + HD + 1] = l_run[tid];
  }
  __threadfence();
  __syncthreads();
  uint32_t* counter = p.counters + b * p.kv_heads + kvh;
  if (tid == 0) {
    const bool last = atomicAdd(counter, 1u) == static_cast<uint32_t>(p.splits - 1);
    if (last) *counter = 0;
    is_last = last;
  }
  __syncthreads();
  QMM_TRACE(trace, 4);               // partials published
  if (!is_last) return;
  __threadfence();

  // ---- the last slice of this (row, head) to finish combines them all ----
  const float* all = p.part + (static_cast<int64_t>(b) * p.kv_heads + kvh) * p.splits * REP * kStat;
  {
    // per head: one warp takes the slices' maxima and sums (lane <-> slice), leaves every slice's
    // weight exp(max_s - max) and the common denominator in shared memory
    const int warp = tid >> 5, lane = tid & 31;
    for (int h = warp; h < REP; h += kAttnThreads / 32) {
      float ms[2], ls[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int sp = lane + 32 * u;
        ms[u] = sp < p.splits ? __ldcg(all + (sp * REP + h) * kStat + HD) : -INFINITY;
        ls[u] = sp < p.splits ? __ldcg(all + (sp * REP + h) * kStat + HD + 1) : 0.0f;
      }
      float mx = fmaxf(ms[0], ms[1]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float den = 0.0f;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const float w = (ms[u] == -INFINITY) ? 0.0f : __expf(ms[u] - mx);
        wsplit[h][lane + 32 * u] = w;
        den = fmaf(w, ls[u], den);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
      if (lane == 0) denom[h] = den;
    }
  }
  __syncthreads();
  const uint32_t stamp = p.push_world > 0
      ? (*reinterpret_cast<const volatile uint32_t*>(p.epoch) << 10) | static_cast<uint32_t>(p.push_site + 1) : 0u;
  for (int i = tid; i < REP * HD / 4; i += kAttnThreads) {        // thread <-> 4 consecutive dimensions
    const int h = i / (HD / 4), d0 = (i - h * (HD / 4)) * 4;
    float4 num = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 8
    for (int sp = 0; sp < p.splits; ++sp) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(all + (sp * REP + h) * kStat + d0));
      const float w = wsplit[h][sp];
      num.x = fmaf(w, v.x, num.x); num.y = fmaf(w, v.y, num.y);
      num.z = fmaf(w, v.z, num.z); num.w = fmaf(w, v.w, num.w);
    }
    const float inv = 1.0f / denom[h];
    const __nv_bfloat162 v0 = __floats2bfloat162_rn(num.x * inv, num.y * inv);
    const __nv_bfloat162 v1 = __floats2bfloat162_rn(num.z * inv, num.w * inv);
    const uint2 o = make_uint2(*reinterpret_cast<const uint32_t*>(&v0), *reinterpret_cast<const uint32_t*>(&v1));
    const int64_t col = static_cast<int64_t>(kvh * REP + h) * HD + d0;
    if (p.out) *reinterpret_cast<uint2*>(p.out + static_cast<int64_t>(b) * p.heads * HD + col) = o;
    if (p.push_world > 0) {
      // to every rank as stamped units {pair, stamp}: data and arrival in one store
      const uint4 unit = make_uint4(o.x, stamp, o.y, stamp);
      for (int r = 0; r < p.push_world; ++r)
        *reinterpret_cast<uint4*>(p.push_dst[r] + b * p.push_row_bytes + col * 4) = unit;
    }
  }
  QMM_TRACE(trace, 6);               // (the combining CTA only)
}

template <int HD, int REP>
int launch_attention(const AttnParams& p, int64_t batch, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(p.splits), static_cast<unsigned>(p.kv_heads), static_cast<unsigned>(batch));
  cfg.blockDim = dim3(REP <= 4 ? 512 : 256);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
#if QMM_STEP_TRACING
  AttnParams traced = p;
  traced.trace = next_trace_block(8);
  cudaError_t e = cudaLaunchKernelEx(&cfg, decode_attention_kernel<HD, REP>, traced);
#else
  cudaError_t e = cudaLaunchKernelEx(&cfg, decode_attention_kernel<HD, REP>, p);
#endif
  if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "decode_attention_kernel launch: %s", cudaGetErrorString(e));
  count_launch();
  return check_launch("decode_attention_kernel");
}

template <int HD>
int launch_rep(const AttnParams& p, int rep, int64_t batch, cudaStream_t stream) {
  switch (rep) {
    case 1: return launch_attention<HD, 1>(p, batch, stream);
    case 2: return launch_attention<HD, 2>(p, batch, stream);
    case 4: return launch_attention<HD, 4>(p, batch, stream);
    case 8: return launch_attention<HD, 8>(p, batch, stream);
  }
  return fail(QMM_ERR_UNSUPPORTED, "decode_attention: %d query heads per key/value head (1, 2, 4 or 8)", rep);
}


// ---------------------------------------------------------------------------------------------
// The same attention for longer slices (several sequences at once: batch x key/value heads fill
// the machine, so a CTA walks hundreds of positions): bandwidth instead of latency. Key and
// value rows stream through a three-stage ring of 64-position chunks (`cp.async`, 16-byte pieces,
// XOR-swizzled so that `ldmatrix` reads are conflict free); scores and the value sum run on
// `mma.sync.m16n8k16` with the query heads of the group as the A rows (at most 8 of 16 used --
// the tensor work is tiny, the point is that a chunk costs a few dozen instructions per warp
// instead of thousands of FMAs). Four warps take 16 positions of a chunk each and keep their own
// running (max, sum, weighted values); they are merged once at the end, together with the decode
// position's own term, which comes from shared memory and never from the cache. Slices publish
// and combine exactly as in the kernel above.
constexpr int kMmaChunk = 64, kMmaThreads = 128, kMmaStages = 3;

__device__ __forceinline__ uint32_t attn_smem_u32(const void* q) { return static_cast<uint32_t>(__cvta_generic_to_shared(q)); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;                     // 0: the 16 bytes are written as zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void ldsm4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
// d += a (16 x 16, rows 8..15 zero) * b (16 x 8)
__device__ __forceinline__ void mma_rows8(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  const uint32_t zero = 0u;
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(zero), "r"(a2), "r"(zero), "r"(b0), "r"(b1));
}

template <int HD, int REP>
__global__ void __launch_bounds__(kMmaThreads)
decode_attention_mma_kernel(const AttnParams p) {
  static_assert(REP <= 8, "the query heads of a group are the first eight A rows");
  constexpr int kRowBytes = HD * 2, kPieces = HD / 8;
  constexpr int kTensorBytes = kMmaChunk * kRowBytes;           // one chunk of keys (or of values)
  constexpr int kStageBytes = 2 * kTensorBytes;
  constexpr int kStat = HD + 4;
  constexpr int kWarps = kMmaThreads / 32;
  extern __shared__ __align__(128) uint8_t attn_smem[];
  uint8_t* stages = attn_smem;                                       // [kMmaStages][K chunk | V chunk]
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(attn_smem + kMmaStages * kStageBytes);   // [8][HD], rotated
  float* knew = reinterpret_cast<float*>(q_s + 8 * HD);              // [HD] the decode position's key (rotated) ...
  float* vnew = knew + HD;                                           // ... and value
  float* s_self = vnew + HD;                                         // [8]
  float* pm = s_self + 8;                                            // [kWarps][8] the warps' maxima, sums
  float* pl = pm + kWarps * 8;
  float* wsplit = pl + kWarps * 8;                                   // [REP][64] (combine)
  float* denom = wsplit + REP * 64;                                  // [REP]
  float* pO = reinterpret_cast<float*>(stages);                      // [kWarps][REP][HD]: reuses the ring after the walk
  __shared__ int is_last;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int total_heads = p.heads + 2 * p.kv_heads;
  const __nv_bfloat16* row = p.qkv + static_cast<int64_t>(b) * total_heads * HD;
  const int64_t len = p.pos + 1;
  const int64_t per = (len + p.splits - 1) / p.splits;
  const int64_t lo = split * per, hi = (lo + per < len) ? lo + per : len;
  __nv_bfloat16* kc = p.k_cache + (static_cast<int64_t>(b) * p.kv_heads + kvh) * p.ctx * HD;
  __nv_bfloat16* vc = p.v_cache + (static_cast<int64_t>(b) * p.kv_heads + kvh) * p.ctx * HD;
  const int nchunks = lo < hi ? static_cast<int>((hi - lo + kMmaChunk - 1) / kMmaChunk) : 0;

  // chunk `ci` into its ring slot: every thread copies its share of the 16-byte pieces; rows past
  // the slice and the decode position's own row (not in the cache yet) arrive as zeros
  auto load_chunk = [&](int ci) {
    if (ci < nchunks) {
      uint8_t* st = stages + (ci % kMmaStages) * kStageBytes;
      const int64_t pos0 = lo + static_cast<int64_t>(ci) * kMmaChunk;
#pragma unroll
      for (int i = 0; i < kMmaChunk * kPieces / kMmaThreads; ++i) {
        const int q = tid + kMmaThreads * i, r = q / kPieces, c = q % kPieces;
        const int64_t pos = pos0 + r;
        const bool valid = pos < hi && pos != p.pos;
        const int64_t from = (valid ? pos : lo) * HD + c * 8;
        const uint32_t off = r * kRowBytes + ((c ^ (r & 7)) << 4);
        cp_async16(attn_smem_u32(st + off), kc + from, valid);
        cp_async16(attn_smem_u32(st + kTensorBytes + off), vc + from, valid);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // the cache holds earlier positions only: the first chunks travel under the predecessor's tail
  load_chunk(0);
  load_chunk(1);
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- rotary embedding of the group's queries and of the key; the value ----
  constexpr int kHalf = HD / 2;
  const float inv_sqrt = rsqrtf(static_cast<float>(HD));
  for (int i = tid; i < (REP + 1) * kHalf; i += kMmaThreads) {
    const int h = i / kHalf, j = i - h * kHalf;
    const __nv_bfloat16* src = h < REP ? row + (kvh * REP + h) * HD : row + (p.heads + kvh) * HD;
    const float a = __bfloat162float(src[j]), c = __bfloat162float(src[j + kHalf]);
    float sn, cs;
    const float freq = exp2f(-2.0f * static_cast<float>(j) / static_cast<float>(HD) * log2f(p.theta));
    sincosf(static_cast<float>(p.pos) * freq, &sn, &cs);
    const __nv_bfloat16 rlo = __float2bfloat16_rn(a * cs - c * sn), rhi = __float2bfloat16_rn(c * cs + a * sn);
    if (h < REP) {
      q_s[h * HD + j] = rlo;
      q_s[h * HD + j + kHalf] = rhi;
    } else {
      knew[j] = __bfloat162float(rlo);
      knew[j + kHalf] = __bfloat162float(rhi);
    }
  }
  for (int i = tid; i < (8 - REP) * HD; i += kMmaThreads) q_s[REP * HD + i] = __float2bfloat16_rn(0.0f);
  for (int i = tid; i < HD; i += kMmaThreads) vnew[i] = __bfloat162float(row[(p.heads + p.kv_heads + kvh) * HD + i]);
  __syncthreads();
  const bool owns = p.pos >= lo && p.pos < hi;
  if (owns) {
    for (int i = tid; i < HD; i += kMmaThreads) {
      kc[p.pos * HD + i] = __float2bfloat16_rn(knew[i]);
      vc[p.pos * HD + i] = __float2bfloat16_rn(vnew[i]);
    }
    // the decode position's own score per head (one warp per head, heads w, w + 4)
    for (int h = warp; h < REP; h += kWarps) {
      float acc = 0.0f;
      for (int d = lane; d < HD; d += 32) acc = fmaf(__bfloat162float(q_s[h * HD + d]), knew[d], acc);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) s_self[h] = acc * inv_sqrt;
    }
  }
  // this lane's query fragments: A rows g (a0: dims 2t, 2t+1 of a 16-wide step; a2: the same + 8)
  uint32_t qa[HD / 16][2];
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
    qa[ks][0] = *reinterpret_cast<const uint32_t*>(q_s + g * HD + ks * 16 + t * 2);
    qa[ks][1] = *reinterpret_cast<const uint32_t*>(q_s + g * HD + ks * 16 + 8 + t * 2);
  }

  float m_run = -INFINITY, l_run = 0.0f;            // of query head g (the four lanes of a row agree)
  float o[HD / 8][4];
#pragma unroll
  for (int nt = 0; nt < HD / 8; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nt][e] = 0.0f;
  const int lm = lane >> 3, lr = lane & 7;          // ldmatrix: this lane addresses row lr of matrix lm

  for (int ci = 0; ci < nchunks; ++ci) {
    asm volatile("cp.async.wait_group 1;" ::: "memory");      // chunk ci has landed (this thread's pieces)
    __syncthreads();                                           // everybody's pieces; and chunk ci - 1 is consumed
    load_chunk(ci + 2);                                        // into the slot chunk ci - 1 used
    const uint32_t ks_base = attn_smem_u32(stages + (ci % kMmaStages) * kStageBytes);
    const uint32_t vs_base = ks_base + kTensorBytes;
    // scores of this warp's 16 positions: two 8-position tiles
    float sc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
    {
      const int r = warp * 16 + (lm >> 1) * 8 + lr;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        uint32_t kb[4];
        ldsm4(kb, ks_base + r * kRowBytes + ((((ks * 2 + (lm & 1)) ^ (r & 7))) << 4));
        mma_rows8(sc[0], qa[ks][0], qa[ks][1], kb[0], kb[1]);
        mma_rows8(sc[1], qa[ks][0], qa[ks][1], kb[2], kb[3]);
      }
    }
    const int64_t pos0 = lo + static_cast<int64_t>(ci) * kMmaChunk + warp * 16 + t * 2;
    float cmax = -INFINITY;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int64_t pos = pos0 + j * 8 + e;
        sc[j][e] = (pos < hi && pos != p.pos) ? sc[j][e] * inv_sqrt : -INFINITY;
        cmax = fmaxf(cmax, sc[j][e]);
      }
    cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, 1));
    cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, 2));
    const float m_new = fmaxf(m_run, cmax);
    const float alpha = (m_run == -INFINITY) ? 0.0f : __expf(m_run - m_new);
    float pr[2][2], csum = 0.0f;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        pr[j][e] = (sc[j][e] == -INFINITY) ? 0.0f : __expf(sc[j][e] - m_new);
        csum += pr[j][e];
      }
    csum += __shfl_xor_sync(0xffffffffu, csum, 1);
    csum += __shfl_xor_sync(0xffffffffu, csum, 2);
    l_run = l_run * alpha + csum;
    m_run = m_new;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
      o[nt][0] *= alpha;
      o[nt][1] *= alpha;
    }
    // weighted values: the probabilities are the A rows now (k = this warp's 16 positions)
    const __nv_bfloat162 p0 = __floats2bfloat162_rn(pr[0][0], pr[0][1]), p1 = __floats2bfloat162_rn(pr[1][0], pr[1][1]);
    const uint32_t pa0 = *reinterpret_cast<const uint32_t*>(&p0), pa2 = *reinterpret_cast<const uint32_t*>(&p1);
    {
      const int r = warp * 16 + (lm & 1) * 8 + lr;
#pragma unroll
      for (int dp = 0; dp < HD / 16; ++dp) {
        uint32_t vb[4];
        ldsm4_trans(vb, vs_base + r * kRowBytes + ((((dp * 2 + (lm >> 1)) ^ (r & 7))) << 4));
        mma_rows8(o[2 * dp], pa0, pa2, vb[0], vb[1]);
        mma_rows8(o[2 * dp + 1], pa0, pa2, vb[2], vb[3]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();                                   // the ring is free: it holds the warps' results from here on

  // ---- the four warps' results and the decode position's own term into one (max, sum, values) ----
  if (g < REP) {
    if (t == 0) {
      pm[warp * 8 + g] = m_run;
      pl[warp * 8 + g] = l_run;
    }
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt)
      *reinterpret_cast<float2*>(pO + (warp * REP + g) * HD + nt * 8 + t * 2) = make_float2(o[nt][0], o[nt][1]);
  }
  __syncthreads();
  float* mine = p.part + ((static_cast<int64_t>(b) * p.kv_heads + kvh) * p.splits + split) * REP * kStat;
  for (int i = tid; i < REP * HD; i += kMmaThreads) {
    const int h = i / HD, d = i - h * HD;
    float mx = owns ? s_self[h] : -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) mx = fmaxf(mx, pm[w * 8 + h]);
    float num = 0.0f, den = 0.0f;
    if (mx != -INFINITY) {
      if (owns) {
        const float ws = __expf(s_self[h] - mx);
        num = ws * vnew[d];
        den = ws;
      }
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const float mw = pm[w * 8 + h];
        const float ww = (mw == -INFINITY) ? 0.0f : __expf(mw - mx);
        num = fmaf(ww, pO[(w * REP + h) * HD + d], num);
        den = fmaf(ww, pl[w * 8 + h], den);
      }
    }
    mine[h * kStat + d] = num;
    if (d == 0) {
      mine[h * kStat + HD] = mx;
      mine[h * kStat + HD + 1] = den;
    }
  }
  __threadfence();
  __syncthreads();
  uint32_t* counter = p.counters + b * p.kv_heads + kvh;
  if (tid == 0) {
    const bool last = atomicAdd(counter, 1u) == static_cast<uint32_t>(p.splits - 1);
    if (last) *counter = 0;
    is_last = last;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();

  // ---- the last slice of this (row, head) to finish combines them all ----
  const float* all = p.part + (static_cast<int64_t>(b) * p.kv_heads + kvh) * p.splits * REP * kStat;
  for (int h = warp; h < REP; h += kWarps) {
    float ms[2], ls[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int sp = lane + 32 * u;
      ms[u] = sp < p.splits ? __ldcg(all + (sp * REP + h) * kStat + HD) : -INFINITY;
      ls[u] = sp < p.splits ? __ldcg(all + (sp * REP + h) * kStat + HD + 1) : 0.0f;
    }
    float mx = fmaxf(ms[0], ms[1]);
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o2));
    float den = 0.0f;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const float w = (ms[u] == -INFINITY) ? 0.0f : __expf(ms[u] - mx);
      wsplit[h * 64 + lane + 32 * u] = w;
      den = fmaf(w, ls[u], den);
    }
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o2);
    if (lane == 0) denom[h] = den;
  }
  __syncthreads();
  const uint32_t stamp = p.push_world > 0
      ? (*reinterpret_cast<const volatile uint32_t*>(p.epoch) << 10) | static_cast<uint32_t>(p.push_site + 1) : 0u;
  for (int i = tid; i < REP * HD / 4; i += kMmaThreads) {
    const int h = i / (HD / 4), d0 = (i - h * (HD / 4)) * 4;
    float4 num = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int sp = 0; sp < p.splits; ++sp) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(all + (sp * REP + h) * kStat + d0));
      const float w = wsplit[h * 64 + sp];
      num.x = fmaf(w, v.x, num.x); num.y = fmaf(w, v.y, num.y);
      num.z = fmaf(w, v.z, num.z); num.w = fmaf(w, v.w, num.w);
    }
    const float inv = 1.0f / denom[h];
    const __nv_bfloat162 v0 = __floats2bfloat162_rn(num.x * inv, num.y * inv);
    const __nv_bfloat162 v1 = __floats2bfloat162_rn(num.z * inv, num.w * inv);
    const uint2 ov = make_uint2(*reinterpret_cast<const uint32_t*>(&v0), *reinterpret_cast<const uint32_t*>(&v1));
    const int64_t col = static_cast<int64_t>(kvh * REP + h) * HD + d0;
    if (p.out) *reinterpret_cast<uint2*>(p.out + static_cast<int64_t>(b) * p.heads * HD + col) = ov;
    if (p.push_world > 0) {
      const uint4 unit = make_uint4(ov.x, stamp, ov.y, stamp);
      for (int r = 0; r < p.push_world; ++r)
        *reinterpret_cast<uint4*>(p.push_dst[r] + b * p.push_row_bytes + col * 4) = unit;
    }
  }
}

template <int HD, int REP>
int launch_attention_mma(const AttnParams& p, int64_t batch, cudaStream_t stream) {
  constexpr size_t smem = kMmaStages * 2 * kMmaChunk * HD * 2 + 8 * HD * 2 + 2 * HD * 4 + (8 + 2 * 4 * 8 + REP * 64 + REP) * 4 + 64;
  static bool configured[kMaxDevices] = {};
  const int dev = current_device();
  if (dev < 0) return QMM_ERR_DEVICE;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(decode_attention_mma_kernel<HD, REP>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(p.splits), static_cast<unsigned>(p.kv_heads), static_cast<unsigned>(batch));
  cfg.blockDim = dim3(kMmaThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, decode_attention_mma_kernel<HD, REP>, p);
  if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "decode_attention_mma_kernel launch: %s", cudaGetErrorString(e));
  count_launch();
  return check_launch("decode_attention_mma_kernel");
}

template <int HD>
int launch_rep_mma(const AttnParams& p, int rep, int64_t batch, cudaStream_t stream) {
  switch (rep) {
    case 1: return launch_attention_mma<HD, 1>(p, batch, stream);
    case 2: return launch_attention_mma<HD, 2>(p, batch, stream);
    case 4: return launch_attention_mma<HD, 4>(p, batch, stream);
    case 8: return launch_attention_mma<HD, 8>(p, batch, stream);
  }
  return fail(QMM_ERR_UNSUPPORTED, "decode_attention: %d query heads per key/value head (1, 2, 4 or 8)", rep);
}

}  // namespace
}  // namespace qmm

using namespace qmm;

extern "C" int64_t qmm_decode_attention_scratch_bytes(int64_t batch, int heads, int kv_heads, int head_dim, int64_t ctx) {
  if (batch < 0 || heads <= 0 || kv_heads <= 0 || head_dim <= 0 || ctx <= 0) return 0;
  const int64_t splits = 64;                                     // the most a call ever uses
  return batch * kv_heads * splits * (heads / kv_heads) * (head_dim + 4) * 4 + (batch * kv_heads + 1) * 4 + 256;
}

extern "C" int qmm_decode_attention(const void* qkv, void* k_cache, void* v_cache, void* out, void* scratch,
                                    int64_t scratch_bytes, int64_t batch, int heads, int kv_heads, int head_dim,
                                    int64_t ctx, int64_t pos, float theta, int push_slot, int push_site,
                                    const qmm_exchange* ex, void* stream) {
  if (!qkv || !k_cache || !v_cache || !scratch) return fail(QMM_ERR_NULL, "decode_attention: null pointer");
  if (batch < 0 || batch > 65535 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || kv_heads > 65535 || pos < 0 || pos >= ctx)
    return fail(QMM_ERR_SHAPE, "decode_attention: bad shape or position");
  if (head_dim != 64 && head_dim != 128) return fail(QMM_ERR_UNSUPPORTED, "decode_attention: head_dim %d (64 or 128)", head_dim);
  if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
       reinterpret_cast<uintptr_t>(scratch)) & 15)
    return fail(QMM_ERR_LAYOUT, "decode_attention: pointers must be 16-byte aligned");
  if (scratch_bytes < qmm_decode_attention_scratch_bytes(batch, heads, kv_heads, head_dim, ctx))
    return fail(QMM_ERR_TOO_LARGE, "decode_attention: scratch of %lld bytes is too small", (long long)scratch_bytes);
  const bool pushes = push_slot >= 0;
  if (!out && !pushes) return fail(QMM_ERR_NULL, "decode_attention: no output");
  if (pushes && (!ex || ex->world < 1 || ex->world > 8 || !ex->peer_bufs || !ex->epoch))
    return fail(QMM_ERR_NULL, "decode_attention: an exchange is needed to push");
  if (batch == 0) return QMM_OK;
  AttnParams p = {};
  p.qkv = static_cast<const __nv_bfloat16*>(qkv);
  p.k_cache = static_cast<__nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<__nv_bfloat16*>(v_cache);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.heads = heads; p.kv_heads = kv_heads; p.ctx = ctx; p.pos = pos; p.theta = theta;
  // slices of the context: enough CTAs to give every SM one, at least 128 positions each
  const int64_t len = pos + 1;
  int64_t splits = (device_sm_count() + batch * kv_heads - 1) / (batch * kv_heads);
  if (splits > (len + 127) / 128) splits = (len + 127) / 128;
  if (splits > 64) splits = 64;
  if (splits < 1) splits = 1;
  // Slices of a few hundred positions and more (several sequences at once) take the streaming
  // kernel, two CTAs per SM; QMM_ATTN_KERNEL=simt / mma forces one.
  int64_t wide = 2 * device_sm_count() / (batch * kv_heads);      // (rounded down: one wave of CTAs)
  if (wide > (len + 255) / 256) wide = (len + 255) / 256;
  if (wide > 64) wide = 64;
  if (wide < 1) wide = 1;
  const char* force = getenv("QMM_ATTN_KERNEL");
  const bool mma = force ? force[0] == 'm' : (len + splits - 1) / splits >= 256;
  if (mma) splits = wide;
  p.splits = static_cast<int>(splits);
  const int rep = heads / kv_heads;
  const int64_t part_bytes = batch * kv_heads * 64 * rep * (head_dim + 4) * 4;
  p.part = static_cast<float*>(scratch);
  p.counters = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(scratch) + ((part_bytes + 255) & ~int64_t(255)));
  if (pushes) {
    if (push_site < 0 || push_site >= 1023) return fail(QMM_ERR_SHAPE, "decode_attention: exchange sites are 0..1022");
    const int64_t slice = static_cast<int64_t>(heads) * head_dim * 4;      // stamped units: 4 bytes per value
    if (batch * slice * ex->world > ex->slot_bytes) return fail(QMM_ERR_SHAPE, "decode_attention: the gathered rows do not fit a slot");
    p.push_world = ex->world; p.push_site = push_site;
    p.push_row_bytes = slice * ex->world;
    p.epoch = static_cast<const uint32_t*>(ex->epoch);
    for (int r = 0; r < ex->world; ++r) {
      if (!ex->peer_bufs[r]) return fail(QMM_ERR_NULL, "decode_attention: bad peer pointer");
      p.push_dst[r] = static_cast<uint8_t*>(ex->peer_bufs[r]) + static_cast<int64_t>(push_slot) * ex->slot_bytes + ex->rank * slice;
    }
  }
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (mma) return head_dim == 128 ? launch_rep_mma<128>(p, rep, batch, st) : launch_rep_mma<64>(p, rep, batch, st);
  return head_dim == 128 ? launch_rep<128>(p, rep, batch, st) : launch_rep<64>(p, rep, batch, st);
}
