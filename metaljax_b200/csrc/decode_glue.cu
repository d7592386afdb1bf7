// Element-wise glue of one decoder step around the fused quantized linears: residual add +
// RMS normalisation, rotary embedding + key/value cache append, and the SwiGLU gate. The
// reference reaches these through its generic op handlers (src/metaljax/ops/elementwise.py,
// src/metaljax/ops/reduce.py); here each is one memory-bound kernel so that a decode step is
// a short chain of launches between the weight streams. bf16 in and out, float32 arithmetic.
//
// Every kernel is launched with programmatic stream serialization, lets its successor start at
// once (`griddepcontrol.launch_dependents`), and touches memory only after
// `griddepcontrol.wait`, so the decode kernel that follows can request its weights while the
// glue kernel is still running.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "qmm_internal.h"
#include "../../include/qmm_decode.h"

namespace qmm {
namespace {

__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(u[i] << 16);
    f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint32_t u[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    u[i] = *reinterpret_cast<const uint32_t*>(&p);
  }
  return make_uint4(u[0], u[1], u[2], u[3]);
}

// h = x (+ residual); residual_out = h (optional); y = h * rsqrt(mean(h^2) + eps) * weight.
// One CTA per row; dim is a multiple of 8.
constexpr int kNormThreads = 256;
__global__ void __launch_bounds__(kNormThreads)
add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* residual_in,
                   const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* residual_out, int64_t dim, float eps) {   // residual_out may be residual_in
  pdl_enter();
  extern __shared__ uint4 row_cache[];               // the row as bf16, dim / 8 pieces, then 8 partial sums
  float* partial = reinterpret_cast<float*>(row_cache + dim / 8);
  const int64_t row = blockIdx.x;
  const int pieces = static_cast<int>(dim / 8);
  float ss = 0.0f;
  for (int p = threadIdx.x; p < pieces; p += kNormThreads) {
    uint4 v = *reinterpret_cast<const uint4*>(x + row * dim + p * 8);
    float f[8];
    unpack8(v, f);
    if (residual_in) {
      float r[8];
      unpack8(*reinterpret_cast<const uint4*>(residual_in + row * dim + p * 8), r);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] += r[i];
      v = pack8(f);
      unpack8(v, f);                                  // the sum as it is stored: bf16
    }
    if (residual_out) *reinterpret_cast<uint4*>(residual_out + row * dim + p * 8) = v;
    row_cache[p] = v;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(f[i], f[i], ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int i = 0; i < kNormThreads / 32; ++i) total += partial[i];
  const float inv = rsqrtf(total / static_cast<float>(dim) + eps);
  for (int p = threadIdx.x; p < pieces; p += kNormThreads) {
    float f[8], w[8];
    unpack8(row_cache[p], f);
    unpack8(*reinterpret_cast<const uint4*>(weight + p * 8), w);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = f[i] * inv * w[i];
    *reinterpret_cast<uint4*>(y + row * dim + p * 8) = pack8(f);
  }
}

// qkv[b] = [q heads | k heads | v heads], each head_dim wide. Rotates q and k (rotate-half
// pairing: element i with i + head_dim/2, angle pos * theta^(-2i/head_dim)), writes q to
// q_out[b, head, :] and k, v to the caches [b, kv_head, pos, :].
__global__ void rope_kv_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                               __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                               int heads, int kv_heads, int head_dim, int64_t ctx, int64_t pos, float theta) {
  pdl_enter();
  const int b = blockIdx.y;
  const int half = head_dim / 2;
  const int total_heads = heads + 2 * kv_heads;
  const int64_t row = static_cast<int64_t>(b) * total_heads * head_dim;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total_heads * half; i += gridDim.x * blockDim.x) {
    const int head = i / half, j = i % half;
    const float lo = __bfloat162float(qkv[row + head * head_dim + j]);
    const float hi = __bfloat162float(qkv[row + head * head_dim + j + half]);
    if (head < heads + kv_heads) {
      float s, c;
      // full-precision power: the angle is pos * freq, so a relative error of freq is multiplied
      // by positions of up to 10^5
      const float freq = exp2f(-2.0f * static_cast<float>(j) / static_cast<float>(head_dim) * log2f(theta));
      sincosf(static_cast<float>(pos) * freq, &s, &c);
      const float rlo = lo * c - hi * s, rhi = hi * c + lo * s;
      if (head < heads) {
        __nv_bfloat16* dst = q_out + (static_cast<int64_t>(b) * heads + head) * head_dim;
        dst[j] = __float2bfloat16_rn(rlo);
        dst[j + half] = __float2bfloat16_rn(rhi);
      } else {
        __nv_bfloat16* dst = k_cache + ((static_cast<int64_t>(b) * kv_heads + (head - heads)) * ctx + pos) * head_dim;
        dst[j] = __float2bfloat16_rn(rlo);
        dst[j + half] = __float2bfloat16_rn(rhi);
      }
    } else {
      __nv_bfloat16* dst = v_cache + ((static_cast<int64_t>(b) * kv_heads + (head - heads - kv_heads)) * ctx + pos) * head_dim;
      dst[j] = __float2bfloat16_rn(lo);
      dst[j + half] = __float2bfloat16_rn(hi);
    }
  }
}

// gate_up[r] = [gate | up], each `ffn` wide: out[r, i] = silu(gate[i]) * up[i].
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out,
                                int64_t rows, int64_t ffn) {
  pdl_enter();
  const int64_t pieces = ffn / 8;
  const int64_t total = rows * pieces;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / pieces, p = i % pieces;
    float g[8], u[8];
    unpack8(*reinterpret_cast<const uint4*>(gate_up + r * 2 * ffn + p * 8), g);
    unpack8(*reinterpret_cast<const uint4*>(gate_up + r * 2 * ffn + ffn + p * 8), u);
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] = g[k] / (1.0f + __expf(-g[k])) * u[k];
    *reinterpret_cast<uint4*>(out + r * ffn + p * 8) = pack8(g);
  }
}

// ---- one-shot all-gather over peer memory ------------------------------------------------
// Every rank copies its slice [rows, slice_bytes] into every rank's gather buffer (plain peer
// stores through NVLink; its own copy included) at column offset rank * slice_bytes of rows
// that are world * slice_bytes apart, then raises a flag word on every rank, then waits until
// all ranks' flags for this call have been raised on itself. The next kernel of the stream
// therefore finds the gathered [rows, world * slice_bytes] matrix complete. One kernel per
// rank, each on its own GPU; the waits are bounded (a second or so of SM clock) and report
// through the status word, after which later calls skip their waits.
//
// state (device memory of this rank, zero-initialised once): [slot] calls completed on that
// slot (slots 0..2), [4] CTAs finished in the current call, [8 + r] CTAs that finished copying
// to rank r in the current call.
constexpr int kAgThreads = 256;

struct AllGatherParams {
  const uint8_t* local;
  uint8_t* peer_buf[8];
  uint32_t* peer_flags[8];       // every rank's flag words: [slot][source rank], 3 x 8
  uint32_t* state;
  int* status;
  int64_t rows, slice_bytes, slot_bytes;
  long long spin_limit;          // SM clocks the wait for the peers may last
  int rank, world, slot;
};

__global__ void __launch_bounds__(kAgThreads) allgather_push_kernel(const AllGatherParams p) {
  pdl_enter();                                        // `local` is the previous kernel's output
  const int peer = blockIdx.x, part = blockIdx.y, parts = gridDim.y;
  const uint32_t seq = reinterpret_cast<volatile uint32_t*>(p.state)[p.slot] + 1;
  // copy this CTA's share of the slice to `peer`
  const int64_t chunks_per_row = p.slice_bytes / 16;
  const int64_t total = p.rows * chunks_per_row;
  const int64_t dst_row = static_cast<int64_t>(p.world) * p.slice_bytes;
  uint8_t* dst = p.peer_buf[peer] + static_cast<int64_t>(p.slot) * p.slot_bytes + static_cast<int64_t>(p.rank) * p.slice_bytes;
  for (int64_t i = static_cast<int64_t>(part) * kAgThreads + threadIdx.x; i < total;
       i += static_cast<int64_t>(parts) * kAgThreads) {
    const int64_t r = i / chunks_per_row, c = i % chunks_per_row;
    const uint4 v = *reinterpret_cast<const uint4*>(p.local + r * p.slice_bytes + c * 16);
    *reinterpret_cast<uint4*>(dst + r * dst_row + c * 16) = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    // the last CTA that finished copying to `peer` raises this rank's flag there
    if (atomicAdd(&p.state[8 + peer], 1u) == static_cast<unsigned>(parts - 1)) {
      p.state[8 + peer] = 0;
      __threadfence_system();
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.peer_flags[peer] + p.slot * 8 + p.rank), "r"(seq) : "memory");
    }
  }
  // CTA (0, 0): wait for every rank's flag of this call on this rank
  if (peer == 0 && part == 0 && threadIdx.x < p.world) {
    const uint32_t* flag = p.peer_flags[p.rank] + p.slot * 8 + threadIdx.x;
    if (*reinterpret_cast<volatile int*>(p.status) == 0) {
      const long long t0 = clock64();
      for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (static_cast<int32_t>(v - seq) >= 0) break;
        if (clock64() - t0 > p.spin_limit) {
          atomicCAS(p.status, 0, 100 + static_cast<int>(threadIdx.x));   // which rank never arrived
          break;
        }
      }
    }
  }
  __syncthreads();
  // the last CTA of the call publishes the call count of this slot and clears the counter
  if (threadIdx.x == 0) {
    const unsigned all = gridDim.x * gridDim.y;
    if (atomicAdd(&p.state[4], 1u) == all - 1) {
      p.state[4] = 0;
      reinterpret_cast<volatile uint32_t*>(p.state)[p.slot] = seq;
    }
  }
}

__global__ void step_begin_kernel(uint32_t* epoch) {
  pdl_enter();
  if (threadIdx.x == 0) *epoch = *epoch + 1u;
}

// ---- greedy sampling: the largest logit of every row and its index ---------------------
// grid (parts, rows): every CTA takes a slice of one row and leaves (value, index) in scratch;
// the last CTA of a row to finish compares the slices and writes the row's result. Ties go to
// the smallest index. NaNs never win (a row of NaNs gives index 0).
constexpr int kArgmaxThreads = 256;

__global__ void argmax_rows_kernel(const __nv_bfloat16* __restrict__ logits, int64_t n, int64_t row_stride,
                                   int64_t index_offset, float* __restrict__ out_val, int64_t* __restrict__ out_idx,
                                   float* part_val, int64_t* part_idx, uint32_t* counters) {
  pdl_enter();
  __shared__ float sval[kArgmaxThreads / 32];
  __shared__ int64_t sidx[kArgmaxThreads / 32];
  __shared__ int is_last;
  const int parts = gridDim.x, part = blockIdx.x;
  const int64_t row = blockIdx.y;
  const __nv_bfloat16* x = logits + row * row_stride;
  const int64_t per = ((n + parts - 1) / parts + 7) & ~int64_t(7);
  const int64_t lo = part * per, hi = lo + per < n ? lo + per : n;
  float best = -INFINITY;
  int64_t where = lo < n ? lo : 0;
  auto take = [&](float v, int64_t i) {
    if (v > best || (v == best && i < where)) { best = v; where = i; }
  };
  const bool vec = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  if (vec) {
    for (int64_t i = lo + threadIdx.x * 8; i < hi; i += kArgmaxThreads * 8) {
      if (i + 8 <= hi) {
        float f[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(x + i)), f);
#pragma unroll
        for (int e = 0; e < 8; ++e) take(f[e], i + e);
      } else {
        for (int64_t j = i; j < hi; ++j) take(__bfloat162float(x[j]), j);
      }
    }
  } else {
    for (int64_t i = lo + threadIdx.x; i < hi; i += kArgmaxThreads) take(__bfloat162float(x[i]), i);
  }
  auto merge = [&](float ov, int64_t oi) {
    if (ov > best || (ov == best && oi < where)) { best = ov; where = oi; }
  };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int64_t oi = __shfl_xor_sync(0xffffffffu, where, o);
    merge(ov, oi);
  }
  if ((threadIdx.x & 31) == 0) { sval[threadIdx.x >> 5] = best; sidx[threadIdx.x >> 5] = where; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kArgmaxThreads / 32; ++w) merge(sval[w], sidx[w]);
    part_val[row * parts + part] = best;
    part_idx[row * parts + part] = where;
    __threadfence();
    const bool last = atomicAdd(&counters[row], 1u) == static_cast<uint32_t>(parts - 1);
    if (last) counters[row] = 0;
    is_last = last;
  }
  __syncthreads();
  if (!is_last || threadIdx.x >= 32) return;
  __threadfence();
  best = -INFINITY;
  where = 0;
  for (int q = threadIdx.x; q < parts; q += 32) merge(__ldcg(part_val + row * parts + q), __ldcg(part_idx + row * parts + q));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int64_t oi = __shfl_xor_sync(0xffffffffu, where, o);
    merge(ov, oi);
  }
  if (threadIdx.x == 0) {
    out_val[row] = best;
    out_idx[row] = where + index_offset;
  }
}

template <typename... Args>
int launch_pdl(const char* what, void (*kernel)(Args...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
               Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args...);
  if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "%s launch: %s", what, cudaGetErrorString(e));
  count_launch();
  return check_launch(what);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace qmm

using namespace qmm;

extern "C" int qmm_decode_add_rmsnorm(const void* x, const void* residual_in, const void* weight, void* y,
                                      void* residual_out, int64_t rows, int64_t dim, float eps, void* stream) {
  if (!x || !weight || !y) return fail(QMM_ERR_NULL, "add_rmsnorm: x, weight and y are required");
  if (rows < 0 || dim <= 0 || dim % 8 || dim > 24576) return fail(QMM_ERR_SHAPE, "add_rmsnorm: dim must be a multiple of 8, at most 24576");
  if (!aligned16(x) || !aligned16(weight) || !aligned16(y) || !aligned16(residual_in) || !aligned16(residual_out))
    return fail(QMM_ERR_LAYOUT, "add_rmsnorm: pointers must be 16-byte aligned");
  if (rows == 0) return QMM_OK;
  const size_t smem = static_cast<size_t>(dim) * 2 + kNormThreads / 32 * sizeof(float);
  static bool configured[kMaxDevices] = {};     // more than the default 48 KiB at the largest dim
  const int dev = current_device();
  if (dev < 0) return QMM_ERR_DEVICE;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 24576 * 2 + 64);
    if (e != cudaSuccess) return fail(QMM_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured[dev] = true;
  }
  return launch_pdl("add_rmsnorm_kernel", add_rmsnorm_kernel, dim3(static_cast<unsigned>(rows)), dim3(kNormThreads),
                    smem, static_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual_in),
                    static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(y),
                    static_cast<__nv_bfloat16*>(residual_out), dim, eps);
}

extern "C" int qmm_decode_rope_kv(const void* qkv, void* q_out, void* k_cache, void* v_cache, int64_t batch,
                                  int heads, int kv_heads, int head_dim, int64_t ctx, int64_t pos, float theta,
                                  void* stream) {
  if (!qkv || !q_out || !k_cache || !v_cache) return fail(QMM_ERR_NULL, "rope_kv: null pointer");
  if (batch < 0 || batch > 65535 || heads <= 0 || kv_heads <= 0 || head_dim <= 0 || head_dim % 2 || pos < 0 || pos >= ctx)
    return fail(QMM_ERR_SHAPE, "rope_kv: bad shape or position");
  if (batch == 0) return QMM_OK;
  const int work = (heads + 2 * kv_heads) * (head_dim / 2);
  return launch_pdl("rope_kv_kernel", rope_kv_kernel, dim3(static_cast<unsigned>((work + 255) / 256), static_cast<unsigned>(batch)),
                    dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(qkv),
                    static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache),
                    static_cast<__nv_bfloat16*>(v_cache), heads, kv_heads, head_dim, ctx, pos, theta);
}

extern "C" int qmm_decode_silu_mul(const void* gate_up, void* out, int64_t rows, int64_t ffn, void* stream) {
  if (!gate_up || !out) return fail(QMM_ERR_NULL, "silu_mul: null pointer");
  if (rows < 0 || ffn <= 0 || ffn % 8) return fail(QMM_ERR_SHAPE, "silu_mul: ffn must be a multiple of 8");
  if (!aligned16(gate_up) || !aligned16(out)) return fail(QMM_ERR_LAYOUT, "silu_mul: pointers must be 16-byte aligned");
  if (rows == 0) return QMM_OK;
  const int64_t total = rows * (ffn / 8);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return launch_pdl("silu_mul_kernel", silu_mul_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0,
                    static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(gate_up),
                    static_cast<__nv_bfloat16*>(out), rows, ffn);
}

extern "C" int64_t qmm_decode_argmax_scratch_bytes(int64_t rows) {
  return rows < 0 ? 0 : rows * 64 * 12 + rows * 4 + 64;
}

extern "C" int qmm_decode_argmax(const void* logits, int64_t rows, int64_t n, int64_t row_stride, int64_t index_offset,
                                 void* out_val, void* out_idx, void* scratch, int64_t scratch_bytes, void* stream) {
  if (!logits || !out_val || !out_idx || !scratch) return fail(QMM_ERR_NULL, "argmax: null pointer");
  if (rows < 0 || rows > 65535 || n < 1 || row_stride < n) return fail(QMM_ERR_SHAPE, "argmax: bad shape");
  if (scratch_bytes < qmm_decode_argmax_scratch_bytes(rows)) return fail(QMM_ERR_TOO_LARGE, "argmax: scratch is too small");
  if (reinterpret_cast<uintptr_t>(scratch) & 15)
    return fail(QMM_ERR_LAYOUT, "argmax: scratch must be 16-byte aligned");
  if (rows == 0) return QMM_OK;
  int64_t parts = (n + 4095) / 4096;
  if (parts > 64) parts = 64;
  const int64_t fill = (2 * device_sm_count() + rows - 1) / rows;         // no more CTAs than two per SM in all
  if (parts > fill) parts = fill < 1 ? 1 : fill;
  uint8_t* sc = static_cast<uint8_t*>(scratch);
  float* part_val = reinterpret_cast<float*>(sc);
  int64_t* part_idx = reinterpret_cast<int64_t*>(sc + rows * 64 * 4);
  uint32_t* counters = reinterpret_cast<uint32_t*>(sc + rows * 64 * 12);
  return launch_pdl("argmax_rows_kernel", argmax_rows_kernel, dim3(static_cast<unsigned>(parts), static_cast<unsigned>(rows)),
                    dim3(kArgmaxThreads), 0, static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(logits), n,
                    row_stride, index_offset, static_cast<float*>(out_val), static_cast<int64_t*>(out_idx), part_val, part_idx,
                    counters);
}

extern "C" int qmm_decode_allgather(const void* local, void* const* peer_bufs, void* const* peer_flags, void* state,
                                    int rank, int world, int slot, int64_t rows, int64_t slice_bytes,
                                    int64_t slot_bytes, void* stream) {
  if (!local || !peer_bufs || !peer_flags || !state) return fail(QMM_ERR_NULL, "allgather: null pointer");
  if (world < 1 || world > 8 || rank < 0 || rank >= world || slot < 0 || slot > 2)
    return fail(QMM_ERR_SHAPE, "allgather: world must be 1..8, slot 0..2");
  if (rows < 0 || slice_bytes <= 0 || slice_bytes % 16 || rows * slice_bytes * world > slot_bytes)
    return fail(QMM_ERR_SHAPE, "allgather: slices are multiples of 16 bytes and must fit the slot");
  if (!aligned16(local)) return fail(QMM_ERR_LAYOUT, "allgather: pointers must be 16-byte aligned");
  if (rows == 0) return QMM_OK;
  AllGatherParams p = {};
  p.local = static_cast<const uint8_t*>(local);
  for (int r = 0; r < world; ++r) {
    if (!peer_bufs[r] || !peer_flags[r] || !aligned16(peer_bufs[r])) return fail(QMM_ERR_NULL, "allgather: bad peer pointer");
    p.peer_buf[r] = static_cast<uint8_t*>(peer_bufs[r]);
    p.peer_flags[r] = static_cast<uint32_t*>(peer_flags[r]);
  }
  p.state = static_cast<uint32_t*>(state);
  p.status = device_status_word();
  if (!p.status) return fail(QMM_ERR_CUDA, "could not allocate the device status word");
  p.rows = rows; p.slice_bytes = slice_bytes; p.slot_bytes = slot_bytes;
  p.spin_limit = wait_limit_clocks();
  p.rank = rank; p.world = world; p.slot = slot;
  int64_t parts = (rows * slice_bytes + 32767) / 32768;
  if (parts > 16) parts = 16;
  return launch_pdl("allgather_push_kernel", allgather_push_kernel, dim3(static_cast<unsigned>(world), static_cast<unsigned>(parts)),
                    dim3(kAgThreads), 0, static_cast<cudaStream_t>(stream), p);
}


extern "C" int qmm_decode_step_begin(const qmm_exchange* ex, void* stream) {
  if (!ex || !ex->epoch) return fail(QMM_ERR_NULL, "step_begin: no exchange");
  return launch_pdl("step_begin_kernel", step_begin_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream),
                    static_cast<uint32_t*>(ex->epoch));
}

extern "C" int qmm_decode_linear(const qmm_problem* problem, const qmm_decode_fusion* fusion, const qmm_exchange* ex,
                                 void* stream) {
  if (!problem || !fusion) return fail(QMM_ERR_NULL, "decode_linear: problem and fusion are required");
  qmm_problem p = *problem;
  const bool waits = fusion->wait_slot >= 0, pushes = fusion->push_slot >= 0;
  if ((waits || pushes) && !ex) return fail(QMM_ERR_NULL, "decode_linear: an exchange is needed for wait_slot / push_slot");
  if (ex && (ex->world < 1 || ex->world > 8 || ex->rank < 0 || ex->rank >= ex->world || !ex->peer_bufs || !ex->epoch))
    return fail(QMM_ERR_SHAPE, "decode_linear: bad exchange (world 1..8, all pointers set)");
  const int world = ex ? ex->world : 1;
  if (waits) p.x = static_cast<const uint8_t*>(ex->peer_bufs[ex->rank]) + static_cast<int64_t>(fusion->wait_slot) * ex->slot_bytes;
  alignas(16) static unsigned char dummy_y[16];
  const bool no_y = !p.y;
  if (no_y) {
    if (!pushes && !(fusion->epilogue == QMM_EPILOGUE_SWIGLU_PAIRS && fusion->epilogue_out))
      return fail(QMM_ERR_NULL, "decode_linear: y is NULL and nothing is pushed");
    p.y = dummy_y;                                    // (passes the pointer checks; never written: see below)
  }
  int rc = check_problem(p);
  if (rc) return rc;
  if (no_y) p.y = nullptr;
  if (p.M != 1 || p.batch != 1 || !gemv_imma_supports(p))
    return fail(QMM_ERR_UNSUPPORTED, "decode_linear: only what the single-row decode kernel takes (M = 1, bf16)");
  if (fusion->prologue < QMM_PROLOGUE_NONE || fusion->prologue > QMM_PROLOGUE_SWIGLU)
    return fail(QMM_ERR_UNSUPPORTED, "decode_linear: unknown prologue %d", fusion->prologue);
  if (fusion->prologue == QMM_PROLOGUE_ADD_RMSNORM && (!fusion->norm_weight || fusion->residual_out == fusion->residual_in))
    return fail(QMM_ERR_NULL, "decode_linear: add + rmsnorm needs norm_weight, and residual_out apart from residual_in");
  if (fusion->prologue == QMM_PROLOGUE_SWIGLU && (p.K % world || (p.K / world) % 8))
    return fail(QMM_ERR_SHAPE, "decode_linear: SwiGLU blocks must be multiples of 8 wide");
  if ((waits && (fusion->wait_site < 0 || fusion->wait_site >= 1023)) || (pushes && (fusion->push_site < 0 || fusion->push_site >= 1023)))
    return fail(QMM_ERR_SHAPE, "decode_linear: exchange sites are 0..1022");
  if (fusion->epilogue != QMM_EPILOGUE_NONE && fusion->epilogue != QMM_EPILOGUE_SWIGLU_PAIRS)
    return fail(QMM_ERR_UNSUPPORTED, "decode_linear: unknown epilogue %d", fusion->epilogue);
  const bool pairs = fusion->epilogue == QMM_EPILOGUE_SWIGLU_PAIRS;
  if (pairs && ((!pushes && !fusion->epilogue_out) || p.N % 16))
    return fail(QMM_ERR_SHAPE, "decode_linear: the SwiGLU epilogue needs somewhere to put its N / 2 values, and N a multiple of 16");
  if (pairs && (reinterpret_cast<uintptr_t>(fusion->epilogue_out) & 15))
    return fail(QMM_ERR_LAYOUT, "decode_linear: epilogue_out must be 16-byte aligned");
  if (pushes && p.N % 8) return fail(QMM_ERR_LAYOUT, "decode_linear: a pushed slice must be a multiple of 8 values");
  const int64_t n_out = pairs ? p.N / 2 : p.N;             // values this rank contributes to the gathered row
  if (pushes && world * n_out * 4 > ex->slot_bytes)         // (a stamped row takes 4 bytes per value)
    return fail(QMM_ERR_SHAPE, "decode_linear: the gathered row does not fit a slot");
  if (waits && p.K * (fusion->prologue == QMM_PROLOGUE_SWIGLU ? 2 : 1) * 4 > ex->slot_bytes)
    return fail(QMM_ERR_SHAPE, "decode_linear: the awaited row does not fit a slot");
  DecodeFusion f = {};
  f.prologue = fusion->prologue;
  f.residual_in = fusion->residual_in; f.residual_out = fusion->residual_out;
  f.norm_weight = fusion->norm_weight; f.eps = fusion->eps;
  f.swiglu_width = static_cast<int>(p.K / world);
  if (ex) f.epoch = static_cast<const uint32_t*>(ex->epoch);
  if (waits) {
    f.wait_world = world; f.wait_site = fusion->wait_site;
  }
  if (pushes) {
    f.push_world = world; f.push_site = fusion->push_site;
    for (int r = 0; r < world; ++r) {
      if (!ex->peer_bufs[r]) return fail(QMM_ERR_NULL, "decode_linear: bad peer pointer");
      f.push_dst[r] = static_cast<uint8_t*>(ex->peer_bufs[r]) + static_cast<int64_t>(fusion->push_slot) * ex->slot_bytes +
                      static_cast<int64_t>(ex->rank) * n_out * 4;
    }
  }
  f.epilogue = pairs ? 1 : 0;
  f.epilogue_out = pairs ? fusion->epilogue_out : nullptr;
  return launch_gemv_imma(p, static_cast<cudaStream_t>(stream), &f);
}
