// Internal declarations shared by the libqmm translation units.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qmm.h"

namespace qmm {

// Records `msg` (printf-style) as the calling thread's last error and returns `code`.
int fail(int code, const char* fmt, ...);

// Bumps the process-wide launch counter reported by qmm_launch_count().
void count_launch(int n = 1);

// Bumps the counter of device-memory allocations made by the library (qmm_alloc_count()).
void count_alloc(int n = 1);

// Per-device facts are cached by device ordinal: a process may drive several GPUs.
constexpr int kMaxDevices = 64;
// The calling thread's current device ordinal, or -1 (with the error recorded).
int current_device();

// The kernel family forced by qmm_set_route_override (a qmm_route_id; QMM_ROUTE_NONE = automatic).
int route_override();

// Checks the CUDA runtime's sticky/launch error after a launch.
int check_launch(const char* what);

// Kernel families. Each validates nothing: `qmm_launch` has already done so.
int launch_simt(const qmm_problem& p, cudaStream_t stream);
// Scratch memory a caller lends for the duration of one call on this thread (set by the entry
// point that works without allocating); NULL when the library may allocate its own.
struct ScratchBlock {
  void* ptr;
  size_t bytes;
  int* status;     // where the kernels of this call record a device wait that ran out
};
const ScratchBlock* scratch_override();
void set_scratch_override(const ScratchBlock* block);

int launch_gemv(const qmm_problem& p, cudaStream_t stream);
bool gemv_supports(const qmm_problem& p);
// What a decode step fuses into a single-row linear: how its activation row is made from the
// previous kernels' outputs, and the exchange of its input and output rows over peer memory.
struct DecodeFusion {
  int prologue;              // 0 none, 1 residual add + RMS norm, 2 SwiGLU
  const void* residual_in;
  void* residual_out;
  const void* norm_weight;
  float eps;
  int swiglu_width;
  const uint32_t* epoch;     // this rank's step counter
  int wait_world, wait_site; // x is a stamped row in this rank's gather slot
  int push_world, push_site; // y also goes, stamped, to every rank's slot
  uint8_t* push_dst[8];
  int epilogue;              // 1: rows alternate gate, up; silu(gate) * up is what is pushed / written
  void* epilogue_out;        //    ... plainly to here ([N / 2] bf16), when not NULL
};

// The single-row (M = 1) integer tensor-core decode kernel; launch_gemv hands it what it takes.
int launch_gemv_imma(const qmm_problem& p, cudaStream_t stream, const DecodeFusion* fusion = nullptr);
bool gemv_imma_supports(const qmm_problem& p);
// qmm_launch's validation of a raw problem (pointers included).
int check_problem(const qmm_problem& p);
int launch_gemm_tc(const qmm_problem& p, cudaStream_t stream);
bool gemm_tc_supports(const qmm_problem& p);
// Development builds (-DQMM_STEP_TRACING=1): every launch of the decode-step kernels takes the
// next block of a caller-provided buffer and its CTAs stamp %globaltimer at fixed points
// (16 stamps per CTA, 512 CTAs per block). Off in the product build: no parameter, no code.
#ifndef QMM_STEP_TRACING
#define QMM_STEP_TRACING 0
#endif
#if QMM_STEP_TRACING
constexpr int kTraceStamps = 16, kTraceCtas = 512;
unsigned long long* next_trace_block(int kind);
#ifdef __CUDACC__
__device__ __forceinline__ void trace_mark(unsigned long long* t, int slot) {
  if (t && threadIdx.x == 0) {
    const unsigned cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    if (cta < kTraceCtas) {
      unsigned long long g;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g));
      t[cta * kTraceStamps + slot] = g;
    }
  }
}
#endif
#define QMM_TRACE(t, slot) trace_mark(t, slot)
#else
#define QMM_TRACE(t, slot) ((void)0)
#endif

// Reads (and clears) the current device's status word.
int read_status_word(int* out);

// Encodes a 2-D TMA descriptor (a CUtensorMap, 128 bytes at `map_out`): `inner` x `outer`
// elements of kind `elem_kind` (a qmm_elem; QMM_U8 for raw bytes), rows `row_bytes` apart,
// copied in boxes of box_inner x box_outer, optionally in the 128-byte swizzle.
int tensor_map_2d(void* map_out, int elem_kind, const void* base, uint64_t inner, uint64_t outer,
                  uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle128);

// The current device's word in which kernels record a bounded wait that ran out (one word per
// device, allocated on first use and kept), or NULL.
int* device_status_word();

// SM clocks a bounded device-side wait may last (qmm_set_wait_limit; default about 2 s).
long long wait_limit_clocks();
void set_wait_limit_clocks(long long clocks);

int device_sm_count();

int launch_dequantize(const uint32_t* w, const void* scales, const void* biases, int table_dtype,
                      void* out, int out_dtype, int64_t rows, int64_t K, int group_size, int bits,
                      int mode, cudaStream_t stream);
int launch_pack_codes(const uint8_t* codes, uint32_t* out, int64_t rows, int64_t K, int bits,
                      cudaStream_t stream);

#ifdef __CUDACC__
// Raw bits of element i of a 16-bit (`wide` false) or 32-bit (`wide` true) table, zero-extended.
// Nothing here depends on the loaded value, so a caller can request many elements before it
// uses the first; callers keep `wide` loop-invariant so that the loads of a batch do not end
// up in separate branches.
__device__ __forceinline__ uint32_t table_raw(const void* p, bool wide, int64_t i) {
  if (wide) return __ldg(static_cast<const uint32_t*>(p) + i);
  return __ldg(static_cast<const uint16_t*>(p) + i);
}

// The float value of such raw bits (QMM_BF16 / QMM_F16 / QMM_F32).
__device__ __forceinline__ float table_value(uint32_t raw, int dtype) {
  if (dtype == QMM_BF16) return __uint_as_float(raw << 16);
  if (dtype == QMM_F16) {
    float f;
    asm("{ .reg .b16 h; cvt.u16.u32 h, %1; cvt.f32.f16 %0, h; }" : "=f"(f) : "r"(raw));
    return f;
  }
  return __uint_as_float(raw);
}
#endif

inline int elem_size(int e) {
  switch (e) {
    case QMM_BF16: case QMM_F16: return 2;
    case QMM_F32: case QMM_U32: case QMM_I32: return 4;
    case QMM_U8: return 1;
  }
  return 0;
}

}  // namespace qmm
