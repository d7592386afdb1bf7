/* libqmm -- fused dequantize-and-matmul for NVIDIA B200 (sm_100a), C ABI.
 *
 * This library stands where the reference (eterevsky/metaljax 0.11.3) calls into
 * Apple's MLX: the recognizer's `emit` ends in ONE `mx.quantized_matmul`
 * (src/metaljax/qmm.py:2491-2492) and the mixture-of-experts rewrite in ONE
 * `mx.gather_qmm` (src/metaljax/moe.py:1320-1322). Each entry point below names
 * the reference call it replaces. Argument meaning (packed layout, group size,
 * bits, mode, transpose=True) is MLX's, so a pack built by the reference's
 * `pack_codes` / `pack_exact` / `mxfp4_scale_bytes` is consumed unchanged.
 *
 * Conventions
 *  - Tensors cross as DLPack `DLTensor` views (`qmm_tensor` below has the same
 *    layout); device tensors must be kDLCUDA on the current device. The caller
 *    allocates outputs and owns all memory; the library borrows for the call and
 *    retains nothing.
 *  - Work is enqueued on `stream` (a `cudaStream_t`, NULL = the legacy default
 *    stream). No call synchronizes the device.
 *  - Every function returns a `qmm_status`; 0 is success. Nothing throws across
 *    the ABI. `qmm_last_error()` returns a thread-local message for the last
 *    non-zero status on the calling thread.
 *  - There is no CPU path: a call on a machine without an sm_100 device fails
 *    with QMM_ERR_CUDA / QMM_ERR_DEVICE.
 *
 * Packed layout (src/metaljax/qmm.py:206-232): a row of K codes is a
 * little-endian bit stream in uint32 words, element i at bits [i*bits,(i+1)*bits).
 * Affine: `w = scales*q + biases` per group of `group_size` along K
 * (src/metaljax/qmm.py:71-75), tables `[.., N, K/group_size]` in bf16, f16 or f32.
 * MXFP4: `w = E2M1[q] * 2^(byte-127)`, one E8M0 byte per 32 elements, no bias
 * table (src/metaljax/qmm.py:167-173, 335-357).
 */
#ifndef QMM_H_
#define QMM_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QMM_VERSION 1

/* ---- DLPack-compatible view (same memory layout as DLTensor) ---------------- */
typedef struct {
  int32_t device_type; /* 1 = kDLCPU, 2 = kDLCUDA */
  int32_t device_id;
} qmm_device;

typedef struct {
  uint8_t code; /* 0 int, 1 uint, 2 float, 4 bfloat */
  uint8_t bits;
  uint16_t lanes;
} qmm_dtype;

typedef struct {
  void* data;
  qmm_device device;
  int32_t ndim;
  qmm_dtype dtype;
  int64_t* shape;
  int64_t* strides; /* in elements; NULL = compact row-major */
  uint64_t byte_offset;
} qmm_tensor;

/* ---- enums ------------------------------------------------------------------ */
typedef enum {
  QMM_OK = 0,
  QMM_ERR_NULL = 1,        /* a required pointer is NULL */
  QMM_ERR_DTYPE = 2,       /* element type not accepted in that position */
  QMM_ERR_SHAPE = 3,       /* ranks / extents do not agree */
  QMM_ERR_LAYOUT = 4,      /* non-contiguous where contiguity is required, or misaligned */
  QMM_ERR_DEVICE = 5,      /* not a CUDA tensor, or tensors on different devices */
  QMM_ERR_GROUP = 6,       /* group_size / bits / mode combination not representable */
  QMM_ERR_UNSUPPORTED = 7, /* valid request this build does not implement */
  QMM_ERR_CUDA = 8,        /* a CUDA runtime call failed (message has the reason) */
  QMM_ERR_TIMEOUT = 9,     /* a bounded device-side wait ran out */
  QMM_ERR_TOO_LARGE = 10   /* a static capacity was exceeded */
} qmm_status;

/* Codes a kernel can leave in the device status word (qmm_poll_status): 1..99 name the wait
 * of a compute kernel that ran out, 100 + r the rank an exchange never heard from, and
 * QMM_DEVICE_BAD_INDEX a gather index outside [0, E) / [0, T): that pair was computed with
 * index 0 instead of reading out of bounds. */
#define QMM_DEVICE_BAD_INDEX 200

/* QMM_MODE_FLOAT: the weight holds values of the activation type, nothing is dequantized; taken
 * by qmm_ragged_mm only (the other entry points refuse it). */
typedef enum { QMM_MODE_AFFINE = 0, QMM_MODE_MXFP4 = 1, QMM_MODE_FLOAT = 2 } qmm_mode;

/* Element types of the raw-pointer entry points. */
typedef enum {
  QMM_BF16 = 0,
  QMM_F16 = 1,
  QMM_F32 = 2,
  QMM_U8 = 3,
  QMM_U32 = 4,
  QMM_I32 = 5
} qmm_elem;

/* Which kernel family a problem is routed to (see qmm_route). */
typedef enum {
  QMM_ROUTE_NONE = 0,
  QMM_ROUTE_GEMV = 1,       /* decode: M <= 16, weight streaming */
  QMM_ROUTE_GEMM_TC = 2,    /* prefill: tcgen05 tensor-core kernel */
  QMM_ROUTE_SIMT = 3,       /* float32 activations / shapes the others decline */
  QMM_ROUTE_GEMV_FMMA = 4   /* only as an override: the decode family's floating-point mma.sync
                             * kernel also where the single-row integer kernel would be chosen */
} qmm_route_id;

/* ---- library ---------------------------------------------------------------- */

/* ABI version of the loaded library (== QMM_VERSION it was built with). */
int qmm_version(void);

/* Message for the calling thread's last failure ("" if none). The reference's
 * counterpart is the Python exception text the PJRT entry turns into a
 * PJRT_Error (plugin/metal_pjrt.cc:185-226). */
const char* qmm_last_error(void);

/* ---- the fused op ----------------------------------------------------------- */

/* Replaces `mx.quantized_matmul(x, w, scales, biases, transpose=True,
 * group_size, bits, mode)` at src/metaljax/qmm.py:2491-2492.
 *
 *   y[.., m, n] = sum_k x[.., m, k] * deq(w)[.., n, k]
 *
 *   x       [M, K] or [B, M, K]   bf16 | f16 | f32, rows contiguous along K
 *   w       [N, K*bits/32] or [B, N, K*bits/32]   uint32 (a 2-D w is shared by
 *           every batch of a 3-D x, as MLX broadcasts leading dimensions)
 *   scales  [.., N, K/group_size]  bf16 | f16 | f32 (affine); uint8 E8M0 (mxfp4)
 *   biases  same shape and type as scales (affine); NULL (mxfp4)
 *   y       [M, N] or [B, M, N]   bf16 | f16 | f32, caller-allocated; the cast to
 *           the dot's result type (src/metaljax/qmm.py:2499-2500) happens in the
 *           kernel's epilogue
 *   transpose   must be 1 (the only form the reference emits)
 *   group_size  32 | 64 | 128 (affine), 32 (mxfp4);  bits 4 | 8 (affine), 4 (mxfp4)
 * Accumulation is float32.
 *
 * Stream order: the kernels are launched with programmatic stream serialization. x (and the
 * index / size arrays of the gathered and ragged forms) are read, and y is written, only after
 * everything queued before the call on `stream` has completed and is visible. The packed
 * weight and its tables are requested earlier -- once the grid queued directly before has
 * finished its thread blocks -- because in the reference's protocol they are constants made
 * once by the pack prologue (src/metaljax/qmm.py:2305-2387), long before the first fused op. A
 * caller that rewrites a weight on the same stream immediately before using it puts an event
 * or any other kernel in between. */
int qmm_quantized_matmul(const qmm_tensor* x, const qmm_tensor* w, const qmm_tensor* scales,
                         const qmm_tensor* biases, qmm_tensor* y, int transpose, int group_size,
                         int bits, int mode, void* stream);

/* Replaces `mx.gather_qmm(x, w, scales, biases, lhs_idx, rhs_idx, transpose=True,
 * group_size, bits, mode)` at src/metaljax/moe.py:1320-1322.
 *
 *   y[p, m, n] = sum_k x[lhs_idx[p], m, k] * deq(w[rhs_idx[p]])[n, k]
 *
 *   x [T, M, K]; w [E, N, K*bits/32]; scales/biases [E, N, K/group_size];
 *   lhs_idx, rhs_idx uint32 or int32 [P]; y [P, M, N]. */
int qmm_gather_qmm(const qmm_tensor* x, const qmm_tensor* w, const qmm_tensor* scales,
                   const qmm_tensor* biases, const qmm_tensor* lhs_idx, const qmm_tensor* rhs_idx,
                   qmm_tensor* y, int transpose, int group_size, int bits, int mode, void* stream);

/* The sorted form of the same gather: `ragged_dot(lhs[m,k], rhs[g,k,n],
 * group_sizes[g])` with a packed rhs. Rows [off[g], off[g+1]) of x, off = prefix sum
 * of group_sizes, meet expert g. The reference reaches this computation through
 * `gather_qmm` with pairs in router order (src/metaljax/moe.py:1432-1433); sorting
 * the pairs by expert first gives this call. Rows past sum(group_sizes) are zeroed.
 *
 *   x [Mtot, K]; w [G, N, K*bits/32]; scales/biases [G, N, K/group_size];
 *   group_sizes int32 [G] on the device; y [Mtot, N]. */
int qmm_ragged_dot(const qmm_tensor* x, const qmm_tensor* w, const qmm_tensor* scales,
                   const qmm_tensor* biases, const qmm_tensor* group_sizes, qmm_tensor* y,
                   int group_size, int bits, int mode, void* stream);

/* The same grouped product for FLOAT experts: replaces `mx.gather_mm(x, w, lhs_idx, rhs_idx)`
 * (src/metaljax/moe.py:1324-1336) once the pairs are sorted by expert, through the ragged
 * tensor-core main loop with the dequantization step bypassed.
 *   x [Mtot, K] bf16 | f16; w [G, N, K] of x's type; group_sizes int32 [G] on the device;
 *   y [Mtot, N] bf16 | f16 | f32. K >= 64 and a multiple of 8. Rows past sum(group_sizes) are
 *   zeroed. QMM_ERR_UNSUPPORTED for anything else (there is no other route for float weights). */
int qmm_ragged_mm(const qmm_tensor* x, const qmm_tensor* w, const qmm_tensor* group_sizes,
                  qmm_tensor* y, void* stream);

/* The two element-wise steps of a gathered expert block, raw pointers (dtype: QMM_BF16 |
 * QMM_F16; 16-byte aligned). The reference runs them as generic pair-space ops after its
 * gathered dots (src/metaljax/moe.py:1425-1461).
 *
 * qmm_moe_silu_mul: out[i] = silu(gate[i]) * up[i] over `elements` values (a multiple of 8),
 * silu rounded to the storage type before the product, as the two-op form rounds it.
 *
 * qmm_moe_routed_sum: out[t, :] = sum over k of weights[t, k] * rows[row_of_pair[t*K + k], :]
 * in float32 (product rounded, then added, k ascending), cast to the storage type; rows is
 * [total_rows, width] (pairs sorted by expert), row_of_pair int64 [tokens * K] maps a pair in
 * router order to its sorted row, weights float32 [tokens, K], width a multiple of 8. An index
 * outside [0, total_rows) is clamped and reported (QMM_ERR_SHAPE from qmm_poll_status). */
int qmm_moe_silu_mul(const void* gate, const void* up, void* out, int64_t elements, int dtype, void* stream);
int qmm_moe_routed_sum(const void* rows, const int64_t* row_of_pair, const float* weights, void* out,
                       int64_t tokens, int k, int64_t width, int64_t total_rows, int dtype, void* stream);

/* Replaces `mx.dequantize(w, scales, biases, group_size, bits[, mode])`, which the
 * reference uses to pin the packed layout (tests/test_qmm.py:121,
 * tests/test_qmm_mxfp4.py:192): out [.., N, K] bf16 | f16 | f32, each element one
 * float32 FMA `scales*q + biases` (or the exact MXFP4 product) rounded once. */
int qmm_dequantize(const qmm_tensor* w, const qmm_tensor* scales, const qmm_tensor* biases,
                   qmm_tensor* out, int group_size, int bits, int mode, void* stream);

/* `qmm_quantized_matmul` for callers that must not allocate. (No counterpart in the
 * reference: MLX allocates inside `mx.quantized_matmul` as it pleases.)
 *
 * Same arguments, meaning, results and status codes as `qmm_quantized_matmul`, restricted to
 * what the tensor-core kernel takes (bf16 / f16 activations, K >= 64; QMM_ERR_UNSUPPORTED
 * otherwise). It exists for call sites where device memory cannot be requested while the call
 * is made -- a serving loop that has handed every byte to its own pool, a real-time thread that
 * may not block in the driver, code running under a tool that forbids allocation between two
 * marks. For a short, narrow product the kernel shares a tile's K range among several CTAs and
 * needs float32 scratch for their partial results; here that scratch is a fixed 8 MiB block of
 * device memory that belongs to the library image, and the call performs no cudaMalloc,
 * cudaMallocAsync, cudaFree or other allocating call.
 *   - A product whose partial results need more than the block (splits * M * N * 4 bytes, with
 *     at most 8 splits; about M * N <= 260k at full split) is refused with QMM_ERR_TOO_LARGE and
 *     a message naming both sizes; nothing is launched.
 *   - The first call on a device looks the block's address up and configures the kernels
 *     (one-time host-side setup); make that first call before any stream capture begins.
 *   - The block is one per device and shared by every caller in the process: two calls of this
 *     entry point that can overlap in time (different streams, different threads) race on it.
 *     Calls on one stream are safe.
 *   - Nothing in the block has to be cleared between calls. Its last 256 bytes hold the status
 *     word of the calls made through this entry point; it is zero when the library is loaded
 *     and becomes non-zero only if a bounded device-side wait runs out (the output of that
 *     call is then undefined). `qmm_poll_status_static` reads and clears it without
 *     allocating; `qmm_poll_status` reports it too. */
int qmm_quantized_matmul_static(const qmm_tensor* x, const qmm_tensor* w, const qmm_tensor* scales,
                                const qmm_tensor* biases, qmm_tensor* y, int transpose,
                                int group_size, int bits, int mode, void* stream);

/* Replaces `pack_codes(codes, bits)` (src/metaljax/qmm.py:206-232) for device
 * tensors: codes uint8 [.., K] -> out uint32 [.., K*bits/32], masked to `bits`. */
int qmm_pack_codes(const qmm_tensor* codes, qmm_tensor* out, int bits, void* stream);

/* ---- raw-pointer form (C/C++ callers such as the PJRT entry) ------------------ */

typedef struct {
  uint32_t struct_size;     /* sizeof(qmm_problem), for forward compatibility */
  int32_t mode;             /* qmm_mode */
  int32_t bits;             /* 4 | 8 */
  int32_t group_size;       /* 32 | 64 | 128 */
  int32_t x_dtype;          /* qmm_elem: BF16 | F16 | F32 */
  int32_t table_dtype;      /* qmm_elem of scales/biases (U8 for mxfp4) */
  int32_t y_dtype;          /* qmm_elem: BF16 | F16 | F32 */
  int32_t num_weights;     /* weight matrices behind `w` (experts E for a gather); 0 = batch
                            * when w_batch_stride != 0, else 1 */
  int64_t batch;            /* B >= 1 */
  int64_t M, K, N;
  const void* x;            /* [B, M, K] */
  const uint32_t* w;        /* [B or 1, N, K*bits/32] */
  const void* scales;       /* [B or 1, N, K/group_size] */
  const void* biases;       /* same, or NULL for mxfp4 */
  void* y;                  /* [B, M, N] */
  int64_t x_batch_stride;   /* elements between batches of x (0 allowed) */
  int64_t w_batch_stride;   /* rows of w between batches: N, or 0 = shared weight */
  int64_t y_batch_stride;   /* elements between batches of y */
  /* gather (both NULL for the dense op): pair p reads x batch lhs_idx[p] and
   * weight rhs_idx[p]; `batch` is then the number of pairs P. */
  const int32_t* lhs_idx;
  const int32_t* rhs_idx;
  /* ragged (NULL otherwise): int32 [batch] on the device; M is then the total row
   * count of x and y, `batch` the number of experts. */
  const int32_t* group_sizes;
  /* gather: batches of x behind `x` (T), so that a bad lhs_idx can be caught on the device;
   * 0 = unknown, lhs_idx is then only checked for being non-negative. */
  int64_t x_batches;
} qmm_problem;

/* Same computation as the three tensor entry points above, from raw pointers. */
int qmm_launch(const qmm_problem* problem, void* stream);

/* The kernel family `qmm_launch` would choose for this problem (a qmm_route_id),
 * after the same validation, without touching the device. Negative = -qmm_status. */
int qmm_route(const qmm_problem* problem);

/* Validates exactly like qmm_quantized_matmul but launches nothing and accepts
 * host tensors: returns the status the real call would give for these shapes and
 * types (device checks excepted). */
int qmm_check_quantized_matmul(const qmm_tensor* x, const qmm_tensor* w,
                               const qmm_tensor* scales, const qmm_tensor* biases,
                               const qmm_tensor* y, int transpose, int group_size, int bits,
                               int mode);

/* Test hook: force every later launch of this process onto one kernel family
 * (a qmm_route_id; QMM_ROUTE_NONE restores the automatic choice). A family that does
 * not support the problem makes the call fail with QMM_ERR_UNSUPPORTED instead of
 * silently taking another route. No counterpart in the reference. */
int qmm_set_route_override(int route);

/* Waits for the device and reports whether a kernel of this library gave up on a bounded
 * device-side wait since the last poll: *status_out is 0, or the code of the wait that
 * ran out (the call then returns QMM_ERR_TIMEOUT). Clears the word. No counterpart in the
 * reference, whose MLX calls are synchronous from Python's point of view. */
int qmm_poll_status(int* status_out);

/* The same for the status word of `qmm_quantized_matmul_static` alone, on the current device:
 * waits for the device, copies the word out of the library's static block, clears it if set.
 * Allocates nothing. No counterpart in the reference. */
int qmm_poll_status_static(int* status_out);

/* Test hook: how many SM clocks the bounded waits of the exchange kernels (qmm_decode.h) may
 * last before they give up and report through the status word (default 4e9, about two
 * seconds; at least 1000). Process-wide. No counterpart in the reference. */
int qmm_set_wait_limit(long long clocks);

/* Number of kernels this library has launched on the calling process since load
 * (monotonic; used by benchmarks to report their launch count). */
uint64_t qmm_launch_count(void);

/* Number of device-memory allocations (cudaMalloc / cudaMallocAsync) the library itself has
 * made since load: the per-device status word on first use, and the float32 partial-sum
 * scratch of a split tensor-core product. `qmm_quantized_matmul_static` never raises it once
 * the device has been used. No counterpart in the reference. */
uint64_t qmm_alloc_count(void);

#ifdef __cplusplus
}
#endif
#endif /* QMM_H_ */
