/* Glue kernels of one decoder step around the fused quantized linears of qmm.h.
 *
 * These have no counterpart at the reference's qmm boundary: the reference runs the same
 * arithmetic through its generic element-wise and reduce handlers
 * (src/metaljax/ops/elementwise.py, src/metaljax/ops/reduce.py). They exist so that a decode
 * step measured end to end (the Llama-shaped harness in metaljax_b200/llama.py) is a short
 * chain of launches between the weight streams. All tensors are bf16, row-major, on the
 * current device; pointers are 16-byte aligned; arithmetic is float32. Status codes and
 * qmm_last_error() are those of qmm.h. Every call launches on `stream` and returns without
 * synchronizing.
 */
#ifndef QMM_DECODE_H_
#define QMM_DECODE_H_

#include <stdint.h>

#include "qmm.h"

#ifdef __cplusplus
extern "C" {
#endif

/* h = x (+ residual_in when non-NULL); residual_out = h when non-NULL;
 * y[r, :] = h[r, :] * rsqrt(mean(h[r, :]^2) + eps) * weight.  x, y: [rows, dim]; weight: [dim].
 * dim is a multiple of 8, at most 24576. */
int qmm_decode_add_rmsnorm(const void* x, const void* residual_in, const void* weight, void* y,
                           void* residual_out, int64_t rows, int64_t dim, float eps, void* stream);

/* qkv: [batch, (heads + 2*kv_heads) * head_dim] = q heads, then k heads, then v heads.
 * Rotary embedding (rotate-half pairing, angle pos * theta^(-2i/head_dim)) on q and k;
 * q -> q_out [batch, heads, head_dim]; k, v -> caches [batch, kv_heads, ctx, head_dim] at
 * position pos (0 <= pos < ctx). */
int qmm_decode_rope_kv(const void* qkv, void* q_out, void* k_cache, void* v_cache, int64_t batch,
                       int heads, int kv_heads, int head_dim, int64_t ctx, int64_t pos, float theta,
                       void* stream);

/* gate_up: [rows, 2*ffn] = gate, then up.  out[r, i] = silu(gate[r, i]) * up[r, i]. */
int qmm_decode_silu_mul(const void* gate_up, void* out, int64_t rows, int64_t ffn, void* stream);

/* Greedy sampling: out_val[r] (float32) = the largest of logits[r, 0..n) (bf16, rows row_stride
 * elements apart) and out_idx[r] (int64) = its index + index_offset (ties: the smallest index).
 * `scratch`: qmm_decode_argmax_scratch_bytes(rows) bytes of device memory, 16-byte aligned,
 * zeroed once before the first call, not shared by calls that can overlap. */
int64_t qmm_decode_argmax_scratch_bytes(int64_t rows);
int qmm_decode_argmax(const void* logits, int64_t rows, int64_t n, int64_t row_stride, int64_t index_offset,
                      void* out_val, void* out_idx, void* scratch, int64_t scratch_bytes, void* stream);

/* One-shot all-gather over peer memory (one call per rank, each on its own GPU): this rank's
 * slice `local` [rows, slice_bytes] is stored into every rank's gather buffer
 * `peer_bufs[r] + slot*slot_bytes` at column offset rank*slice_bytes of rows world*slice_bytes
 * apart; then a flag is raised on every rank and the kernel waits (bounded; a timeout is
 * reported by qmm_poll_status) until every rank's flag for this call has been raised here, so
 * the next kernel of the stream reads the complete [rows, world*slice_bytes] matrix.
 *   peer_bufs[r], peer_flags[r]  rank r's gather buffer (3 slots of slot_bytes) and flag words
 *                                (24 uint32, zero-initialised once), mapped into this process
 *                                (CUDA IPC / symmetric memory); world entries each
 *   state                        16 uint32 of this rank's own device memory, zeroed once
 *   slot                         0..2; consecutive calls must use different slots, and every
 *                                rank must make the same sequence of calls.
 * slice_bytes is a multiple of 16. */
int qmm_decode_allgather(const void* local, void* const* peer_bufs, void* const* peer_flags, void* state,
                         int rank, int world, int slot, int64_t rows, int64_t slice_bytes,
                         int64_t slot_bytes, void* stream);

/* ---- the exchange folded into the kernels (single-row decode) ------------------------------
 *
 * With the weights sharded on their output rows, every linear's slice has to reach every rank
 * before the next kernel reads the whole row. Instead of a separate all-gather kernel, the
 * producing kernel stores its slice straight into every rank's gather slot from its epilogue
 * (plain peer stores over NVLink) and the consuming kernel, which requests its weights first,
 * reads the row as it arrives. No counterpart in the reference, which is single-device.
 *
 * A gathered row travels as 8-byte units {two bf16 values, 32-bit stamp}; the stamp is
 * (epoch << 10) | (site + 1), where `epoch` counts decode steps (qmm_decode_step_begin advances
 * it on the device, so a step captured in a CUDA graph can be replayed) and `site` numbers the
 * exchanges of one step (< 1023). A reader takes a unit when it carries the stamp it expects
 * (a bounded wait; a timeout is reported by qmm_poll_status as 100): data and "it has arrived"
 * cross the link in one store, so there is no separate flag, fence or counter. A slot therefore
 * holds 4 bytes per value. Every rank makes the same sequence of calls; consecutive exchanges
 * must use different slots (two slots alternating are enough, any rotation works). */
typedef struct {
  void* const* peer_bufs;   /* [world] every rank's gather area (`slot_bytes` per slot, zeroed once), mapped here */
  void* epoch;              /* this rank's step counter: one uint32 of device memory, zeroed once */
  int64_t slot_bytes;       /* multiple of 16 */
  int32_t rank, world;      /* world <= 8 */
} qmm_exchange;

typedef enum { QMM_PROLOGUE_NONE = 0, QMM_PROLOGUE_ADD_RMSNORM = 1, QMM_PROLOGUE_SWIGLU = 2 } qmm_prologue;
typedef enum { QMM_EPILOGUE_NONE = 0, QMM_EPILOGUE_SWIGLU_PAIRS = 1 } qmm_epilogue;

typedef struct {
  int32_t prologue;         /* qmm_prologue: what the linear's activation row is made from
                             *   NONE         x as it stands, [1, K]
                             *   ADD_RMSNORM  h = x (+ residual_in); residual_out = h (written once, by one CTA;
                             *                must not be the buffer residual_in points to); row = rmsnorm(h) * norm_weight
                             *   SWIGLU       x holds `world` blocks of [gate | up], each half K / world wide;
                             *                row = silu(gate) * up, block after block */
  int32_t wait_slot;        /* >= 0: x is the stamped row in gather slot `wait_slot` of this rank, */
  int32_t wait_site;        /*       written by exchange `wait_site`; < 0: x is problem->x */
  int32_t push_slot;        /* >= 0: y (this rank's N columns of a row of world * N) also goes to slot `push_slot` */
  int32_t push_site;        /*       of every rank, as exchange `push_site`; problem->y may then be NULL */
  const void* residual_in;
  void* residual_out;
  const void* norm_weight;  /* [K] bf16 */
  float eps;
  int32_t epilogue;         /* qmm_epilogue: what is pushed
                             *   NONE          the N outputs
                             *   SWIGLU_PAIRS  the weight's rows alternate gate_j, up_j (rows 2j, 2j + 1): the
                             *                 N / 2 values silu(y[2j]) * y[2j + 1], each y rounded to bf16 first
                             *                 (what a separate SwiGLU of the stored outputs computes); they go to
                             *                 epilogue_out and / or, with push_slot >= 0, to the gather slots (this
                             *                 rank's N / 2 columns of a row of world * N / 2); N a multiple of 16;
                             *                 problem->y, if given, still receives the N plain outputs */
  void* epilogue_out;       /* [N / 2] bf16, or NULL */
} qmm_decode_fusion;

/* Advances this rank's step counter: once at the start of every decode step, on the step's
 * stream, before the step's first exchange. */
int qmm_decode_step_begin(const qmm_exchange* ex, void* stream);

/* One sharded linear of a single-row decode step: `qmm_launch(problem)` with the activation row
 * produced, and the output row exchanged, inside the kernel as `fusion` says. M = 1, bf16
 * activations, bf16 (affine) or E8M0 (mxfp4) tables; QMM_ERR_UNSUPPORTED otherwise (the caller
 * then runs the unfused sequence). `ex` may be NULL when fusion->wait_slot and push_slot are < 0. */
int qmm_decode_linear(const qmm_problem* problem, const qmm_decode_fusion* fusion, const qmm_exchange* ex,
                      void* stream);

/* Rotary embedding + cache append + grouped-query attention of one decode position, one kernel:
 * what qmm_decode_rope_kv followed by softmax(q k^T / sqrt(head_dim)) v over positions 0..pos
 * computes. qkv as for qmm_decode_rope_kv; out [batch, heads * head_dim] bf16 (query head i
 * attends through key/value head i / (heads / kv_heads)), or NULL when the row is only pushed.
 * head_dim 64 or 128; heads / kv_heads 1, 2, 4 or 8. The context is cut into slices that run as
 * separate CTAs (slices of a few hundred positions and more -- many sequences at once -- take a
 * streaming tensor-core form of the kernel, short ones a latency form; same results within
 * rounding); their partial results meet in `scratch`, device memory the caller provides:
 * qmm_decode_attention_scratch_bytes(...) bytes, zeroed once before the first call, not shared
 * by calls that can overlap. With push_slot >= 0 the row also goes to every rank's gather slot
 * (this rank's heads are a column block of the gathered row) as exchange `push_site` of `ex`. */
int64_t qmm_decode_attention_scratch_bytes(int64_t batch, int heads, int kv_heads, int head_dim, int64_t ctx);
int qmm_decode_attention(const void* qkv, void* k_cache, void* v_cache, void* out, void* scratch,
                         int64_t scratch_bytes, int64_t batch, int heads, int kv_heads, int head_dim,
                         int64_t ctx, int64_t pos, float theta, int push_slot, int push_site,
                         const qmm_exchange* ex, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* QMM_DECODE_H_ */
