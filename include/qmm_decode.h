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

#ifdef __cplusplus
}
#endif
#endif /* QMM_DECODE_H_ */
