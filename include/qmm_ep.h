/* Dispatch and combine of an expert-parallel mixture-of-experts block over peer memory.
 *
 * The reference is single-device: these entry points replace nothing in it. They serve the
 * expert-parallel form of the gathered expert block (`metaljax_b200/parallel.py`), where every
 * rank routes its own tokens and expert e lives on rank e / (experts / world): instead of
 * all-to-all collectives whose sizes the host has to read back, the ranks store rows straight
 * into each other's buffers over NVLink (one process per GPU; every rank maps every rank's
 * buffers, e.g. through torch symmetric memory), and the sizes never leave the devices.
 *
 * Every rank makes the same sequence of calls. A call pair is
 *   qmm_ep_dispatch  -> this rank's receive buffer holds the rows of its experts, laid out
 *                       (local expert, source rank, source order); group_sizes_out [experts/world]
 *                       (int32, device) is what the grouped product over them takes
 *   ... the expert products on peer_recv[rank] (capacity_rows rows; rows past the sum of the
 *       group sizes are not meaningful) ...
 *   qmm_ep_combine   -> this rank's return buffer holds the result row of each of its pairs, in
 *                       the order of its own pairs sorted by expert
 * Waits are bounded (qmm_set_wait_limit) and report through qmm_poll_status (codes 110..112); a
 * row that would not fit a buffer is dropped and reported (QMM_ERR_SHAPE). */
#ifndef QMM_EP_H_
#define QMM_EP_H_

#include "qmm.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
  void* const* peer_counts;  /* [world] rank r's table: world * experts * 8 bytes, zeroed once */
  void* const* peer_flags;   /* [world] rank r's flags: 2 * world uint32, zeroed once */
  void* const* peer_recv;    /* [world] rank r's receive buffer: capacity_rows rows */
  void* const* peer_ret;     /* [world] rank r's return buffer: max_pairs rows */
  void* epoch;               /* this rank's call counter: one uint32 of device memory, zeroed once */
  void* scratch;             /* this rank's: 16 bytes of device memory, zeroed once */
  int64_t capacity_rows;     /* rows a receive buffer holds (>= the most pairs that can meet on one rank) */
  int64_t max_pairs;         /* rows a return buffer holds (>= this rank's pairs per call) */
  int32_t rank, world;       /* world <= 8 */
  int32_t experts;           /* all experts: a multiple of world, <= 256 */
} qmm_ep_exchange;

/* x [tokens, row_bytes] (16-byte aligned rows); token_of_row int64 [pairs]: the token of each of
 * this rank's pairs, pairs sorted by (global) expert; counts int32 [experts]: pairs per expert. */
int qmm_ep_dispatch(const qmm_ep_exchange* ex, const void* x, int64_t tokens, int64_t row_bytes,
                    const int64_t* token_of_row, const int32_t* counts, int64_t pairs,
                    int32_t* group_sizes_out, void* stream);

/* rows [capacity_rows, row_bytes]: the results, in the receive buffer's row order. */
int qmm_ep_combine(const qmm_ep_exchange* ex, const void* rows, int64_t row_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* QMM_EP_H_ */
