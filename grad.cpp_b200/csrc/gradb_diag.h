/* Entry points that exist only in the diagnostics build of the library (libgradb_diag.so, built with
 * -DGRADB_DIAGNOSTICS). That build also checks device-side indices (a violated bound records a code in the session's
 * status word, skips the access, and the call returns GRADB_ERR_INVALID "a device-side index check failed"), reads the
 * overrides GRADB_TC_TILE / GRADB_ATTN_SPLITS and, with GRADB_B1_TRACE=1, records the single-sequence kernel's stage
 * timestamps. None of this is in the product library or its header. */
#ifndef GRADB_DIAG_H
#define GRADB_DIAG_H

#include "../../include/gradb.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Nanosecond timestamps CTA 0 of the single-sequence persistent kernel left at its stage boundaries during the most
 * recent step (session created with GRADB_B1_TRACE=1). Returns how many were recorded. */
gradb_status gradb_session_stage_trace(gradb_session* session, uint64_t* stamps_out, int capacity, int* count_out);

/* Makes a bounded device-side wait run out, to exercise the status-word path: the pipelined cached-attention kernel
 * polls each tile's arrival at most spin_limit times (0 = the normal limit) and every warp leaves out the copy of
 * its skip_tile-th tile (-1 = none), so the wait for that tile expires; the kernel records code 301, waits for its
 * other copies and returns; the call that launched it returns GRADB_ERR_DEVICE_WAIT. Nothing faults or hangs. */
gradb_status gradb_diag_attention_wait(gradb_session* session, unsigned spin_limit, int skip_tile);

/* Non-finite values among the session's current logits and residual rows of sequences 0..n_seq-1. */
gradb_status gradb_diag_count_nonfinite(gradb_session* session, int n_seq, long long* count_out);

/* Overwrites one entry of a sequence's id history on the device without the range check the product entry points
 * make, so that the device-side index check of the penalty stage can be seen to catch it. */
gradb_status gradb_diag_poke_history(gradb_session* session, int seq, int index, int32_t id);

/* Clock cycles CTA 0 of the persistent many-row GEMM has spent per role since the last reset, summed over launches,
 * as 8 rows of 16 counters, one row per epilogue kind (0 Q|K|V, 1 residual, 2 GELU, 3 SwiGLU, 4 logits, 5 log-sum-exp):
 * [0] tiles, MMA lane: [1] waiting for a drained accumulator, [2] waiting for operands, [3] whole loop;
 * TMA lane: [4] waiting for a free ring stage, [5] whole loop; first epilogue warp: [6] waiting for an accumulator,
 * [7] accumulator -> staged tile, [8] barrier, [9] row pass, [10] barrier.
 * The call also reads GRADB_DIAG_WIDE_SKIP (bits: 1 no accumulator -> staged tile pass, 2 no row pass, 4 no MMAs,
 * 8 no copies and no waiting for them) for the launches that follow: parts of the kernel timed alone, results
 * meaningless. */
gradb_status gradb_diag_wide_clocks(uint64_t* out128, int reset);

/* Clock cycles one warp of CTA 0 of the tensor-core prompt attention kernel has spent per part of an element (one
 * 128 x 128 tile of scores) since the last reset: [0] elements, [1] waiting for the scores, [2] scores -> registers,
 * mask and maximum, [3] first barrier, [4] previous O_tile, [5] write-out at an item change, [6] exponentials -> P,
 * [7] waiting for V, [8] transpose, [9] store wait and fences, [10] second barrier. */
gradb_status gradb_diag_attn_clocks(uint64_t* out16, int reset);

/* Clock cycles sequence 0's CTA of the sampled selection kernel has spent per part since the last reset, for calls
 * that take the few-candidates path after top-k: [0] calls, [1] logits -> shared memory, [2] penalty, [3] temperature,
 * [4] k-th value (for k <= 256: threshold, list, k-th value and the survivors' order; [5] then stays zero),
 * [5] count and compact, [6] softmax / nucleus / draw on the survivors, [7] bookkeeping; and of those that run the
 * stage on the full row: [8] maximum and exponentials, [9] softmax denominator, [10] probabilities, [11] sort,
 * [12] nucleus cutoff, [13] mask + kept mass + renormalisation, [14] all of [8]-[13] and the draw; [15] the largest
 * [14] of any sequence's CTA in one call (the kernel lasts as long as its slowest sequence). */
gradb_status gradb_diag_select_clocks(uint64_t* out16, int reset);

#ifdef __cplusplus
}
#endif
#endif
