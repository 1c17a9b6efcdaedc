/* b200moe diagnostics: entry points that exist only in a library built with -DB200_DIAGNOSTICS
 * (B200MOE_DIAG=1 python sm120-fp4_b200/build.py). The product build does not export them. They have no counterpart in the
 * reference project. */
#ifndef B200MOE_DIAG_H
#define B200MOE_DIAG_H
#include "b200moe.h"

#ifdef __cplusplus
extern "C" {
#endif

/* issue-cost measurement of tcgen05 scale copies and MMAs (diagnostic; no counterpart in the reference): cycles_dev[0] =
 * cycles to issue `reps` rounds of {ncp copies, nmma MMAs 128 x N x 64, ncommit commits}, cycles_dev[1] = cycles until all completed
 * (device int64 x 4; [2], [3] = the same for the second issuing thread). flags: 1 two accumulators, 2 wait on a completed
 * mbarrier every round, 4 tcgen05 fence every round, 8 wait for the round's own commit, 16 copies from a second thread,
 * 32 converged warps with one elected lane instead of single diverged threads. */
int b200moe_umma_cost(int N, int reps, int ncp, int nmma, int flags, int ncommit, long long* cycles_dev, void* stream);

/* per-worker cycle counters of the last decode launch (8 int64 per worker: consumer wait, math, fix-up, phase-1 end,
 * producer wait, producer grid wait, producer end, consumer end). Filled only by a library built with -DB200_TIMERS (a
 * diagnostic build; the reference has no counterpart); returns the number of workers copied. Synchronises the stream. */
int b200moe_layer_debug_counters(const b200moe_layer* layer, const void* workspace, long long* out, int max_workers, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_DIAG_H */
