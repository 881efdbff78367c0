/*
 * Hooks for this library's own tests and benchmark.  Not part of the C ABI a backend crate
 * binds (include/yaxus_cuda.h): nothing here is needed to use the library, the symbols may
 * change between builds, and a release build may drop them.
 */
#ifndef YX_HOOKS_H
#define YX_HOOKS_H

#include "../../include/yaxus_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Runs the split-key planner (the counterpart of `AttentionCase::plan`,
 * crates/yaxus-backend-gpu/src/plan.rs:275-309) on host arrays; needs no device.  Each item is
 * written as YX_PROBE_ITEM_WORDS words: tile_begin, tile_end, key_lo, key_hi, pt_off, kv_head,
 * n_rows, padded rows, CTA, then 16 pass rows and their 16 partial slots.  share_prefix: 0 off,
 * 1 on with the default rows per shared item, above 1 that many rows per shared item. */
#define YX_PROBE_ITEM_WORDS 41
int yx_plan_probe(uint32_t rows, const uint32_t *pos_host, const uint32_t *pt_off_host, const uint32_t *pages_host,
                  uint32_t n_pages, int hkv, int group, int64_t window, uint64_t key_lo, uint64_t key_hi,
                  int max_rows, int n_ctas, int share_prefix, int esize, int cost32, int cost64, int item_cost,
                  int min_piece, yx_plan_info *info, uint32_t *items_out, uint32_t max_items);

/* The planner's short way (a plan patched in place when the next pass has the shape of the last
 * one) against plans built from scratch: runs `steps` decode steps from the given pass, every row one
 * key further each step, through one plan object, and builds a fresh plan beside it every time.
 * Returns the number of steps whose plans differed (0 is the only good answer), or -1 on a
 * malformed pass; *patched_out receives how many steps took the short way.  Needs no device. */
int yx_hook_plan_steps(uint32_t rows, const uint32_t *pos_host, const uint32_t *pt_off_host, const uint32_t *pages_host,
                       uint32_t n_pages, int hkv, int group, int64_t window, int max_rows, int n_ctas, int steps,
                       int *patched_out);

/* Measurement only.  Makes the context's next plans be built from scratch, as they are in a decode
 * loop whenever a row's keys grow into a new 64-key tile (a benchmark that repeats one pass would
 * otherwise always take the planner's short way). */
int yx_hook_forget_plan_shape(yx_ctx *ctx);

/* Measurement only.  on != 0: yx_attend runs its split-key kernel and skips the merge of the
 * triples (the call then produces no output), so that back-to-back calls time that kernel alone. */
int yx_hook_skip_merge(yx_ctx *ctx, int on);

/* Makes a bounded device-side wait run out without starving any real kernel: one CTA waits on
 * an mbarrier nobody arrives on, for at most `limit_cycles` SM cycles, then gives up the way
 * the attention kernels do (failure recorded in the context's status word, the kernel returns
 * normally).  The next yx_sync must report YX_ERR_DEVICE and the context must stay usable
 * after yx_clear_error. */
int yx_hook_expire_wait(yx_ctx *ctx, uint64_t limit_cycles);

/* Per-CTA timestamps of the split-key and tile kernels are written to `dev_buf` while it is set.
 * Only a library built with -DYX_TRACE stamps anything; otherwise the call returns
 * YX_ERR_UNSUPPORTED. */
int yx_hook_set_trace(yx_ctx *ctx, void *dev_buf);

/* Host time the context has spent in the phases of its attention calls since the last reset, in
 * nanoseconds: [0] checks, [1] planning, [2] laying the plan out in its staging buffer, [3] the
 * upload call, [4] the append launch, [5] the attention kernel launches, [6] the merge launch.
 * Measured only by a library built with -DYX_TRACE; otherwise YX_ERR_UNSUPPORTED. */
int yx_hook_host_times(yx_ctx *ctx, double *out8, int reset);

#ifdef __cplusplus
}
#endif
#endif
