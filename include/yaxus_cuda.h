/*
 * libyaxus_cuda: attention over yaxus's paged, prefix-shared KV cache on NVIDIA B200 (sm_100a).
 *
 * This is the C ABI a `yaxus-backend-cuda` crate binds to implement the hot-path methods of
 * yaxus's `trait Backend` (crates/yaxus-model/src/lib.rs:95-171): `new_kv`, `copy_page`,
 * `begin_pass`, `attention`, plus the read-back and tensor plumbing those need.  The page
 * tables, page allocator and prefix sharing stay in yaxus-model (crates/yaxus-model/src/kv.rs)
 * and reach this library only as `PassMeta` arrays and `PageCopy` pairs.
 *
 * Conventions
 *  - Every function returns YX_OK or an error code; the first error of a context also sticks
 *    (yx_status / yx_last_error) because the trait's `attention`, `copy_page` and `begin_pass`
 *    cannot fail by signature and the reference defers device errors to the next read-back
 *    (crates/yaxus-model/src/lib.rs:187-197).  Nothing here aborts the process.
 *  - All work is enqueued on the context's stream; only yx_sync and yx_download with
 *    `wait != 0` wait for the device.  A context is not thread-safe (the reference drives a
 *    backend from one inference thread: its design notes, section on the engine thread).
 *  - Pointers named *_dev are device pointers; *_host are host pointers.
 *  - head_dim must be 128 and the page is 128 tokens, as in the reference's GPU backend
 *    (crates/yaxus-backend-gpu/src/lib.rs:72, crates/yaxus-model/src/kv.rs:17).
 *  - There is no CPU fallback: without a CUDA device every entry point fails.
 */
#ifndef YAXUS_CUDA_H
#define YAXUS_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define YX_PAGE 128
#define YX_HEAD_DIM 128

typedef struct yx_ctx yx_ctx;
typedef struct yx_kv yx_kv;

enum yx_error {
    YX_OK = 0,
    YX_ERR_INVALID = 1,     /* bad argument (the reference would panic on an assert) */
    YX_ERR_CUDA = 2,        /* a CUDA runtime call failed */
    YX_ERR_OOM = 3,         /* device allocation failed */
    YX_ERR_STATE = 4,       /* call out of order, e.g. attention without begin_pass */
    YX_ERR_DEVICE = 5,      /* a kernel reported a failed check (bad page index, a wait that gave up) */
    YX_ERR_NCCL = 6,
    YX_ERR_UNSUPPORTED = 7
};

enum yx_dtype { YX_F32 = 0, YX_F16 = 1, YX_BF16 = 2 };

/* Rope (crates/yaxus-model/src/config.rs:174-179) for head_dim 128. */
typedef struct yx_rope {
    float inv_freq[YX_HEAD_DIM / 2];
    float concentration;
} yx_rope;

/* LayerMeta (crates/yaxus-model/src/config.rs:163-170).  window <= 0 means full attention;
 * otherwise the query at p sees keys in (p - window, p]. */
typedef struct yx_layer {
    int32_t window;
    yx_rope rope;
} yx_layer;

/* Kernel choices, the counterpart of the reference's `Tuning`
 * (crates/yaxus-backend-gpu/src/device.rs:96-167).  Zero means "library default". */
typedef struct yx_tuning {
    int32_t force_path;      /* 0 auto, 1 SIMT split-key, 2 tensor split-key, 3 tcgen05 tiles */
    int32_t ctas_per_sm;     /* persistent CTAs per SM for the split-key kernels (0: default, 4 for the SIMT kernel and
                                for the tensor kernel one per SM with one SM left spare for the call behind) */
    int32_t share_prefix;    /* 0 default (on), 1 on, 2 off: read pages shared by several rows once */
    int32_t tile_min_rows;   /* rows of one sequence from which the tcgen05 tile kernel is used */
    int32_t cost32;          /* planner cost of a 64-key tile of an item with 32 padded query rows, */
    int32_t cost64;          /* and with 64, in 16ths of the cost of a 16-row item's tile */
    int32_t stages;          /* 64-key tiles in flight per SM in the tensor split-key kernel (2..5) */
    int32_t share_rows;      /* pass rows a shared-prefix item may hold (0: 16 / group, one MMA tile) */
    int32_t item_cost;       /* planner cost of starting an item, in 16ths of a tile, plus one (0: default) */
    int32_t fused_merge;     /* 1: the split-key kernel merges the triples itself; 0: a combine kernel does */
    int32_t tile_single;     /* 1: the tcgen05 tile kernel takes one query head per CTA (default: two) */
    int32_t min_piece;       /* fewest 64-key tiles the planner makes an item of when it cuts a run (0: default) */
    int32_t overlap_calls;   /* 2: an attention call that directly follows another one on the stream waits for it
                                before it reads anything; 3: it waits before its first write (0: default, that or,
                                where the call ahead filled every SM, before its CTAs leave) */
} yx_tuning;

/* What the last yx_attend / yx_attention call planned; for tests and benchmarks. */
typedef struct yx_plan_info {
    int32_t path;            /* 1 SIMT, 2 tensor split-key, 3 tcgen05 tiles (+2 if mixed) */
    int32_t n_ctas;
    int32_t n_items;
    int32_t n_parts;         /* partial (m,l,o) triples merged by the combine kernel */
    int64_t tiles;           /* 64-key tiles streamed */
    int64_t unique_kv_bytes; /* K+V bytes the plan reads, each shared page counted once */
    int64_t logical_kv_bytes;/* the same with every row's keys counted separately per row group */
    int32_t launches;        /* kernels launched by the call */
    int32_t shared_groups;   /* row groups made of several sequences over shared pages */
} yx_plan_info;

/* ---- context ------------------------------------------------------------------------ */

/* One context per GPU (the reference's `Gpu` device object, crates/yaxus-backend-gpu/src/lib.rs:235-246).
 * `stream` is a cudaStream_t to enqueue on, or NULL to create a private non-blocking stream
 * (to share the legacy default stream pass cudaStreamLegacy, not NULL). */
int yx_ctx_create(int device, void *stream, yx_ctx **out);
void yx_ctx_destroy(yx_ctx *ctx);
/* Sticky first error; YX_OK / "" when none. */
int yx_status(const yx_ctx *ctx);
const char *yx_last_error(const yx_ctx *ctx);
void yx_clear_error(yx_ctx *ctx);
/* Waits for the stream and folds kernel-reported failures into the sticky error: the check
 * the reference makes at read-back (crates/yaxus-model/src/lib.rs:187-197). */
int yx_sync(yx_ctx *ctx);
void *yx_stream(const yx_ctx *ctx);
int yx_set_tuning(yx_ctx *ctx, const yx_tuning *tuning);
int yx_last_plan(const yx_ctx *ctx, yx_plan_info *out);
/* Kernels this context has launched so far. */
int64_t yx_launch_count(const yx_ctx *ctx);
/* Per-kernel device time, the counterpart of the reference's YAXUS_PROFILE=2 timestamp
 * queries (crates/yaxus-backend-gpu/src/profile.rs:1-64).  Between begin and end every
 * split-key kernel and every combine kernel is bracketed by CUDA events on the stream;
 * yx_profile_end waits for the stream and returns the summed milliseconds and the number of
 * attention calls measured (at most 4096; later calls are not timed). */
int yx_profile_begin(yx_ctx *ctx);
int yx_profile_end(yx_ctx *ctx, float *split_ms, float *combine_ms, int *calls);

/* ---- tensors: the backend's `Tensor` plumbing and `SyncReadback::to_host`
 *      (crates/yaxus-model/src/lib.rs:177-185) ------------------------------------------ */
int yx_tensor_alloc(yx_ctx *ctx, size_t bytes, void **out_dev);
int yx_tensor_free(yx_ctx *ctx, void *dev);
/* Stream-ordered copies.  Host memory should be pinned for them to be asynchronous. */
int yx_upload(yx_ctx *ctx, void *dst_dev, const void *src_host, size_t bytes);
int yx_download(yx_ctx *ctx, void *dst_host, const void *src_dev, size_t bytes, int wait);
int yx_host_alloc(yx_ctx *ctx, size_t bytes, void **out_host);
int yx_host_free(yx_ctx *ctx, void *host);

/* ---- KV storage ---------------------------------------------------------------------- */

/* Backend::new_kv (crates/yaxus-model/src/lib.rs:118; cpu lib.rs:464-470): zeroed K and V
 * arenas of `pages` pages for each of `n_layers` layers.  `dtype` is the storage type: YX_F32
 * is the reference's; YX_F16 / YX_BF16 round on append (round-to-nearest-even).  The
 * physical layout is private; slot semantics (`page * 128 + pos % 128`) are the reference's. */
int yx_kv_create(yx_ctx *ctx, int n_layers, const yx_layer *layers, uint32_t pages, int hkv,
                 int head_dim, int dtype, uint32_t max_pos, yx_kv **out);
void yx_kv_destroy(yx_ctx *ctx, yx_kv *kv);
/* Backend::copy_page (lib.rs:120; cpu lib.rs:472-479): page src -> dst in every layer, K and V. */
int yx_kv_copy_page(yx_ctx *ctx, yx_kv *kv, uint32_t src, uint32_t dst);
/* Import / export of `n_pages` consecutive pages of one layer in the reference's layout
 * `[n_pages*128][hkv*128]` (cpu lib.rs:464-470), as raw storage elements (4 bytes each for
 * YX_F32, 2 otherwise).  Synchronous; for tests and for moving an existing cache in or out. */
int yx_kv_read_pages(yx_ctx *ctx, yx_kv *kv, int layer, uint32_t first_page, uint32_t n_pages, void *k_host,
                     void *v_host);
int yx_kv_write_pages(yx_ctx *ctx, yx_kv *kv, int layer, uint32_t first_page, uint32_t n_pages, const void *k_host,
                      const void *v_host);

/* ---- a pass -------------------------------------------------------------------------- */

/* Backend::begin_pass (lib.rs:123) with PassMeta's arrays (lib.rs:63-75).  The arrays are
 * copied before the call returns; the upload is ordered on the stream after the kernels of
 * earlier passes.  Rows of one sequence must be consecutive with consecutive positions. */
int yx_begin_pass(yx_ctx *ctx, uint32_t rows, const uint32_t *pos_host, const uint32_t *kv_slot_host,
                  const uint32_t *pt_off_host, const uint32_t *pages_host, uint32_t n_pages);

/* Backend::attention (lib.rs:132-140; cpu lib.rs:515-530): qkv `[rows][(hq+2hkv)*128]` f32;
 * per-head RMSNorm with weights (1 + g) and RoPE at each row's position on q and k; k and v
 * written to each row's slot of `layer`; then causal (sliding-window if the layer has a
 * window) GQA attention.  out `[rows][hq*128]` f32. */
int yx_attention(yx_ctx *ctx, yx_kv *kv, int layer, const float *qkv_dev, const float *q_norm_dev,
                 const float *k_norm_dev, int hq, float eps, float *out_dev);

/* The two halves of `attention`, for callers that already hold final q, k and v.
 * yx_kv_append: the scatter at the end of write_rows (cpu lib.rs:374-382): k_rows, v_rows
 * `[rows][hkv*128]` of `src_dtype` (YX_F32 or the cache's own type) to the rows' slots. */
int yx_kv_append(yx_ctx *ctx, yx_kv *kv, int layer, const void *k_rows_dev, const void *v_rows_dev,
                 int src_dtype);
/* attend (cpu lib.rs:389-427): q `[rows][hq*128]` of q_dtype, out likewise of out_dtype.
 * window: < 0 uses the layer's, 0 none, > 0 that many keys. */
int yx_attend(yx_ctx *ctx, yx_kv *kv, int layer, const void *q_dev, int q_dtype, int hq, int64_t window,
              void *out_dev, int out_dtype);

/* ---- split-key partials and their merge ---------------------------------------------- */

/* The (m, l, o) triple of the reference's split attention
 * (crates/yaxus-backend-gpu/src/shaders.rs:1466-1579) for the keys in [key_lo, key_hi) only:
 * m,l `[rows][hq]`, o `[rows][hq][128]` unnormalised; a (row, head) without a live key gets
 * (m, l) = (-1e30, 0).  Page-table entries of pages outside the range are never read. */
int yx_attend_partial(yx_ctx *ctx, yx_kv *kv, int layer, const void *q_dev, int q_dtype, int hq,
                      int64_t window, uint64_t key_lo, uint64_t key_hi, float *m_dev, float *l_dev,
                      float *o_dev);
/* attn_combine (shaders.rs:1581-1637): merges n_parts triples laid out `[n_parts][n]`,
 * `[n_parts][n][128]` (n = rows*hq), dropping parts with l <= 0 by value. */
int yx_lse_combine(yx_ctx *ctx, int n_parts, const float *m_dev, const float *l_dev, const float *o_dev,
                   size_t n, void *out_dev, int out_dtype);

/* ---- long-context decode with the keys split across GPUs ------------------------------ */

/* No counterpart in the reference (it is single-GPU).  One process per GPU; rank 0 makes an
 * id, every rank passes the same 128 bytes to yx_comm_create. */
int yx_comm_unique_id(void *out_id128);
int yx_comm_create(yx_ctx *ctx, int n_ranks, int rank, const void *id128);
int yx_comm_destroy(yx_ctx *ctx);
/* yx_attend_partial over this rank's [key_lo, key_hi), an NCCL all-gather of the triples,
 * and yx_lse_combine on every rank. */
int yx_attend_allgather(yx_ctx *ctx, yx_kv *kv, int layer, const void *q_dev, int q_dtype, int hq,
                        int64_t window, uint64_t key_lo, uint64_t key_hi, void *out_dev, int out_dtype);

/* ---- attention without allocation ----------------------------------------------------------- */

/* ---- The other operators of the reference's `Backend` trait --------------------------------
 * What `Model::forward` calls either side of attention (crates/yaxus-model/src/lib.rs:124-171), with
 * the CPU backend's arithmetic (crates/yaxus-backend-cpu/src/lib.rs:485-562).  Activations are
 * row-major f32 on the device; matrix weights and the embedding table are bf16 `[N, K]` as the
 * model files store them (upload them with yx_tensor_alloc + yx_upload: `load_weight`, cpu
 * lib.rs:455-462; the quantised formats of the reference are not taken); norm vectors are f32, as
 * for yx_attention.  All calls enqueue on the context's stream; only yx_argmax_rows waits. */

/* `embed` (lib.rs:125; cpu :485-497): out[r] = f32(table[ids[r]]), `table` bf16 [vocab, h].  The
 * reference takes the ids from the pass; here they come with the call and are copied at once. */
int yx_embed(yx_ctx *ctx, const void *table_bf16_dev, uint32_t vocab, uint32_t h, const uint32_t *ids_host,
             uint32_t rows, float *out_dev);
/* `rmsnorm` (lib.rs:126; cpu :296-302, :499-507): out = (offset + w) * (x * rsqrt(mean(x^2) + eps)). */
int yx_rmsnorm(yx_ctx *ctx, const float *x_dev, const float *w_dev, uint32_t rows, uint32_t cols, float offset,
               float eps, float *out_dev);
/* `add_norm` (lib.rs:149-162): x += rmsnorm(delta, post_w, post_offset); out = rmsnorm(x, pre_w,
 * pre_offset).  One kernel. */
int yx_add_norm(yx_ctx *ctx, float *x_dev, const float *delta_dev, const float *post_w_dev, float post_offset,
                const float *pre_w_dev, float pre_offset, float eps, uint32_t rows, uint32_t cols, float *out_dev);
/* `matmul` (lib.rs:128; cpu :314-357, :509-514): out [rows, n] = x [rows, k] . w[n, k]^T, f32 sums. */
int yx_matmul(yx_ctx *ctx, const float *x_dev, const void *w_bf16_dev, uint32_t rows, uint32_t n, uint32_t k,
              float *out_dev);
/* `matmul_glu` (lib.rs:164-168): swiglu(x . w^T) for w = [gate; up]; out is [rows, n / 2]. */
int yx_matmul_glu(yx_ctx *ctx, const float *x_dev, const void *w_bf16_dev, uint32_t rows, uint32_t n, uint32_t k,
                  float *out_dev);
/* `swiglu` (lib.rs:142; cpu :532-542): [rows, 2 inner] -> [rows, inner], g / (1 + exp(-g)) * u. */
int yx_swiglu(yx_ctx *ctx, const float *x_dev, uint32_t rows, uint32_t inner, float *out_dev);
/* `add_assign` (lib.rs:144; cpu :544-547): a += b over n elements. */
int yx_add_assign(yx_ctx *ctx, float *a_dev, const float *b_dev, size_t n);
/* `select_rows` (lib.rs:170; cpu :549-552): out[i] = x[rows[i]]. */
int yx_select_rows(yx_ctx *ctx, const float *x_dev, uint32_t src_rows, uint32_t cols, const uint32_t *rows_host,
                   uint32_t n, float *out_dev);
/* `SyncReadback::argmax_rows` (lib.rs:177-185; cpu :430-441, :556-558): the first largest value of
 * every row, NaNs skipped, 0 for a row without a number.  Waits for the device, and so reports
 * whatever error the stream's earlier work raised.  `to_host` is yx_download with wait = 1. */
int yx_argmax_rows(yx_ctx *ctx, const float *logits_dev, uint32_t rows, uint32_t cols, uint32_t *out_host);

/* No counterpart in the reference.  Same result as yx_attend (cpu lib.rs:389-427) for passes of
 * at most YX_STATIC_MAX_ROW_HEADS (row, query head) pairs, but the call allocates nothing: the
 * partial triples of its split-key kernel (YX_STATIC_SPLITS runs of keys per row and KV head) live
 * in an array built into the library's device image (4 MiB + 64 KiB per device), not in a
 * workspace from the allocator.  For callers that have handed all free device memory to the KV
 * page pool, or that cannot take the device-wide stall of an allocation inside their decode loop.
 * Larger passes are rejected with YX_ERR_INVALID and a message naming the limit.
 * The context's device must be the current device.  The first call on a device looks the
 * array's address up; make it before any stream capture begins.  Where the CUDA runtime loads
 * modules lazily, that first call is also where the driver commits the 4 MiB of the array: free
 * device memory drops once, there, and not again.  The array is one per device context (one per
 * device for a process that only uses the runtime API): calls whose kernels may overlap on a
 * device race on it, so order them on one stream or with events.  Nothing in it needs clearing
 * between calls. */
#define YX_STATIC_SPLITS 8
#define YX_STATIC_MAX_ROW_HEADS 1024
int yx_attend_static(yx_ctx *ctx, yx_kv *kv, int layer, const void *q_dev, int q_dtype, int hq, int64_t window,
                     void *out_dev, int out_dtype);

#ifdef __cplusplus
}
#endif
#endif
