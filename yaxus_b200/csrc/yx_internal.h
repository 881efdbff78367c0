// Internal declarations shared by the translation units of libyaxus_cuda.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/yaxus_cuda.h"

namespace yx {

constexpr int PAGE = YX_PAGE;   // tokens per page (crates/yaxus-model/src/kv.rs:17)
constexpr int D = YX_HEAD_DIM;  // head_dim
constexpr int TILE_KEYS = 64;   // keys per streamed tile (half a page)
constexpr int MAX_ITEM_ROWS = 16;

// ----------------------------------------------------------------------------------------
// KV storage layout (private to the library; `Kv` is opaque to yaxus-model).
//
// Per layer there is one K and one V arena.  A (page, kv head) block holds the page's 128
// tokens of that head contiguously, so that a split-key CTA streams whole blocks with bulk
// copies instead of gathering 256-byte pieces from token-major rows.
//   f32  : [page][hkv][tok 128][128 f32]                      (64 KiB per block)
//   16bit: [page][hkv][dhalf 2][tok 128][64 elements = 128 B] (32 KiB per block)
//          with the eight 16-byte chunks of every 128-byte row stored at chunk ^ (tok & 7).
// The 16-bit form is exactly the 128-byte-swizzled shared-memory layout that ldmatrix reads
// without bank conflicts and that tcgen05 matrix descriptors name as SWIZZLE_128B, so a bulk
// copy of any run of rows lands ready for the tensor cores.
// ----------------------------------------------------------------------------------------
__host__ __device__ inline size_t kv_block_elems() { return (size_t)PAGE * D; }

// Element offset of (page, kvh, tok, dim) inside a layer's arena, 16-bit storage.
__host__ __device__ inline size_t kv_off16(uint32_t page, int hkv, int kvh, int tok, int dim) {
    size_t blk = ((size_t)page * hkv + kvh) * kv_block_elems();
    int dh = dim >> 6, c = (dim & 63) >> 3, e = dim & 7;
    return blk + (size_t)dh * (PAGE * 64) + (size_t)tok * 64 + (size_t)((c ^ (tok & 7)) << 3) + e;
}
// Element offset, f32 storage.
__host__ __device__ inline size_t kv_off32(uint32_t page, int hkv, int kvh, int tok, int dim) {
    return ((size_t)page * hkv + kvh) * kv_block_elems() + (size_t)tok * D + dim;
}

// ----------------------------------------------------------------------------------------
// Plan of one attention call (host-built, uploaded with the pass).
// ----------------------------------------------------------------------------------------

// One piece of split-key work: some rows of the pass (they share a page table over the
// item's keys) against the keys of tiles [tile_begin, tile_end) of one KV head.
struct alignas(16) Item {
    uint32_t tile_begin;   // in units of TILE_KEYS keys of logical position
    uint32_t tile_end;     // exclusive
    uint32_t key_lo;       // first key any row of the item may see (inclusive)
    uint32_t key_hi;       // last key any row of the item may see (inclusive)
    uint32_t pt_off;       // offset of the page table in the pass's `pages`
    uint16_t kv_head;
    uint16_t n_rows;
    uint16_t rows[MAX_ITEM_ROWS];        // pass rows
    uint32_t part[MAX_ITEM_ROWS];        // partial slot of each row for this KV head
    uint32_t mt;                         // padded query rows (n_rows * group rounded up): 16, 32 or 64
    uint32_t flags;                      // bit 0: other items read the same pages; bits 1..31: the first position
                                         // the item's sequences append in this pass (keys from there on may be new)
};
static_assert(sizeof(Item) == 128, "Item is 128 bytes");

// Where the combine kernel finds the partials of one (row, kv head).
struct Merge {
    uint32_t first;  // first partial slot
    uint32_t count;  // slots
};

// ---- the same plan, resolved for the streaming kernel --------------------------------------
// The tensor split-key kernel never walks a page table: the host, which holds the tables
// anyway, resolves every 64-key tile to the (page, KV head) block it lives in, so that the
// kernel's copy engine is fed from one flat array and nothing on the device waits on a
// dependent lookup.

// What one persistent CTA works through.
struct CtaHdr {
    uint32_t item_begin, item_end;   // ItemRec range
    uint32_t tile_begin, tile_end;   // TileDesc range (the items' tiles, in order)
};

// One 64-key tile: where it is and which of its rows hold keys of the item.
struct TileDesc {
    uint32_t block;   // page * hkv + kv_head: index of the 32 KiB block in the K and V arenas
    uint32_t info;    // bit 0: which half of the page; bits 1-7: first row; bits 8-15: rows (1..64);
                      // bit 16: other items read the same tile (keep it in L2);
                      // bit 17: the tile may hold rows that this pass appends (see TILE_FRESH)
};
// A tile is "fresh" when it covers positions at or after the first row its sequence has in this
// pass: the kernel that ran just before the attention kernel (the append) may have written it.
// Every other tile was complete before that kernel started, so the attention kernel may copy it
// before it waits for its grid dependency.
// Where the merge kernel's time stamps start in a diagnostic trace buffer (u64 slots; the split-key
// kernel has 16 per CTA below it), four per merge CTA.
constexpr int TRACE_MERGE_BASE = 160 * 16;
constexpr uint32_t TILE_REUSED = 1u << 16;
constexpr uint32_t TILE_FRESH = 1u << 17;

// An item as the kernel reads it: a header and six words per pass row.  On the device the records
// are packed at the size of the plan's longest one (rounded up to 16 bytes, one bulk copy each).
struct alignas(16) ItemRec {
    uint32_t w[128];
};
constexpr int IR_TILES = 0;       // tiles of the item
constexpr int IR_KEY0 = 1;        // logical position of the first tile's first key
constexpr int IR_HEAD_ROWS = 2;   // kv_head | n_rows << 16
constexpr int IR_MT = 3;          // padded query rows: 16, 32, 64
constexpr int IR_ROW0 = 4;        // then six words per pass row:
constexpr int IR_ROW_WORDS = 6;   //   first key seen, last key seen, partial slot, pass row, first slot, slots
constexpr int IRR_KLO = 0, IRR_KHI = 1, IRR_PART = 2, IRR_ROW = 3, IRR_FIRST = 4, IRR_COUNT = 5;

// What a persistent CTA of the split-key kernel needs before its first global load returns; it
// travels in kernel-parameter space: the CTA's span, its first tiles and the rows of its first
// item.  A cold global load at kernel start costs over a microsecond, and three of them in a
// chain (span -> descriptors -> data) were once the largest single cost of the kernel.
constexpr int PROLOGUE_TILES = 4;
struct CtaPrologue {
    CtaHdr hdr;
    TileDesc first[PROLOGUE_TILES];
    uint32_t head_rows, mt;            // of the first item: kv_head | n_rows << 16, padded query rows
    uint16_t rows[MAX_ITEM_ROWS];      // its pass rows
};

// One item of the tiled (tcgen05) kernel: up to 128 consecutive rows of one sequence for one
// query head, against pages [page_begin, page_end) of the sequence's table.
struct TileItem {
    uint32_t row0;        // first pass row
    uint32_t n_rows;      // 1..128; row r sits at position pos0 + r
    uint32_t pos0;
    uint32_t pt_off;
    uint16_t head;        // query head
    uint16_t kv_head;
    uint32_t page_begin, page_end;
    uint32_t pad_;
};
static_assert(sizeof(TileItem) == 32, "TileItem is 32 bytes");

struct Plan {
    int path = 0;
    int n_ctas = 0;
    std::vector<Item> items;
    std::vector<uint32_t> cta_begin;    // n_ctas + 1 offsets into items
    std::vector<Merge> merges;          // [rows][hkv]
    uint32_t n_parts = 0;
    // resolved form (filled when PlanParams::resolve is set)
    std::vector<TileItem> tile_items;   // rows handled by the tiled kernel (not in `items`), grouped by CTA
    std::vector<uint32_t> tile_cta_begin;   // offsets into tile_items per persistent CTA, plus the end
    std::vector<CtaHdr> cta_hdr;
    std::vector<TileDesc> tiles;
    std::vector<ItemRec> recs;
    std::vector<CtaPrologue> prologue;  // one per CTA (resolved form)
    std::vector<uint32_t> scratch_dense, scratch_seen, scratch_once;   // planner scratch, kept for its capacity
    std::vector<uint64_t> scratch_table;
    std::vector<TileItem> scratch_tile_items;
    std::vector<uint32_t> scratch_lengths, scratch_links;
    uint64_t last_limit = 0;            // per-CTA load limit the last plan settled on (starting point of the next search)
    // What the last plan was built from, so that a pass with the same shape (the next decode step:
    // every row one key further, no new tile, no new page) only has its key ranges patched in.
    struct UnitSig { uint32_t pt_off, t0, n, n_rows, reused, fresh_tile; };
    bool sig_valid = false;
    uint32_t sig_rows_in_pass = 0;
    int sig_params[10] = {};
    int64_t sig_window = 0;
    std::vector<UnitSig> sig_units;
    std::vector<uint16_t> sig_unit_rows;
    std::vector<uint32_t> sig_pages;
    std::vector<uint32_t> item_unit;    // the unit each item is a piece of
    std::vector<uint32_t> item_tile0;   // index of each item's first tile descriptor
    bool patched = false;               // the last build took the short way
    bool single_use = false;            // every tile not marked as reused is read by exactly one item
    bool has_empty_rows = false;        // some (row, kv head) has no item: no live key in the range
    yx_plan_info info{};
};

struct PassHost {
    uint32_t rows = 0;
    std::vector<uint32_t> pos, kv_slot, pt_off, pages;
    // taken once at begin_pass, so that every attention call of the pass checks them in O(1)
    uint32_t max_pos_seen = 0;    // largest position of a row
    uint32_t max_page_seen = 0;   // largest page id in `pages`
    uint32_t max_slot_seen = 0;   // largest kv_slot of a row
};

struct PlanParams {
    int hkv, group;          // group = hq / hkv
    int64_t window;          // <= 0: none
    uint64_t key_lo, key_hi; // extra restriction [key_lo, key_hi) (UINT64_MAX = none)
    int max_rows;            // rows per item (1 for the SIMT kernel)
    int n_ctas;              // persistent CTAs to fill
    bool share_prefix;
    int esize;               // bytes per stored element
    int w32, w64;            // cost of a tile of an item with 32 / 64 padded rows, in 16ths of a 16-row tile's
    bool resolve;            // also build the resolved form for the streaming kernel
    int tile_min_rows;       // groups of at least this many rows go to the tiled kernel (0 = none)
    bool tile_pairs;         // tile items take two query heads of a KV head each (needs an even group)
    int tile_ctas;           // persistent CTAs of the tiled kernel (0: one per item)
    int share_rows;          // pass rows a shared item may hold (0 = one 16-row MMA tile's worth)
    int item_cost;           // fixed cost of an item, in 16ths of a 16-row tile's
    int min_piece;           // fewest tiles worth an item of their own
};

// Builds the split-key plan.  Throws std::string on a malformed pass.
void build_split_plan(const PassHost &pass, const PlanParams &pp, Plan &out);

}  // namespace yx

// ----------------------------------------------------------------------------------------
// Objects behind the opaque handles.
// ----------------------------------------------------------------------------------------
struct yx_kv {
    int n_layers = 0, hkv = 0, dtype = 0, esize = 4;
    uint32_t pages = 0, max_pos = 0;
    size_t layer_bytes = 0;            // bytes of one K (or V) arena
    std::vector<yx_layer> layers;
    char *k_base = nullptr;            // [layer][arena]
    char *v_base = nullptr;
    void *rope_dev = nullptr;          // yx_rope per layer
    // Set (and never cleared) by the kernels that write V when a bf16 value of magnitude 65536 or
    // more, or a non-finite one, goes into the cache: such a value does not fit f16, and the tile
    // kernel then keeps V in bf16 (two MMAs per product) instead of converting it (one).
    uint32_t *wide_v_dev = nullptr;
    char *k(int layer) const { return k_base + (size_t)layer * layer_bytes; }
    char *v(int layer) const { return v_base + (size_t)layer * layer_bytes; }
};

struct yx_dev_status {
    int code;      // first failed device check (0 = none)
    int where;     // kernel-specific location
    int a, b;
    unsigned int expired;   // one bit per `where` (mod 32) of every wait that ran out, not just the first
};

struct ncclComm;

struct yx_ctx;
#ifdef YX_TRACE
void host_clock_start(yx_ctx *ctx);
void host_clock_lap(yx_ctx *ctx, int phase);   // adds the time since the last start or lap to host_ns[phase]
#else
inline void host_clock_start(yx_ctx *) {}
inline void host_clock_lap(yx_ctx *, int) {}
#endif

struct yx_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    int status = 0;
    std::string error;
    yx_tuning tuning{};
    yx_plan_info last_plan{};
    int64_t launches = 0;
    bool smem_configured[12] = {};          // per-kernel opt-in to large dynamic shared memory
    void *trace_buf = nullptr;             // device buffer for per-CTA kernel timestamps (builds with -DYX_TRACE)
    // Host time spent in the phases of an attention call, in ns (builds with -DYX_TRACE): 0 pass checks,
    // 1 planning, 2 laying the plan out in the staging buffer, 3 its upload call, 4 the append launch,
    // 5 the attention kernel launches, 6 the merge launch.
    double host_ns[8] = {};
    int64_t host_mark = 0;
    bool skip_merge = false;               // measurement hook: leave the merge of the triples out
    // What this context last put on its stream, for the split-key kernel's early K/V copies: it may
    // copy tiles before waiting for the kernel ahead of it only if that kernel cannot have written
    // them (an append of the current pass writes the marked tiles only; attention kernels write none).
    // LAST_SPLIT_KEY is LAST_ATTEND narrowed: the call launched the split-key kernel (and its merge) and
    // nothing else.  The split-key kernel of the next call may then do all its reading without waiting
    // (see AttendArgs::late_wait).
    enum { LAST_OTHER = 0, LAST_APPEND, LAST_ATTEND, LAST_KV_WRITE, LAST_SPLIT_KEY };
    int last_launch = LAST_OTHER;
    // What the last attention call wrote (its output and, for partial calls, its triples): a call whose
    // queries lie in there reads the result of the call ahead and must wait for it like any other.
    struct Range {
        uintptr_t lo = 0, hi = 0;
    } last_written[4];
    uint64_t last_append_serial = 0;

    yx_dev_status *dev_status = nullptr;   // pinned, mapped

    // per-kernel timing (yx_profile_begin / yx_profile_end)
    bool profiling = false;
    std::vector<cudaEvent_t> prof_events;  // 4 per call: split start/stop, combine start/stop
    size_t prof_used = 0;

    // pass metadata
    yx::PassHost pass;
    bool have_pass = false;
    uint64_t pass_serial = 0;
    uint32_t *d_meta = nullptr;            // pos | kv_slot | pt_off | pages
    size_t d_meta_cap = 0;
    uint32_t *d_pos = nullptr, *d_slot = nullptr, *d_ptoff = nullptr, *d_pages = nullptr;

    // pinned staging ring for stream-ordered uploads
    struct Stage {
        void *host = nullptr;
        size_t cap = 0;
        cudaEvent_t done = nullptr;
        bool busy = false;
    };
    std::vector<Stage> ring;
    size_t ring_next = 0;

    // cached plans of the current pass
    struct CachedPlan {
        uint64_t pass_serial = 0;
        int hkv = 0, group = 0, max_rows = 0, n_ctas = 0, esize = 0, w32 = 0, w64 = 0;
        int64_t window = 0;
        uint64_t key_lo = 0, key_hi = 0;
        bool share = false, resolve = false;
        int share_rows = 0, item_cost = 0, min_piece = 0;
        yx::Plan plan;
        char *dev = nullptr;       // items | cta_begin | merges | cta_hdr | tiles | recs
        size_t dev_cap = 0;
        yx::Item *d_items = nullptr;
        uint32_t *d_cta_begin = nullptr;
        yx::Merge *d_merges = nullptr;
        yx::CtaHdr *d_cta_hdr = nullptr;
        yx::TileDesc *d_tiles = nullptr;
        const char *d_recs = nullptr;   // records packed at rec_stride bytes each
        uint32_t rec_stride = 0;
        yx::TileItem *d_tile_items = nullptr;
        uint32_t *d_tile_cta_begin = nullptr;
        int tile_min_rows = 0;
        bool tile_pairs = false;
    };
    std::vector<CachedPlan> plans;

    // scratch: partial triples
    float *ws_o = nullptr;   // [n_parts][group][128]
    float *ws_ml = nullptr;  // [n_parts][group][2]
    size_t ws_o_cap = 0, ws_ml_cap = 0;
    int ws_set = 0;          // which of the two sets of partial buffers the last attention call took
    int last_split_ctas = 0; // CTAs of the last call's split-key kernel (0: that call had none)
    float *q_tmp = nullptr;  // normalised, rotated q of yx_attention
    size_t q_tmp_cap = 0;
    uint32_t *counters = nullptr;   // arrival counters of the fused merge; all zero between launches
    size_t counters_cap = 0;
    float *mm_part = nullptr;              // per-k-chunk partial sums of the matmul
    size_t mm_part_cap = 0;
    void *mm_packed = nullptr;             // the pass rows of a matmul as bf16 MMA fragments
    size_t mm_packed_cap = 0;
    void *lt_handle = nullptr;             // cublasLtHandle_t, made at the first matmul of many rows
    void *lt_workspace = nullptr;
    size_t lt_workspace_cap = 0;
    uint32_t *idx_dev = nullptr;           // token ids / row indices / argmax results of the model operators
    size_t idx_cap = 0;

    // multi-GPU
    ncclComm *comm = nullptr;
    int n_ranks = 1, rank = 0;
    float *gather_buf = nullptr;
    size_t gather_cap = 0;
};

namespace yx {

int fail(yx_ctx *ctx, int code, const std::string &msg);
// When profiling, records the next timing event of the current attention call (which = 0..3).
void profile_mark(yx_ctx *ctx, int which);
int check_cuda(yx_ctx *ctx, cudaError_t e, const char *what);
// Stream-ordered upload of `bytes` from pageable host memory through the pinned ring.
int upload_ordered(yx_ctx *ctx, void *dst_dev, const void *src_host, size_t bytes);
int ensure_buffer(yx_ctx *ctx, void **buf, size_t *cap, size_t bytes);
// yx_attend over the keys [key_lo, key_hi) only: what one rank alone has to do for yx_attend_allgather.
int attend_key_range(yx_ctx *ctx, yx_kv *kv, int layer, const void *q, int q_dtype, int hq, int64_t window, uint64_t key_lo,
                     uint64_t key_hi, void *out, int out_dtype);
// Destroys the context's cuBLASLt handle, if it made one.
void release_matmul_library(yx_ctx *ctx);

// Kernel launchers (each returns a yx_error and counts its launches in ctx->launches).
int launch_append(yx_ctx *ctx, yx_kv *kv, int layer, const void *k_rows, const void *v_rows, int src_dtype);
int launch_qk_rope_append(yx_ctx *ctx, yx_kv *kv, int layer, const float *qkv, const float *q_norm,
                          const float *k_norm, int hq, float eps, float *q_out);
int launch_copy_page(yx_ctx *ctx, yx_kv *kv, uint32_t src, uint32_t dst);
int launch_page_io(yx_ctx *ctx, yx_kv *kv, int layer, uint32_t first_page, uint32_t n_pages, void *k_lin, void *v_lin,
                   bool write);

struct AttendArgs {
    uint32_t rows;           // rows of the pass (of q and out)
    const void *q;
    int q_dtype;
    int hq;
    int group;
    const char *k_arena;
    const char *v_arena;
    int hkv;
    int kv_dtype;
    uint32_t kv_pages;
    int64_t window;
    uint64_t key_lo, key_hi;
    const Item *items;
    const uint32_t *cta_begin;
    int n_ctas;
    float *part_o;
    float *part_ml;
    // resolved plan and fused merge (tensor kernel)
    const CtaHdr *cta_hdr;
    const TileDesc *tiles;
    const char *recs;        // item records, rec_stride bytes apart (only the words the items' rows use are uploaded)
    uint32_t rec_stride;
    bool single_use;
    const Plan *plan;        // host copy, for what is passed in kernel-parameter space
    int n_stages;            // copy ring depth (0 = default)
    bool early_kv;           // unmarked tiles may be copied before the grid dependency wait
    bool late_wait;          // the kernels ahead are a split-key attention call of this context and its merge, and
                             // everything before that call is complete once this kernel runs: keys, values,
                             // queries and the plan are read at once, and the grid dependency is waited for only
                             // before the first write (the partial buffers, which the merge ahead still reads).
                             // Not set when the queries overlap what that call writes.
    bool wait_at_end;        // with late_wait: the CTAs wait before they leave instead of before their first write
                             // (the call ahead had a CTA on every SM: see attend_impl)
    bool fused;              // merge inside the split-key kernel
    uint32_t *counters;      // one per (pass row, kv head), zero between launches
    void *out;               // normalised output, or null
    int out_dtype;
    float *m_out, *l_out, *o_out;   // merged triple, or null
};
struct TileArgs {
    const void *q;
    int q_dtype, hq, group, hkv, kv_dtype;
    const char *k_arena, *v_arena;
    uint32_t kv_pages;
    int64_t window;
    const TileItem *items;
    int n_items;
    const uint32_t *cta_begin;   // n_ctas + 1 offsets into items (persistent kernel)
    int n_ctas;
    void *out;
    int out_dtype;
    bool pairs;              // items name the first of two query heads of one KV head
    const uint32_t *wide_v;  // the cache's "V holds values f16 cannot" flag (device)
};
int launch_prefill_tc(yx_ctx *ctx, const TileArgs &a);
int launch_attend_simt(yx_ctx *ctx, const AttendArgs &a);
int launch_attend_mma(yx_ctx *ctx, const AttendArgs &a);
// Writes the empty mark (-1e30, 0, 0) for n (row, head) triples.
int launch_fill_empty(yx_ctx *ctx, size_t n, float *m, float *l, float *o);
int launch_combine(yx_ctx *ctx, const Merge *merges, const float *part_o, const float *part_ml, int rows,
                   int hq, int group, void *out, int out_dtype, float *m_out, float *l_out, float *o_out, bool chained = false);
// Parts with strides (in floats) sm, sl, so between consecutive parts of m, l and o.
int launch_combine_strided(yx_ctx *ctx, int n_parts, const float *m, const float *l, const float *o, size_t sm,
                           size_t sl, size_t so, size_t n, void *out, int out_dtype);

}  // namespace yx
