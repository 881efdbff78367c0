// The C ABI of libyaxus_cuda: contexts, KV storage, pass metadata and the attention entry
// points.  Kernels live in kv_ops.cu, attend_simt.cu, attend_mma.cu (split-key, 16-bit caches),
// prefill_tc.cu (tcgen05 tiles for prompt chunks) and combine.cu.
#include <string.h>

#include <algorithm>
#include <new>

#include "yx_internal.h"

namespace yx {

int fail(yx_ctx *ctx, int code, const std::string &msg) {
    if (ctx && ctx->status == YX_OK) {
        ctx->status = code;
        ctx->error = msg;
    }
    return code;
}

int check_cuda(yx_ctx *ctx, cudaError_t e, const char *what) {
    if (e == cudaSuccess) return YX_OK;
    int code = e == cudaErrorMemoryAllocation ? YX_ERR_OOM : YX_ERR_CUDA;
    return fail(ctx, code, std::string(what) + ": " + cudaGetErrorString(e));
}

void profile_mark(yx_ctx *ctx, int which) {
    if (!ctx->profiling) return;
    size_t idx = ctx->prof_used * 4 + which;
    if (idx >= ctx->prof_events.size()) return;
    cudaEventRecord(ctx->prof_events[idx], ctx->stream);
    if (which == 3) ctx->prof_used++;
}

int ensure_buffer(yx_ctx *ctx, void **buf, size_t *cap, size_t bytes) {
    if (bytes <= *cap && *buf) return YX_OK;
    size_t want = std::max<size_t>(bytes, 256);
    want = want + want / 2;
    if (*buf) {
        // Kernels queued earlier may still use the old buffer.
        if (int rc = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "sync before growing a buffer")) return rc;
        cudaFree(*buf);
        *buf = nullptr;
        *cap = 0;
    }
    void *p = nullptr;
    if (int rc = check_cuda(ctx, cudaMalloc(&p, want), "cudaMalloc (workspace)")) return rc;
    *buf = p;
    *cap = want;
    return YX_OK;
}

// The reference writes pass metadata through its command stream so that it lands after the
// kernels of earlier passes (crates/yaxus-backend-gpu/src/dev/wgpu/mod.rs:284-294).  Here a
// ring of pinned buffers does the same: the caller's arrays are copied at once, the
// host-to-device copy is ordered on the stream, and a buffer is reused only after its copy.
// A pinned staging buffer of at least `bytes`, free to write (its previous upload has left it).
int stage_acquire(yx_ctx *ctx, size_t bytes, void **host) {
    if (ctx->ring.empty()) ctx->ring.resize(8);
    yx_ctx::Stage &st = ctx->ring[ctx->ring_next];
    if (st.busy) {
        if (int rc = check_cuda(ctx, cudaEventSynchronize(st.done), "wait for a staging buffer")) return rc;
        st.busy = false;
    }
    if (st.cap < bytes) {
        if (st.host) cudaFreeHost(st.host);
        st.host = nullptr;
        st.cap = 0;
        size_t want = std::max<size_t>(bytes + bytes / 2, 4096);
        if (int rc = check_cuda(ctx, cudaMallocHost(&st.host, want), "cudaMallocHost (staging)")) return rc;
        st.cap = want;
    }
    if (!st.done)
        if (int rc = check_cuda(ctx, cudaEventCreateWithFlags(&st.done, cudaEventDisableTiming), "cudaEventCreate")) return rc;
    *host = st.host;
    return YX_OK;
}

// Sends the buffer stage_acquire last returned, stream-ordered, and moves on to the next one.
int stage_commit(yx_ctx *ctx, void *dst_dev, size_t bytes) {
    yx_ctx::Stage &st = ctx->ring[ctx->ring_next];
    ctx->ring_next = (ctx->ring_next + 1) % ctx->ring.size();
    if (int rc = check_cuda(ctx, cudaMemcpyAsync(dst_dev, st.host, bytes, cudaMemcpyHostToDevice, ctx->stream), "upload"))
        return rc;
    if (int rc = check_cuda(ctx, cudaEventRecord(st.done, ctx->stream), "cudaEventRecord")) return rc;
    st.busy = true;
    ctx->last_launch = yx_ctx::LAST_OTHER;
    return YX_OK;
}

int upload_ordered(yx_ctx *ctx, void *dst_dev, const void *src_host, size_t bytes) {
    if (bytes == 0) return YX_OK;
    void *host = nullptr;
    if (int rc = stage_acquire(ctx, bytes, &host)) return rc;
    memcpy(host, src_host, bytes);
    return stage_commit(ctx, dst_dev, bytes);
}

namespace {

bool valid_dtype(int d) { return d == YX_F32 || d == YX_F16 || d == YX_BF16; }

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
        else prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

int fold_device_status(yx_ctx *ctx) {
    if (ctx->dev_status && ctx->dev_status->code != 0) {
        yx_dev_status s = *ctx->dev_status;
        ctx->dev_status->code = 0;
        ctx->dev_status->expired = 0;
        // A kernel that gave up may have left arrival counters of the fused merge non-zero.
        if (ctx->counters) cudaMemsetAsync(ctx->counters, 0, ctx->counters_cap, ctx->stream);
        return fail(ctx, YX_ERR_DEVICE,
                    "a kernel reported a failed check: code " + std::to_string(s.code) + " at " +
                        std::to_string(s.where) + " (" + std::to_string(s.a) + ", " + std::to_string(s.b) + ")" +
                        (s.expired ? ", waits that ran out: mask " + std::to_string(s.expired) : std::string()));
    }
    return YX_OK;
}

// Finds or builds the split-key plan of the current pass for these parameters, and makes
// sure it is on the device.
int get_plan(yx_ctx *ctx, const PlanParams &pp, yx_ctx::CachedPlan **out) {
    for (auto &cp : ctx->plans) {
        if (cp.pass_serial == ctx->pass_serial && cp.hkv == pp.hkv && cp.group == pp.group &&
            cp.max_rows == pp.max_rows && cp.n_ctas == pp.n_ctas && cp.window == pp.window &&
            cp.key_lo == pp.key_lo && cp.key_hi == pp.key_hi && cp.share == pp.share_prefix && cp.esize == pp.esize &&
            cp.w32 == pp.w32 && cp.w64 == pp.w64 && cp.resolve == pp.resolve && cp.share_rows == pp.share_rows && cp.item_cost == pp.item_cost && cp.min_piece == pp.min_piece && cp.tile_min_rows == pp.tile_min_rows && cp.tile_pairs == pp.tile_pairs) {
            *out = &cp;
            return YX_OK;
        }
    }
    // Reuse the slot of an older pass, else add one (a pass rarely needs more than two:
    // full-attention layers and sliding-window layers).
    yx_ctx::CachedPlan *slot = nullptr;
    for (auto &cp : ctx->plans)
        if (cp.pass_serial != ctx->pass_serial) {
            slot = &cp;
            break;
        }
    if (!slot) {
        if (ctx->plans.size() >= 8) {
            slot = &ctx->plans[0];
        } else {
            ctx->plans.emplace_back();
            slot = &ctx->plans.back();
        }
    }
    host_clock_lap(ctx, 0);
    try {
        build_split_plan(ctx->pass, pp, slot->plan);
    } catch (const std::string &msg) {
        slot->pass_serial = 0;
        return fail(ctx, YX_ERR_INVALID, "attention plan: " + msg);
    } catch (const std::bad_alloc &) {
        slot->pass_serial = 0;
        return fail(ctx, YX_ERR_OOM, "attention plan: out of host memory");
    }
    host_clock_lap(ctx, 1);
    slot->pass_serial = ctx->pass_serial;
    slot->hkv = pp.hkv;
    slot->group = pp.group;
    slot->max_rows = pp.max_rows;
    slot->n_ctas = pp.n_ctas;
    slot->window = pp.window;
    slot->key_lo = pp.key_lo;
    slot->key_hi = pp.key_hi;
    slot->share = pp.share_prefix;
    slot->esize = pp.esize;
    slot->w32 = pp.w32;
    slot->w64 = pp.w64;
    slot->resolve = pp.resolve;
    slot->share_rows = pp.share_rows;
    slot->item_cost = pp.item_cost;
    slot->min_piece = pp.min_piece;
    slot->tile_min_rows = pp.tile_min_rows;
    slot->tile_pairs = pp.tile_pairs;

    const Plan &pl = slot->plan;
    auto pad16 = [](size_t n) { return (n + 15) / 16 * 16; };
    const size_t items_b = pp.resolve ? 0 : pl.items.size() * sizeof(Item);
    const size_t cta_b = pp.resolve ? 0 : pad16(pl.cta_begin.size() * sizeof(uint32_t));
    const size_t mer_b = pad16(pl.merges.size() * sizeof(Merge));
    const size_t hdr_b = pad16(pl.cta_hdr.size() * sizeof(CtaHdr));
    const size_t til_b = pad16(pl.tiles.size() * sizeof(TileDesc));
    // Item records go up packed: only the words that the item with the most rows uses, each.
    int most_rows = 1;
    for (const Item &it : pl.items) most_rows = std::max(most_rows, (int)it.n_rows);
    const size_t rec_stride = pad16((size_t)(IR_ROW0 + IR_ROW_WORDS * most_rows) * 4);
    const size_t rec_b = pp.resolve ? pl.items.size() * rec_stride : 0;
    const size_t tit_b = pl.tile_items.size() * sizeof(TileItem);
    const size_t tcb_b = pad16(pl.tile_cta_begin.size() * sizeof(uint32_t));
    const size_t total = items_b + cta_b + mer_b + hdr_b + til_b + rec_b + tit_b + tcb_b;
    if (int rc = ensure_buffer(ctx, (void **)&slot->dev, &slot->dev_cap, total)) {
        slot->pass_serial = 0;
        return rc;
    }
    // The parts are laid out straight in a pinned staging buffer (padding bytes are never read).
    char *blob = nullptr;
    if (total > 0)
        if (int rc = stage_acquire(ctx, total, (void **)&blob)) {
            slot->pass_serial = 0;
            return rc;
        }
    size_t at = 0;
    auto put = [&](const void *src, size_t bytes, size_t padded) {
        if (bytes) memcpy(blob + at, src, bytes);
        size_t here = at;
        at += padded;
        return here;
    };
    const size_t o_items = put(pl.items.data(), items_b, items_b);
    const size_t o_cta = put(pl.cta_begin.data(), cta_b ? pl.cta_begin.size() * sizeof(uint32_t) : 0, cta_b);
    const size_t o_mer = put(pl.merges.data(), pl.merges.size() * sizeof(Merge), mer_b);
    const size_t o_hdr = put(pl.cta_hdr.data(), pl.cta_hdr.size() * sizeof(CtaHdr), hdr_b);
    const size_t o_til = put(pl.tiles.data(), pl.tiles.size() * sizeof(TileDesc), til_b);
    const size_t o_rec = at;
    if (rec_b) {
        for (size_t i = 0; i < pl.items.size(); i++) memcpy(blob + at + i * rec_stride, pl.recs[i].w, rec_stride);
        at += rec_b;
    }
    const size_t o_tit = put(pl.tile_items.data(), tit_b, tit_b);
    const size_t o_tcb = put(pl.tile_cta_begin.data(), pl.tile_cta_begin.size() * sizeof(uint32_t), tcb_b);
    host_clock_lap(ctx, 2);
    if (int rc = total > 0 ? stage_commit(ctx, slot->dev, total) : YX_OK) {
        slot->pass_serial = 0;
        return rc;
    }
    host_clock_lap(ctx, 3);
    slot->d_items = (Item *)(slot->dev + o_items);
    slot->d_cta_begin = (uint32_t *)(slot->dev + o_cta);
    slot->d_merges = (Merge *)(slot->dev + o_mer);
    slot->d_cta_hdr = (CtaHdr *)(slot->dev + o_hdr);
    slot->d_tiles = (TileDesc *)(slot->dev + o_til);
    slot->d_recs = slot->dev + o_rec;
    slot->rec_stride = (uint32_t)rec_stride;
    slot->d_tile_items = (TileItem *)(slot->dev + o_tit);
    slot->d_tile_cta_begin = (uint32_t *)(slot->dev + o_tcb);
    *out = slot;
    return YX_OK;
}

int pick_path(const yx_ctx *ctx, const yx_kv *kv) {
    int f = ctx->tuning.force_path;
    if (kv->dtype == YX_F32) return 1;
    if (f == 1) return 1;
    return 2;
}

// What yx_attention does to the step's rows before it attends: norm, RoPE, append, queries to `q`.
struct RopeAppend {
    const float *qkv, *q_norm, *k_norm;
    float eps;
};

// Shared body of yx_attend / yx_attend_partial / yx_attention: (the rows' norm, RoPE and append,)
// the split-key kernel, then the merge.  With `pre`, the plan is made and uploaded first and the
// three kernels follow one another on the stream with no copy between them: the attention kernel
// is then a programmatic dependent of the append and starts its copies beside it.
int attend_impl(yx_ctx *ctx, yx_kv *kv, int layer, const void *q, int q_dtype, int hq, int64_t window,
                uint64_t key_lo, uint64_t key_hi, void *out, int out_dtype, float *m_out, float *l_out,
                float *o_out, const RopeAppend *pre = nullptr) {
    if (!ctx || !kv) return YX_ERR_INVALID;
    if (ctx->status != YX_OK) return ctx->status;
    if (!ctx->have_pass) return fail(ctx, YX_ERR_STATE, "attention without begin_pass");
    if (layer < 0 || layer >= kv->n_layers) return fail(ctx, YX_ERR_INVALID, "layer out of range");
    if (!valid_dtype(q_dtype) || !valid_dtype(out_dtype)) return fail(ctx, YX_ERR_INVALID, "bad dtype");
    if (hq <= 0 || hq % kv->hkv != 0) return fail(ctx, YX_ERR_INVALID, "hq must be a positive multiple of hkv");
    const int group = hq / kv->hkv;
    if (group > 16) return fail(ctx, YX_ERR_UNSUPPORTED, "more than 16 query heads per KV head");
    if (ctx->pass.rows == 0) return YX_OK;
    if (!q || (!out && !o_out)) return fail(ctx, YX_ERR_INVALID, "null tensor");
    if (window < 0) window = kv->layers[layer].window;
    if (ctx->pass.max_pos_seen >= kv->max_pos) return fail(ctx, YX_ERR_INVALID, "a row's position exceeds max_pos");
    DeviceGuard guard(ctx->device);

    const int path = pick_path(ctx, kv);
    const int64_t launches0 = ctx->launches;
    PlanParams pp{};
    pp.hkv = kv->hkv;
    pp.group = group;
    pp.window = window > 0 ? window : 0;
    pp.key_lo = key_lo;
    pp.key_hi = key_hi;
    pp.esize = kv->esize;
    const int per_sm = ctx->tuning.ctas_per_sm > 0 ? ctx->tuning.ctas_per_sm : (path == 1 ? 4 : 1);
    pp.n_ctas = ctx->sm_count * per_sm;
    // The tensor split-key kernel is planned for one CTA fewer than there are SMs unless the
    // tuning asks for a count.  These calls run back to back, each one's grid launched while the
    // one ahead still runs; a plan that keeps every SM busy to its last tile leaves that grid no
    // SM to place its first CTA on, and the interval between such calls was 19.5 us where plans
    // of the same batch for 140..147 CTAs all gave 18.8 us (the kernel is bound by HBM, not by
    // the number of CTAs).  With an SM spare one CTA of the call behind always runs a call ahead.
    if (path == 2 && ctx->tuning.ctas_per_sm <= 0 && pp.n_ctas > 1) pp.n_ctas -= 1;
    // (a slot of the split-key kernel holds 32 query rows of f32 or 64 of a 16-bit type)
    pp.max_rows = path == 1 ? 1 : std::max(1, std::min(MAX_ITEM_ROWS, (q_dtype == YX_F32 ? 32 : 64) / group));
    pp.share_prefix = path != 1 && ctx->tuning.share_prefix != 2;
    pp.w32 = ctx->tuning.cost32 > 0 ? ctx->tuning.cost32 : 16;
    pp.w64 = ctx->tuning.cost64 > 0 ? ctx->tuning.cost64 : 40;
    pp.resolve = path == 2;
    pp.share_rows = ctx->tuning.share_rows;
    // Prompt-sized runs of rows on a 16-bit cache go to the tcgen05 kernel; it writes final
    // outputs, so it is not used when triples are asked for.
    pp.tile_min_rows = 0;
    if (path == 2 && out && !o_out && ctx->tuning.force_path != 2)
        pp.tile_min_rows = ctx->tuning.force_path == 3 ? 1 : (ctx->tuning.tile_min_rows > 0 ? ctx->tuning.tile_min_rows : 64);
    // Two heads per item unless the group is odd or f32 queries need their low part (bf16 caches).
    pp.tile_ctas = ctx->sm_count;
    pp.tile_pairs = group % 2 == 0 && !(kv->dtype == YX_BF16 && q_dtype == YX_F32) && ctx->tuning.tile_single != 1;
    pp.min_piece = ctx->tuning.min_piece > 0 ? ctx->tuning.min_piece : (path == 2 ? 2 : 1);
    pp.item_cost = ctx->tuning.item_cost > 0 ? ctx->tuning.item_cost - 1 : (path == 2 ? 14 : 0);
    // (taken before get_plan, whose upload of a new plan is itself an ordering point on the stream)
    const bool predecessor_is_split_key_call = ctx->last_launch == yx_ctx::LAST_SPLIT_KEY;
    const bool predecessor_wrote_marked_tiles_only =
        ctx->last_launch == yx_ctx::LAST_ATTEND || ctx->last_launch == yx_ctx::LAST_SPLIT_KEY ||
        (ctx->last_launch == yx_ctx::LAST_APPEND && ctx->last_append_serial == ctx->pass_serial);
    yx_ctx::CachedPlan *cp = nullptr;
    if (int rc = get_plan(ctx, pp, &cp)) return rc;
    const Plan &pl = cp->plan;

    // Every page id the plan will read must be inside the arena.  (With a key range, entries of
    // pages outside the range may be placeholders: the kernels' own check covers what is read.)
    if (ctx->pass.max_page_seen >= kv->pages && !ctx->pass.pages.empty() && key_lo == 0 && key_hi == UINT64_MAX)
        return fail(ctx, YX_ERR_INVALID, "page id outside the KV arena");

    // Two sets of partial buffers, taken in turn by successive calls: a split-key kernel that runs
    // while the merge of the call ahead still reads that call's triples writes its own elsewhere
    // (see AttendArgs::late_wait).
    const size_t o_bytes = ((size_t)std::max<uint32_t>(pl.n_parts, 1) * group * D * sizeof(float) + 255) / 256 * 256;
    const size_t ml_bytes = ((size_t)std::max<uint32_t>(pl.n_parts, 1) * group * 2 * sizeof(float) + 255) / 256 * 256;
    if (int rc = ensure_buffer(ctx, (void **)&ctx->ws_o, &ctx->ws_o_cap, 2 * o_bytes)) return rc;
    if (int rc = ensure_buffer(ctx, (void **)&ctx->ws_ml, &ctx->ws_ml_cap, 2 * ml_bytes)) return rc;
    ctx->ws_set ^= 1;
    float *const part_o = ctx->ws_o + (size_t)ctx->ws_set * (o_bytes / sizeof(float));
    float *const part_ml = ctx->ws_ml + (size_t)ctx->ws_set * (ml_bytes / sizeof(float));
    if (path == 2) {
        // Arrival counters of the fused merge: zero when allocated, and every launch leaves
        // them zero again.
        size_t need = (size_t)ctx->pass.rows * kv->hkv * sizeof(uint32_t);
        if (need > ctx->counters_cap || !ctx->counters) {
            if (int rc = ensure_buffer(ctx, (void **)&ctx->counters, &ctx->counters_cap, need)) return rc;
            if (int rc = check_cuda(ctx, cudaMemsetAsync(ctx->counters, 0, ctx->counters_cap, ctx->stream), "zero counters"))
                return rc;
        }
    }

    bool early_kv = predecessor_wrote_marked_tiles_only;
    if (pre) {
        // write_rows, then attend (cpu lib.rs:526-529): all rows' K/V land before any row attends.
        if (int rc = launch_qk_rope_append(ctx, kv, layer, pre->qkv, pre->q_norm, pre->k_norm, hq, pre->eps, (float *)q))
            return rc;
        host_clock_lap(ctx, 4);
        ctx->last_launch = yx_ctx::LAST_APPEND;
        ctx->last_append_serial = ctx->pass_serial;
        early_kv = true;   // an append of this pass writes marked tiles only
    }

    AttendArgs a{};
    a.rows = ctx->pass.rows;
    a.q = q;
    a.q_dtype = q_dtype;
    a.hq = hq;
    a.group = group;
    a.k_arena = kv->k(layer);
    a.v_arena = kv->v(layer);
    a.hkv = kv->hkv;
    a.kv_dtype = kv->dtype;
    a.kv_pages = kv->pages;
    a.window = pp.window;
    a.key_lo = key_lo;
    a.key_hi = key_hi;
    a.items = cp->d_items;
    a.cta_begin = cp->d_cta_begin;
    a.n_ctas = pl.n_ctas;
    a.part_o = part_o;
    a.part_ml = part_ml;
    a.cta_hdr = cp->d_cta_hdr;
    a.tiles = cp->d_tiles;
    a.recs = cp->d_recs;
    a.rec_stride = cp->rec_stride;
    a.single_use = pl.single_use;
    a.plan = &pl;
    a.n_stages = ctx->tuning.stages;
    a.early_kv = early_kv;
    a.fused = ctx->tuning.fused_merge == 1;
    // (anything this call put on the stream before the kernel - a new plan, a grown buffer, zeroed
    // counters - is an ordering point of its own and was counted in ctx->launches or reset last_launch)
    a.late_wait = predecessor_is_split_key_call && ctx->last_launch == yx_ctx::LAST_SPLIT_KEY && !a.fused &&
                  ctx->tuning.overlap_calls != 2 && !ctx->profiling;
    {
        // ... unless these queries are what the call ahead wrote (its merge may still be running).
        const uintptr_t q_lo = (uintptr_t)q, q_hi = q_lo + (size_t)ctx->pass.rows * hq * D * (q_dtype == YX_F32 ? 4 : 2);
        for (const auto &w : ctx->last_written)
            if (w.hi > w.lo && q_lo < w.hi && w.lo < q_hi) a.late_wait = false;
        const size_t n = (size_t)ctx->pass.rows * hq;
        const size_t out_b = n * D * (out_dtype == YX_F32 ? 4 : 2);
        ctx->last_written[0] = {(uintptr_t)out, out ? (uintptr_t)out + out_b : 0};
        ctx->last_written[1] = {(uintptr_t)o_out, o_out ? (uintptr_t)o_out + n * D * 4 : 0};
        ctx->last_written[2] = {(uintptr_t)m_out, m_out ? (uintptr_t)m_out + n * 4 : 0};
        ctx->last_written[3] = {(uintptr_t)l_out, l_out ? (uintptr_t)l_out + n * 4 : 0};
    }
    // When the kernel of the call ahead had a CTA for every SM, no CTA of this kernel can run before
    // one of that kernel's has left, which it does only once everything ahead of it is complete
    // (the merge that last read the set of partial buffers this call writes included).  The wait can
    // then move from before a CTA's first write to before it leaves.
    a.wait_at_end = a.late_wait && ctx->last_split_ctas >= ctx->sm_count && ctx->tuning.overlap_calls != 3;
    ctx->last_split_ctas = path == 2 && !pl.items.empty() ? pl.n_ctas : 0;
    a.counters = ctx->counters;
    a.out = out;
    a.out_dtype = out_dtype;
    a.m_out = m_out;
    a.l_out = l_out;
    a.o_out = o_out;
    profile_mark(ctx, 0);
    host_clock_lap(ctx, 0);
    if (!pl.tile_items.empty()) {
        TileArgs t{};
        t.q = q;
        t.q_dtype = q_dtype;
        t.hq = hq;
        t.group = group;
        t.hkv = kv->hkv;
        t.kv_dtype = kv->dtype;
        t.k_arena = kv->k(layer);
        t.v_arena = kv->v(layer);
        t.kv_pages = kv->pages;
        t.window = pp.window;
        t.items = cp->d_tile_items;
        t.n_items = (int)pl.tile_items.size();
        t.cta_begin = cp->d_tile_cta_begin;
        t.n_ctas = (int)pl.tile_cta_begin.size() - 1;
        t.out = out;
        t.out_dtype = out_dtype;
        t.pairs = pp.tile_pairs;
        t.wide_v = kv->wide_v_dev;
        if (int rc = launch_prefill_tc(ctx, t)) return rc;
    }
    // With every row in the tiled kernel's hands and no partial triples asked for, the merge
    // has nothing to do.
    const bool need_combine = (!pl.items.empty() || o_out != nullptr) && !ctx->skip_merge;
    if (path == 2) {
        // Rows without a live key in the range get no item, so nothing would write them.
        if (a.fused && o_out && pl.has_empty_rows)
            if (int rc = launch_fill_empty(ctx, (size_t)ctx->pass.rows * hq, m_out, l_out, o_out)) return rc;
        if (!pl.items.empty())
            if (int rc = launch_attend_mma(ctx, a)) return rc;
        host_clock_lap(ctx, 5);
        profile_mark(ctx, 1);
        profile_mark(ctx, 2);
        if (!a.fused && need_combine)
            if (int rc = launch_combine(ctx, cp->d_merges, part_o, part_ml, (int)ctx->pass.rows, hq, group, out,
                                        out_dtype, m_out, l_out, o_out, a.late_wait != 0))
                return rc;
        host_clock_lap(ctx, 6);
        profile_mark(ctx, 3);
    } else {
        if (!pl.items.empty())
            if (int rc = launch_attend_simt(ctx, a)) return rc;
        profile_mark(ctx, 1);
        profile_mark(ctx, 2);
        if (need_combine)
            if (int rc = launch_combine(ctx, cp->d_merges, part_o, part_ml, (int)ctx->pass.rows, hq, group, out,
                                        out_dtype, m_out, l_out, o_out))
                return rc;
        profile_mark(ctx, 3);
    }
    if (ctx->launches != launches0)
        ctx->last_launch = path == 2 && !pl.items.empty() && pl.tile_items.empty() && !a.fused ? yx_ctx::LAST_SPLIT_KEY : yx_ctx::LAST_ATTEND;
    ctx->last_plan = pl.info;
    ctx->last_plan.path = pl.tile_items.empty() ? path : (pl.items.empty() ? 3 : 5);
    ctx->last_plan.launches = (int)(ctx->launches - launches0);
    return YX_OK;
}

}  // namespace

int attend_key_range(yx_ctx *ctx, yx_kv *kv, int layer, const void *q, int q_dtype, int hq, int64_t window, uint64_t key_lo,
                     uint64_t key_hi, void *out, int out_dtype) {
    return attend_impl(ctx, kv, layer, q, q_dtype, hq, window, key_lo, key_hi, out, out_dtype, nullptr, nullptr, nullptr);
}

}  // namespace yx

using namespace yx;

extern "C" {

int yx_ctx_create(int device, void *stream, yx_ctx **out) {
    if (!out) return YX_ERR_INVALID;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) return YX_ERR_CUDA;   // no CPU fallback
    if (device < 0 || device >= n) return YX_ERR_INVALID;
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return YX_ERR_CUDA;
    if (prop.major != 10) return YX_ERR_UNSUPPORTED;   // built for sm_100a only
    yx_ctx *ctx = new (std::nothrow) yx_ctx();
    if (!ctx) return YX_ERR_OOM;
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    DeviceGuard guard(device);
    if (stream) {
        ctx->stream = (cudaStream_t)stream;
    } else {
        if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
            delete ctx;
            return YX_ERR_CUDA;
        }
        ctx->own_stream = true;
    }
    if (cudaHostAlloc((void **)&ctx->dev_status, sizeof(yx_dev_status), cudaHostAllocMapped) != cudaSuccess) {
        if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
        delete ctx;
        return YX_ERR_OOM;
    }
    memset(ctx->dev_status, 0, sizeof(yx_dev_status));
    *out = ctx;
    return YX_OK;
}

void yx_ctx_destroy(yx_ctx *ctx) {
    if (!ctx) return;
    DeviceGuard guard(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    yx_comm_destroy(ctx);
    for (auto &st : ctx->ring) {
        if (st.host) cudaFreeHost(st.host);
        if (st.done) cudaEventDestroy(st.done);
    }
    for (auto &cp : ctx->plans)
        if (cp.dev) cudaFree(cp.dev);
    if (ctx->d_meta) cudaFree(ctx->d_meta);
    if (ctx->ws_o) cudaFree(ctx->ws_o);
    if (ctx->ws_ml) cudaFree(ctx->ws_ml);
    if (ctx->q_tmp) cudaFree(ctx->q_tmp);
    if (ctx->counters) cudaFree(ctx->counters);
    if (ctx->mm_part) cudaFree(ctx->mm_part);
    if (ctx->mm_packed) cudaFree(ctx->mm_packed);
    if (ctx->lt_workspace) cudaFree(ctx->lt_workspace);
    release_matmul_library(ctx);
    if (ctx->idx_dev) cudaFree(ctx->idx_dev);
    if (ctx->gather_buf) cudaFree(ctx->gather_buf);
    if (ctx->dev_status) cudaFreeHost(ctx->dev_status);
    for (auto &e : ctx->prof_events)
        if (e) cudaEventDestroy(e);
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

int yx_status(const yx_ctx *ctx) { return ctx ? ctx->status : YX_ERR_INVALID; }
const char *yx_last_error(const yx_ctx *ctx) { return ctx ? ctx->error.c_str() : "null context"; }
void yx_clear_error(yx_ctx *ctx) {
    if (ctx) {
        ctx->status = YX_OK;
        ctx->error.clear();
    }
}

int yx_sync(yx_ctx *ctx) {
    if (!ctx) return YX_ERR_INVALID;
    DeviceGuard guard(ctx->device);
    if (int rc = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize")) return rc;
    if (int rc = fold_device_status(ctx)) return rc;
    return ctx->status;
}

void *yx_stream(const yx_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }

int yx_set_tuning(yx_ctx *ctx, const yx_tuning *t) {
    if (!ctx) return YX_ERR_INVALID;
    ctx->tuning = t ? *t : yx_tuning{};
    for (auto &cp : ctx->plans) cp.pass_serial = 0;
    return YX_OK;
}

int yx_last_plan(const yx_ctx *ctx, yx_plan_info *out) {
    if (!ctx || !out) return YX_ERR_INVALID;
    *out = ctx->last_plan;
    return YX_OK;
}

int64_t yx_launch_count(const yx_ctx *ctx) { return ctx ? ctx->launches : 0; }

int yx_profile_begin(yx_ctx *ctx) {
    if (!ctx) return YX_ERR_INVALID;
    DeviceGuard guard(ctx->device);
    if (ctx->prof_events.empty()) {
        ctx->prof_events.resize(4 * 4096, nullptr);
        for (auto &e : ctx->prof_events)
            if (int rc = check_cuda(ctx, cudaEventCreate(&e), "cudaEventCreate (profile)")) return rc;
    }
    ctx->prof_used = 0;
    ctx->profiling = true;
    return YX_OK;
}

int yx_profile_end(yx_ctx *ctx, float *split_ms, float *combine_ms, int *calls) {
    if (!ctx) return YX_ERR_INVALID;
    DeviceGuard guard(ctx->device);
    ctx->profiling = false;
    if (int rc = yx_sync(ctx)) return rc;
    float a = 0.f, b = 0.f;
    for (size_t i = 0; i < ctx->prof_used; i++) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, ctx->prof_events[4 * i], ctx->prof_events[4 * i + 1]) == cudaSuccess) a += ms;
        if (cudaEventElapsedTime(&ms, ctx->prof_events[4 * i + 2], ctx->prof_events[4 * i + 3]) == cudaSuccess) b += ms;
    }
    if (split_ms) *split_ms = a;
    if (combine_ms) *combine_ms = b;
    if (calls) *calls = (int)ctx->prof_used;
    return YX_OK;
}

// ---- tensors ---------------------------------------------------------------------------

int yx_tensor_alloc(yx_ctx *ctx, size_t bytes, void **out_dev) {
    if (!ctx || !out_dev) return YX_ERR_INVALID;
    DeviceGuard guard(ctx->device);
    *out_dev = nullptr;
    return check_cuda(ctx, cudaMalloc(out_dev, std::max<size_t>(bytes, 16)), "cudaMalloc (tensor)");
}

int yx_tensor_free(yx_ctx *ctx, void *dev) {
    if (!ctx) return YX_ERR_INVALID;
    DeviceGuard guard(ctx->device);
    return dev ? check_cuda(ctx, cudaFree(dev), "cudaFree") : YX_OK;
}

int yx_upload(yx_ctx *ctx, void *dst_dev, const void *src_host, size_t bytes) {
    if (!ctx || (bytes && (!dst_dev || !src_host))) return YX_ERR_INVALID;
    DeviceGuard guard(ctx->device);
    ctx->last_launch = yx_ctx::LAST_OTHER;
    return check_cuda(ctx, cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream), "upload");
}

int yx_download(yx_ctx *ctx, void *dst_host, const void *src_dev, size_t bytes, int wait) {
    if (!ctx || (bytes && (!dst_host || !src_dev))) return YX_ERR_INVALID;
    DeviceGuard guard(ctx->device);
    ctx->last_launch = yx_ctx::LAST_OTHER;
    if (int rc = check_cuda(ctx, cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream), "download"))
        return rc;
    return wait ? yx_sync(ctx) : YX_OK;
}

int yx_host_alloc(yx_ctx *ctx, size_t bytes, void **out_host) {
    if (!ctx || !out_host) return YX_ERR_INVALID;
    DeviceGuard guard(ctx->device);
    return check_cuda(ctx, cudaMallocHost(out_host, std::max<size_t>(bytes, 16)), "cudaMallocHost");
}

int yx_host_free(yx_ctx *ctx, void *host) {
    if (!ctx) return YX_ERR_INVALID;
    return host ? check_cuda(ctx, cudaFreeHost(host), "cudaFreeHost") : YX_OK;
}

// ---- KV storage ------------------------------------------------------------------------

int yx_kv_create(yx_ctx *ctx, int n_layers, const yx_layer *layers, uint32_t pages, int hkv, int head_dim,
                 int dtype, uint32_t max_pos, yx_kv **out) {
    if (!ctx || !out) return YX_ERR_INVALID;
    *out = nullptr;
    if (n_layers <= 0 || !layers || pages == 0 || hkv <= 0) return fail(ctx, YX_ERR_INVALID, "new_kv: bad sizes");
    if (head_dim != D) return fail(ctx, YX_ERR_UNSUPPORTED, "new_kv: head_dim must be 128");
    if (!valid_dtype(dtype)) return fail(ctx, YX_ERR_INVALID, "new_kv: bad dtype");
    DeviceGuard guard(ctx->device);
    yx_kv *kv = new (std::nothrow) yx_kv();
    if (!kv) return fail(ctx, YX_ERR_OOM, "new_kv: out of host memory");
    kv->n_layers = n_layers;
    kv->hkv = hkv;
    kv->dtype = dtype;
    kv->esize = dtype == YX_F32 ? 4 : 2;
    kv->pages = pages;
    kv->max_pos = max_pos;
    kv->layers.assign(layers, layers + n_layers);
    kv->layer_bytes = (size_t)pages * hkv * kv_block_elems() * kv->esize;
    size_t total = kv->layer_bytes * n_layers;
    int rc = check_cuda(ctx, cudaMalloc((void **)&kv->k_base, total), "new_kv: cudaMalloc K");
    if (!rc) rc = check_cuda(ctx, cudaMalloc((void **)&kv->v_base, total), "new_kv: cudaMalloc V");
    if (!rc) rc = check_cuda(ctx, cudaMalloc(&kv->rope_dev, sizeof(yx_rope) * n_layers), "new_kv: cudaMalloc rope");
    if (!rc) rc = check_cuda(ctx, cudaMalloc((void **)&kv->wide_v_dev, 256), "new_kv: cudaMalloc flag");
    if (!rc) rc = check_cuda(ctx, cudaMemsetAsync(kv->wide_v_dev, 0, 256, ctx->stream), "new_kv: zero flag");
    // Zeroed like the reference's arenas (cpu lib.rs:466-468).
    if (!rc) rc = check_cuda(ctx, cudaMemsetAsync(kv->k_base, 0, total, ctx->stream), "new_kv: zero K");
    if (!rc) rc = check_cuda(ctx, cudaMemsetAsync(kv->v_base, 0, total, ctx->stream), "new_kv: zero V");
    if (!rc) {
        std::vector<yx_rope> ropes(n_layers);
        for (int l = 0; l < n_layers; l++) ropes[l] = layers[l].rope;
        rc = upload_ordered(ctx, kv->rope_dev, ropes.data(), sizeof(yx_rope) * n_layers);
    }
    if (rc) {
        yx_kv_destroy(ctx, kv);
        return rc;
    }
    *out = kv;
    return YX_OK;
}

void yx_kv_destroy(yx_ctx *ctx, yx_kv *kv) {
    if (!kv) return;
    if (ctx) {
        DeviceGuard guard(ctx->device);
        cudaStreamSynchronize(ctx->stream);
        if (kv->k_base) cudaFree(kv->k_base);
        if (kv->v_base) cudaFree(kv->v_base);
        if (kv->rope_dev) cudaFree(kv->rope_dev);
        if (kv->wide_v_dev) cudaFree(kv->wide_v_dev);
    }
    delete kv;
}

int yx_kv_copy_page(yx_ctx *ctx, yx_kv *kv, uint32_t src, uint32_t dst) {
    if (!ctx || !kv) return YX_ERR_INVALID;
    if (ctx->status != YX_OK) return ctx->status;
    if (src >= kv->pages || dst >= kv->pages) return fail(ctx, YX_ERR_INVALID, "copy_page: page outside the arena");
    if (src == dst) return YX_OK;
    DeviceGuard guard(ctx->device);
    ctx->last_launch = yx_ctx::LAST_KV_WRITE;
    return launch_copy_page(ctx, kv, src, dst);
}

static int page_io(yx_ctx *ctx, yx_kv *kv, int layer, uint32_t first, uint32_t n_pages, void *k_host, void *v_host,
                   bool write) {
    if (!ctx || !kv || !k_host || !v_host) return YX_ERR_INVALID;
    if (layer < 0 || layer >= kv->n_layers || n_pages == 0 || (uint64_t)first + n_pages > kv->pages)
        return fail(ctx, YX_ERR_INVALID, "page io: out of range");
    DeviceGuard guard(ctx->device);
    ctx->last_launch = yx_ctx::LAST_KV_WRITE;
    size_t bytes = (size_t)n_pages * PAGE * kv->hkv * D * kv->esize;
    void *lin = nullptr;
    if (int rc = check_cuda(ctx, cudaMalloc(&lin, 2 * bytes), "page io: cudaMalloc")) return rc;
    char *k_lin = (char *)lin, *v_lin = k_lin + bytes;
    int rc = YX_OK;
    if (write) {
        rc = check_cuda(ctx, cudaMemcpyAsync(k_lin, k_host, bytes, cudaMemcpyHostToDevice, ctx->stream), "page io");
        if (!rc) rc = check_cuda(ctx, cudaMemcpyAsync(v_lin, v_host, bytes, cudaMemcpyHostToDevice, ctx->stream), "page io");
        if (!rc) rc = launch_page_io(ctx, kv, layer, first, n_pages, k_lin, v_lin, true);
    } else {
        rc = launch_page_io(ctx, kv, layer, first, n_pages, k_lin, v_lin, false);
        if (!rc) rc = check_cuda(ctx, cudaMemcpyAsync(k_host, k_lin, bytes, cudaMemcpyDeviceToHost, ctx->stream), "page io");
        if (!rc) rc = check_cuda(ctx, cudaMemcpyAsync(v_host, v_lin, bytes, cudaMemcpyDeviceToHost, ctx->stream), "page io");
    }
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    cudaFree(lin);
    if (rc) return rc;
    return check_cuda(ctx, e, "page io: sync");
}

int yx_kv_read_pages(yx_ctx *ctx, yx_kv *kv, int layer, uint32_t first, uint32_t n_pages, void *k_host, void *v_host) {
    return page_io(ctx, kv, layer, first, n_pages, k_host, v_host, false);
}
int yx_kv_write_pages(yx_ctx *ctx, yx_kv *kv, int layer, uint32_t first, uint32_t n_pages, const void *k_host,
                      const void *v_host) {
    return page_io(ctx, kv, layer, first, n_pages, (void *)k_host, (void *)v_host, true);
}

// ---- a pass ----------------------------------------------------------------------------

int yx_begin_pass(yx_ctx *ctx, uint32_t rows, const uint32_t *pos, const uint32_t *kv_slot, const uint32_t *pt_off,
                  const uint32_t *pages, uint32_t n_pages) {
    if (!ctx) return YX_ERR_INVALID;
    if (ctx->status != YX_OK) return ctx->status;
    if (rows && (!pos || !kv_slot || !pt_off)) return fail(ctx, YX_ERR_INVALID, "begin_pass: null array");
    if (n_pages && !pages) return fail(ctx, YX_ERR_INVALID, "begin_pass: null page table");
    if (rows > 65535) return fail(ctx, YX_ERR_UNSUPPORTED, "begin_pass: more than 65535 rows");
    uint32_t max_pos = 0, max_slot = 0, max_page = 0;
    for (uint32_t r = 0; r < rows; r++) {
        if ((uint64_t)pt_off[r] + pos[r] / PAGE >= n_pages)
            return fail(ctx, YX_ERR_INVALID, "begin_pass: a row's page table runs past `pages`");
        // kv_slot must be the slot of the row's own position (PassMeta, lib.rs:69-70).
        if (kv_slot[r] != pages[pt_off[r] + pos[r] / PAGE] * (uint32_t)PAGE + pos[r] % PAGE)
            return fail(ctx, YX_ERR_INVALID, "begin_pass: kv_slot is not slot(pages, pos)");
        max_pos = std::max(max_pos, pos[r]);
        max_slot = std::max(max_slot, kv_slot[r]);
    }
    for (uint32_t i = 0; i < n_pages; i++) max_page = std::max(max_page, pages[i]);
    DeviceGuard guard(ctx->device);
    PassHost &p = ctx->pass;
    p.rows = rows;
    p.pos.assign(pos, pos + rows);          // the vectors keep their capacity from pass to pass
    p.kv_slot.assign(kv_slot, kv_slot + rows);
    p.pt_off.assign(pt_off, pt_off + rows);
    p.pages.assign(pages, pages + n_pages);
    p.max_pos_seen = max_pos;
    p.max_slot_seen = max_slot;
    p.max_page_seen = max_page;
    ctx->pass_serial++;
    ctx->have_pass = true;

    const size_t words = (size_t)3 * rows + n_pages;
    if (int rc = ensure_buffer(ctx, (void **)&ctx->d_meta, &ctx->d_meta_cap, std::max<size_t>(words, 4) * 4)) return rc;
    ctx->d_pos = ctx->d_meta;
    ctx->d_slot = ctx->d_meta + rows;
    ctx->d_ptoff = ctx->d_meta + 2 * (size_t)rows;
    ctx->d_pages = ctx->d_meta + 3 * (size_t)rows;
    if (words == 0) return YX_OK;
    // The arrays go straight into a pinned staging buffer: one copy, one upload, no allocation.
    uint32_t *blob = nullptr;
    if (int rc = stage_acquire(ctx, words * 4, (void **)&blob)) return rc;
    if (rows) {
        memcpy(blob, pos, rows * 4);
        memcpy(blob + rows, kv_slot, rows * 4);
        memcpy(blob + 2 * (size_t)rows, pt_off, rows * 4);
    }
    if (n_pages) memcpy(blob + 3 * (size_t)rows, pages, (size_t)n_pages * 4);
    return stage_commit(ctx, ctx->d_meta, words * 4);
}

int yx_kv_append(yx_ctx *ctx, yx_kv *kv, int layer, const void *k_rows, const void *v_rows, int src_dtype) {
    if (!ctx || !kv) return YX_ERR_INVALID;
    if (ctx->status != YX_OK) return ctx->status;
    if (!ctx->have_pass) return fail(ctx, YX_ERR_STATE, "kv_append without begin_pass");
    if (layer < 0 || layer >= kv->n_layers) return fail(ctx, YX_ERR_INVALID, "layer out of range");
    if (src_dtype != YX_F32 && src_dtype != kv->dtype)
        return fail(ctx, YX_ERR_INVALID, "kv_append: rows must be f32 or of the cache's type");
    if (ctx->pass.rows == 0) return YX_OK;
    if (!k_rows || !v_rows) return fail(ctx, YX_ERR_INVALID, "null tensor");
    if (ctx->pass.max_slot_seen / PAGE >= kv->pages) return fail(ctx, YX_ERR_INVALID, "kv_slot outside the KV arena");
    DeviceGuard guard(ctx->device);
    ctx->last_launch = yx_ctx::LAST_APPEND;
    ctx->last_append_serial = ctx->pass_serial;
    return launch_append(ctx, kv, layer, k_rows, v_rows, src_dtype);
}

int yx_attend(yx_ctx *ctx, yx_kv *kv, int layer, const void *q, int q_dtype, int hq, int64_t window, void *out,
              int out_dtype) {
    return attend_impl(ctx, kv, layer, q, q_dtype, hq, window, 0, UINT64_MAX, out, out_dtype, nullptr, nullptr, nullptr);
}

int yx_attend_partial(yx_ctx *ctx, yx_kv *kv, int layer, const void *q, int q_dtype, int hq, int64_t window,
                      uint64_t key_lo, uint64_t key_hi, float *m, float *l, float *o) {
    if (!m || !l || !o) return ctx ? fail(ctx, YX_ERR_INVALID, "null partial output") : YX_ERR_INVALID;
    return attend_impl(ctx, kv, layer, q, q_dtype, hq, window, key_lo, key_hi, nullptr, YX_F32, m, l, o);
}

int yx_attention(yx_ctx *ctx, yx_kv *kv, int layer, const float *qkv, const float *q_norm, const float *k_norm,
                 int hq, float eps, float *out) {
    if (!ctx || !kv) return YX_ERR_INVALID;
    if (ctx->status != YX_OK) return ctx->status;
    if (!ctx->have_pass) return fail(ctx, YX_ERR_STATE, "attention without begin_pass");
    if (layer < 0 || layer >= kv->n_layers) return fail(ctx, YX_ERR_INVALID, "layer out of range");
    if (hq <= 0 || hq % kv->hkv != 0) return fail(ctx, YX_ERR_INVALID, "hq must be a positive multiple of hkv");
    if (ctx->pass.rows == 0) return YX_OK;
    if (!qkv || !q_norm || !k_norm || !out) return fail(ctx, YX_ERR_INVALID, "null tensor");
    if (ctx->pass.max_slot_seen / PAGE >= kv->pages) return fail(ctx, YX_ERR_INVALID, "kv_slot outside the KV arena");
    host_clock_start(ctx);
    DeviceGuard guard(ctx->device);
    size_t q_bytes = (size_t)ctx->pass.rows * hq * D * sizeof(float);
    if (int rc = ensure_buffer(ctx, (void **)&ctx->q_tmp, &ctx->q_tmp_cap, q_bytes)) return rc;
    host_clock_lap(ctx, 0);
    const RopeAppend pre{qkv, q_norm, k_norm, eps};
    return attend_impl(ctx, kv, layer, ctx->q_tmp, YX_F32, hq, -1, 0, UINT64_MAX, out, YX_F32, nullptr, nullptr, nullptr, &pre);
}

int yx_lse_combine(yx_ctx *ctx, int n_parts, const float *m, const float *l, const float *o, size_t n, void *out,
                   int out_dtype) {
    if (!ctx) return YX_ERR_INVALID;
    if (ctx->status != YX_OK) return ctx->status;
    if (n_parts <= 0 || !m || !l || !o || !out || !valid_dtype(out_dtype))
        return fail(ctx, YX_ERR_INVALID, "lse_combine: bad arguments");
    if (n == 0) return YX_OK;
    DeviceGuard guard(ctx->device);
    return launch_combine_strided(ctx, n_parts, m, l, o, n, n, n * D, n, out, out_dtype);
}

}  // extern "C"
