// Hooks for the library's own tests and benchmark (yx_hooks.h): the planner on host arrays, a
// switch that leaves the merge out of an attention call, a kernel whose bounded wait runs out,
// and the time-stamp buffer of a diagnostic build.
#include <string.h>

#include "yx_device.cuh"
#include "yx_hooks.h"

extern "C" int yx_plan_probe(uint32_t rows, const uint32_t *pos, const uint32_t *pt_off, const uint32_t *pages,
                             uint32_t n_pages, int hkv, int group, int64_t window, uint64_t key_lo, uint64_t key_hi,
                             int max_rows, int n_ctas, int share_prefix, int esize, int cost32, int cost64,
                             int item_cost, int min_piece, yx_plan_info *info, uint32_t *items_out, uint32_t max_items) {
    if (rows && (!pos || !pt_off)) return YX_ERR_INVALID;
    yx::PassHost pass;
    pass.rows = rows;
    pass.pos.assign(pos, pos + rows);
    pass.pt_off.assign(pt_off, pt_off + rows);
    pass.pages.assign(pages, pages + n_pages);
    yx::PlanParams pp{};
    pp.hkv = hkv;
    pp.group = group;
    pp.window = window > 0 ? window : 0;
    pp.key_lo = key_lo;
    pp.key_hi = key_hi;
    pp.max_rows = max_rows;
    pp.n_ctas = n_ctas;
    pp.share_prefix = share_prefix != 0;
    pp.esize = esize;
    pp.w32 = cost32 > 0 ? cost32 : 16;
    pp.w64 = cost64 > 0 ? cost64 : 16;
    pp.resolve = true;
    pp.min_piece = min_piece > 0 ? min_piece : 1;
    pp.item_cost = item_cost > 0 ? item_cost : 0;
    pp.share_rows = share_prefix > 1 ? share_prefix : 0;   // values above 1 name the rows a shared item may hold
    yx::Plan plan;
    try {
        yx::build_split_plan(pass, pp, plan);
    } catch (const std::string &) {
        return YX_ERR_INVALID;
    }
    if (info) *info = plan.info;
    if (items_out) {
        uint32_t cta = 0;
        for (uint32_t i = 0; i < plan.items.size() && i < max_items; i++) {
            while (cta + 1 < plan.cta_begin.size() && plan.cta_begin[cta + 1] <= i) cta++;
            const yx::Item &it = plan.items[i];
            uint32_t *o = items_out + (size_t)i * YX_PROBE_ITEM_WORDS;
            o[0] = it.tile_begin;
            o[1] = it.tile_end;
            o[2] = it.key_lo;
            o[3] = it.key_hi;
            o[4] = it.pt_off;
            o[5] = it.kv_head;
            o[6] = it.n_rows;
            o[7] = it.mt;
            o[8] = cta;
            for (int r = 0; r < yx::MAX_ITEM_ROWS; r++) {
                o[9 + r] = it.rows[r];
                o[9 + yx::MAX_ITEM_ROWS + r] = it.part[r];
            }
        }
    }
    return YX_OK;
}

namespace {

bool same_plan(const yx::Plan &a, const yx::Plan &b) {
    using namespace yx;
    if (a.tiles.size() != b.tiles.size() || a.items.size() != b.items.size() || a.n_ctas != b.n_ctas || a.n_parts != b.n_parts ||
        a.prologue.size() != b.prologue.size() || a.merges.size() != b.merges.size() || a.cta_hdr.size() != b.cta_hdr.size())
        return false;
    if (memcmp(a.tiles.data(), b.tiles.data(), a.tiles.size() * sizeof(TileDesc))) return false;
    if (memcmp(a.items.data(), b.items.data(), a.items.size() * sizeof(Item))) return false;
    if (memcmp(a.prologue.data(), b.prologue.data(), a.prologue.size() * sizeof(CtaPrologue))) return false;
    if (memcmp(a.merges.data(), b.merges.data(), a.merges.size() * sizeof(Merge))) return false;
    if (memcmp(a.cta_hdr.data(), b.cta_hdr.data(), a.cta_hdr.size() * sizeof(CtaHdr))) return false;
    for (size_t i = 0; i < a.items.size(); i++) {   // the words of a record that are read
        if (memcmp(a.recs[i].w, b.recs[i].w, 16)) return false;
        if (memcmp(a.recs[i].w + IR_ROW0, b.recs[i].w + IR_ROW0, a.items[i].n_rows * IR_ROW_WORDS * 4)) return false;
    }
    return a.info.unique_kv_bytes == b.info.unique_kv_bytes && a.info.logical_kv_bytes == b.info.logical_kv_bytes &&
           a.info.tiles == b.info.tiles && a.single_use == b.single_use && a.has_empty_rows == b.has_empty_rows;
}

}  // namespace

extern "C" int yx_hook_plan_steps(uint32_t rows, const uint32_t *pos, const uint32_t *pt_off, const uint32_t *pages,
                                  uint32_t n_pages, int hkv, int group, int64_t window, int max_rows, int n_ctas, int steps,
                                  int *patched_out) {
    if (rows && (!pos || !pt_off)) return -1;
    yx::PassHost pass;
    pass.rows = rows;
    pass.pos.assign(pos, pos + rows);
    pass.pt_off.assign(pt_off, pt_off + rows);
    pass.pages.assign(pages, pages + n_pages);
    yx::PlanParams pp{};
    pp.hkv = hkv;
    pp.group = group;
    pp.window = window > 0 ? window : 0;
    pp.key_lo = 0;
    pp.key_hi = UINT64_MAX;
    pp.max_rows = max_rows;
    pp.n_ctas = n_ctas;
    pp.share_prefix = true;
    pp.esize = 2;
    pp.w32 = 16;
    pp.w64 = 40;
    pp.resolve = true;
    pp.min_piece = 2;
    pp.item_cost = 14;
    yx::Plan running;
    int patched = 0, differing = 0;
    try {
        for (int s = 0; s < steps; s++) {
            yx::build_split_plan(pass, pp, running);
            yx::Plan fresh;
            yx::build_split_plan(pass, pp, fresh);
            patched += running.patched ? 1 : 0;
            differing += same_plan(running, fresh) ? 0 : 1;
            for (uint32_t &p : pass.pos) p++;
        }
    } catch (const std::string &) {
        return -1;
    }
    if (patched_out) *patched_out = patched;
    return differing;
}

extern "C" int yx_hook_forget_plan_shape(yx_ctx *ctx) {
    if (!ctx) return YX_ERR_INVALID;
    for (auto &cp : ctx->plans) cp.plan.sig_valid = false;
    return YX_OK;
}

extern "C" int yx_hook_skip_merge(yx_ctx *ctx, int on) {
    if (!ctx) return YX_ERR_INVALID;
    ctx->skip_merge = on != 0;
    return YX_OK;
}

namespace {

// One CTA, one mbarrier that nobody arrives on, the same bounded wait the attention kernels use
// with a caller-chosen limit.  No memory traffic, nothing to drain: when the wait gives up the
// failure is in the status word and the kernel returns normally.
__global__ void expire_wait_kernel(yx_dev_status *status, long long limit) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    const uint32_t b = yx::dev::smem_u32(&bar);
    if (threadIdx.x == 0) {
        abort_flag = 0;
        yx::dev::mbar_init(b, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) yx::dev::mbar_wait_slow(b, 0, &abort_flag, status, 900, limit);
}

}  // namespace

extern "C" int yx_hook_expire_wait(yx_ctx *ctx, uint64_t limit_cycles) {
    if (!ctx) return YX_ERR_INVALID;
    if (ctx->status != YX_OK) return ctx->status;
    // Never more than about a second, whatever is asked for.
    const long long limit = (long long)(limit_cycles > 2000000000ull ? 2000000000ull : limit_cycles);
    int prev = -1;
    cudaGetDevice(&prev);
    if (prev != ctx->device) cudaSetDevice(ctx->device);
    expire_wait_kernel<<<1, 32, 0, ctx->stream>>>(ctx->dev_status, limit);
    int rc = yx::check_cuda(ctx, cudaGetLastError(), "expire_wait kernel");
    if (prev != ctx->device) cudaSetDevice(prev);
    if (!rc) ctx->launches++;
    return rc;
}

#ifdef YX_TRACE
#include <chrono>
static int64_t host_now_ns() {
    return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
void host_clock_start(yx_ctx *ctx) { ctx->host_mark = host_now_ns(); }
void host_clock_lap(yx_ctx *ctx, int phase) {
    const int64_t now = host_now_ns();
    ctx->host_ns[phase & 7] += (double)(now - ctx->host_mark);
    ctx->host_mark = now;
}
#endif

extern "C" int yx_hook_host_times(yx_ctx *ctx, double *out8, int reset) {
    if (!ctx || !out8) return YX_ERR_INVALID;
#ifdef YX_TRACE
    for (int i = 0; i < 8; i++) {
        out8[i] = ctx->host_ns[i];
        if (reset) ctx->host_ns[i] = 0.0;
    }
    return YX_OK;
#else
    (void)reset;
    return YX_ERR_UNSUPPORTED;
#endif
}

extern "C" int yx_hook_set_trace(yx_ctx *ctx, void *dev_buf) {
    if (!ctx) return YX_ERR_INVALID;
#ifdef YX_TRACE
    ctx->trace_buf = dev_buf;
    return YX_OK;
#else
    (void)dev_buf;
    return YX_ERR_UNSUPPORTED;
#endif
}
