// yx_attend_static: attend (crates/yaxus-backend-cpu/src/lib.rs:389-427) for small passes with
// no allocation of any kind inside the call.
//
// It is a variant of the CUDA-core split-key kernel: every (pass row, KV head) has its keys cut
// into a fixed number of runs, one CTA per run writes the partial triple (m, l, o) of each query
// head of the group, and a second kernel merges the runs.  The partial triples do not live in
// a workspace obtained from the allocator but in a device array that is part of this module's
// image, so the call needs no memory beyond what the process already holds.
//
// Who needs that: an engine sizes its KV page pool to whatever device memory is left once the
// weights are resident, so an attention call that grows a workspace later can meet an empty
// device; and a device allocation stalls every stream of the device while it is served, which a
// decode loop that was promised a steady step time cannot afford.  Such a caller wants every
// byte settled before the loop starts.
//
// Set-up: the first call on a device looks the scratch array's address up.  Make that first
// call before any stream capture begins.  Later calls only launch the two kernels.
//
// Concurrency: the scratch array is one per device context (a process that only uses the
// runtime API has one context per device).  Two calls whose kernels may overlap in the same
// context (different streams, different yx_ctx objects, different threads) race on it and give
// wrong results; order them on one stream or with events.  The address is looked up again when
// the calling thread's current CUDA context is not the one it was looked up in (after a device
// reset, or under a driver-API context): a symbol's address belongs to a context.
//
// Nothing in the scratch has to start at zero: every triple a merge reads was written by the
// first kernel of the same call (a run without a live key writes the empty mark -1e30, 0).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <dlfcn.h>

#include <mutex>
#include <string>

#include "yx_device.cuh"
#include "yx_internal.h"

namespace yx {
namespace {

constexpr int SPLITS = YX_STATIC_SPLITS;
constexpr int MAX_ROW_HEADS = YX_STATIC_MAX_ROW_HEADS;
constexpr int WARPS = 4;
constexpr int HC = 4;   // query heads per sweep over the keys
constexpr float LOG2E = 1.4426950408889634f;
constexpr int MAX_DEVICES = 64;

// [row * hkv + kv head][run][head in group]: o 128 floats, then (m, l) pairs.  4 MiB + 64 KiB.
struct StaticScratch {
    float o[(size_t)MAX_ROW_HEADS * SPLITS * D];
    float ml[(size_t)MAX_ROW_HEADS * SPLITS * 2];
};
static __device__ __align__(256) StaticScratch g_static_scratch;

std::mutex g_lookup_lock;
StaticScratch *g_scratch_addr[MAX_DEVICES] = {};
void *g_scratch_ctx[MAX_DEVICES] = {};   // the CUDA context each address was looked up in

// The calling thread's current CUDA context, or null if the driver library cannot be asked (the
// runtime has it loaded already; nothing is linked against it).
void *current_cuda_context() {
    using Fn = int (*)(void **);
    static Fn fn = [] {
        void *h = dlopen("libcuda.so.1", RTLD_LAZY | RTLD_NOLOAD);
        return h ? (Fn)dlsym(h, "cuCtxGetCurrent") : (Fn) nullptr;
    }();
    void *c = nullptr;
    if (fn && fn(&c) == 0) return c;
    return nullptr;
}

// The array's address on `device`, which must be the current device.  Looked up once per device
// and context; a changed context means a different copy of the array at a different address.
cudaError_t scratch_on(int device, StaticScratch **out) {
    std::lock_guard<std::mutex> hold(g_lookup_lock);
    void *now = current_cuda_context();
    if (!g_scratch_addr[device] || g_scratch_ctx[device] != now) {
        StaticScratch *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **)&p, g_static_scratch);
        if (e != cudaSuccess) return e;
        g_scratch_addr[device] = p;
        // the runtime may have made the context current only inside the call above
        g_scratch_ctx[device] = now ? now : current_cuda_context();
    }
    *out = g_scratch_addr[device];
    return cudaSuccess;
}

__device__ __forceinline__ float4 load_kv4(const char *arena, int kv_dtype, uint32_t page, int hkv, int kvh, int tok,
                                           int lane) {
    const int dim = lane * 4;
    if (kv_dtype == YX_F32) return *(const float4 *)((const float *)arena + kv_off32(page, hkv, kvh, tok, dim));
    return dev::load4_as_f32(arena, kv_dtype, kv_off16(page, hkv, kvh, tok, dim));
}

// grid (rows * hkv, SPLITS); a warp takes every fourth key of the run, a lane four dims.
__global__ void __launch_bounds__(WARPS * 32)
attend_static_split_kernel(const void *__restrict__ q, int q_dtype, int hq, int group, const char *__restrict__ k_arena,
                           const char *__restrict__ v_arena, int hkv, int kv_dtype, uint32_t kv_pages, uint32_t window,
                           const uint32_t *__restrict__ pos, const uint32_t *__restrict__ pt_off,
                           const uint32_t *__restrict__ pages, StaticScratch *scratch, yx_dev_status *status) {
    __shared__ float sm_o[WARPS][HC][D];
    __shared__ float sm_ml[WARPS][HC][2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float scale = 0.08838834764831845f;   // 1 / sqrt(128), the reference's f32 value
    const uint32_t row = blockIdx.x / (uint32_t)hkv;
    const int kvh = (int)(blockIdx.x % (uint32_t)hkv);
    const uint32_t p = pos[row], pto = pt_off[row];
    uint32_t lo = 0;
    if (window > 0 && p + 1 > window) lo = p + 1 - window;
    // keys lo..=p in SPLITS runs of equal length (the last ones may be empty)
    const uint32_t n_keys = p - lo + 1;
    const uint32_t per = (n_keys + SPLITS - 1) / SPLITS;
    const uint64_t k0 = (uint64_t)lo + (uint64_t)blockIdx.y * per;
    const uint64_t k1 = min(k0 + per, (uint64_t)p + 1);   // exclusive
    for (int h0 = 0; h0 < group; h0 += HC) {
        float4 qv[HC], o[HC];
        float m[HC], l[HC];
#pragma unroll
        for (int g = 0; g < HC; g++) {
            const int hh = min(h0 + g, group - 1);
            qv[g] = dev::load4_as_f32(q, q_dtype, ((size_t)row * hq + kvh * group + hh) * D + lane * 4);
            m[g] = -INFINITY;
            l[g] = 0.0f;
            o[g] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        for (uint64_t key = k0 + warp; key < k1; key += WARPS) {
            const uint32_t page = pages[pto + (uint32_t)(key / PAGE)];
            if (page >= kv_pages) {   // recorded, the access is skipped
                if (lane == 0 && atomicCAS(&status->code, 0, 1) == 0) {
                    status->where = 600;
                    status->a = (int)page;
                    status->b = (int)row;
                }
                continue;
            }
            const int tok = (int)(key % PAGE);
            const float4 kk = load_kv4(k_arena, kv_dtype, page, hkv, kvh, tok, lane);
            const float4 vv = load_kv4(v_arena, kv_dtype, page, hkv, kvh, tok, lane);
            float s[HC];
#pragma unroll
            for (int g = 0; g < HC; g++) s[g] = qv[g].x * kk.x + qv[g].y * kk.y + qv[g].z * kk.z + qv[g].w * kk.w;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1)
#pragma unroll
                for (int g = 0; g < HC; g++) s[g] += __shfl_xor_sync(0xffffffffu, s[g], off);
#pragma unroll
            for (int g = 0; g < HC; g++) {
                const float sc = s[g] * scale;
                const float mn = fmaxf(m[g], sc);
                const float a = exp2f((m[g] - mn) * LOG2E);   // 0 on the first key (m = -inf)
                const float e = exp2f((sc - mn) * LOG2E);
                l[g] = l[g] * a + e;
                o[g].x = o[g].x * a + e * vv.x;
                o[g].y = o[g].y * a + e * vv.y;
                o[g].z = o[g].z * a + e * vv.z;
                o[g].w = o[g].w * a + e * vv.w;
                m[g] = mn;
            }
        }
#pragma unroll
        for (int g = 0; g < HC; g++) {
            *(float4 *)&sm_o[warp][g][lane * 4] = o[g];
            if (lane == 0) {
                sm_ml[warp][g][0] = m[g];
                sm_ml[warp][g][1] = l[g];
            }
        }
        __syncthreads();
        // Thread t merges dim t of the four warps' triples, head by head.
        const int t = threadIdx.x;
#pragma unroll
        for (int g = 0; g < HC; g++) {
            if (h0 + g >= group) break;
            float mx = -INFINITY;
#pragma unroll
            for (int w = 0; w < WARPS; w++) mx = fmaxf(mx, sm_ml[w][g][0]);
            float ls = 0.0f, acc = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; w++) {
                const float mw = sm_ml[w][g][0];
                const float f = mw == -INFINITY ? 0.0f : exp2f((mw - mx) * LOG2E);
                ls += sm_ml[w][g][1] * f;
                acc += sm_o[w][g][t] * f;
            }
            const size_t slot = ((size_t)blockIdx.x * SPLITS + blockIdx.y) * group + h0 + g;
            scratch->o[slot * D + t] = acc;
            if (t == 0) {
                scratch->ml[slot * 2] = mx == -INFINITY ? -1e30f : mx;   // the reference's empty mark
                scratch->ml[slot * 2 + 1] = ls;
            }
        }
        __syncthreads();
    }
}

// One CTA of 128 threads per (row, query head): thread t merges dim t of the SPLITS runs.
// Runs with l <= 0 are dropped by value (crates/yaxus-backend-gpu/src/shaders.rs:1597-1598).
__global__ void __launch_bounds__(D)
attend_static_merge_kernel(const StaticScratch *__restrict__ scratch, int hq, int group, void *out, int out_dtype) {
    __shared__ float sm_out[D];
    const uint32_t row = blockIdx.x / (uint32_t)hq;
    const int h = (int)(blockIdx.x % (uint32_t)hq), kvh = h / group, g = h % group;
    const int hkv = hq / group, t = threadIdx.x;
    const size_t first = ((size_t)(row * hkv + kvh) * SPLITS) * group + g;
    float mx = -1e30f;
#pragma unroll
    for (int s = 0; s < SPLITS; s++) {
        const size_t slot = first + (size_t)s * group;
        if (scratch->ml[slot * 2 + 1] > 0.0f) mx = fmaxf(mx, scratch->ml[slot * 2]);
    }
    float l = 0.0f, acc = 0.0f;
#pragma unroll
    for (int s = 0; s < SPLITS; s++) {
        const size_t slot = first + (size_t)s * group;
        const float el = scratch->ml[slot * 2 + 1];
        if (el > 0.0f) {
            const float w = exp2f((scratch->ml[slot * 2] - mx) * LOG2E);
            l += el * w;
            acc += scratch->o[slot * D + t] * w;
        }
    }
    sm_out[t] = l > 0.0f ? acc / l : 0.0f;
    __syncthreads();
    if (t < D / 4)
        dev::store4(out, out_dtype, ((size_t)row * hq + h) * D + t * 4,
                    make_float4(sm_out[t * 4], sm_out[t * 4 + 1], sm_out[t * 4 + 2], sm_out[t * 4 + 3]));
}

}  // namespace
}  // namespace yx

using namespace yx;

extern "C" int yx_attend_static(yx_ctx *ctx, yx_kv *kv, int layer, const void *q, int q_dtype, int hq, int64_t window,
                                void *out, int out_dtype) {
    if (!ctx || !kv) return YX_ERR_INVALID;
    if (ctx->status != YX_OK) return ctx->status;
    if (!ctx->have_pass) return fail(ctx, YX_ERR_STATE, "yx_attend_static without begin_pass");
    if (layer < 0 || layer >= kv->n_layers) return fail(ctx, YX_ERR_INVALID, "yx_attend_static: layer out of range");
    if (hq <= 0 || hq % kv->hkv != 0) return fail(ctx, YX_ERR_INVALID, "yx_attend_static: hq must be a positive multiple of hkv");
    if (q_dtype < YX_F32 || q_dtype > YX_BF16 || out_dtype < YX_F32 || out_dtype > YX_BF16)
        return fail(ctx, YX_ERR_INVALID, "yx_attend_static: bad dtype");
    const uint32_t rows = ctx->pass.rows;
    if (rows == 0) return YX_OK;
    if (!q || !out) return fail(ctx, YX_ERR_INVALID, "yx_attend_static: null tensor");
    if ((uint64_t)rows * (uint64_t)hq > (uint64_t)MAX_ROW_HEADS)
        return fail(ctx, YX_ERR_INVALID,
                    "yx_attend_static: rows * hq = " + std::to_string((uint64_t)rows * hq) +
                        " exceeds YX_STATIC_MAX_ROW_HEADS = " + std::to_string(MAX_ROW_HEADS) +
                        " (the size of the built-in scratch); use yx_attend");
    if (ctx->device < 0 || ctx->device >= MAX_DEVICES) return fail(ctx, YX_ERR_INVALID, "yx_attend_static: device index out of range");
    int current = -1;
    if (int rc = check_cuda(ctx, cudaGetDevice(&current), "yx_attend_static: current device")) return rc;
    if (current != ctx->device)
        return fail(ctx, YX_ERR_STATE, "yx_attend_static: the context's device must be the current device");
    // The same host-side checks as yx_attend (the kernel's own record-and-skip is the second line).
    if (ctx->pass.max_pos_seen >= kv->max_pos) return fail(ctx, YX_ERR_INVALID, "a row's position exceeds max_pos");
    if (ctx->pass.max_page_seen >= kv->pages && !ctx->pass.pages.empty())
        return fail(ctx, YX_ERR_INVALID, "page id outside the KV arena");
    StaticScratch *scratch = nullptr;
    if (int rc = check_cuda(ctx, scratch_on(ctx->device, &scratch), "yx_attend_static: scratch address")) return rc;
    int64_t w = window < 0 ? (int64_t)kv->layers[layer].window : window;
    if (w > (int64_t)UINT32_MAX) w = (int64_t)UINT32_MAX;   // wider than any position: the same as none
    const int group = hq / kv->hkv;
    attend_static_split_kernel<<<dim3(rows * (uint32_t)kv->hkv, SPLITS), WARPS * 32, 0, ctx->stream>>>(
        q, q_dtype, hq, group, kv->k(layer), kv->v(layer), kv->hkv, kv->dtype, kv->pages, (uint32_t)(w > 0 ? w : 0),
        ctx->d_pos, ctx->d_ptoff, ctx->d_pages, scratch, ctx->dev_status);
    ctx->launches++;
    if (int rc = check_cuda(ctx, cudaGetLastError(), "attend_static split kernel")) return rc;
    attend_static_merge_kernel<<<rows * (uint32_t)hq, D, 0, ctx->stream>>>(scratch, hq, group, out, out_dtype);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "attend_static merge kernel");
}
