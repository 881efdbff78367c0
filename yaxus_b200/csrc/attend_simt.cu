// Split-key attention on CUDA cores, for f32 KV storage (the reference's own cache type) and
// as a second, independent implementation the tensor-core kernel is checked against.
//
// Same contract as the reference's `attn_split` (crates/yaxus-backend-gpu/src/shaders.rs:1466-1579):
// per item (rows, one KV head, a run of keys) it emits, for every query head of the KV head's
// group, the running maximum m, the sum of exponentials l and the unnormalised output o.
// A CTA of four warps walks the items the planner gave it.  A warp takes every fourth key, eight of
// them in flight;
// a lane holds four of the 128 dims, so a K or V row is one coalesced 512-byte (f32) or
// 256-byte (16-bit) read per warp; the four warps' triples are merged in shared memory.
// K and V are read straight from global memory: each byte is used once per head chunk.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "yx_internal.h"

namespace yx {
namespace {

constexpr int WARPS = 4;
constexpr int HC = 4;  // query heads per sweep over the keys
constexpr int KU = 8;  // keys a warp has in flight
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float4 load4(const char *arena, int kv_dtype, uint32_t page, int hkv, int kvh, int tok,
                                        int lane) {
    int dim = lane * 4;
    if (kv_dtype == YX_F32) return *(const float4 *)((const float *)arena + kv_off32(page, hkv, kvh, tok, dim));
    uint2 raw = *(const uint2 *)((const uint16_t *)arena + kv_off16(page, hkv, kvh, tok, dim));
    float4 r;
    if (kv_dtype == YX_F16) {
        float2 a = __half22float2(*(const __half2 *)&raw.x), b = __half22float2(*(const __half2 *)&raw.y);
        r = make_float4(a.x, a.y, b.x, b.y);
    } else {
        float2 a = __bfloat1622float2(*(const __nv_bfloat162 *)&raw.x), b = __bfloat1622float2(*(const __nv_bfloat162 *)&raw.y);
        r = make_float4(a.x, a.y, b.x, b.y);
    }
    return r;
}

__device__ __forceinline__ float4 load_q4(const void *q, int q_dtype, size_t elem) {
    if (q_dtype == YX_F32) return *(const float4 *)((const float *)q + elem);
    uint2 raw = *(const uint2 *)((const uint16_t *)q + elem);
    if (q_dtype == YX_F16) {
        float2 a = __half22float2(*(const __half2 *)&raw.x), b = __half22float2(*(const __half2 *)&raw.y);
        return make_float4(a.x, a.y, b.x, b.y);
    }
    float2 a = __bfloat1622float2(*(const __nv_bfloat162 *)&raw.x), b = __bfloat1622float2(*(const __nv_bfloat162 *)&raw.y);
    return make_float4(a.x, a.y, b.x, b.y);
}

__global__ void __launch_bounds__(WARPS * 32)
attend_simt_kernel(const void *__restrict__ q, int q_dtype, int hq, int group, const char *__restrict__ k_arena,
                   const char *__restrict__ v_arena, int hkv, int kv_dtype, uint32_t kv_pages, uint32_t window,
                   const uint32_t *__restrict__ pos, const uint32_t *__restrict__ pages, const Item *__restrict__ items,
                   const uint32_t *__restrict__ cta_begin, float *__restrict__ part_o, float *__restrict__ part_ml,
                   yx_dev_status *status) {
    __shared__ float sm_o[WARPS][HC][D];
    __shared__ float sm_ml[WARPS][HC][2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float scale = 0.08838834764831845f;   // 1 / sqrt(128), the reference's f32 value
    // A programmatic dependent of the kernel before it: resident while that kernel finishes, it
    // waits here for everything earlier to be complete, and only then lets the merge kernel behind
    // it become resident in turn.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t ib = cta_begin[blockIdx.x], ie = cta_begin[blockIdx.x + 1];
    for (uint32_t ii = ib; ii < ie; ii++) {
        const Item it = items[ii];
        const int kvh = it.kv_head;
        for (int r = 0; r < it.n_rows; r++) {
            const uint32_t row = it.rows[r];
            const uint32_t p = pos[row];
            uint32_t lo = 0;
            if (window > 0 && p + 1 > window) lo = p + 1 - window;
            uint32_t k0 = max(max(lo, it.key_lo), it.tile_begin * TILE_KEYS);
            uint32_t k1 = min(min(p, it.key_hi), it.tile_end * TILE_KEYS - 1);   // inclusive
            for (int h0 = 0; h0 < group; h0 += HC) {
                float4 qv[HC];
                float m[HC], l[HC];
                float4 o[HC];
#pragma unroll
                for (int g = 0; g < HC; g++) {
                    int hh = min(h0 + g, group - 1);
                    qv[g] = load_q4(q, q_dtype, ((size_t)row * hq + kvh * group + hh) * D + lane * 4);
                    m[g] = -INFINITY;
                    l[g] = 0.0f;
                    o[g] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
                // KU keys of this warp at a time: their page ids, then their K and V rows, are asked
                // for together, so a round costs two memory latencies instead of two per key.
                for (uint64_t key0 = (uint64_t)k0 + warp; key0 <= k1; key0 += (uint64_t)WARPS * KU) {
                    float4 kk[KU], vv[KU];
                    bool live[KU];
                    uint32_t page[KU];
#pragma unroll
                    for (int u = 0; u < KU; u++) {
                        const uint64_t key = key0 + (uint64_t)u * WARPS;
                        live[u] = key <= k1;
                        page[u] = live[u] ? pages[it.pt_off + (uint32_t)(key / PAGE)] : 0u;
                    }
#pragma unroll
                    for (int u = 0; u < KU; u++) {
                        const uint64_t key = key0 + (uint64_t)u * WARPS;
                        if (live[u] && page[u] >= kv_pages) {   // recorded, the access is skipped
                            if (lane == 0 && atomicCAS(&status->code, 0, 1) == 0) {
                                status->where = 100;
                                status->a = (int)page[u];
                                status->b = (int)row;
                            }
                            live[u] = false;
                        }
                        kk[u] = vv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (live[u]) {
                            const int tok = (int)(key % PAGE);
                            kk[u] = load4(k_arena, kv_dtype, page[u], hkv, kvh, tok, lane);
                            vv[u] = load4(v_arena, kv_dtype, page[u], hkv, kvh, tok, lane);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < KU; u++) {
                        if (!live[u]) continue;   // (uniform over the warp)
                        float s[HC];
#pragma unroll
                        for (int g = 0; g < HC; g++)
                            s[g] = qv[g].x * kk[u].x + qv[g].y * kk[u].y + qv[g].z * kk[u].z + qv[g].w * kk[u].w;
#pragma unroll
                        for (int off = 16; off > 0; off >>= 1)
#pragma unroll
                            for (int g = 0; g < HC; g++) s[g] += __shfl_xor_sync(0xffffffffu, s[g], off);
#pragma unroll
                        for (int g = 0; g < HC; g++) {
                            float sc = s[g] * scale;
                            float mn = fmaxf(m[g], sc);
                            float a = exp2f((m[g] - mn) * LOG2E);   // 0 on the first key (m = -inf)
                            float e = exp2f((sc - mn) * LOG2E);
                            l[g] = l[g] * a + e;
                            o[g].x = o[g].x * a + e * vv[u].x;
                            o[g].y = o[g].y * a + e * vv[u].y;
                            o[g].z = o[g].z * a + e * vv[u].z;
                            o[g].w = o[g].w * a + e * vv[u].w;
                            m[g] = mn;
                        }
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
                        float mw = sm_ml[w][g][0];
                        float f = mw == -INFINITY ? 0.0f : exp2f((mw - mx) * LOG2E);
                        ls += sm_ml[w][g][1] * f;
                        acc += sm_o[w][g][t] * f;
                    }
                    size_t slot = (size_t)it.part[r] * group + h0 + g;
                    part_o[slot * D + t] = acc;
                    if (t == 0) {
                        // An item without a live key for this row: the reference's empty mark.
                        part_ml[slot * 2] = mx == -INFINITY ? -1e30f : mx;
                        part_ml[slot * 2 + 1] = ls;
                    }
                }
                __syncthreads();
            }
        }
    }
}

}  // namespace

int launch_attend_simt(yx_ctx *ctx, const AttendArgs &a) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)a.n_ctas);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const uint32_t window = (uint32_t)std::max<int64_t>(a.window, 0);
    if (int rc = check_cuda(ctx,
                            cudaLaunchKernelEx(&cfg, attend_simt_kernel, a.q, a.q_dtype, a.hq, a.group, (const char *)a.k_arena,
                                               (const char *)a.v_arena, a.hkv, a.kv_dtype, a.kv_pages, window,
                                               (const uint32_t *)ctx->d_pos, (const uint32_t *)ctx->d_pages, a.items, a.cta_begin,
                                               a.part_o, a.part_ml, ctx->dev_status),
                            "attend_simt kernel launch"))
        return rc;
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "attend_simt kernel");
}

}  // namespace yx
