// Merge of split-key partials: the reference's `attn_combine`
// (crates/yaxus-backend-gpu/src/shaders.rs:1581-1637).  One warp per (row, query head), a
// lane holds four of the 128 dims.  Parts with l <= 0 are dropped by value, because an empty
// part's o was never written (shaders.rs:1597-1598).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "yx_device.cuh"

namespace yx {
namespace {

__device__ __forceinline__ void store_out(void *out, int out_dtype, size_t elem, float4 v) {
    if (out_dtype == YX_F32) {
        *(float4 *)((float *)out + elem) = v;
    } else if (out_dtype == YX_F16) {
        __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
        uint2 pk = make_uint2(*(uint32_t *)&a, *(uint32_t *)&b);
        *(uint2 *)((uint16_t *)out + elem) = pk;
    } else {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 pk = make_uint2(*(uint32_t *)&a, *(uint32_t *)&b);
        *(uint2 *)((uint16_t *)out + elem) = pk;
    }
}

// Parts of (row, head) are slots first..first+count of its (row, kv head); the triple of
// slot s and head-in-group g sits at index s * group + g.  Lane c reads the (m, l) of part c,
// the warp agrees on the maximum and the weights, and only then are the o vectors read, all
// loads independent of one another: the merge costs two memory latencies, not two per part.
// LOOP: the grid has fewer warps than there are (row, head) pairs, and a warp takes several in turn.
template <bool LOOP>
__global__ void __launch_bounds__(128) combine_kernel(const Merge *__restrict__ merges, const float *__restrict__ part_o,
                               const float *__restrict__ part_ml, uint32_t n, int hq, int group, void *out,
                               int out_dtype, float *m_out, float *l_out, float *o_out, unsigned long long *trace) {
    // (diagnostic build: when this CTA entered and when its wait returned)
    if (YX_TR(trace != nullptr) && threadIdx.x == 0) trace[TRACE_MERGE_BASE + 4 * blockIdx.x] = dev::gtime();
    uint32_t idx = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t warps = (gridDim.x * blockDim.x) >> 5;   // the grid may be smaller than the work: see launch_combine
    int lane = threadIdx.x & 31;
    if (idx >= n) return;
    // The first pair's record is asked for before the wait (host-written: not the split-key kernel's output).
    Merge mg = merges[(size_t)(idx / (uint32_t)hq) * (hq / group) + (idx % (uint32_t)hq) / group];
    // Launched as a programmatic dependent of the split-key kernel: it is resident beside that
    // kernel's CTAs (four warps of 48 registers a thread: one warp fits in what three warps of the
    // split-key kernel leave of each register file partition) long before they finish.  The
    // kernel behind this one, usually the next attention call, may be made resident in turn.  The
    // triples are read only after the whole grid before this one is complete and its writes are
    // visible.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (YX_TR(trace != nullptr) && threadIdx.x == 0) trace[TRACE_MERGE_BASE + 4 * blockIdx.x + 1] = dev::gtime();
    for (bool first = true; idx < n; idx = LOOP ? idx + warps : n, first = false) {
    const int g = (int)(idx % (uint32_t)hq) % group;
    if (!first) mg = merges[(size_t)(idx / (uint32_t)hq) * (hq / group) + (idx % (uint32_t)hq) / group];
    if (mg.count == 0 && !o_out) continue;   // the row was another kernel's (tiled path)
    float mx = -1e30f, l = 0.0f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    // The first few vectors are asked for together with the (m, l) pairs: a row and KV head has
    // two or three parts on average, and the merge then costs one memory latency instead of two.
    // (A part that turns out empty is loaded but not used: its vector may never have been written.)
    constexpr int EARLY = 4;
    float4 early[EARLY];
#pragma unroll
    for (int j = 0; j < EARLY; j++) {
        early[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if ((uint32_t)j < mg.count) early[j] = *(const float4 *)(part_o + ((size_t)(mg.first + j) * group + g) * D + lane * 4);
    }
    for (uint32_t c0 = 0; c0 < mg.count; c0 += 32) {
        const uint32_t c = c0 + lane;
        float em = -1e30f, el = 0.0f;
        if (c < mg.count) {
            float2 v = *(const float2 *)(part_ml + ((size_t)(mg.first + c) * group + g) * 2);
            em = v.x;
            el = v.y;
        }
        const bool live = el > 0.0f;
        float cm = live ? em : -1e30f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
        const float nm = fmaxf(mx, cm);
        const float r = __expf(mx - nm);
        const float w = live ? __expf(em - nm) : 0.0f;
        float ls = el * w;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, o);
        l = l * r + ls;
        acc.x *= r;
        acc.y *= r;
        acc.z *= r;
        acc.w *= r;
        mx = nm;
        const int nc = (int)min(32u, mg.count - c0);
        int j0 = 0;
        if (c0 == 0) {
#pragma unroll
            for (int j = 0; j < EARLY; j++) {
                const float wj = __shfl_sync(0xffffffffu, w, j);
                if (j < nc && wj > 0.0f) {
                    acc.x += early[j].x * wj;
                    acc.y += early[j].y * wj;
                    acc.z += early[j].z * wj;
                    acc.w += early[j].w * wj;
                }
            }
            j0 = EARLY;
        }
#pragma unroll 4
        for (int j = j0; j < nc; j++) {
            const float wj = __shfl_sync(0xffffffffu, w, j);
            if (wj > 0.0f) {   // an empty part's o was never written
                float4 po = *(const float4 *)(part_o + ((size_t)(mg.first + c0 + j) * group + g) * D + lane * 4);
                acc.x += po.x * wj;
                acc.y += po.y * wj;
                acc.z += po.z * wj;
                acc.w += po.w * wj;
            }
        }
    }
    if (out) {
        float inv = 1.0f / l;   // a row always sees its own key, so l > 0 for whole attention
        store_out(out, out_dtype, (size_t)idx * D + lane * 4, make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv));
    }
    if (o_out) {
        *(float4 *)(o_out + (size_t)idx * D + lane * 4) = acc;
        if (lane == 0) {
            m_out[idx] = mx;
            l_out[idx] = l;
        }
    }
    }
    if (YX_TR(trace != nullptr) && threadIdx.x == 0) trace[TRACE_MERGE_BASE + 4 * blockIdx.x + 2] = dev::gtime();
}

// Part c of element idx: m[c * sm + idx], l[c * sl + idx], o[c * so + idx * 128 ..].
__global__ void combine_flat_kernel(int n_parts, const float *__restrict__ m, const float *__restrict__ l,
                                    const float *__restrict__ o, size_t sm, size_t sl, size_t so, size_t n, void *out,
                                    int out_dtype) {
    size_t idx = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (idx >= n) return;
    float mx = -1e30f, ls = 0.0f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c = 0; c < n_parts; c++) {
        float em = m[(size_t)c * sm + idx], el = l[(size_t)c * sl + idx];
        if (!(el > 0.0f)) continue;
        float4 po = *(const float4 *)(o + (size_t)c * so + idx * D + lane * 4);
        float nm = fmaxf(mx, em);
        float r = __expf(mx - nm), w = __expf(em - nm);
        ls = ls * r + el * w;
        acc.x = acc.x * r + po.x * w;
        acc.y = acc.y * r + po.y * w;
        acc.z = acc.z * r + po.z * w;
        acc.w = acc.w * r + po.w * w;
        mx = nm;
    }
    float inv = 1.0f / ls;
    store_out(out, out_dtype, idx * D + lane * 4, make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv));
}

__global__ void fill_empty_kernel(size_t n, float *m, float *l, float *o) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n * D) o[i] = 0.0f;
    if (i < n) {
        m[i] = -1e30f;
        l[i] = 0.0f;
    }
}

}  // namespace

int launch_fill_empty(yx_ctx *ctx, size_t n, float *m, float *l, float *o) {
    size_t blocks = (n * D + 255) / 256;
    fill_empty_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(n, m, l, o);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "fill_empty kernel");
}

int launch_combine(yx_ctx *ctx, const Merge *merges, const float *part_o, const float *part_ml, int rows, int hq,
                   int group, void *out, int out_dtype, float *m_out, float *l_out, float *o_out, bool chained) {
    uint32_t n = (uint32_t)rows * (uint32_t)hq;
    uint32_t blocks = (n * 32 + 127) / 128;
    // In a run of back-to-back attention calls the next call's kernel is this kernel's programmatic
    // dependent: it cannot start before every CTA of this grid has started, and beside a CTA of
    // the split-key kernel an SM has room for one of these only.  A verification pass (80 rows, 640
    // CTAs) then held the next call back until the split-key kernel's CTAs had left: 35.8 us a
    // call where a grid of one CTA per SM, each taking several (row, head) pairs in turn, gives
    // 29.5 us (grids of 1.5 to 3 CTAs per SM: 37-39 us).  Up to about seven pairs a warp this pays
    // (128 rows: 36.4 against 41.3 us); with nine (160 rows: 39.1 against 37.3 us) the merge is too
    // long to hide, and such passes, like prompt-sized ones, keep the full grid.
    const bool loop = chained && blocks > (uint32_t)ctx->sm_count && blocks <= 8u * (uint32_t)ctx->sm_count;
    if (loop) blocks = (uint32_t)ctx->sm_count;
    if (!ctx->smem_configured[2]) {
        // Same shared-memory carve-out as the split-key kernel it follows, so that the SMs are
        // not reconfigured between the two on every attention call.
        cudaFuncSetAttribute(combine_kernel<false>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(combine_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        ctx->smem_configured[2] = true;
    }
    // Programmatic stream serialisation: the launch is set up while the kernel before it still
    // runs, which hides a launch latency that is a tenth of a decode step.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (int rc = check_cuda(ctx, cudaLaunchKernelEx(&cfg, loop ? combine_kernel<true> : combine_kernel<false>, merges, part_o, part_ml, n, hq, group, out, out_dtype, m_out, l_out, o_out,
                                                    (unsigned long long *)ctx->trace_buf),
                            "combine kernel launch"))
        return rc;
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "combine kernel");
}

int launch_combine_strided(yx_ctx *ctx, int n_parts, const float *m, const float *l, const float *o, size_t sm,
                           size_t sl, size_t so, size_t n, void *out, int out_dtype) {
    size_t blocks = (n * 32 + 127) / 128;
    if (!ctx->smem_configured[3]) {
        cudaFuncSetAttribute(combine_flat_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        ctx->smem_configured[3] = true;
    }
    combine_flat_kernel<<<(unsigned)blocks, 128, 0, ctx->stream>>>(n_parts, m, l, o, sm, sl, so, n, out, out_dtype);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "combine_flat kernel");
}

}  // namespace yx
