// KV page writes: plain append, fused norm + RoPE + append, page copy, page import/export.
// All of them are pure index work over small amounts of data; what matters is that the slot
// arithmetic is exactly the reference's (crates/yaxus-model/src/kv.rs:20-22) and that stores
// are 16-byte vectors.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "yx_internal.h"

namespace yx {
namespace {

__device__ __forceinline__ uint16_t to_storage(float x, int dtype) {
    // Round to nearest even, as the oracle rounds on the host.
    if (dtype == YX_F16) return __half_as_ushort(__float2half_rn(x));
    return __bfloat16_as_ushort(__float2bfloat16_rn(x));
}

// A packed pair of bf16 values holds one that f16 cannot: magnitude 65536 or more, infinite or NaN.
__device__ __forceinline__ bool bf16_pair_is_wide(uint32_t w) { return (w & 0x7fffu) >= 0x4780u || ((w >> 16) & 0x7fffu) >= 0x4780u; }

// One thread per 8 consecutive dims of one (row, kv head) of K or V.
// grid.x covers rows * hkv * 16 chunks, grid.y: 0 = K, 1 = V.
__global__ void append_kernel(const void *__restrict__ k_rows, const void *__restrict__ v_rows, int src_dtype,
                              const uint32_t *__restrict__ kv_slot, uint32_t rows, int hkv, int kv_dtype,
                              char *__restrict__ k_arena, char *__restrict__ v_arena, uint32_t *__restrict__ wide_v) {
    // The attention kernel that follows is launched as a programmatic dependent: it may be made
    // resident now, and copies K/V tiles that this kernel does not write while this kernel runs.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t total = rows * (uint32_t)hkv * 16u;
    if (idx >= total) return;
    const bool is_v = blockIdx.y == 1;
    uint32_t chunk = idx & 15u;
    uint32_t h = (idx >> 4) % (uint32_t)hkv;
    uint32_t row = (idx >> 4) / (uint32_t)hkv;
    uint32_t slot = kv_slot[row];
    uint32_t page = slot / PAGE;
    int tok = (int)(slot % PAGE);
    int dim = (int)chunk * 8;
    const char *src = (const char *)(is_v ? v_rows : k_rows);
    char *arena = is_v ? v_arena : k_arena;
    size_t src_elem = ((size_t)row * hkv + h) * D + dim;
    if (kv_dtype == YX_F32) {
        const float4 *s = (const float4 *)(src + src_elem * 4);
        float4 a = s[0], b = s[1];
        float4 *d = (float4 *)(arena + kv_off32(page, hkv, (int)h, tok, dim) * 4);
        d[0] = a;
        d[1] = b;
        return;
    }
    uint4 packed;
    if (src_dtype == YX_F32) {
        const float4 *s = (const float4 *)(src + src_elem * 4);
        float4 a = s[0], b = s[1];
        packed.x = (uint32_t)to_storage(a.x, kv_dtype) | ((uint32_t)to_storage(a.y, kv_dtype) << 16);
        packed.y = (uint32_t)to_storage(a.z, kv_dtype) | ((uint32_t)to_storage(a.w, kv_dtype) << 16);
        packed.z = (uint32_t)to_storage(b.x, kv_dtype) | ((uint32_t)to_storage(b.y, kv_dtype) << 16);
        packed.w = (uint32_t)to_storage(b.z, kv_dtype) | ((uint32_t)to_storage(b.w, kv_dtype) << 16);
    } else {
        packed = *(const uint4 *)(src + src_elem * 2);
    }
    if (is_v && kv_dtype == YX_BF16 &&
        (bf16_pair_is_wide(packed.x) || bf16_pair_is_wide(packed.y) || bf16_pair_is_wide(packed.z) || bf16_pair_is_wide(packed.w)))
        atomicOr(wide_v, 1u);
    *(uint4 *)(arena + kv_off16(page, hkv, (int)h, tok, dim) * 2) = packed;
}

// write_rows (crates/yaxus-backend-cpu/src/lib.rs:359-385) ≡ qk_rope
// (crates/yaxus-backend-gpu/src/shaders.rs:285-341).  One warp per (row, head) over the
// hq + 2*hkv heads of a qkv row.  Lane l holds dims {2l, 2l+1, 2l+64, 2l+65}: both members of
// two rotation pairs.  cos/sin follow crates/yaxus-model/src/config.rs:213-219: f32 angle,
// f64 cos/sin, f32 result times the concentration.
__global__ void qk_rope_append_kernel(const float *__restrict__ qkv, const float *__restrict__ q_norm,
                                      const float *__restrict__ k_norm, const uint32_t *__restrict__ pos,
                                      const uint32_t *__restrict__ kv_slot, uint32_t rows, int hq, int hkv,
                                      float eps, const yx_rope *__restrict__ rope, int kv_dtype,
                                      char *__restrict__ k_arena, char *__restrict__ v_arena,
                                      float *__restrict__ q_out, uint32_t *__restrict__ wide_v) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // see append_kernel
    const int heads = hq + 2 * hkv;
    uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (warp >= rows * (uint32_t)heads) return;
    uint32_t row = warp / (uint32_t)heads;
    int head = (int)(warp % (uint32_t)heads);
    const float *x = qkv + ((size_t)row * heads + head) * D;
    float2 lo = *(const float2 *)(x + 2 * lane);
    float2 hi = *(const float2 *)(x + 64 + 2 * lane);
    const bool is_q = head < hq, is_k = !is_q && head < hq + hkv;
    float r0 = lo.x, r1 = lo.y, r2 = hi.x, r3 = hi.y;
    if (is_q || is_k) {
        float ss = lo.x * lo.x + lo.y * lo.y + hi.x * hi.x + hi.y * hi.y;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        float r = 1.0f / sqrtf(ss / (float)D + eps);
        const float *w = is_q ? q_norm : k_norm;
        float2 wl = *(const float2 *)(w + 2 * lane), wh = *(const float2 *)(w + 64 + 2 * lane);
        // Separate roundings (no fused multiply-add), as in the reference's Rust arithmetic.
        float a0 = __fmul_rn(1.0f + wl.x, __fmul_rn(lo.x, r)), a1 = __fmul_rn(1.0f + wl.y, __fmul_rn(lo.y, r));
        float b0 = __fmul_rn(1.0f + wh.x, __fmul_rn(hi.x, r)), b1 = __fmul_rn(1.0f + wh.y, __fmul_rn(hi.y, r));
        float p = (float)pos[row];
        float ang0 = __fmul_rn(p, rope->inv_freq[2 * lane]), ang1 = __fmul_rn(p, rope->inv_freq[2 * lane + 1]);
        float conc = rope->concentration;
        float c0 = __fmul_rn((float)cos((double)ang0), conc), s0 = __fmul_rn((float)sin((double)ang0), conc);
        float c1 = __fmul_rn((float)cos((double)ang1), conc), s1 = __fmul_rn((float)sin((double)ang1), conc);
        r0 = __fsub_rn(__fmul_rn(a0, c0), __fmul_rn(b0, s0));
        r2 = __fadd_rn(__fmul_rn(b0, c0), __fmul_rn(a0, s0));
        r1 = __fsub_rn(__fmul_rn(a1, c1), __fmul_rn(b1, s1));
        r3 = __fadd_rn(__fmul_rn(b1, c1), __fmul_rn(a1, s1));
    }
    if (is_q) {
        float *q = q_out + ((size_t)row * hq + head) * D;
        *(float2 *)(q + 2 * lane) = make_float2(r0, r1);
        *(float2 *)(q + 64 + 2 * lane) = make_float2(r2, r3);
        return;
    }
    int h = is_k ? head - hq : head - hq - hkv;
    char *arena = is_k ? k_arena : v_arena;
    uint32_t slot = kv_slot[row];
    uint32_t page = slot / PAGE;
    int tok = (int)(slot % PAGE);
    if (kv_dtype == YX_F32) {
        float *d = (float *)arena + kv_off32(page, hkv, h, tok, 0);
        *(float2 *)(d + 2 * lane) = make_float2(r0, r1);
        *(float2 *)(d + 64 + 2 * lane) = make_float2(r2, r3);
    } else {
        uint32_t a = (uint32_t)to_storage(r0, kv_dtype) | ((uint32_t)to_storage(r1, kv_dtype) << 16);
        uint32_t b = (uint32_t)to_storage(r2, kv_dtype) | ((uint32_t)to_storage(r3, kv_dtype) << 16);
        if (!is_k && kv_dtype == YX_BF16 && (bf16_pair_is_wide(a) || bf16_pair_is_wide(b))) atomicOr(wide_v, 1u);
        uint16_t *base = (uint16_t *)arena;
        *(uint32_t *)(base + kv_off16(page, hkv, h, tok, 2 * lane)) = a;
        *(uint32_t *)(base + kv_off16(page, hkv, h, tok, 64 + 2 * lane)) = b;
    }
}

// copy_page (cpu lib.rs:472-479): a page is one contiguous run of hkv blocks in this layout,
// so the copy is a straight 16-byte-vector copy per layer for K and for V.
// grid.y = layer * 2 + (0 K, 1 V).
__global__ void copy_page_kernel(char *k_base, char *v_base, size_t layer_bytes, size_t page_bytes, uint32_t src,
                                 uint32_t dst) {
    int layer = blockIdx.y >> 1;
    char *arena = ((blockIdx.y & 1) ? v_base : k_base) + (size_t)layer * layer_bytes;
    const uint4 *s = (const uint4 *)(arena + (size_t)src * page_bytes);
    uint4 *d = (uint4 *)(arena + (size_t)dst * page_bytes);
    size_t n = page_bytes / 16;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) d[i] = s[i];
}

// Page import/export between the private layout and the reference's `[tok][hkv*128]`.
// One thread per element.
__global__ void page_io_kernel(char *k_arena, char *v_arena, int hkv, int kv_dtype, uint32_t first_page,
                               uint32_t n_pages, char *k_lin, char *v_lin, int write, uint32_t *wide_v) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t per_page = (size_t)PAGE * hkv * D;
    if (idx >= per_page * n_pages) return;
    char *arena = blockIdx.y ? v_arena : k_arena;
    char *lin = blockIdx.y ? v_lin : k_lin;
    uint32_t page = first_page + (uint32_t)(idx / per_page);
    uint32_t in_page = (uint32_t)(idx % per_page);
    int dim = in_page % D;
    int h = (in_page / D) % hkv;
    int tok = in_page / (D * hkv);
    if (kv_dtype == YX_F32) {
        float *a = (float *)arena + kv_off32(page, hkv, h, tok, dim);
        float *l = (float *)lin + idx;
        if (write) *a = *l;
        else *l = *a;
    } else {
        uint16_t *a = (uint16_t *)arena + kv_off16(page, hkv, h, tok, dim);
        uint16_t *l = (uint16_t *)lin + idx;
        if (write) {
            *a = *l;
            if (blockIdx.y && kv_dtype == YX_BF16 && (*l & 0x7fffu) >= 0x4780u) atomicOr(wide_v, 1u);
        } else {
            *l = *a;
        }
    }
}

}  // namespace

int launch_append(yx_ctx *ctx, yx_kv *kv, int layer, const void *k_rows, const void *v_rows, int src_dtype) {
    uint32_t rows = ctx->pass.rows;
    uint32_t total = rows * (uint32_t)kv->hkv * 16u;
    dim3 grid((total + 255) / 256, 2);
    if (!ctx->smem_configured[4]) {
        // Keep the carve-out of the attention kernels these run between.
        cudaFuncSetAttribute(append_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(qk_rope_append_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        ctx->smem_configured[4] = true;
    }
    append_kernel<<<grid, 256, 0, ctx->stream>>>(k_rows, v_rows, src_dtype, ctx->d_slot, rows, kv->hkv, kv->dtype,
                                                  kv->k(layer), kv->v(layer), kv->wide_v_dev);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "append kernel");
}

int launch_qk_rope_append(yx_ctx *ctx, yx_kv *kv, int layer, const float *qkv, const float *q_norm,
                          const float *k_norm, int hq, float eps, float *q_out) {
    uint32_t rows = ctx->pass.rows;
    uint64_t warps = (uint64_t)rows * (hq + 2 * kv->hkv);
    uint32_t blocks = (uint32_t)((warps * 32 + 255) / 256);
    if (!ctx->smem_configured[4]) {
        cudaFuncSetAttribute(append_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(qk_rope_append_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        ctx->smem_configured[4] = true;
    }
    qk_rope_append_kernel<<<blocks, 256, 0, ctx->stream>>>(qkv, q_norm, k_norm, ctx->d_pos, ctx->d_slot, rows, hq,
                                                          kv->hkv, eps, (const yx_rope *)kv->rope_dev + layer,
                                                          kv->dtype, kv->k(layer), kv->v(layer), q_out, kv->wide_v_dev);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "qk_rope_append kernel");
}

int launch_copy_page(yx_ctx *ctx, yx_kv *kv, uint32_t src, uint32_t dst) {
    size_t page_bytes = (size_t)kv->hkv * kv_block_elems() * kv->esize;
    dim3 grid((unsigned)std::min<size_t>(64, (page_bytes / 16 + 255) / 256), (unsigned)kv->n_layers * 2);
    copy_page_kernel<<<grid, 256, 0, ctx->stream>>>(kv->k_base, kv->v_base, kv->layer_bytes, page_bytes, src, dst);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "copy_page kernel");
}

int launch_page_io(yx_ctx *ctx, yx_kv *kv, int layer, uint32_t first_page, uint32_t n_pages, void *k_lin, void *v_lin,
                   bool write) {
    size_t total = (size_t)n_pages * PAGE * kv->hkv * D;
    dim3 grid((unsigned)((total + 255) / 256), 2);
    page_io_kernel<<<grid, 256, 0, ctx->stream>>>(kv->k(layer), kv->v(layer), kv->hkv, kv->dtype, first_page, n_pages,
                                                   (char *)k_lin, (char *)v_lin, write ? 1 : 0, kv->wide_v_dev);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "page_io kernel");
}

}  // namespace yx
