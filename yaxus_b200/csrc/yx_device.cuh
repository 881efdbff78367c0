// Device-side helpers shared by the attention kernels: mbarriers with bounded waits, bulk
// asynchronous copies, ldmatrix / mma.sync wrappers, storage-type packing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "yx_internal.h"

namespace yx {
namespace dev {

constexpr long long WAIT_CYCLES = 4000000000ll;   // about two seconds at 2 GHz

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Transpose of an 8x8 matrix of 16-bit elements held one row pair per thread across the warp.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns at once when the CTA has given up; on expiry it raises the CTA's
// abort flag and records where in the context's status word.  Nothing spins forever.  The
// spinning part is out of line: it is cold code, and the attention kernels pay for every
// instruction-cache line they touch.
static __device__ __noinline__ void mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                            yx_dev_status *status, int where) {
    if (*abort_flag) return;
    long long t0 = clock64();
    for (uint32_t spins = 1;; spins++) {
        if (mbar_try(bar, parity)) return;
        if ((spins & 255u) == 0) {
            if (*abort_flag) return;
            if (clock64() - t0 > WAIT_CYCLES) {
                *abort_flag = 1;
                if (atomicCAS(&status->code, 0, 2) == 0) {
                    status->where = where;
                    status->a = (int)blockIdx.x;
                    status->b = (int)parity;
                }
                return;
            }
        }
    }
}
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                          yx_dev_status *status, int where) {
    if (mbar_try(bar, parity)) return;
    mbar_wait_slow(bar, parity, abort_flag, status, where);
}

__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar, uint64_t pol) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar), "l"(pol)
        : "memory");
}

__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t &a, uint32_t &b, uint32_t &c, uint32_t &d) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(a), "=r"(b), "=r"(c), "=r"(d)
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm2(uint32_t addr, uint32_t &a, uint32_t &b) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(a), "=r"(b) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t &a, uint32_t &b, uint32_t &c, uint32_t &d) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(a), "=r"(b), "=r"(c), "=r"(d)
                 : "r"(addr));
}

template <bool BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (BF16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float x, float y) {
    if constexpr (BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
        return *(uint32_t *)&v;
    } else {
        __half2 v = __floats2half2_rn(x, y);
        return *(uint32_t *)&v;
    }
}
template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t u) {
    if constexpr (BF16) return __bfloat1622float2(*(__nv_bfloat162 *)&u);
    else return __half22float2(*(__half2 *)&u);
}

// Four consecutive elements of a tensor of `dtype` as f32.
__device__ __forceinline__ float4 load4_as_f32(const void *base, int dtype, size_t elem) {
    if (dtype == YX_F32) return *(const float4 *)((const float *)base + elem);
    uint2 raw = *(const uint2 *)((const uint16_t *)base + elem);
    float2 a, b;
    if (dtype == YX_F16) {
        a = __half22float2(*(const __half2 *)&raw.x);
        b = __half22float2(*(const __half2 *)&raw.y);
    } else {
        a = __bfloat1622float2(*(const __nv_bfloat162 *)&raw.x);
        b = __bfloat1622float2(*(const __nv_bfloat162 *)&raw.y);
    }
    return make_float4(a.x, a.y, b.x, b.y);
}

// Four consecutive outputs in the tensor's type.
__device__ __forceinline__ void store4(void *out, int out_dtype, size_t elem, float4 v) {
    if (out_dtype == YX_F32) {
        *(float4 *)((float *)out + elem) = v;
    } else if (out_dtype == YX_F16) {
        __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
        *(uint2 *)((uint16_t *)out + elem) = make_uint2(*(uint32_t *)&a, *(uint32_t *)&b);
    } else {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        *(uint2 *)((uint16_t *)out + elem) = make_uint2(*(uint32_t *)&a, *(uint32_t *)&b);
    }
}

// 2^x by the special-function unit (two units in the last place; -inf gives 0).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Merge of `count` partial triples (slots first..first+count of one (row, kv head), head g of
// `group`) by one warp: lane c reads the (m, l) of part c, the warp agrees on the maximum and
// the weights, then the o vectors are read with independent loads.  Parts with l <= 0 are
// dropped by value: their o was never written
// (crates/yaxus-backend-gpu/src/shaders.rs:1597-1598).  Loads bypass L1 (.cg): the parts may
// have been written by other SMs during this very kernel.
__device__ __forceinline__ void merge_parts(const float *part_o, const float *part_ml, uint32_t first, uint32_t count,
                                            int group, int g, int lane, float &mx, float &l, float4 &acc) {
    mx = -1e30f;
    l = 0.0f;
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t c0 = 0; c0 < count; c0 += 32) {
        const uint32_t c = c0 + lane;
        float em = -1e30f, el = 0.0f;
        if (c < count) {
            float2 v = __ldcg((const float2 *)(part_ml + ((size_t)(first + c) * group + g) * 2));
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
        const int nc = (int)min(32u, count - c0);
#pragma unroll 4
        for (int j = 0; j < nc; j++) {
            const float wj = __shfl_sync(0xffffffffu, w, j);
            if (wj > 0.0f) {
                float4 po = __ldcg((const float4 *)(part_o + ((size_t)(first + c0 + j) * group + g) * D + lane * 4));
                acc.x += po.x * wj;
                acc.y += po.y * wj;
                acc.z += po.z * wj;
                acc.w += po.w * wj;
            }
        }
    }
}

// Four merges at once by one warp (tasks with on[k] false are skipped): all (m, l) loads are
// issued before any is used, then all o loads, so the four cost two round trips together.
// Parts beyond 32 per task fall back to the one-at-a-time routine.
__device__ __forceinline__ void merge_parts4(const float *part_o, const float *part_ml, const uint32_t (&first)[4],
                                             const uint32_t (&count)[4], const bool (&on)[4], int group,
                                             const int (&g)[4], int lane, float (&mx)[4], float (&l)[4],
                                             float4 (&acc)[4]) {
    bool small = true;
#pragma unroll
    for (int k = 0; k < 4; k++) small = small && (!on[k] || count[k] <= 32);
    if (!small) {
#pragma unroll
        for (int k = 0; k < 4; k++)
            if (on[k]) merge_parts(part_o, part_ml, first[k], count[k], group, g[k], lane, mx[k], l[k], acc[k]);
        return;
    }
    float2 ml[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        ml[k] = make_float2(-1e30f, 0.0f);
        if (on[k] && (uint32_t)lane < count[k])
            ml[k] = __ldcg((const float2 *)(part_ml + ((size_t)(first[k] + lane) * group + g[k]) * 2));
    }
    float w[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const bool live = ml[k].y > 0.0f;
        float cm = live ? ml[k].x : -1e30f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
        w[k] = live ? __expf(ml[k].x - cm) : 0.0f;
        float ls = ml[k].y * w[k];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, o);
        mx[k] = cm;
        l[k] = ls;
        acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    uint32_t most = 0;
#pragma unroll
    for (int k = 0; k < 4; k++) most = max(most, on[k] ? count[k] : 0u);
    for (uint32_t j = 0; j < most; j++) {
        float4 po[4];
        float wj[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            wj[k] = __shfl_sync(0xffffffffu, w[k], j & 31);
            po[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (on[k] && j < count[k] && wj[k] > 0.0f)
                po[k] = __ldcg((const float4 *)(part_o + ((size_t)(first[k] + j) * group + g[k]) * D + lane * 4));
            else
                wj[k] = 0.0f;
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {
            acc[k].x += po[k].x * wj[k];
            acc[k].y += po[k].y * wj[k];
            acc[k].z += po[k].z * wj[k];
            acc[k].w += po[k].w * wj[k];
        }
    }
}

}  // namespace dev
}  // namespace yx
