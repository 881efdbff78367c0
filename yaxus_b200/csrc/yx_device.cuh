// Device-side helpers shared by the attention kernels: mbarriers with bounded waits, bulk
// asynchronous copies, ldmatrix / mma.sync wrappers, storage-type packing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "yx_internal.h"

// Time stamps inside the kernels exist only in a diagnostic build (-DYX_TRACE); in the shipped
// library the condition is a compile-time false and the stamping code is dropped.
#ifdef YX_TRACE
#define YX_TR(cond) (cond)
#else
#define YX_TR(cond) false
#endif

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

// Bounded wait (`limit` SM cycles).  Returns at once when the CTA has given up; on expiry it raises
// the CTA's abort flag and records where in the context's status word.  Nothing spins forever.  The
// spinning part is out of line: it is cold code, and the attention kernels pay for every
// instruction-cache line they touch.
static __device__ __noinline__ void mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                            yx_dev_status *status, int where, long long limit = WAIT_CYCLES) {
    if (*abort_flag) return;
    long long t0 = clock64();
    for (uint32_t spins = 1;; spins++) {
        if (mbar_try(bar, parity)) return;
        if ((spins & 255u) == 0) {
            if (*abort_flag) return;
            if (clock64() - t0 > limit) {
                *abort_flag = 1;
                atomicOr(&status->expired, 1u << (where & 31));
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

}  // namespace dev
}  // namespace yx
