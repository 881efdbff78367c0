// The operators of the reference's `Backend` trait either side of attention
// (crates/yaxus-model/src/lib.rs:124-171), as the CPU backend computes them
// (crates/yaxus-backend-cpu/src/lib.rs:485-562): embedding gather, RMSNorm, the fused residual
// step, matmul against bf16 weights, SwiGLU, add, row gather, argmax.
//
// All of them are bandwidth-bound.  The only one with real traffic is the matmul: at decode a
// pass has at most 16 rows, so `x [T,K] . w[N,K]^T` streams the weight matrix once and does
// 2 T flops per weight byte.  It is taken transposed, out^T = W x^T, with `mma.sync.m16n8k16`:
// the 16-row side holds weight rows (always full), the 8-column side holds pass rows, as in the
// split-key attention kernel.  Activations stay f32 in the interface; a small kernel first turns
// them into a high and a low bf16 part (x = hi + lo to 16 bits of mantissa), laid out in the
// order the MMA's B fragments want, and every weight fragment is used twice.
// Weights go from global memory straight into A fragments with 16-byte loads: a thread takes
// eight consecutive k of one weight row, which permutes k inside a step the same way for both
// operands, so the products pair up correctly.
//
// Passes of more than 32 rows (prompt chunks) are a plain GEMM and go to cuBLASLt, loaded at run
// time like NCCL; the activations' high and low bf16 parts are two GEMMs into one f32 result.
// Without the library the row kernel takes the rows 32 at a time, streaming the weights again
// for each block.
#include <cublasLt.h>
#include <cuda_bf16.h>
#include <dlfcn.h>

#include <algorithm>

#include "yx_internal.h"

namespace yx {
namespace {

constexpr int MM_WARPS = 4;
constexpr int MM_AHEAD = 4;               // steps of weights in flight per thread
constexpr int MM_CTAS_PER_SM = 5;
constexpr int MM_STEP = 32;              // k per warp step: one 16-byte load per thread and row half
constexpr int MM_PAIR = 64;              // two steps: the four threads of a weight row read one whole 128-byte line
constexpr int MM_MAX_T = 32;             // pass rows per launch (four 8-column tiles)

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// The activations of up to 32 pass rows as the MMA's B fragments want them: per 32-k step and
// 8-row column tile a 512-byte block of high parts and one of low parts, lane-major (lane =
// 4 g + t holds the eight k that thread t of a weight row's four loads in that step: steps come in
// pairs over 64 k, thread t owning k = 16 t .. 16 t + 15 of the pair, the lower eight in the even step).
// Rows past T are zero.
template <int NT>
__global__ void pack_rows_kernel(const float *__restrict__ x, uint32_t T, uint32_t K, uint4 *__restrict__ packed) {
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;   // one thread per 16-byte pair of blocks
    const uint32_t steps = K / MM_STEP;
    if (idx >= steps * NT * 32u) return;
    const uint32_t lane = idx & 31u, tile = (idx >> 5) % NT, s = (idx >> 5) / NT;
    const uint32_t n = tile * 8 + (lane >> 2), k0 = (s >> 1) * MM_PAIR + (lane & 3u) * 16 + (s & 1u) * 8;
    uint32_t hi[4], lo[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        float v[2] = {0.0f, 0.0f};
        if (n < T) {
            const float2 p = *(const float2 *)(x + (size_t)n * K + k0 + 2 * j);
            v[0] = p.x;
            v[1] = p.y;
        }
        const __nv_bfloat16 h0 = __float2bfloat16_rn(v[0]), h1 = __float2bfloat16_rn(v[1]);
        const __nv_bfloat16 l0 = __float2bfloat16_rn(v[0] - __bfloat162float(h0)), l1 = __float2bfloat16_rn(v[1] - __bfloat162float(h1));
        hi[j] = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
        lo[j] = (uint32_t)__bfloat16_as_ushort(l0) | ((uint32_t)__bfloat16_as_ushort(l1) << 16);
    }
    uint4 *dst = packed + ((size_t)(s * NT + tile) * 2u) * 32u + lane;
    dst[0] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    dst[32] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
}

// part[ky][t][n] = sum over k-chunk ky of x[t][k] * w[n][k].  NT = 8-column tiles of pass rows.
// The work is cut into items of 16 weight rows x one chunk of kc columns, dealt round-robin to the
// warps of a grid that just fills the machine.  A warp's weights come straight from global memory
// into A fragments, AHEAD steps in flight, and the prefetch runs on into the warp's next item, so
// the stream never drains; the packed activations are read through L1.  kc is a multiple of 32 AHEAD.
template <int NT>
__global__ void __launch_bounds__(MM_WARPS * 32, 5) matmul_rows_kernel(const uint4 *__restrict__ packed, const __nv_bfloat16 *__restrict__ w,
                                                                        uint32_t T, uint32_t N, uint32_t K, uint32_t kc, uint32_t chunks,
                                                                        float *__restrict__ part) {
    constexpr int AHEAD = MM_AHEAD;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const uint32_t steps = kc / MM_STEP;
    const uint32_t total = ((N + 15u) / 16u) * chunks, n_warps = gridDim.x * MM_WARPS;
    uint32_t item = blockIdx.x * MM_WARPS + warp;
    if (item >= total) return;
    auto at = [](uint32_t s) { return (size_t)(s >> 1) * MM_PAIR + (s & 1u) * 8; };   // element offset of step s
    // Rows past N repeat the last row (their results are not stored).
    auto row_ptr = [&](uint32_t it, uint32_t half) {
        const uint32_t r = min((it / chunks) * 16u + g + half * 8u, N - 1u);
        return w + (size_t)r * K + (size_t)(it % chunks) * kc + t4 * 16;
    };
    // The prefetch position: AHEAD steps ahead of the consumer.
    uint32_t pf_item = item, pf_step = 0;
    const __nv_bfloat16 *pf_a = row_ptr(item, 0), *pf_b = row_ptr(item, 1);
    uint4 wa[AHEAD], wb[AHEAD];
#pragma unroll
    for (int i = 0; i < AHEAD; i++) {   // (steps >= AHEAD)
        wa[i] = ldg_stream(pf_a + at(pf_step));
        wb[i] = ldg_stream(pf_b + at(pf_step));
        pf_step++;
    }
    for (; item < total; item += n_warps) {
        const uint32_t ky = item % chunks, row0 = (item / chunks) * 16u;
        const uint4 *xp = packed + (size_t)ky * steps * NT * 64u + lane;
        float acc[NT][4];
#pragma unroll
        for (int n = 0; n < NT; n++) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
        for (uint32_t s0 = 0; s0 < steps; s0 += AHEAD) {
#pragma unroll
            for (int i = 0; i < AHEAD; i++) {
                const uint32_t s = s0 + i;
                const uint4 a = wa[i], b = wb[i];
                if (pf_step == steps) {   // on to this warp's next item
                    pf_step = 0;
                    pf_item += n_warps;
                    if (pf_item < total) {
                        pf_a = row_ptr(pf_item, 0);
                        pf_b = row_ptr(pf_item, 1);
                    }
                }
                if (pf_item < total) {
                    wa[i] = ldg_stream(pf_a + at(pf_step));
                    wb[i] = ldg_stream(pf_b + at(pf_step));
                    pf_step++;
                }
#pragma unroll
                for (int n = 0; n < NT; n++) {
                    const uint4 hi = __ldg(xp + ((size_t)s * NT + n) * 64u);
                    const uint4 lo = __ldg(xp + ((size_t)s * NT + n) * 64u + 32u);
                    mma_bf16(acc[n], a.x, b.x, a.y, b.y, hi.x, hi.y);
                    mma_bf16(acc[n], a.z, b.z, a.w, b.w, hi.z, hi.w);
                    mma_bf16(acc[n], a.x, b.x, a.y, b.y, lo.x, lo.y);
                    mma_bf16(acc[n], a.z, b.z, a.w, b.w, lo.z, lo.w);
                }
            }
        }
        // c0,c1: weight row g, pass rows 2 t4, 2 t4 + 1 of the tile; c2,c3: weight row g + 8.
        float *dst = part + (size_t)ky * T * N;
#pragma unroll
        for (int n = 0; n < NT; n++) {
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const uint32_t tok = n * 8 + t4 * 2 + (c & 1), row = row0 + g + (c >> 1) * 8;
                if (tok < T && row < N) dst[(size_t)tok * N + row] = acc[n][c];
            }
        }
    }
}

// out[t][j] = sum over chunks of part[.][t][j], or with glu: silu(sum[t][j]) * sum[t][I + j], I = N / 2
// (cpu lib.rs:532-542).
__global__ void matmul_finish_kernel(const float *__restrict__ part, uint32_t chunks, uint32_t T, uint32_t N, int glu,
                                     float *__restrict__ out) {
    const uint32_t cols = glu ? N / 2 : N;
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * cols) return;
    const uint32_t t = idx / cols, j = idx - t * cols;
    float a = 0.0f, b = 0.0f;
    for (uint32_t c = 0; c < chunks; c++) {
        const float *p = part + ((size_t)c * T + t) * N;
        a += p[j];
        if (glu) b += p[cols + j];
    }
    out[idx] = glu ? a / (1.0f + expf(-a)) * b : a;
}

// Any shape the tensor-core kernel does not take (K not a multiple of 128): a warp per output.
__global__ void matmul_any_kernel(const float *__restrict__ x, const __nv_bfloat16 *__restrict__ w, uint32_t T, uint32_t N,
                                  uint32_t K, float *__restrict__ out) {
    const uint32_t o = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (o >= T * N) return;
    const uint32_t t = o / N, n = o - t * N;
    float s = 0.0f;
    for (uint32_t k = lane; k < K; k += 32) s += __bfloat162float(w[(size_t)n * K + k]) * x[(size_t)t * K + k];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
    if (lane == 0) out[o] = s;
}

__global__ void swiglu_kernel(const float *__restrict__ x, uint32_t rows, uint32_t inner, float *__restrict__ out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * inner) return;
    const size_t r = idx / inner, j = idx - r * inner;
    const float g = x[r * 2 * inner + j], u = x[r * 2 * inner + inner + j];
    out[idx] = g / (1.0f + expf(-g)) * u;
}

__global__ void add_assign_kernel(float *__restrict__ a, const float *__restrict__ b, size_t n) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) a[idx] += b[idx];
}

// out[r] = f32(table[ids[r]]) (cpu lib.rs:485-497); an id outside the table is recorded and its row zeroed.
__global__ void embed_kernel(const __nv_bfloat16 *__restrict__ table, uint32_t vocab, uint32_t h, const uint32_t *__restrict__ ids,
                             float *__restrict__ out, yx_dev_status *status) {
    const uint32_t r = blockIdx.x, id = ids[r];
    if (id >= vocab) {
        if (threadIdx.x == 0 && atomicCAS(&status->code, 0, 1) == 0) {
            status->where = 400;
            status->a = (int)id;
            status->b = (int)r;
        }
        for (uint32_t c = threadIdx.x; c < h; c += blockDim.x) out[(size_t)r * h + c] = 0.0f;
        return;
    }
    for (uint32_t c = threadIdx.x; c < h; c += blockDim.x) out[(size_t)r * h + c] = __bfloat162float(table[(size_t)id * h + c]);
}

__global__ void select_rows_kernel(const float *__restrict__ x, uint32_t src_rows, uint32_t cols, const uint32_t *__restrict__ rows,
                                   float *__restrict__ out, yx_dev_status *status) {
    const uint32_t r = blockIdx.x, src = rows[r];
    if (src >= src_rows) {
        if (threadIdx.x == 0 && atomicCAS(&status->code, 0, 1) == 0) {
            status->where = 401;
            status->a = (int)src;
            status->b = (int)r;
        }
        return;
    }
    for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) out[(size_t)r * cols + c] = x[(size_t)src * cols + c];
}

__device__ __forceinline__ float block_sum(float v, float *scratch) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    __syncthreads();   // the scratch may still be read from the call before
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float s = 0.0f;
    for (int i = 0; i < n_warps; i++) s += scratch[i];
    return s;
}

// One CTA per row.  With `x_inout`: d = rmsnorm(delta, post); x += d; out = rmsnorm(x, pre)
// (crates/yaxus-model/src/lib.rs:149-162).  Without: out = rmsnorm(delta, post) (cpu lib.rs:296-302).
__global__ void __launch_bounds__(256) norm_kernel(float *__restrict__ x_inout, const float *__restrict__ delta,
                                                   const float *__restrict__ post_w, float post_offset,
                                                   const float *__restrict__ pre_w, float pre_offset, float eps, uint32_t cols,
                                                   float *__restrict__ out) {
    __shared__ float scratch[8];
    const size_t base = (size_t)blockIdx.x * cols;
    float ss = 0.0f;
    for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = delta[base + c];
        ss += v * v;
    }
    const float r1 = 1.0f / sqrtf(block_sum(ss, scratch) / (float)cols + eps);
    if (!x_inout) {
        for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) out[base + c] = (post_offset + post_w[c]) * (delta[base + c] * r1);
        return;
    }
    float ss2 = 0.0f;
    for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = x_inout[base + c] + (post_offset + post_w[c]) * (delta[base + c] * r1);
        x_inout[base + c] = v;
        ss2 += v * v;
    }
    const float r2 = 1.0f / sqrtf(block_sum(ss2, scratch) / (float)cols + eps);
    for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) out[base + c] = (pre_offset + pre_w[c]) * (x_inout[base + c] * r2);
}

// The first largest value of each row; NaNs never win, a row of NaNs gives 0 (cpu lib.rs:430-441).
__global__ void __launch_bounds__(256) argmax_rows_kernel(const float *__restrict__ x, uint32_t cols, uint32_t *__restrict__ out) {
    __shared__ float best_v[8];
    __shared__ uint32_t best_i[8];
    const float *row = x + (size_t)blockIdx.x * cols;
    float bv = -INFINITY;
    uint32_t bi = 0xffffffffu;   // nothing above -inf seen yet
    for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = row[c];
        if (v > bv) {
            bv = v;
            bi = c;
        }
    }
    auto better = [](float v, uint32_t i, float w, uint32_t j) { return v > w || (v == w && i < j); };
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, d);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, d);
        if (better(ov, oi, bv, bi)) {
            bv = ov;
            bi = oi;
        }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        best_v[warp] = bv;
        best_i[warp] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < (int)(blockDim.x >> 5); i++)
            if (better(best_v[i], best_i[i], bv, bi)) {
                bv = best_v[i];
                bi = best_i[i];
            }
        out[blockIdx.x] = bi == 0xffffffffu ? 0u : bi;
    }
}

int launched(yx_ctx *ctx, const char *what) {
    ctx->launches++;
    ctx->last_launch = yx_ctx::LAST_OTHER;
    return check_cuda(ctx, cudaGetLastError(), what);
}

// ---- cuBLASLt, for passes of many rows --------------------------------------------------------
struct Lt {
    void *lib = nullptr;
    bool tried = false;
    cublasStatus_t (*create)(cublasLtHandle_t *) = nullptr;
    cublasStatus_t (*destroy)(cublasLtHandle_t) = nullptr;
    cublasStatus_t (*desc_create)(cublasLtMatmulDesc_t *, cublasComputeType_t, cudaDataType_t) = nullptr;
    cublasStatus_t (*desc_destroy)(cublasLtMatmulDesc_t) = nullptr;
    cublasStatus_t (*desc_set)(cublasLtMatmulDesc_t, cublasLtMatmulDescAttributes_t, const void *, size_t) = nullptr;
    cublasStatus_t (*layout_create)(cublasLtMatrixLayout_t *, cudaDataType_t, uint64_t, uint64_t, int64_t) = nullptr;
    cublasStatus_t (*layout_destroy)(cublasLtMatrixLayout_t) = nullptr;
    cublasStatus_t (*pref_create)(cublasLtMatmulPreference_t *) = nullptr;
    cublasStatus_t (*pref_destroy)(cublasLtMatmulPreference_t) = nullptr;
    cublasStatus_t (*pref_set)(cublasLtMatmulPreference_t, cublasLtMatmulPreferenceAttributes_t, const void *, size_t) = nullptr;
    cublasStatus_t (*heuristic)(cublasLtHandle_t, cublasLtMatmulDesc_t, cublasLtMatrixLayout_t, cublasLtMatrixLayout_t,
                                cublasLtMatrixLayout_t, cublasLtMatrixLayout_t, cublasLtMatmulPreference_t, int,
                                cublasLtMatmulHeuristicResult_t *, int *) = nullptr;
    cublasStatus_t (*matmul)(cublasLtHandle_t, cublasLtMatmulDesc_t, const void *, const void *, cublasLtMatrixLayout_t,
                             const void *, cublasLtMatrixLayout_t, const void *, const void *, cublasLtMatrixLayout_t, void *,
                             cublasLtMatrixLayout_t, const cublasLtMatmulAlgo_t *, void *, size_t, cudaStream_t) = nullptr;
    bool ok() const { return matmul != nullptr; }
};

Lt load_lt() {
    Lt l;
    l.tried = true;
    const char *names[] = {"libcublasLt.so.12", "libcublasLt.so", "/usr/local/cuda/lib64/libcublasLt.so.12"};
    for (const char *n : names) {
        l.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (l.lib) break;
    }
    if (!l.lib) return l;
    auto sym = [&](const char *n) { return dlsym(l.lib, n); };
    l.create = (decltype(l.create))sym("cublasLtCreate");
    l.destroy = (decltype(l.destroy))sym("cublasLtDestroy");
    l.desc_create = (decltype(l.desc_create))sym("cublasLtMatmulDescCreate");
    l.desc_destroy = (decltype(l.desc_destroy))sym("cublasLtMatmulDescDestroy");
    l.desc_set = (decltype(l.desc_set))sym("cublasLtMatmulDescSetAttribute");
    l.layout_create = (decltype(l.layout_create))sym("cublasLtMatrixLayoutCreate");
    l.layout_destroy = (decltype(l.layout_destroy))sym("cublasLtMatrixLayoutDestroy");
    l.pref_create = (decltype(l.pref_create))sym("cublasLtMatmulPreferenceCreate");
    l.pref_destroy = (decltype(l.pref_destroy))sym("cublasLtMatmulPreferenceDestroy");
    l.pref_set = (decltype(l.pref_set))sym("cublasLtMatmulPreferenceSetAttribute");
    l.heuristic = (decltype(l.heuristic))sym("cublasLtMatmulAlgoGetHeuristic");
    auto mm = (decltype(l.matmul))sym("cublasLtMatmul");
    if (l.create && l.destroy && l.desc_create && l.desc_destroy && l.desc_set && l.layout_create && l.layout_destroy &&
        l.pref_create && l.pref_destroy && l.pref_set && l.heuristic)
        l.matmul = mm;
    return l;
}

// (initialised once, by whichever thread comes first)
Lt &lt() {
    static Lt l = load_lt();
    return l;
}

// x [T][K] f32 -> hi [T][K] and lo [T][K] bf16, x = hi + lo to 16 bits of mantissa.
__global__ void split_rows_kernel(const float *__restrict__ x, size_t n, __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const float v = x[idx];
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    hi[idx] = h;
    lo[idx] = __float2bfloat16_rn(v - __bfloat162float(h));
}

constexpr size_t LT_WORKSPACE = 32u << 20;

// out [T][N] (row-major f32) = x . w^T through cuBLASLt.  In its column-major terms the result is
// the N x T matrix w^T(K x N, transposed) times x^T (K x T).  Returns -1 when the library or a
// kernel for the shape is not there (the caller then uses the row kernel), else a yx_error.
int matmul_lt(yx_ctx *ctx, const float *x, const __nv_bfloat16 *w, uint32_t T, uint32_t N, uint32_t K, float *out) {
    Lt &l = lt();
    if (!l.ok()) return -1;
    if (!ctx->lt_handle) {
        cublasLtHandle_t h = nullptr;
        if (l.create(&h) != CUBLAS_STATUS_SUCCESS) return -1;
        ctx->lt_handle = h;
    }
    if (int rc = ensure_buffer(ctx, (void **)&ctx->mm_packed, &ctx->mm_packed_cap, (size_t)T * K * 4)) return rc;
    if (int rc = ensure_buffer(ctx, (void **)&ctx->lt_workspace, &ctx->lt_workspace_cap, LT_WORKSPACE)) return rc;
    __nv_bfloat16 *hi = (__nv_bfloat16 *)ctx->mm_packed, *lo = hi + (size_t)T * K;
    const size_t n = (size_t)T * K;
    split_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(x, n, hi, lo);
    if (int rc = launched(ctx, "matmul: activation split kernel")) return rc;

    cublasLtMatmulDesc_t desc = nullptr;
    cublasLtMatrixLayout_t la = nullptr, lb = nullptr, lc = nullptr;
    cublasLtMatmulPreference_t pref = nullptr;
    int result = -1;
    do {
        if (l.desc_create(&desc, CUBLAS_COMPUTE_32F, CUDA_R_32F) != CUBLAS_STATUS_SUCCESS) break;
        const cublasOperation_t ta = CUBLAS_OP_T, tb = CUBLAS_OP_N;
        if (l.desc_set(desc, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof ta) != CUBLAS_STATUS_SUCCESS) break;
        if (l.desc_set(desc, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof tb) != CUBLAS_STATUS_SUCCESS) break;
        if (l.layout_create(&la, CUDA_R_16BF, K, N, K) != CUBLAS_STATUS_SUCCESS) break;   // w: K x N, column-major
        if (l.layout_create(&lb, CUDA_R_16BF, K, T, K) != CUBLAS_STATUS_SUCCESS) break;   // x parts: K x T
        if (l.layout_create(&lc, CUDA_R_32F, N, T, N) != CUBLAS_STATUS_SUCCESS) break;    // out: N x T
        if (l.pref_create(&pref) != CUBLAS_STATUS_SUCCESS) break;
        const size_t ws = LT_WORKSPACE;
        if (l.pref_set(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &ws, sizeof ws) != CUBLAS_STATUS_SUCCESS) break;
        cublasLtMatmulHeuristicResult_t heur{};
        int found = 0;
        if (l.heuristic((cublasLtHandle_t)ctx->lt_handle, desc, la, lb, lc, lc, pref, 1, &heur, &found) != CUBLAS_STATUS_SUCCESS || found == 0)
            break;
        const float one = 1.0f, zero = 0.0f;
        cublasStatus_t st = l.matmul((cublasLtHandle_t)ctx->lt_handle, desc, &one, w, la, hi, lb, &zero, out, lc, out, lc, &heur.algo,
                                     ctx->lt_workspace, LT_WORKSPACE, ctx->stream);
        if (st == CUBLAS_STATUS_SUCCESS)
            st = l.matmul((cublasLtHandle_t)ctx->lt_handle, desc, &one, w, la, lo, lb, &one, out, lc, out, lc, &heur.algo,
                          ctx->lt_workspace, LT_WORKSPACE, ctx->stream);
        if (st != CUBLAS_STATUS_SUCCESS) {
            result = fail(ctx, YX_ERR_CUDA, "matmul: cublasLtMatmul failed with status " + std::to_string((int)st));
            break;
        }
        ctx->launches += 2;
        ctx->last_launch = yx_ctx::LAST_OTHER;
        result = YX_OK;
    } while (false);
    if (pref) l.pref_destroy(pref);
    if (lc) l.layout_destroy(lc);
    if (lb) l.layout_destroy(lb);
    if (la) l.layout_destroy(la);
    if (desc) l.desc_destroy(desc);
    return result;
}

template <int NT>
int launch_matmul_rows(yx_ctx *ctx, const float *x, const __nv_bfloat16 *w, uint32_t T, uint32_t N, uint32_t K, float *part,
                       uint32_t kc, uint32_t chunks) {
    const size_t packed_bytes = (size_t)(K / MM_STEP) * NT * 2 * 512;
    if (int rc = ensure_buffer(ctx, (void **)&ctx->mm_packed, &ctx->mm_packed_cap, packed_bytes)) return rc;
    const uint32_t pack_threads = (K / MM_STEP) * NT * 32u;
    pack_rows_kernel<NT><<<(pack_threads + 255) / 256, 256, 0, ctx->stream>>>(x, T, K, (uint4 *)ctx->mm_packed);
    if (int rc = launched(ctx, "matmul: activation packing kernel")) return rc;
    const uint32_t items = ((N + 15u) / 16u) * chunks;
    const uint32_t grid = std::min<uint32_t>((items + MM_WARPS - 1) / MM_WARPS, (uint32_t)ctx->sm_count * MM_CTAS_PER_SM);
    matmul_rows_kernel<NT><<<grid, MM_WARPS * 32, 0, ctx->stream>>>((const uint4 *)ctx->mm_packed, w, T, N, K, kc, chunks, part);
    return launched(ctx, "matmul kernel");
}

struct Guard {
    int prev = -1;
    explicit Guard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
        else prev = -1;
    }
    ~Guard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

int ready(yx_ctx *ctx) {
    if (!ctx) return YX_ERR_INVALID;
    return ctx->status;
}

int matmul_impl(yx_ctx *ctx, const float *x, const void *w_bf16, uint32_t T, uint32_t N, uint32_t K, int glu, float *out) {
    if (int rc = ready(ctx)) return rc;
    if (T == 0 || N == 0) return YX_OK;
    if (!x || !w_bf16 || !out || K == 0) return fail(ctx, YX_ERR_INVALID, "matmul: null tensor or empty inner dimension");
    if (glu && N % 2 != 0) return fail(ctx, YX_ERR_INVALID, "matmul_glu: the weight must hold gate and up rows (even N)");
    Guard guard(ctx->device);
    const __nv_bfloat16 *w = (const __nv_bfloat16 *)w_bf16;
    const uint32_t cols = glu ? N / 2 : N;
    if (K % (MM_STEP * MM_AHEAD) != 0 || ((uintptr_t)w & 15u) != 0 || ((uintptr_t)x & 7u) != 0) {
        float *dst = out;
        if (glu) {
            if (int rc = ensure_buffer(ctx, (void **)&ctx->mm_part, &ctx->mm_part_cap, (size_t)T * N * sizeof(float))) return rc;
            dst = ctx->mm_part;
        }
        const uint64_t threads = (uint64_t)T * N * 32;
        matmul_any_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, ctx->stream>>>(x, w, T, N, K, dst);
        if (int rc = launched(ctx, "matmul kernel (any shape)")) return rc;
        if (glu) {
            const uint64_t n = (uint64_t)T * cols;
            swiglu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(dst, T, cols, out);
            return launched(ctx, "swiglu kernel");
        }
        return YX_OK;
    }
    if (T > MM_MAX_T && ctx->tuning.force_path != 2) {
        float *dst = out;
        if (glu) {
            if (int rc = ensure_buffer(ctx, (void **)&ctx->mm_part, &ctx->mm_part_cap, (size_t)T * N * sizeof(float))) return rc;
            dst = ctx->mm_part;
        }
        const int rc = matmul_lt(ctx, x, w, T, N, K, dst);
        if (rc > 0) return rc;
        if (rc == YX_OK) {
            if (!glu) return YX_OK;
            const uint64_t n = (uint64_t)T * cols;
            swiglu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(dst, T, cols, out);
            return launched(ctx, "swiglu kernel");
        }
        // (no cuBLASLt, or no kernel of its for this shape: the row kernel below)
    }
    // K is cut into chunks (an item is 16 weight rows of one chunk) until every resident warp has
    // a few items to take, which evens the warps' loads out; no more than eight chunks, whose
    // partial sums the finishing kernel adds up.
    const uint32_t row_items = (N + 15) / 16, warps = (uint32_t)ctx->sm_count * MM_CTAS_PER_SM * MM_WARPS;
    uint32_t kc = K;
    while (kc % (2 * MM_STEP * MM_AHEAD) == 0 && K / (kc / 2) <= 8 && row_items * (K / kc) < 4 * warps) kc /= 2;
    const uint32_t chunks = K / kc;
    // Pass rows go 32 at a time; each block of them streams the weights again.
    for (uint32_t t0 = 0; t0 < T; t0 += MM_MAX_T) {
        const uint32_t tn = std::min<uint32_t>(MM_MAX_T, T - t0);
        if (int rc = ensure_buffer(ctx, (void **)&ctx->mm_part, &ctx->mm_part_cap, (size_t)chunks * MM_MAX_T * N * sizeof(float)))
            return rc;
        const float *xt = x + (size_t)t0 * K;
        int rc = tn <= 8    ? launch_matmul_rows<1>(ctx, xt, w, tn, N, K, ctx->mm_part, kc, chunks)
                 : tn <= 16 ? launch_matmul_rows<2>(ctx, xt, w, tn, N, K, ctx->mm_part, kc, chunks)
                            : launch_matmul_rows<4>(ctx, xt, w, tn, N, K, ctx->mm_part, kc, chunks);
        if (rc) return rc;
        const uint64_t n = (uint64_t)tn * cols;
        matmul_finish_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(ctx->mm_part, chunks, tn, N, glu,
                                                                                  out + (size_t)t0 * cols);
        if (int rc2 = launched(ctx, "matmul finish kernel")) return rc2;
    }
    return YX_OK;
}

}  // namespace

void release_matmul_library(yx_ctx *ctx) {
    if (ctx->lt_handle && lt().ok()) lt().destroy((cublasLtHandle_t)ctx->lt_handle);
    ctx->lt_handle = nullptr;
}

}  // namespace yx

using namespace yx;

extern "C" {

int yx_matmul(yx_ctx *ctx, const float *x_dev, const void *w_bf16_dev, uint32_t rows, uint32_t n, uint32_t k, float *out_dev) {
    return matmul_impl(ctx, x_dev, w_bf16_dev, rows, n, k, 0, out_dev);
}

int yx_matmul_glu(yx_ctx *ctx, const float *x_dev, const void *w_bf16_dev, uint32_t rows, uint32_t n, uint32_t k,
                  float *out_dev) {
    return matmul_impl(ctx, x_dev, w_bf16_dev, rows, n, k, 1, out_dev);
}

int yx_swiglu(yx_ctx *ctx, const float *x_dev, uint32_t rows, uint32_t inner, float *out_dev) {
    if (int rc = ready(ctx)) return rc;
    const uint64_t n = (uint64_t)rows * inner;
    if (n == 0) return YX_OK;
    if (!x_dev || !out_dev) return fail(ctx, YX_ERR_INVALID, "swiglu: null tensor");
    Guard guard(ctx->device);
    swiglu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(x_dev, rows, inner, out_dev);
    return launched(ctx, "swiglu kernel");
}

int yx_add_assign(yx_ctx *ctx, float *a_dev, const float *b_dev, size_t n) {
    if (int rc = ready(ctx)) return rc;
    if (n == 0) return YX_OK;
    if (!a_dev || !b_dev) return fail(ctx, YX_ERR_INVALID, "add_assign: null tensor");
    Guard guard(ctx->device);
    add_assign_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(a_dev, b_dev, n);
    return launched(ctx, "add_assign kernel");
}

int yx_rmsnorm(yx_ctx *ctx, const float *x_dev, const float *w_dev, uint32_t rows, uint32_t cols, float offset, float eps,
               float *out_dev) {
    if (int rc = ready(ctx)) return rc;
    if (rows == 0) return YX_OK;
    if (!x_dev || !w_dev || !out_dev || cols == 0) return fail(ctx, YX_ERR_INVALID, "rmsnorm: null tensor or no columns");
    Guard guard(ctx->device);
    norm_kernel<<<rows, 256, 0, ctx->stream>>>(nullptr, x_dev, w_dev, offset, nullptr, 0.0f, eps, cols, out_dev);
    return launched(ctx, "rmsnorm kernel");
}

int yx_add_norm(yx_ctx *ctx, float *x_dev, const float *delta_dev, const float *post_w_dev, float post_offset,
                const float *pre_w_dev, float pre_offset, float eps, uint32_t rows, uint32_t cols, float *out_dev) {
    if (int rc = ready(ctx)) return rc;
    if (rows == 0) return YX_OK;
    if (!x_dev || !delta_dev || !post_w_dev || !pre_w_dev || !out_dev || cols == 0)
        return fail(ctx, YX_ERR_INVALID, "add_norm: null tensor or no columns");
    Guard guard(ctx->device);
    norm_kernel<<<rows, 256, 0, ctx->stream>>>(x_dev, delta_dev, post_w_dev, post_offset, pre_w_dev, pre_offset, eps, cols, out_dev);
    return launched(ctx, "add_norm kernel");
}

int yx_embed(yx_ctx *ctx, const void *table_bf16_dev, uint32_t vocab, uint32_t h, const uint32_t *ids_host, uint32_t rows,
             float *out_dev) {
    if (int rc = ready(ctx)) return rc;
    if (rows == 0) return YX_OK;
    if (!table_bf16_dev || !ids_host || !out_dev || h == 0) return fail(ctx, YX_ERR_INVALID, "embed: null tensor");
    for (uint32_t r = 0; r < rows; r++)
        if (ids_host[r] >= vocab) return fail(ctx, YX_ERR_INVALID, "embed: a token id is outside the table");
    Guard guard(ctx->device);
    if (int rc = ensure_buffer(ctx, (void **)&ctx->idx_dev, &ctx->idx_cap, (size_t)rows * 4)) return rc;
    if (int rc = upload_ordered(ctx, ctx->idx_dev, ids_host, (size_t)rows * 4)) return rc;
    embed_kernel<<<rows, 256, 0, ctx->stream>>>((const __nv_bfloat16 *)table_bf16_dev, vocab, h, ctx->idx_dev, out_dev,
                                                ctx->dev_status);
    return launched(ctx, "embed kernel");
}

int yx_select_rows(yx_ctx *ctx, const float *x_dev, uint32_t src_rows, uint32_t cols, const uint32_t *rows_host, uint32_t n,
                   float *out_dev) {
    if (int rc = ready(ctx)) return rc;
    if (n == 0 || cols == 0) return YX_OK;
    if (!x_dev || !rows_host || !out_dev) return fail(ctx, YX_ERR_INVALID, "select_rows: null tensor");
    for (uint32_t r = 0; r < n; r++)
        if (rows_host[r] >= src_rows) return fail(ctx, YX_ERR_INVALID, "select_rows: a row index is outside the tensor");
    Guard guard(ctx->device);
    if (int rc = ensure_buffer(ctx, (void **)&ctx->idx_dev, &ctx->idx_cap, (size_t)n * 4)) return rc;
    if (int rc = upload_ordered(ctx, ctx->idx_dev, rows_host, (size_t)n * 4)) return rc;
    select_rows_kernel<<<n, 256, 0, ctx->stream>>>(x_dev, src_rows, cols, ctx->idx_dev, out_dev, ctx->dev_status);
    return launched(ctx, "select_rows kernel");
}

int yx_argmax_rows(yx_ctx *ctx, const float *logits_dev, uint32_t rows, uint32_t cols, uint32_t *out_host) {
    if (int rc = ready(ctx)) return rc;
    if (rows == 0) return YX_OK;
    if (!logits_dev || !out_host || cols == 0) return fail(ctx, YX_ERR_INVALID, "argmax_rows: null tensor or no columns");
    Guard guard(ctx->device);
    if (int rc = ensure_buffer(ctx, (void **)&ctx->idx_dev, &ctx->idx_cap, (size_t)rows * 4)) return rc;
    argmax_rows_kernel<<<rows, 256, 0, ctx->stream>>>(logits_dev, cols, ctx->idx_dev);
    if (int rc = launched(ctx, "argmax_rows kernel")) return rc;
    // A read-back: the one place the model waits for the device (crates/yaxus-model/src/lib.rs:177-185).
    if (int rc = check_cuda(ctx, cudaMemcpyAsync(out_host, ctx->idx_dev, (size_t)rows * 4, cudaMemcpyDeviceToHost, ctx->stream),
                            "argmax_rows: read-back"))
        return rc;
    return yx_sync(ctx);
}

}  // extern "C"
