// Tiled causal attention for many-row passes (prompt chunks) over 16-bit paged KV caches, on
// the fifth-generation tensor cores: tcgen05.mma with accumulators in tensor memory (TMEM),
// operands staged in shared memory by bulk asynchronous copies (TMA).  The counterpart of the
// reference's `attn_tile` (crates/yaxus-backend-gpu/src/shaders.rs:422-630), which is an f32
// SIMT kernel over 32-row tiles.
//
// One CTA works on one item: up to 128 consecutive rows of one sequence (one M = 128 tile of
// queries) for one query head, against that sequence's pages up to the last row's position.
// Six warps:
//   warps 0-3  softmax: thread t owns query row t and TMEM lane t.  It reads the scores of a
//              128-key tile from TMEM, masks, keeps the running maximum and sum in f32,
//              writes the probabilities back to TMEM as 16-bit pairs (over the scores), and
//              rescales the output accumulator when the maximum has grown by more than 2^8
//              since the last rescale ("lazy" rescaling: until then the probabilities are
//              simply allowed to exceed 1).
//   warp 4     producer: page ids fetched 32 at a time, one 32 KiB bulk copy per K page and per
//              V page (the cache layout is the 128-byte-swizzled operand layout already).
//   warp 5     MMA issuer: S_j = Q K_j^T (M128 N128 K128, both operands K-major from shared
//              memory) into one of two TMEM score buffers, then O += P_{j-1} V_{j-1} (P from
//              TMEM, V MN-major from shared memory).  S_j is issued before P_{j-1}V_{j-1}, so
//              the softmax of tile j-1 overlaps the tensor work of tile j.
// TMEM columns: [0,128) S0 / P0, [128,256) S1 / P1, [256,384) O.
//
// Every mbarrier wait is bounded; on expiry the CTA records where, stops waiting anywhere,
// still frees its TMEM and returns.

#include "yx_device.cuh"

namespace yx {
namespace {

using namespace dev;

constexpr int BM = 128;                  // query rows per item
constexpr int BN = 128;                  // keys per tile = one page
constexpr int K_STAGES = 3, V_STAGES = 2;
constexpr int PAGE_BYTES = PAGE * D * 2; // one (page, kv head) block of K or of V: 32 KiB
constexpr int HALF_BYTES = PAGE * 128;   // one 64-dim half
constexpr int SOFTMAX_WARPS = 4, PRODUCER_WARP = 4, MMA_WARP = 5;
constexpr int THREADS = 6 * 32;
constexpr int TMEM_COLS = 512;
constexpr int COL_S0 = 0, COL_S1 = 128, COL_O = 256;
// barriers: q_full, k_full[3], k_empty[3], v_full[2], v_empty[2], s_full[2], p_full[2], pv_done
constexpr int N_BARS = 1 + 2 * K_STAGES + 2 * V_STAGES + 2 + 2 + 1;
constexpr int SMEM_BYTES = PAGE_BYTES * (2 + K_STAGES + V_STAGES) + N_BARS * 8 + 64;   // Q high, Q low, K ring, V ring

struct TileParams {
    const void *q;
    int q_dtype, hq, group, hkv;
    const char *k_arena, *v_arena;
    uint32_t n_blocks;
    uint32_t window;
    const uint32_t *pages;
    const TileItem *items;
    void *out;
    int out_dtype;
    int bf16;            // cache type: 1 bf16, 0 f16
    int q_lo;            // queries carry a low part (f32 queries on a bf16 cache): S = Qh K^T + Ql K^T
    int p_lo;            // probabilities carry a low part (bf16 cache): O += Ph V + Pl V
    yx_dev_status *status;
    long long *trace;   // diagnostics: clock stamps of CTA 0's pipeline, or null
    const uint32_t *cta_begin;   // items of persistent CTA c: [cta_begin[c], cta_begin[c + 1])
    const uint32_t *wide_v;      // non-zero: the bf16 cache holds V values that f16 cannot
};

// Shared-memory matrix descriptor: start address, leading / stride byte offsets (16-byte
// units), descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffff) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor, kind::f16: f32 accumulator, 16-bit A and B of the cache's type.
__device__ __forceinline__ uint32_t instr_desc(int bf16, int b_mn_major) {
    const uint32_t fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(BN >> 3) << 17) |
           ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                 "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
                 : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
                 "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc)
                 : "memory");
}
// The same instructions with the descriptors' constant high words and precomputed low words
// (start address and leading offset): the issuing thread then spends one add per operand, which
// matters because a single thread issues every MMA of the CTA.
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
    return ((saddr & 0x3ffff) >> 4) | (((lbo_bytes >> 4) & 0x3fff) << 16);
}
constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);   // stride 1024 B, version 1, 128-byte swizzle
__device__ __forceinline__ void umma_ss_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem),
                 "r"(a_lo), "r"(b_lo), "r"(DESC_HI), "r"(idesc), "r"(acc)
                 : "memory");
}
__device__ __forceinline__ void umma_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 db, {%2, %3};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(d_tmem),
                 "r"(a_tmem), "r"(b_lo), "r"(DESC_HI), "r"(idesc), "r"(acc)
                 : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_pair(float x, float y, int bf16) {
    if (bf16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
        return *(uint32_t *)&v;
    }
    __half2 v = __floats2half2_rn(x, y);
    return *(uint32_t *)&v;
}

__device__ __forceinline__ float2 unpack_pair(uint32_t u, int bf16) {
    if (bf16) return __bfloat1622float2(*(__nv_bfloat162 *)&u);
    return __half22float2(*(__half2 *)&u);
}

__global__ void __launch_bounds__(THREADS, 1) prefill_tc_kernel(const TileParams P) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t s_q = smem_u32(smem);
    const uint32_t s_ql = s_q + PAGE_BYTES;
    const uint32_t s_k = s_ql + PAGE_BYTES;
    const uint32_t s_v = s_k + K_STAGES * PAGE_BYTES;
    const uint32_t bars = s_v + V_STAGES * PAGE_BYTES;
    const uint32_t b_q_full = bars;
    const uint32_t b_k_full = bars + 8, b_k_empty = b_k_full + 8 * K_STAGES;
    const uint32_t b_v_full = b_k_empty + 8 * K_STAGES, b_v_empty = b_v_full + 8 * V_STAGES;
    const uint32_t b_s_full = b_v_empty + 8 * V_STAGES, b_p_full = b_s_full + 16, b_pv_done = b_p_full + 16;
    volatile int *abortp = &abort_flag;

    const TileItem it = P.items[blockIdx.x];
    const uint32_t n_tiles = it.page_end - it.page_begin;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(b_q_full, 1);
        for (int s = 0; s < K_STAGES; s++) {
            mbar_init(b_k_full + 8 * s, 1);
            mbar_init(b_k_empty + 8 * s, 1);
        }
        for (int s = 0; s < V_STAGES; s++) {
            mbar_init(b_v_full + 8 * s, 1);
            mbar_init(b_v_empty + 8 * s, 1);
        }
        for (int s = 0; s < 2; s++) {
            mbar_init(b_s_full + 8 * s, 1);
            mbar_init(b_p_full + 8 * s, SOFTMAX_WARPS * 32);
        }
        mbar_init(b_pv_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Stale rows of a ragged V page meet zero probabilities: they must hold finite numbers.
    for (int i = threadIdx.x; i < V_STAGES * PAGE_BYTES / 16; i += THREADS)
        ((uint4 *)(smem + (2 + K_STAGES) * PAGE_BYTES))[i] = make_uint4(0, 0, 0, 0);
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "n"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    const float sl2 = 0.08838834764831845f * 1.4426950408889634f;   // log2(e) / sqrt(128)

    if (warp == PRODUCER_WARP) {
        // ---- producer ------------------------------------------------------------------------
        const uint32_t kvh = it.kv_head;
        const uint32_t last_key = it.pos0 + it.n_rows - 1;   // newest key any row sees
        uint32_t kph = 0, vph = 0;
        int ks = 0, vs = 0;
        for (uint32_t c = 0; c < n_tiles; c += 32) {
            const uint32_t mine = it.page_begin + c + lane;
            const uint32_t my_page = mine < it.page_end ? P.pages[it.pt_off + mine] : 0u;
            const uint32_t n = min(32u, n_tiles - c);
            for (uint32_t j = 0; j < n; j++) {
                const uint32_t page = __shfl_sync(0xffffffffu, my_page, j);
                const uint32_t pg = it.page_begin + c + j;
                const uint32_t rows = min((uint32_t)PAGE, last_key + 1 - pg * PAGE);
                int stop = 0;
                if (lane == 0) {
                    const bool bad = page * (uint32_t)P.hkv + kvh >= P.n_blocks;
                    if (bad && atomicCAS(&P.status->code, 0, 1) == 0) {
                        P.status->where = 300;
                        P.status->a = (int)page;
                        P.status->b = (int)blockIdx.x;
                    }
                    const size_t off = ((size_t)page * P.hkv + kvh) * PAGE_BYTES;
                    // K
                    mbar_wait(b_k_empty + 8 * ks, kph ^ 1u, abortp, P.status, 31);
                    if (!*abortp) {
                        const uint32_t bar = b_k_full + 8 * ks, dst = s_k + ks * PAGE_BYTES;
                        if (bad) {
                            mbar_expect_tx(bar, 0);
                        } else if (rows == PAGE) {
                            mbar_expect_tx(bar, PAGE_BYTES);
                            bulk_g2s(dst, P.k_arena + off, PAGE_BYTES, bar);
                        } else {
                            mbar_expect_tx(bar, 2 * rows * 128);
                            bulk_g2s(dst, P.k_arena + off, rows * 128, bar);
                            bulk_g2s(dst + HALF_BYTES, P.k_arena + off + HALF_BYTES, rows * 128, bar);
                        }
                    }
                    // V
                    mbar_wait(b_v_empty + 8 * vs, vph ^ 1u, abortp, P.status, 32);
                    if (!*abortp) {
                        const uint32_t bar = b_v_full + 8 * vs, dst = s_v + vs * PAGE_BYTES;
                        if (bad) {
                            mbar_expect_tx(bar, 0);
                        } else if (rows == PAGE) {
                            mbar_expect_tx(bar, PAGE_BYTES);
                            bulk_g2s(dst, P.v_arena + off, PAGE_BYTES, bar);
                        } else {
                            mbar_expect_tx(bar, 2 * rows * 128);
                            bulk_g2s(dst, P.v_arena + off, rows * 128, bar);
                            bulk_g2s(dst + HALF_BYTES, P.v_arena + off + HALF_BYTES, rows * 128, bar);
                        }
                    }
                    stop = *abortp;
                }
                if (__shfl_sync(0xffffffffu, stop, 0)) break;
                if (++ks == K_STAGES) { ks = 0; kph ^= 1u; }
                if (++vs == V_STAGES) { vs = 0; vph ^= 1u; }
            }
            if (*abortp) break;
        }
    } else if (warp == MMA_WARP) {
        // ---- MMA issuer ----------------------------------------------------------------------
        if (lane == 0) {
            const uint32_t idesc_qk = instr_desc(P.bf16, 0), idesc_pv = instr_desc(P.bf16, 1);
            mbar_wait(b_q_full, 0, abortp, P.status, 33);
            tc_fence_after();
            uint32_t kph = 0, vph = 0;
            int ks = 0, vs = 0;
            auto issue_pv = [&](uint32_t j) {   // O (+)= P_j V_j
                const uint32_t b = j & 1u;
                mbar_wait(b_p_full + 8 * b, (j >> 1) & 1u, abortp, P.status, 34);
                mbar_wait(b_v_full + 8 * vs, vph, abortp, P.status, 35);
                tc_fence_after();
                const uint32_t v_base = s_v + vs * PAGE_BYTES;
#pragma unroll
                for (int k = 0; k < 8; k++) {   // 16 keys per step: two 8-row groups of the MN-major V tile
                    const uint64_t vdesc = smem_desc(v_base + k * 16 * 128, HALF_BYTES, 1024);
                    umma_ts(tmem + COL_O, tmem + (b ? COL_S1 : COL_S0) + k * 8, vdesc, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
                    if (P.p_lo) umma_ts(tmem + COL_O, tmem + (b ? COL_S1 : COL_S0) + 64 + k * 8, vdesc, idesc_pv, 1u);
                }
                umma_commit(b_v_empty + 8 * vs);
                umma_commit(b_pv_done);
                if (++vs == V_STAGES) { vs = 0; vph ^= 1u; }
            };
            for (uint32_t j = 0; j < n_tiles && !*abortp; j++) {
                const uint32_t b = j & 1u;
                mbar_wait(b_k_full + 8 * ks, kph, abortp, P.status, 36);
                tc_fence_after();
                const uint32_t k_base = s_k + ks * PAGE_BYTES;
#pragma unroll
                for (int k = 0; k < 8; k++) {   // 16 dims (32 bytes) per step; dims 64.. in the second half
                    const uint32_t off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
                    const uint64_t kdesc = smem_desc(k_base + off, 16, 1024);
                    umma_ss(tmem + (b ? COL_S1 : COL_S0), smem_desc(s_q + off, 16, 1024), kdesc, idesc_qk, k > 0 ? 1u : 0u);
                    if (P.q_lo) umma_ss(tmem + (b ? COL_S1 : COL_S0), smem_desc(s_ql + off, 16, 1024), kdesc, idesc_qk, 1u);
                }
                umma_commit(b_k_empty + 8 * ks);
                umma_commit(b_s_full + 8 * b);
                if (++ks == K_STAGES) { ks = 0; kph ^= 1u; }
                if (j > 0) issue_pv(j - 1);
            }
            if (n_tiles > 0 && !*abortp) issue_pv(n_tiles - 1);
        }
    } else {
        // ---- softmax: thread t owns query row t -----------------------------------------------
        const int r = threadIdx.x;
        const bool valid = (uint32_t)r < it.n_rows;
        const uint32_t pos = it.pos0 + (valid ? r : 0);
        uint32_t klo = 0;
        if (P.window > 0 && pos + 1 > P.window) klo = pos + 1 - P.window;
        const uint32_t khi = pos;
        const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);

        // The query tile, converted to the cache's type, into the swizzled operand layout.
        {
            const size_t base = ((size_t)(it.row0 + (valid ? r : 0)) * P.hq + it.head) * D;
#pragma unroll 4
            for (int c = 0; c < 16; c++) {   // sixteen 16-byte chunks of the row
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
                if (valid) {
                    a = load4_as_f32(P.q, P.q_dtype, base + c * 8);
                    b = load4_as_f32(P.q, P.q_dtype, base + c * 8 + 4);
                }
                const uint32_t w0 = pack_pair(a.x, a.y, P.bf16), w1 = pack_pair(a.z, a.w, P.bf16),
                               w2 = pack_pair(b.x, b.y, P.bf16), w3 = pack_pair(b.z, b.w, P.bf16);
                const uint32_t addr = s_q + (c >> 3) * HALF_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
                if (P.q_lo) {   // what the 16-bit rounding dropped
                    const float2 h0 = unpack_pair(w0, P.bf16), h1 = unpack_pair(w1, P.bf16), h2 = unpack_pair(w2, P.bf16),
                                 h3 = unpack_pair(w3, P.bf16);
                    const uint32_t l0 = pack_pair(a.x - h0.x, a.y - h0.y, P.bf16), l1 = pack_pair(a.z - h1.x, a.w - h1.y, P.bf16),
                                   l2 = pack_pair(b.x - h2.x, b.y - h2.y, P.bf16), l3 = pack_pair(b.z - h3.x, b.w - h3.y, P.bf16);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr + PAGE_BYTES), "r"(l0), "r"(l1), "r"(l2), "r"(l3) : "memory");
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("bar.sync 1, %0;" ::"n"(SOFTMAX_WARPS * 32) : "memory");
            if (threadIdx.x == 0) mbar_arrive(b_q_full);
        }

        float m_used = -INFINITY, l = 0.f;
        for (uint32_t j = 0; j < n_tiles; j++) {
            const uint32_t b = j & 1u;
            const uint32_t col_s = b ? COL_S1 : COL_S0;
            mbar_wait(b_s_full + 8 * b, (j >> 1) & 1u, abortp, P.status, 37);
            tc_fence_after();
            uint32_t sr[4][32];
#pragma unroll
            for (int c = 0; c < 4; c++) tmem_ld32(lane_addr + col_s + c * 32, sr[c]);
            tmem_ld_wait();
            const uint32_t key0 = (it.page_begin + j) * PAGE;
            const bool need_mask = key0 < klo || key0 + PAGE - 1 > khi;
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; c++)
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    float s = __uint_as_float(sr[c][i]);
                    if (need_mask) {
                        const uint32_t key = key0 + c * 32 + i;
                        if (key < klo || key > khi) s = -INFINITY;
                    }
                    sr[c][i] = __float_as_uint(s);
                    mx = fmaxf(mx, s);
                }
            // Lazy rescaling: keep the old reference maximum while the new one is within 2^8.
            float alpha = 1.f;
            bool rescale = false;
            if (mx > m_used && (m_used == -INFINITY || (mx - m_used) * sl2 > 8.f)) {
                alpha = m_used == -INFINITY ? 0.f : fast_exp2((m_used - mx) * sl2);
                rescale = m_used != -INFINITY;   // nothing accumulated yet otherwise
                m_used = mx;
                l *= alpha;
            }
            const float ms = (m_used == -INFINITY ? 0.f : m_used) * sl2;
            // Probabilities over the scores they came from: 128 keys as 64 packed columns, and
            // (bf16 caches) what the 8-bit mantissa dropped as 64 more.
            float sum = 0.f;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                uint32_t pr[32], pl[32];
#pragma unroll
                for (int c = 2 * h; c < 2 * h + 2; c++)
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float p0 = fast_exp2(__uint_as_float(sr[c][i]) * sl2 - ms);
                        const float p1 = fast_exp2(__uint_as_float(sr[c][i + 1]) * sl2 - ms);
                        sum += p0 + p1;
                        const uint32_t w = pack_pair(p0, p1, P.bf16);
                        pr[(c & 1) * 16 + (i >> 1)] = w;
                        if (P.p_lo) {
                            const float2 hf = unpack_pair(w, P.bf16);
                            pl[(c & 1) * 16 + (i >> 1)] = pack_pair(p0 - hf.x, p1 - hf.y, P.bf16);
                        }
                    }
                tmem_st32(lane_addr + col_s + h * 32, pr);
                if (P.p_lo) tmem_st32(lane_addr + col_s + 64 + h * 32, pl);
            }
            l += sum;
            tmem_st_wait();
            // The accumulator is quiet between P_{j-1}V_{j-1} and P_jV_j: rescale it here.
            if (j > 0) {
                mbar_wait(b_pv_done, (j - 1) & 1u, abortp, P.status, 38);
                tc_fence_after();
                if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
                    for (int c = 0; c < 4; c++) {
                        uint32_t orow[32];
                        tmem_ld32(lane_addr + COL_O + c * 32, orow);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; i++) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
                        tmem_st32(lane_addr + COL_O + c * 32, orow);
                    }
                    tmem_st_wait();
                }
            }
            tc_fence_before();
            mbar_arrive(b_p_full + 8 * b);
        }
        // Output: O / l, in the tensor's type.
        if (n_tiles > 0) {
            mbar_wait(b_pv_done, (n_tiles - 1) & 1u, abortp, P.status, 39);
            tc_fence_after();
            const float inv = 1.0f / l;
            const size_t obase = ((size_t)(it.row0 + (valid ? r : 0)) * P.hq + it.head) * D;
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
                uint32_t orow[32];
                tmem_ld32(lane_addr + COL_O + c * 32, orow);
                tmem_ld_wait();
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        store4(P.out, P.out_dtype, obase + c * 32 + i,
                               make_float4(__uint_as_float(orow[i]) * inv, __uint_as_float(orow[i + 1]) * inv,
                                           __uint_as_float(orow[i + 2]) * inv, __uint_as_float(orow[i + 3]) * inv));
                }
            }
        }
    }
    // Everyone is done with tensor memory before it is given back.
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        if (*abortp) {
            // MMAs and copies issued before giving up may still be running.
            for (int i = 0; i < 64; i++) __nanosleep(1000);
        }
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(TMEM_COLS) : "memory");
    }
}


// =============================================================================================
// Two query tiles per CTA: the same 128 rows for two query heads of one KV head.  Each K and V
// page is staged once for 256 query rows, two softmax warpgroups work while the tensor core
// alternates between the tiles, and TMEM is used in full: S/P of tile A [0,128), of tile B
// [128,256), O of A [256,384), O of B [384,512).  Issue order, per page j:
//   S_A(j) S_B(j) | P_A(j)V_j  S_A(j+1) | P_B(j)V_j  S_B(j+1) | ...
// so that a warpgroup's next scores are on their way while the other's probabilities are used.
// Ten warps: 0-3 softmax of A, 4-7 softmax of B, 8 producer, 9 MMA issuer.
// =============================================================================================
constexpr int T2_K_STAGES = 2, T2_V_STAGES = 3;
constexpr int T2_PRODUCER = 8, T2_MMA = 9, T2_CONVERT = 10;
constexpr int T2_THREADS = 10 * 32;
constexpr int T2_THREADS_CONVERT = 12 * 32;   // with the two warps that convert V pages (see VCONV below)
// barriers: q_full, k_full[2], v_full[3], s_full_a, s_full_b[2], p_half[2][2], pv_done[2], v_ready[3]
constexpr int T2_BARS = 1 + T2_K_STAGES + T2_V_STAGES + 1 + T2_K_STAGES + 4 + 2 + T2_V_STAGES;
constexpr int T2_SMEM_BYTES = PAGE_BYTES * (2 + T2_K_STAGES + T2_V_STAGES) + T2_BARS * 8 + 64;

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Scores of keys outside [klo, khi] become -inf, in place in TMEM.  Only ragged tiles (the
// diagonal, a window's lower edge) come here, so the loop is rolled: small code matters more
// than speed.
__device__ __noinline__ void mask_scores(uint32_t s_addr, uint32_t key0, uint32_t klo, uint32_t khi) {
#pragma unroll 1
    for (int c = 0; c < 4; c++) {
        uint32_t sr[32];
        tmem_ld32(s_addr + c * 32, sr);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i++) {
            const uint32_t key = key0 + c * 32 + i;
            if (key < klo || key > khi) sr[i] = 0xff800000u;
        }
        tmem_st32(s_addr + c * 32, sr);
    }
    tmem_st_wait();
}

// 32 scores of one query row (one chunk of a tile) become probabilities, in place: pair i
// (scores 2i, 2i+1) becomes a packed 16-bit pair in word i, which the pairs before i no longer
// need.  For bf16, what the 8-bit mantissa dropped goes to word 16 + i once the whole chunk is
// read.  Straight-line and free of run-time type switches: the softmax warps are bound by
// instruction fetch and issue.
// Two f32 lanes in one 64-bit register, for the packed FMA-pipe instructions of sm_100
// (fma.rn.f32x2, add.f32x2, sub.f32x2): one issue slot for two results.
__device__ __forceinline__ uint64_t pack_f2(float a, float b) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(a), "f"(b));
    return d;
}
__device__ __forceinline__ void unpack_f2(uint64_t d, float &a, float &b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(d));
}
__device__ __forceinline__ uint64_t fma_f2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add_f2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t sub_f2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

template <bool BF16>
__device__ __forceinline__ void exp_chunk(uint32_t (&sr)[32], float sl2, float ms, float &sum0, float &sum1) {
    if constexpr (BF16) {
        // bf16: the low parts make this loop issue-bound, and the packed instructions (scale and
        // shift, running sums, the residual) save three issue slots of twelve per pair.
        uint32_t lo[16];
        const uint64_t scale2 = pack_f2(sl2, sl2), shift2 = pack_f2(-ms, -ms);
        uint64_t sums = pack_f2(sum0, sum1);
#pragma unroll
        for (int i = 0; i < 16; i++) {
            float x0, x1;
            unpack_f2(fma_f2(pack_f2(__uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1])), scale2, shift2), x0, x1);
            const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
            const uint64_t p2 = pack_f2(p0, p1);
            sums = add_f2(sums, p2);
            __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
            const uint32_t w = *(uint32_t *)&v;
            float r0, r1;
            unpack_f2(sub_f2(p2, pack_f2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u))), r0, r1);
            __nv_bfloat162 lv = __floats2bfloat162_rn(r0, r1);
            lo[i] = *(uint32_t *)&lv;
            sr[i] = w;
        }
        unpack_f2(sums, sum0, sum1);
#pragma unroll
        for (int i = 0; i < 16; i++) sr[16 + i] = lo[i];
    } else {
        // f16: bound by the chain of TMEM round trips, not by issue slots; scalar code measured faster.
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(sr[2 * i]), sl2, -ms));
            const float p1 = fast_exp2(fmaf(__uint_as_float(sr[2 * i + 1]), sl2, -ms));
            sum0 += p0;
            sum1 += p1;
            __half2 v = __floats2half2_rn(p0, p1);
            sr[i] = *(uint32_t *)&v;
        }
    }
}

// 32 columns to TMEM: words [o, o + 16) of x, then of y (no copy through a third array).
__device__ __forceinline__ void tmem_st32_pair(uint32_t taddr, const uint32_t (&x)[32], const uint32_t (&y)[32], int o) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(x[o + 0]), "r"(x[o + 1]), "r"(x[o + 2]), "r"(x[o + 3]), "r"(x[o + 4]), "r"(x[o + 5]), "r"(x[o + 6]), "r"(x[o + 7]),
        "r"(x[o + 8]), "r"(x[o + 9]), "r"(x[o + 10]), "r"(x[o + 11]), "r"(x[o + 12]), "r"(x[o + 13]), "r"(x[o + 14]), "r"(x[o + 15]),
        "r"(y[o + 0]), "r"(y[o + 1]), "r"(y[o + 2]), "r"(y[o + 3]), "r"(y[o + 4]), "r"(y[o + 5]), "r"(y[o + 6]), "r"(y[o + 7]),
        "r"(y[o + 8]), "r"(y[o + 9]), "r"(y[o + 10]), "r"(y[o + 11]), "r"(y[o + 12]), "r"(y[o + 13]), "r"(y[o + 14]), "r"(y[o + 15])
        : "memory");
}

// Probabilities of 64 keys (two chunks) to TMEM: 32 packed columns at `p_addr`, and for bf16
// their low parts 64 columns further on.  The stores are only issued: the caller waits for them
// (tcgen05.wait::st) before it tells the tensor core.
template <bool BF16>
__device__ __forceinline__ void store_half(uint32_t p_addr, const uint32_t (&x)[32], const uint32_t (&y)[32]) {
    tmem_st32_pair(p_addr, x, y, 0);
    if (BF16) tmem_st32_pair(p_addr + 64, x, y, 16);
}

// Two packed bf16 values as two packed f16 values.  Exact for magnitudes in [2^-14, 65536); smaller
// ones lose at most 2^-25, larger ones clamp to the largest f16 (a cache that holds such values
// runs the other variant of the kernel; what clamps here is stale data behind a ragged page, which
// meets zero probabilities and only has to stay finite).
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t w) {
    uint32_t d;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(__uint_as_float(w & 0xffff0000u)), "f"(__uint_as_float(w << 16)));
    return d;
}

// BF16: the cache (and Q) are bf16, else f16.  VCONV (bf16 caches only): two more warps turn every
// V page into f16 in shared memory as it lands, probabilities are written as f16, and P V is ONE
// f16 MMA per K-step; without it a bf16 cache pays two (probabilities as a high and a low bf16
// part), because 8 bits of mantissa are not enough for them.  bf16 -> f16 is exact for every value
// below 65536 in magnitude; whether the cache holds anything larger is recorded by the kernels
// that write V (the cache's `wide_v` flag), and the bf16 kernel below picks the variant from it.
template <bool BF16, bool VCONV>
__device__ __forceinline__ void tc2_body(const TileParams P) {
    static_assert(BF16 || !VCONV, "only bf16 pages are converted");
    constexpr bool PB = BF16 && !VCONV;   // probabilities and V go to the tensor core as bf16 (two parts)
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t s_qa = smem_u32(smem), s_qb = s_qa + PAGE_BYTES;
    const uint32_t s_k = s_qb + PAGE_BYTES;
    const uint32_t s_v = s_k + T2_K_STAGES * PAGE_BYTES;
    const uint32_t bars = s_v + T2_V_STAGES * PAGE_BYTES;
    const uint32_t b_q_full = bars;
    // Every tcgen05.commit costs the tensor pipe a bubble, so one completion signal serves
    // several waiters.  S of tile B for page g (barrier s_full_b[g & 1]) is the last MMA issued
    // that reads K stage g & 1, and it is issued after P V of both tiles for page g - 1: its
    // completion tells softmax warpgroup B that scores are ready and the producer that K stage
    // g & 1 and V stage (g - 1) % 3 are free.  Likewise S of page g + 1 complete means P V of
    // page g complete, which is all a rescale of the accumulator needs.  Only the last P V of
    // each item gets a commit of its own (pv_done).
    const uint32_t b_k_full = bars + 8, b_v_full = b_k_full + 8 * T2_K_STAGES;
    const uint32_t b_s_full_a = b_v_full + 8 * T2_V_STAGES, b_s_full_b = b_s_full_a + 8;
    const uint32_t b_p_half = b_s_full_b + 8 * T2_K_STAGES, b_pv_done = b_p_half + 32;
    const uint32_t b_v_ready = b_pv_done + 16;   // V stage converted (VCONV): one arrival per converting warp
    volatile int *abortp = &abort_flag;

    // The CTA is persistent: the host dealt it items [item0, item_end) of the list.  `g` counts
    // the CTA's pages across its items: ring stages and barrier phases follow g, not the page's
    // index in its item.
    const uint32_t item0 = P.cta_begin[blockIdx.x], item_end = P.cta_begin[blockIdx.x + 1];
    const bool tr0 = YX_TR(P.trace != nullptr) && blockIdx.x == 0 && threadIdx.x == 0;
    if (tr0) P.trace[1536] = clock64();

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(b_q_full, 2);
        for (int s = 0; s < T2_K_STAGES; s++) {
            mbar_init(b_k_full + 8 * s, 1);
            mbar_init(b_s_full_b + 8 * s, 1);
        }
        for (int s = 0; s < T2_V_STAGES; s++) {
            mbar_init(b_v_full + 8 * s, 1);
            mbar_init(b_v_ready + 8 * s, 2);
        }
        mbar_init(b_s_full_a, 1);
        for (int t = 0; t < 2; t++) {
            mbar_init(b_p_half + 16 * t, 4);       // one arrival per softmax warp,
            mbar_init(b_p_half + 16 * t + 8, 4);   // for each 64-key half of the tile
            mbar_init(b_pv_done + 8 * t, 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Rows of a V stage that a ragged page leaves unwritten meet zero probabilities: they must
    // hold finite numbers (afterwards they hold earlier pages' values, which are).
    for (int i = threadIdx.x; i < T2_V_STAGES * PAGE_BYTES / 16; i += blockDim.x)
        ((uint4 *)(smem + (2 + T2_K_STAGES) * PAGE_BYTES))[i] = make_uint4(0, 0, 0, 0);
    if (warp == T2_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "n"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    const float sl2 = 0.08838834764831845f * 1.4426950408889634f;
    if (tr0) P.trace[1537] = clock64();

    if (warp == T2_PRODUCER) {
        // ---- producer: one K page and one V page per tile, for both query tiles ---------------
        uint32_t g = 0;
        for (uint32_t n = 0; item0 + n < item_end && !*abortp; n++) {
            const TileItem it = P.items[item0 + n];
            const uint32_t n_tiles = it.page_end - it.page_begin;
            const uint32_t kvh = it.kv_head;
            const uint32_t last_key = it.pos0 + it.n_rows - 1;
            for (uint32_t c = 0; c < n_tiles; c += 32) {
                const uint32_t mine = it.page_begin + c + lane;
                const uint32_t my_page = mine < it.page_end ? P.pages[it.pt_off + mine] : 0u;
                const uint32_t cnt = min(32u, n_tiles - c);
                for (uint32_t jj = 0; jj < cnt; jj++, g++) {
                    const uint32_t page = __shfl_sync(0xffffffffu, my_page, jj);
                    const uint32_t pg = it.page_begin + c + jj;
                    const uint32_t rows = min((uint32_t)PAGE, last_key + 1 - pg * PAGE);
                    int stop = 0;
                    if (lane == 0) {
                        const bool bad = page * (uint32_t)P.hkv + kvh >= P.n_blocks;
                        if (bad && atomicCAS(&P.status->code, 0, 1) == 0) {
                            P.status->where = 310;
                            P.status->a = (int)page;
                            P.status->b = (int)blockIdx.x;
                        }
                        const size_t off = ((size_t)page * P.hkv + kvh) * PAGE_BYTES;
                        // K stage g & 1 and V stage g % 3 are free once S of tile B for page g - 2 is done.
                        if (g >= 2) mbar_wait(b_s_full_b + 8 * (g & 1), ((g - 2) >> 1) & 1u, abortp, P.status, 41);
                        if (!*abortp) {
                            for (int kv = 0; kv < 2; kv++) {
                                const uint32_t bar = kv ? b_v_full + 8 * (g % 3) : b_k_full + 8 * (g & 1);
                                const uint32_t dst = kv ? s_v + (g % 3) * PAGE_BYTES : s_k + (g & 1) * PAGE_BYTES;
                                const char *src = (kv ? P.v_arena : P.k_arena) + off;
                                if (bad) {
                                    mbar_expect_tx(bar, 0);
                                } else if (rows == PAGE) {
                                    mbar_expect_tx(bar, PAGE_BYTES);
                                    bulk_g2s(dst, src, PAGE_BYTES, bar);
                                } else {
                                    mbar_expect_tx(bar, 2 * rows * 128);
                                    bulk_g2s(dst, src, rows * 128, bar);
                                    bulk_g2s(dst + HALF_BYTES, src + HALF_BYTES, rows * 128, bar);
                                }
                            }
                        }
                        stop = *abortp;
                    }
                    if (__shfl_sync(0xffffffffu, stop, 0)) break;
                }
                if (*abortp) break;
            }
        }
    } else if (warp == T2_MMA) {
        // ---- MMA issuer ----------------------------------------------------------------------
        if (lane == 0) {
            const uint32_t idesc_qk = instr_desc(BF16, 0), idesc_pv = instr_desc(PB, 1);
            // Low descriptor words of the tiles at offset 0; a K-step adds a constant.
            const uint32_t qa_lo = desc_lo(s_qa, 16), qb_lo = desc_lo(s_qb, 16), k_lo = desc_lo(s_k, 16),
                           v_lo = desc_lo(s_v, HALF_BYTES);
            auto issue_s = [&](int t, uint32_t stage) {   // S_t = Q_t K^T
                const uint32_t q_lo = t ? qb_lo : qa_lo, kk_lo = k_lo + stage * (PAGE_BYTES >> 4);
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const uint32_t off = ((k >> 2) * HALF_BYTES + (k & 3) * 32) >> 4;
                    umma_ss_lo(tmem + t * 128, q_lo + off, kk_lo + off, idesc_qk, k > 0 ? 1u : 0u);
                }
                umma_commit(t ? b_s_full_b + 8 * stage : b_s_full_a);
            };
            auto stamp = [&](uint32_t g, int e) {
                if (YX_TR(P.trace != nullptr) && blockIdx.x == 0 && g < 64) P.trace[(2 * 64 + g) * 8 + e] = clock64();
            };
            // O_t (+)= P_t V, a 64-key half at a time; `first`: the item's first page
            auto issue_pv = [&](int t, uint32_t g, bool first, bool last) {
                const uint32_t vv_lo = v_lo + (g % 3) * (PAGE_BYTES >> 4);
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    mbar_wait(b_p_half + 16 * t + 8 * h, g & 1u, abortp, P.status, 44 + t);
                    if (h == 0) stamp(g, t ? 5 : 1);
                    tc_fence_after();
#pragma unroll
                    for (int k = 4 * h; k < 4 * h + 4; k++) {
                        const uint32_t vk_lo = vv_lo + ((k * 16 * 128) >> 4);
                        umma_ts_lo(tmem + 256 + t * 128, tmem + t * 128 + k * 8, vk_lo, idesc_pv, (!first || k > 0) ? 1u : 0u);
                        if (PB) umma_ts_lo(tmem + 256 + t * 128, tmem + t * 128 + 64 + k * 8, vk_lo, idesc_pv, 1u);
                    }
                }
                if (last) umma_commit(b_pv_done + 8 * t);
            };
            uint32_t g = 0;
            for (uint32_t n = 0; item0 + n < item_end && !*abortp; n++) {
                const TileItem it = P.items[item0 + n];
                const uint32_t n_tiles = it.page_end - it.page_begin;
                mbar_wait(b_q_full, n & 1u, abortp, P.status, 43);
                mbar_wait(b_k_full + 8 * (g & 1), (g >> 1) & 1u, abortp, P.status, 46);
                tc_fence_after();
                issue_s(0, g & 1);
                issue_s(1, g & 1);
                for (uint32_t j = 0; j < n_tiles && !*abortp; j++, g++) {
                    const bool more = j + 1 < n_tiles;
                    mbar_wait((VCONV ? b_v_ready : b_v_full) + 8 * (g % 3), (g / 3) & 1u, abortp, P.status, 47);
                    stamp(g, 0);
                    issue_pv(0, g, j == 0, !more);
                    stamp(g, 2);
                    if (more) {
                        mbar_wait(b_k_full + 8 * ((g + 1) & 1), ((g + 1) >> 1) & 1u, abortp, P.status, 48);
                        stamp(g, 3);
                        tc_fence_after();
                        issue_s(0, (g + 1) & 1);
                    }
                    stamp(g, 4);
                    issue_pv(1, g, j == 0, !more);
                    stamp(g, 6);
                    if (more) issue_s(1, (g + 1) & 1);
                    stamp(g, 7);
                }
            }
        }
    } else if (!VCONV && warp >= T2_CONVERT) {
        // (the bf16 kernel is launched with the converting variant's twelve warps; here they idle)
    } else if (VCONV && warp >= T2_CONVERT) {
        // ---- V pages, bf16 -> f16 in place, a 64-dim half of the page per warp ------------------
        const uint32_t half = (uint32_t)(warp - T2_CONVERT) * HALF_BYTES;
        uint32_t g = 0;
        for (uint32_t n = 0; item0 + n < item_end && !*abortp; n++) {
            const TileItem it = P.items[item0 + n];
            const uint32_t n_tiles = it.page_end - it.page_begin;
            for (uint32_t j = 0; j < n_tiles && !*abortp; j++, g++) {
                mbar_wait(b_v_full + 8 * (g % 3), (g / 3) & 1u, abortp, P.status, 60);
                if (*abortp) break;
                const uint32_t base = s_v + (g % 3) * PAGE_BYTES + half;
#pragma unroll 4
                for (int i = lane; i < HALF_BYTES / 16; i += 32) {
                    uint32_t a, b, c, d;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(base + 16u * i));
                    a = bf16x2_to_f16x2(a);
                    b = bf16x2_to_f16x2(b);
                    c = bf16x2_to_f16x2(c);
                    d = bf16x2_to_f16x2(d);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + 16u * i), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
                }
                // the tensor core reads the page through the async proxy
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(b_v_ready + 8 * (g % 3));
            }
        }
    } else {
        // ---- softmax warpgroups: warps 0-3 tile A (head), warps 4-7 tile B (head + 1) -----------
        const int t = warp >> 2;
        const int r = threadIdx.x & 127;
        const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t s_addr = lane_addr + t * 128, o_addr = lane_addr + 256 + t * 128;
        const uint32_t s_q = t ? s_qb : s_qa;
        const size_t qrow = (size_t)P.hq * D;
        const bool q_direct = P.q_dtype == (BF16 ? YX_BF16 : YX_F16);
        auto wg_sync = [&]() {   // one named barrier per warpgroup
            if (t == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
            else asm volatile("bar.sync 2, 128;" ::: "memory");
        };
        auto chunk_addr = [&](int row, int c) {
            return s_q + (c >> 3) * HALF_BYTES + row * 128 + (((c & 7) ^ (row & 7)) << 4);
        };
        // Q tile in the operand layout.  Work is dealt by 16-byte chunk, not by row: 16 consecutive
        // threads read one row's 256 contiguous bytes.  A tile of the cache's own type is copied
        // global -> shared asynchronously (16 bytes per copy, rows past the item's end zero-filled),
        // so the next item's tile can be fetched while the current item finishes; other types are
        // converted on the way through registers.
        auto q_async = [&](const TileItem &ti) {
            const size_t qbase = ((size_t)ti.row0 * P.hq + ti.head + t) * D;
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const int idx = i * 128 + r, row = idx >> 4, c = idx & 15;
                const bool ok = (uint32_t)row < ti.n_rows;
                const uint16_t *src = (const uint16_t *)P.q + qbase + (ok ? row : 0) * qrow + c * 8;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(chunk_addr(row, c)), "l"(src), "r"(ok ? 16 : 0) : "memory");
            }
        };
        auto q_convert = [&](const TileItem &ti) {
            const size_t qbase = ((size_t)ti.row0 * P.hq + ti.head + t) * D;
#pragma unroll 1
            for (int i0 = 0; i0 < 16; i0 += 4) {
                float4 lo4[4], hi4[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int idx = (i0 + i) * 128 + r, row = idx >> 4, c = idx & 15;
                    lo4[i] = hi4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if ((uint32_t)row < ti.n_rows) {
                        lo4[i] = load4_as_f32(P.q, P.q_dtype, qbase + row * qrow + c * 8);
                        hi4[i] = load4_as_f32(P.q, P.q_dtype, qbase + row * qrow + c * 8 + 4);
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int idx = (i0 + i) * 128 + r, row = idx >> 4, c = idx & 15;
                    const uint32_t w0 = pack_pair(lo4[i].x, lo4[i].y, BF16), w1 = pack_pair(lo4[i].z, lo4[i].w, BF16),
                                   w2 = pack_pair(hi4[i].x, hi4[i].y, BF16), w3 = pack_pair(hi4[i].z, hi4[i].w, BF16);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(chunk_addr(row, c)), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
                }
            }
        };
        // Makes the staged tile visible to the tensor core and tells the MMA issuer.
        auto q_publish = [&]() {
            asm volatile("cp.async.wait_all;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            wg_sync();
            if (r == 0) mbar_arrive(b_q_full);
        };

        uint32_t g = 0;
        TileItem it{};
        if (item0 < item_end) {
            it = P.items[item0];
            if (q_direct) q_async(it);
            else q_convert(it);
            q_publish();
        }
        if (tr0) P.trace[1538] = clock64();
        for (uint32_t n = 0; item0 + n < item_end && !*abortp; n++) {
            const uint32_t n_tiles = it.page_end - it.page_begin;
            const bool valid = (uint32_t)r < it.n_rows;
            const uint32_t head = it.head + t;
            const uint32_t pos = it.pos0 + (valid ? r : 0);
            uint32_t klo = 0;
            if (P.window > 0 && pos + 1 > P.window) klo = pos + 1 - P.window;
            const uint32_t khi = pos;
            const bool have_next = item0 + n + 1 < item_end;
            TileItem next{};
            if (have_next) next = P.items[item0 + n + 1];
            float m_used = -INFINITY, l = 0.f;
            for (uint32_t j = 0; j < n_tiles; j++, g++) {
                if (t == 0) mbar_wait(b_s_full_a, g & 1u, abortp, P.status, 49);
                else mbar_wait(b_s_full_b + 8 * (g & 1), (g >> 1) & 1u, abortp, P.status, 50);
                const bool tr = YX_TR(P.trace != nullptr) && blockIdx.x == 0 && r == 0 && g < 64;
                if (tr) P.trace[(t * 64 + g) * 8 + 0] = clock64();
                tc_fence_after();
                // The item's last scores are computed: nothing reads its Q tile any more, and the
                // next item's can start to arrive.
                if (j + 1 == n_tiles && have_next && q_direct) q_async(next);
                const uint32_t key0 = (it.page_begin + j) * PAGE;
                // Warp-uniform decision: the TMEM accesses inside are warp-wide (.sync.aligned) and
                // must not sit under a per-lane condition.
                if (__any_sync(0xffffffffu, key0 < klo || key0 + PAGE - 1 > khi)) mask_scores(s_addr, key0, klo, khi);
                // The tile's scores, read once and held in registers.
                uint32_t s0[32], s1[32], s2[32], s3[32];
                tmem_ld32(s_addr, s0);
                tmem_ld32(s_addr + 32, s1);
                tmem_ld32(s_addr + 64, s2);
                tmem_ld32(s_addr + 96, s3);
                tmem_ld_wait();
                float ma = -INFINITY, mb = -INFINITY, mc = -INFINITY, md = -INFINITY;
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    ma = max3(ma, __uint_as_float(s0[i]), __uint_as_float(s0[i + 1]));
                    mb = max3(mb, __uint_as_float(s1[i]), __uint_as_float(s1[i + 1]));
                    mc = max3(mc, __uint_as_float(s2[i]), __uint_as_float(s2[i + 1]));
                    md = max3(md, __uint_as_float(s3[i]), __uint_as_float(s3[i + 1]));
                }
                const float mx = fmaxf(fmaxf(ma, mb), fmaxf(mc, md));
                // Lazy rescaling: the reference maximum moves only when the new one is more than
                // 2^8 above it, so that most tiles leave the accumulator alone.
                float alpha = 1.f;
                bool rescale = false;
                if (mx > m_used && (m_used == -INFINITY || (mx - m_used) * sl2 > 8.f)) {
                    alpha = m_used == -INFINITY ? 0.f : fast_exp2((m_used - mx) * sl2);
                    rescale = m_used != -INFINITY;   // nothing accumulated yet otherwise
                    m_used = mx;
                    l *= alpha;
                }
                if (j > 0 && __any_sync(0xffffffffu, rescale)) {
                    // The accumulator is quiet: these scores were computed after P(j-1)V, and P(j)V
                    // waits for this tile's probabilities.
#pragma unroll 1
                    for (int c = 0; c < 4; c++) {
                        uint32_t orow[32];
                        tmem_ld32(o_addr + c * 32, orow);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; i++) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
                        tmem_st32(o_addr + c * 32, orow);
                    }
                    tmem_st_wait();
                }
                const float ms = (m_used == -INFINITY ? 0.f : m_used) * sl2;
                float sum0 = 0.f, sum1 = 0.f;
                // Keys [0, 64) first, handed to the tensor core while the other half is computed.
                exp_chunk<PB>(s0, sl2, ms, sum0, sum1);
                exp_chunk<PB>(s1, sl2, ms, sum0, sum1);
                store_half<PB>(s_addr, s0, s1);
                // the stores' latency passes under the next chunk's exponentials
                exp_chunk<PB>(s2, sl2, ms, sum0, sum1);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(b_p_half + 16 * t);
                if (tr) P.trace[(t * 64 + g) * 8 + 1] = clock64();
                exp_chunk<PB>(s3, sl2, ms, sum0, sum1);
                store_half<PB>(s_addr + 32, s2, s3);
                tmem_st_wait();
                l += sum0 + sum1;
                tc_fence_before();
                __syncwarp();
                if (tr) P.trace[(t * 64 + g) * 8 + 2] = clock64();
                if (lane == 0) mbar_arrive(b_p_half + 16 * t + 8);
            }
            // The next item's Q tile is published before this item's epilogue: its first scores
            // are computed meanwhile.  (Its first P V cannot start before this warpgroup has left
            // the epilogue and delivered probabilities, so the accumulator read below is safe.)
            if (have_next) {
                if (!q_direct) q_convert(next);
                q_publish();
            }
            mbar_wait(b_pv_done + 8 * t, n & 1u, abortp, P.status, 53 + t);
            if (tr0 && n == 0) P.trace[1539] = clock64();
            tc_fence_after();
            // Each thread writes its own row, 16 bytes at a time.
            const float inv = 1.0f / l;
            const size_t obase = ((size_t)(it.row0 + (valid ? r : 0)) * P.hq + head) * D;
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
                uint32_t orow_r[32];
                tmem_ld32(o_addr + c * 32, orow_r);
                tmem_ld_wait();
                if (valid) {
                    if (P.out_dtype == YX_F32) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *(float4 *)((float *)P.out + obase + c * 32 + i) =
                                make_float4(__uint_as_float(orow_r[i]) * inv, __uint_as_float(orow_r[i + 1]) * inv,
                                            __uint_as_float(orow_r[i + 2]) * inv, __uint_as_float(orow_r[i + 3]) * inv);
                    } else {
                        const bool ob = P.out_dtype == YX_BF16;
#pragma unroll
                        for (int i = 0; i < 32; i += 8)
                            *(uint4 *)((uint16_t *)P.out + obase + c * 32 + i) =
                                make_uint4(pack_pair(__uint_as_float(orow_r[i]) * inv, __uint_as_float(orow_r[i + 1]) * inv, ob),
                                           pack_pair(__uint_as_float(orow_r[i + 2]) * inv, __uint_as_float(orow_r[i + 3]) * inv, ob),
                                           pack_pair(__uint_as_float(orow_r[i + 4]) * inv, __uint_as_float(orow_r[i + 5]) * inv, ob),
                                           pack_pair(__uint_as_float(orow_r[i + 6]) * inv, __uint_as_float(orow_r[i + 7]) * inv, ob));
                    }
                }
            }
            if (tr0 && n == 0) P.trace[1540] = clock64();
            it = next;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (tr0) P.trace[1541] = clock64();
    if (warp == T2_MMA) {
        if (*abortp) {
            for (int i = 0; i < 64; i++) __nanosleep(1000);
        }
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(TMEM_COLS) : "memory");
    }
}

// f16 caches.
__global__ void __launch_bounds__(T2_THREADS, 1) prefill_tc2_f16_kernel(const TileParams P) {
    // Launched as a programmatic dependent of the kernel before it (the append of this pass's rows):
    // everything that kernel wrote is read only after this wait.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    tc2_body<false, false>(P);
}

// The two-part variant for bf16 caches, out of line: it is the rare path, and kept apart it does not
// weigh on the register allocation of the variant that normally runs.
__device__ __noinline__ void tc2_two_part(const TileParams &P) { tc2_body<true, false>(P); }

// bf16 caches: V pages converted to f16 on the way in, unless the cache holds a value f16 cannot.
__global__ void __launch_bounds__(T2_THREADS_CONVERT, 1) prefill_tc2_bf16_kernel(const TileParams P) {
    asm volatile("griddepcontrol.wait;" ::: "memory");   // (the flag below is the append kernel's to set)
    if (*(volatile const uint32_t *)P.wide_v != 0u) tc2_two_part(P);
    else tc2_body<true, true>(P);
}

}  // namespace

int launch_prefill_tc(yx_ctx *ctx, const TileArgs &a) {
    if (!ctx->smem_configured[6]) {
        if (int rc = check_cuda(ctx, cudaFuncSetAttribute(prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES),
                                "prefill_tc: shared memory attribute"))
            return rc;
        ctx->smem_configured[6] = true;
    }
    TileParams P{};
    P.q = a.q;
    P.q_dtype = a.q_dtype;
    P.hq = a.hq;
    P.group = a.group;
    P.hkv = a.hkv;
    P.k_arena = a.k_arena;
    P.v_arena = a.v_arena;
    P.n_blocks = a.kv_pages * (uint32_t)a.hkv;
    P.window = (uint32_t)std::max<int64_t>(a.window, 0);
    P.pages = ctx->d_pages;
    P.items = a.items;
    P.out = a.out;
    P.out_dtype = a.out_dtype;
    P.bf16 = a.kv_dtype == YX_BF16 ? 1 : 0;
    P.p_lo = P.bf16;
    P.q_lo = P.bf16 && a.q_dtype == YX_F32;
    P.status = ctx->dev_status;
    P.trace = (long long *)ctx->trace_buf;
    P.wide_v = a.wide_v;
    if (a.pairs) {
        // Each item names the first of two query heads of one KV head.
        if (!ctx->smem_configured[7]) {
            if (int rc = check_cuda(ctx, cudaFuncSetAttribute(prefill_tc2_f16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T2_SMEM_BYTES),
                                    "prefill_tc2: shared memory attribute"))
                return rc;
            if (int rc = check_cuda(ctx, cudaFuncSetAttribute(prefill_tc2_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T2_SMEM_BYTES),
                                    "prefill_tc2: shared memory attribute"))
                return rc;
            ctx->smem_configured[7] = true;
        }
        P.cta_begin = a.cta_begin;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)a.n_ctas);   // persistent: at most one CTA per SM
        cfg.blockDim = dim3(P.bf16 ? T2_THREADS_CONVERT : T2_THREADS);
        cfg.dynamicSmemBytes = T2_SMEM_BYTES;
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t le = P.bf16 ? cudaLaunchKernelEx(&cfg, prefill_tc2_bf16_kernel, P) : cudaLaunchKernelEx(&cfg, prefill_tc2_f16_kernel, P);
        if (int rc = check_cuda(ctx, le, "prefill_tc2 kernel launch")) return rc;
    } else {
        prefill_tc_kernel<<<a.n_items, THREADS, SMEM_BYTES, ctx->stream>>>(P);
    }
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "prefill_tc kernel");
}

}  // namespace yx
