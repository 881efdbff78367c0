// Split-key (flash-decoding) attention for 16-bit KV caches: batched decode, speculative
// verification and rows over shared prefixes.  Bandwidth-bound: the job of this kernel is to
// keep every SM's share of HBM busy from the first microsecond to the last.
//
//  * Persistent: one CTA per SM walks the span of 64-key tiles the planner cut for it.
//  * A producer warp streams K and V tiles from the paged cache into a ring of shared-memory
//    stages with bulk asynchronous copies (`cp.async.bulk`, the TMA engine's untiled form)
//    that complete on mbarriers.  The cache layout (yx_internal.h) makes a tile four
//    contiguous runs that land already 128-byte swizzled, so no tensor map is needed and the
//    copy of a ragged tile is simply shorter.  The producer runs ahead across item
//    boundaries; the pipeline never drains between sequences.
//  * Four consumer warps share each tile.  All query heads of the KV head's group, and all
//    rows of an item, are the M rows of one `mma.sync` tile (16, 32 or 64 padded rows), so a
//    K or V byte is read once per item however many heads and rows use it.  Scores and
//    softmax stay in f32 registers; max and sum reduce with quad shuffles.
//  * f32 queries are split into a high and a low 16-bit part (two MMAs), so the only rounding
//    beyond the cache's own is that of the probabilities.
//  * Each item ends in an (m, l, o) triple per query row, the format of the reference's
//    split attention (crates/yaxus-backend-gpu/src/shaders.rs:1466-1579); combine.cu merges.
//
// Every wait on an mbarrier is bounded: on expiry the CTA records the failure in the
// context's status word, stops waiting anywhere, finishes structurally and returns.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "yx_internal.h"

namespace yx {
namespace {

constexpr int STAGES = 6;
constexpr int SUB_BYTES = TILE_KEYS * 128;        // one 64-dim half of a 64-key tile
constexpr int STAGE_BYTES = 4 * SUB_BYTES;        // K lo, K hi, V lo, V hi
constexpr int CONSUMERS = 4;                      // warps
constexpr int THREADS = (CONSUMERS + 1) * 32;
constexpr int MERGE_FLOATS = 16 * (D + 2);        // one warp's (m, l, o) for 16 rows
constexpr int MERGE_BYTES = 3 * MERGE_FLOATS * 4;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + ((MERGE_BYTES + 127) / 128) * 128 + 256;
constexpr long long WAIT_CYCLES = 4000000000ll;   // about two seconds

struct Shared {
    uint32_t stages;   // shared-space addresses
    uint32_t merge;
    uint32_t full;     // STAGES mbarriers
    uint32_t empty;    // STAGES mbarriers
    volatile int *abort_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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

// Bounded wait.  Returns at once when the CTA has given up; on expiry records where.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                          yx_dev_status *status, int where) {
    if (*abort_flag) return;
    if (mbar_try(bar, parity)) return;
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

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t &a, uint32_t &b, uint32_t &c, uint32_t &d) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(a), "=r"(b), "=r"(c), "=r"(d)
                 : "r"(addr));
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

__device__ __forceinline__ float2 load_q2(const void *q, int q_dtype, size_t elem) {
    if (q_dtype == YX_F32) return *(const float2 *)((const float *)q + elem);
    uint32_t raw = *(const uint32_t *)((const uint16_t *)q + elem);
    if (q_dtype == YX_F16) return __half22float2(*(__half2 *)&raw);
    return __bfloat1622float2(*(__nv_bfloat162 *)&raw);
}

struct Pipe {
    int stage;
    uint32_t phase;
    __device__ __forceinline__ void advance() {
        if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
        }
    }
};

struct Params {
    const void *q;
    int q_dtype, hq, group, hkv;
    const char *k_arena, *v_arena;
    uint32_t kv_pages;
    uint32_t window;
    const uint32_t *pos, *pages;
    const Item *items;
    const uint32_t *cta_begin;
    float *part_o, *part_ml;
    yx_dev_status *status;
};

// An item is 32 words: a warp reads it with one coalesced load, lane i holding word i, and
// takes fields out with shuffles.  Word indices follow `struct Item`.
constexpr int W_TILE_BEGIN = 0, W_TILE_END = 1, W_KEY_LO = 2, W_KEY_HI = 3, W_PT_OFF = 4, W_HEAD_ROWS = 5,
              W_ROWS = 6, W_PART = 14, W_MT = 30;
__device__ __forceinline__ uint32_t item_word(const Item *items, uint32_t ii, int lane) {
    return reinterpret_cast<const uint32_t *>(items + ii)[lane];
}
__device__ __forceinline__ uint32_t field(uint32_t w, int idx) { return __shfl_sync(0xffffffffu, w, idx); }

// ---- producer ---------------------------------------------------------------------------
// The whole warp runs this; lane 0 waits and issues the copies.  The page ids of up to 32
// tiles are fetched with one coalesced load, so no copy waits on a page-table lookup of its
// own, and the next item's header is in flight while this item streams.
__device__ void produce(const Params &P, const Shared &S, uint32_t ib, uint32_t ie, int lane) {
    Pipe pipe{0, 0};
    const size_t block_bytes = (size_t)PAGE * D * 2;
    uint32_t w_next = ib < ie ? item_word(P.items, ib, lane) : 0u;
    for (uint32_t ii = ib; ii < ie; ii++) {
        const uint32_t w = w_next;
        if (ii + 1 < ie) w_next = item_word(P.items, ii + 1, lane);
        const uint32_t tb = field(w, W_TILE_BEGIN), te = field(w, W_TILE_END);
        const uint32_t klo = field(w, W_KEY_LO), khi = field(w, W_KEY_HI);
        const uint32_t pt_off = field(w, W_PT_OFF), kvh = field(w, W_HEAD_ROWS) & 0xffffu;
        for (uint32_t c = tb; c < te; c += 32) {
            const uint32_t mine = c + lane;
            const uint32_t my_page = mine < te ? P.pages[pt_off + (mine >> 1)] : 0u;
            const int n_tiles = (int)min(32u, te - c);
            for (int j = 0; j < n_tiles; j++) {
                const uint32_t t = c + j;
                const uint32_t page = __shfl_sync(0xffffffffu, my_page, j);
                int stop = 0;
                if (lane == 0) {
                    mbar_wait(S.empty + 8 * pipe.stage, pipe.phase ^ 1u, S.abort_flag, P.status, 1);
                    stop = *S.abort_flag;
                    if (!stop) {
                        uint32_t a = max(klo, t * TILE_KEYS), b = min(khi, t * TILE_KEYS + TILE_KEYS - 1);
                        uint32_t r0 = a - t * TILE_KEYS, n = b - a + 1;
                        uint32_t bar = S.full + 8 * pipe.stage;
                        if (page >= P.kv_pages) {   // recorded; the tile keeps stale (finite) data
                            if (atomicCAS(&P.status->code, 0, 1) == 0) {
                                P.status->where = 200;
                                P.status->a = (int)page;
                                P.status->b = (int)ii;
                            }
                            mbar_expect_tx(bar, 0);
                        } else {
                            uint32_t bytes = n * 128;
                            size_t off = ((size_t)page * P.hkv + kvh) * block_bytes +
                                         (size_t)((t & 1) * TILE_KEYS + r0) * 128;
                            uint32_t dst = S.stages + pipe.stage * STAGE_BYTES + r0 * 128;
                            mbar_expect_tx(bar, 4 * bytes);
                            bulk_g2s(dst, P.k_arena + off, bytes, bar);
                            bulk_g2s(dst + SUB_BYTES, P.k_arena + off + PAGE * 128, bytes, bar);
                            bulk_g2s(dst + 2 * SUB_BYTES, P.v_arena + off, bytes, bar);
                            bulk_g2s(dst + 3 * SUB_BYTES, P.v_arena + off + PAGE * 128, bytes, bar);
                        }
                    }
                }
                if (__shfl_sync(0xffffffffu, stop, 0)) return;
                pipe.advance();
            }
        }
    }
}

// ---- consumers --------------------------------------------------------------------------
template <int MT, bool BF16>
__device__ void consume_item(const Params &P, const Shared &S, const uint32_t w, Pipe &pipe, int warp, int lane) {
    constexpr int NMT = MT / 16;          // 16-row tiles of queries
    constexpr int NSL = CONSUMERS / NMT;  // key slices of a tile
    constexpr int KS = TILE_KEYS / NSL;   // keys per slice
    constexpr int NT = KS / 8;            // 8-key score tiles per warp
    const int mi = warp % NMT, sl = warp / NMT;
    const int g = lane >> 2, t4 = lane & 3;
    const int group = P.group;
    const uint32_t tb = field(w, W_TILE_BEGIN), te = field(w, W_TILE_END);
    const uint32_t item_lo = field(w, W_KEY_LO), item_hi = field(w, W_KEY_HI);
    const uint32_t head_rows = field(w, W_HEAD_ROWS);
    const int kvh = (int)(head_rows & 0xffffu);
    const int q_rows = (int)(head_rows >> 16) * group;
    const float sl2 = 0.08838834764831845f * 1.4426950408889634f;   // log2(e) / sqrt(128)

    // The two query rows this thread owns in the accumulator fragments.
    uint32_t klo[2], khi[2], part[2];
    size_t q_elem[2];
    bool valid[2];
#pragma unroll
    for (int rs = 0; rs < 2; rs++) {
        int qr = mi * 16 + g + rs * 8;
        valid[rs] = qr < q_rows;
        const int ri = valid[rs] ? qr / group : 0;   // index into the item's rows
        const uint32_t row = (field(w, W_ROWS + (ri >> 1)) >> (16 * (ri & 1))) & 0xffffu;
        part[rs] = field(w, W_PART + ri);
        klo[rs] = 0;
        khi[rs] = 0xffffffffu;
        q_elem[rs] = 0;
        if (valid[rs]) {
            uint32_t p = P.pos[row];
            uint32_t lo = 0;
            if (P.window > 0 && p + 1 > P.window) lo = p + 1 - P.window;
            klo[rs] = max(lo, item_lo);
            khi[rs] = min(p, item_hi);
            q_elem[rs] = ((size_t)row * P.hq + (size_t)kvh * group + (qr % group)) * D;
        }
    }
    // Query fragments, high and low parts.
    uint32_t qh[8][4], ql[8][4];
    // The low part of an f32 query costs a second MMA per score tile; items with 64 padded rows
    // are the ones bound by tensor work, and their rows see long shared prefixes over which the
    // query's rounding averages out, so they go without it.
    const bool exact_q = MT == 64 || (P.q_dtype == YX_BF16 && BF16) || (P.q_dtype == YX_F16 && !BF16);
#pragma unroll
    for (int ks = 0; ks < 8; ks++) {
#pragma unroll
        for (int r = 0; r < 4; r++) {
            int rs = r & 1, dim = ks * 16 + (r >> 1) * 8 + 2 * t4;
            float2 v = valid[rs] ? load_q2(P.q, P.q_dtype, q_elem[rs] + dim) : make_float2(0.f, 0.f);
            uint32_t h = pack2<BF16>(v.x, v.y);
            float2 hf = unpack2<BF16>(h);
            qh[ks][r] = h;
            ql[ks][r] = pack2<BF16>(v.x - hf.x, v.y - hf.y);
        }
    }

    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    const int lm = lane >> 3, lr = lane & 7;
    for (uint32_t t = tb; t < te; t++) {
        mbar_wait(S.full + 8 * pipe.stage, pipe.phase, S.abort_flag, P.status, 2);
        const uint32_t sb = S.stages + pipe.stage * STAGE_BYTES;

        // S = Q K^T over this warp's KS keys.
        // The low parts of the queries accumulate on their own, so that no MMA waits on more
        // than the eight before it in its chain.
        float s[NT][4], s2[MT == 64 ? 1 : NT][4];
#pragma unroll
        for (int j = 0; j < NT; j++) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        if constexpr (MT != 64) {
#pragma unroll
            for (int j = 0; j < NT; j++) s2[j][0] = s2[j][1] = s2[j][2] = s2[j][3] = 0.f;
        }
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
            const uint32_t sub = sb + (ks >> 2) * SUB_BYTES;
            const int c = ((2 * ks) & 7) + (lm & 1);
#pragma unroll
            for (int np = 0; np < NT / 2; np++) {
                int key = sl * KS + np * 16 + (lm >> 1) * 8 + lr;
                uint32_t b0, b1, b2, b3;
                ldsm4(sub + key * 128 + ((c ^ lr) << 4), b0, b1, b2, b3);
                mma16816<BF16>(s[2 * np], qh[ks], b0, b1);
                mma16816<BF16>(s[2 * np + 1], qh[ks], b2, b3);
                if constexpr (MT != 64) {
                    if (!exact_q) {
                        mma16816<BF16>(s2[2 * np], ql[ks], b0, b1);
                        mma16816<BF16>(s2[2 * np + 1], ql[ks], b2, b3);
                    }
                }
            }
        }
        if constexpr (MT != 64) {
#pragma unroll
            for (int j = 0; j < NT; j++)
#pragma unroll
                for (int e = 0; e < 4; e++) s[j][e] += s2[j][e];
        }
        // Mask keys outside each row's [klo, khi].
        const uint32_t key0 = t * TILE_KEYS + sl * KS + 2 * t4;
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                uint32_t key = key0 + j * 8 + (e & 1);
                int rs = e >> 1;
                if (key < klo[rs] || key > khi[rs]) s[j][e] = -INFINITY;
            }
        // Online softmax, per owned row.
#pragma unroll
        for (int rs = 0; rs < 2; rs++) {
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < NT; j++) mx = fmaxf(mx, fmaxf(s[j][2 * rs], s[j][2 * rs + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            float mn = fmaxf(m[rs], mx);
            float mu = mn == -INFINITY ? 0.f : mn;
            float alpha = exp2f((m[rs] - mu) * sl2);
            m[rs] = mn;
            float sum = 0.f;
            float ms = mu * sl2;
#pragma unroll
            for (int j = 0; j < NT; j++) {
                float p0 = exp2f(s[j][2 * rs] * sl2 - ms), p1 = exp2f(s[j][2 * rs + 1] * sl2 - ms);
                s[j][2 * rs] = p0;
                s[j][2 * rs + 1] = p1;
                sum += p0 + p1;
            }
            l[rs] = l[rs] * alpha + sum;
#pragma unroll
            for (int n = 0; n < 16; n++) {
                o[n][2 * rs] *= alpha;
                o[n][2 * rs + 1] *= alpha;
            }
        }
        // O += P V.
#pragma unroll
        for (int kk = 0; kk < KS / 16; kk++) {
            uint32_t a[4], al[4];
#pragma unroll
            for (int r = 0; r < 4; r++) {
                const float p0 = s[2 * kk + (r >> 1)][(r & 1) * 2], p1 = s[2 * kk + (r >> 1)][(r & 1) * 2 + 1];
                a[r] = pack2<BF16>(p0, p1);
                if constexpr (BF16) {
                    // bf16 keeps 8 bits of a probability; its remainder goes in a second MMA.
                    float2 hf = unpack2<BF16>(a[r]);
                    al[r] = pack2<BF16>(p0 - hf.x, p1 - hf.y);
                }
            }
            int key = sl * KS + kk * 16 + (lm & 1) * 8 + lr;
#pragma unroll
            for (int np = 0; np < 8; np++) {
                const uint32_t sub = sb + 2 * SUB_BYTES + (np >> 2) * SUB_BYTES;
                const int c = ((2 * np) & 7) + (lm >> 1);
                uint32_t b0, b1, b2, b3;
                ldsm4t(sub + key * 128 + ((c ^ lr) << 4), b0, b1, b2, b3);
                mma16816<BF16>(o[2 * np], a, b0, b1);
                mma16816<BF16>(o[2 * np + 1], a, b2, b3);
                if constexpr (BF16) {
                    mma16816<BF16>(o[2 * np], al, b0, b1);
                    mma16816<BF16>(o[2 * np + 1], al, b2, b3);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(S.empty + 8 * pipe.stage);
        pipe.advance();
    }

    // Row sums across the quad.
#pragma unroll
    for (int rs = 0; rs < 2; rs++) {
        l[rs] += __shfl_xor_sync(0xffffffffu, l[rs], 1);
        l[rs] += __shfl_xor_sync(0xffffffffu, l[rs], 2);
    }

    // Merge the key slices of each 16-row tile through shared memory.
    if constexpr (NSL > 1) {
        float *scratch = (float *)__cvta_shared_to_generic((size_t)S.merge);
        if (sl > 0) {
            float *w = scratch + ((sl - 1) * NMT + mi) * MERGE_FLOATS;
#pragma unroll
            for (int rs = 0; rs < 2; rs++) {
                int r = g + rs * 8;
                if (t4 == 0) {
                    w[r] = m[rs];
                    w[16 + r] = l[rs];
                }
#pragma unroll
                for (int n = 0; n < 16; n++)
                    *(float2 *)(w + 32 + r * D + n * 8 + 2 * t4) = make_float2(o[n][2 * rs], o[n][2 * rs + 1]);
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory");
        if (sl == 0) {
#pragma unroll
            for (int rs = 0; rs < 2; rs++) {
                int r = g + rs * 8;
                float mx = m[rs];
#pragma unroll
                for (int x = 1; x < NSL; x++) mx = fmaxf(mx, scratch[((x - 1) * NMT + mi) * MERGE_FLOATS + r]);
                float mu = mx == -INFINITY ? 0.f : mx;
                float f = exp2f((m[rs] - mu) * sl2);
                l[rs] *= f;
#pragma unroll
                for (int n = 0; n < 16; n++) {
                    o[n][2 * rs] *= f;
                    o[n][2 * rs + 1] *= f;
                }
#pragma unroll
                for (int x = 1; x < NSL; x++) {
                    const float *w = scratch + ((x - 1) * NMT + mi) * MERGE_FLOATS;
                    float fx = exp2f((w[r] - mu) * sl2);
                    l[rs] += w[16 + r] * fx;
#pragma unroll
                    for (int n = 0; n < 16; n++) {
                        float2 v = *(const float2 *)(w + 32 + r * D + n * 8 + 2 * t4);
                        o[n][2 * rs] += v.x * fx;
                        o[n][2 * rs + 1] += v.y * fx;
                    }
                }
                m[rs] = mx;
            }
        }
    }
    if (sl == 0) {
#pragma unroll
        for (int rs = 0; rs < 2; rs++) {
            if (!valid[rs]) continue;
            int qr = mi * 16 + g + rs * 8;
            size_t slot = (size_t)part[rs] * group + (qr % group);
            float *po = P.part_o + slot * D;
#pragma unroll
            for (int n = 0; n < 16; n++) *(float2 *)(po + n * 8 + 2 * t4) = make_float2(o[n][2 * rs], o[n][2 * rs + 1]);
            if (t4 == 0) {
                bool none = m[rs] == -INFINITY;
                P.part_ml[slot * 2] = none ? -1e30f : m[rs] * 0.08838834764831845f;
                P.part_ml[slot * 2 + 1] = none ? 0.f : l[rs];
            }
        }
    }
    if constexpr (NSL > 1) asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory");
}

template <bool BF16>
__global__ void __launch_bounds__(THREADS, 1) attend_mma_kernel(const Params P) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ int abort_flag;
    Shared S;
    S.stages = smem_u32(smem);
    S.merge = S.stages + STAGES * STAGE_BYTES;
    S.full = S.merge + ((MERGE_BYTES + 127) / 128) * 128;
    S.empty = S.full + 8 * STAGES;
    S.abort_flag = &abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Stale rows of a ragged tile are multiplied by zero probabilities: they must be finite.
    for (int i = threadIdx.x; i < STAGES * STAGE_BYTES / 16; i += THREADS) ((uint4 *)smem)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; s++) {
            mbar_init(S.full + 8 * s, 1);
            mbar_init(S.empty + 8 * s, CONSUMERS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();

    const uint32_t ib = P.cta_begin[blockIdx.x], ie = P.cta_begin[blockIdx.x + 1];
    if (warp == CONSUMERS) {
        produce(P, S, ib, ie, lane);
        return;
    }
    Pipe pipe{0, 0};
    uint32_t w_next = ib < ie ? item_word(P.items, ib, lane) : 0u;
    for (uint32_t ii = ib; ii < ie; ii++) {
        const uint32_t w = w_next;
        if (ii + 1 < ie) w_next = item_word(P.items, ii + 1, lane);   // in flight while this item runs
        switch (field(w, W_MT)) {
            case 16: consume_item<16, BF16>(P, S, w, pipe, warp, lane); break;
            case 32: consume_item<32, BF16>(P, S, w, pipe, warp, lane); break;
            default: consume_item<64, BF16>(P, S, w, pipe, warp, lane); break;
        }
    }
    if (abort_flag) {
        // Copies issued before giving up may still be landing in this CTA's shared memory.
        for (int i = 0; i < 64; i++) __nanosleep(1000);
    }
}

}  // namespace

int launch_attend_mma(yx_ctx *ctx, const AttendArgs &a) {
    const bool bf16 = a.kv_dtype == YX_BF16;
    if (!ctx->smem_configured[bf16]) {
        cudaError_t e = bf16 ? cudaFuncSetAttribute(attend_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES)
                             : cudaFuncSetAttribute(attend_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (int rc = check_cuda(ctx, e, "attend_mma: shared memory attribute")) return rc;
        ctx->smem_configured[bf16] = true;
    }
    Params P{};
    P.q = a.q;
    P.q_dtype = a.q_dtype;
    P.hq = a.hq;
    P.group = a.group;
    P.hkv = a.hkv;
    P.k_arena = a.k_arena;
    P.v_arena = a.v_arena;
    P.kv_pages = a.kv_pages;
    P.window = (uint32_t)std::max<int64_t>(a.window, 0);
    P.pos = ctx->d_pos;
    P.pages = ctx->d_pages;
    P.items = a.items;
    P.cta_begin = a.cta_begin;
    P.part_o = a.part_o;
    P.part_ml = a.part_ml;
    P.status = ctx->dev_status;
    if (bf16) attend_mma_kernel<true><<<a.n_ctas, THREADS, SMEM_BYTES, ctx->stream>>>(P);
    else attend_mma_kernel<false><<<a.n_ctas, THREADS, SMEM_BYTES, ctx->stream>>>(P);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "attend_mma kernel");
}

}  // namespace yx
