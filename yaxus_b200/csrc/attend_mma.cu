// Split-key (flash-decoding) attention for 16-bit KV caches: batched decode, speculative
// verification and rows over shared prefixes.  Bandwidth-bound: the job of this kernel is to
// keep every SM's share of HBM busy from the first microsecond to the last.
//
//  * Persistent: one CTA per SM walks the span of 64-key tiles the planner cut for it.
//  * Nothing on the device walks a page table.  The host planner resolves every tile to its
//    (page, KV head) block; the producer warp reads 32 tile descriptors with one coalesced
//    load and feeds the copy engine from them, across item boundaries, never draining.
//  * K and V tiles come in by bulk asynchronous copies (`cp.async.bulk`, the TMA engine's
//    untiled form) that complete on mbarriers.  The cache layout (yx_internal.h) makes a tile
//    four contiguous runs that land already 128-byte swizzled, so no tensor map is needed and
//    the copy of a ragged tile is simply shorter.  Tiles that no other item reads are copied
//    with an L2 evict-first hint, so that the stream does not push the plan, the queries and
//    the partial results out of L2.
//  * A helper warp stages the queries of the next item in shared memory (converted to the
//    cache's 16-bit type, f32 queries as a high and a low part), so that consumers never wait
//    on global memory at an item boundary.
//  * Four consumer warps share each tile.  All query heads of the KV head's group, and all
//    rows of an item, are the M rows of one `mma.sync` tile (16, 32 or 64 padded rows), so a
//    K or V byte is read once per item however many heads and rows use it.  Scores and
//    softmax stay in f32 registers; max and sum reduce with quad shuffles.
//  * Each item ends in an (m, l, o) triple per query row, the format of the reference's
//    split attention (crates/yaxus-backend-gpu/src/shaders.rs:1466-1579).  The merge of the
//    triples (the reference's `attn_combine`, shaders.rs:1581-1637) is fused: the CTA that
//    delivers the last triple of a (row, KV head) merges them and writes the output, found
//    by an arrival counter in global scratch that the merging CTA resets.
//
// Every wait on an mbarrier is bounded: on expiry the CTA records the failure in the
// context's status word, stops waiting anywhere, finishes structurally and returns.
#include "yx_device.cuh"

namespace yx {
namespace {

using namespace dev;

constexpr int STAGES = 5;
constexpr int SUB_BYTES = TILE_KEYS * 128;        // one 64-dim half of a 64-key tile
constexpr int STAGE_BYTES = 4 * SUB_BYTES;        // K lo, K hi, V lo, V hi
constexpr int CONSUMERS = 4;                      // warps 0..3
constexpr int PRODUCER = CONSUMERS;               // warp 4
constexpr int QWARP = CONSUMERS + 1;              // warp 5
constexpr int THREADS = (CONSUMERS + 2) * 32;
constexpr int Q_SLOTS = 2;
constexpr int Q_SLOT_BYTES = 16384;               // 64 rows x 256 B, or 32 rows high + 32 rows low
constexpr int Q_LOW_OFFSET = 8192;
constexpr int MERGE_FLOATS = 16 * (D + 2);        // one warp's (m, l, o) for 16 rows
constexpr int MERGE_BYTES = ((3 * MERGE_FLOATS * 4 + 127) / 128) * 128;
constexpr int N_BARRIERS = 2 * STAGES + 2 * Q_SLOTS;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + Q_SLOTS * Q_SLOT_BYTES + MERGE_BYTES + 128 + N_BARRIERS * 8;

struct Shared {
    uint32_t stages, q, merge, flags;   // shared-space addresses
    uint32_t full, empty, qfull, qempty;
    volatile int *abort_flag;
};

struct Pipe {
    int stage;
    uint32_t phase;
    __device__ __forceinline__ void advance(int n) {
        if (++stage == n) {
            stage = 0;
            phase ^= 1u;
        }
    }
};

// What a CTA needs before its first global load returns, passed in kernel-parameter space:
// its span, its first two tiles and the rows of its first item.  A cold global load at kernel
// start costs over a microsecond; three of them in a chain (span -> descriptors -> data) were
// the largest single cost of a 15-microsecond kernel.
constexpr int MAX_PROLOGUE_CTAS = 160;
struct CtaPrologue {
    CtaHdr hdr;
    TileDesc first[2];
    uint32_t head_rows, mt;
    uint16_t rows[MAX_ITEM_ROWS];
};

struct Params {
    const void *q;
    int q_dtype, hq, group, hkv;
    const char *k_arena, *v_arena;
    uint32_t n_blocks;               // (page, kv head) blocks in an arena
    const CtaHdr *cta_hdr;
    const TileDesc *tiles;
    const ItemRec *recs;
    int single_use;
    float *part_o, *part_ml;
    uint32_t *counters;
    void *out;
    int out_dtype;
    float *m_out, *l_out, *o_out;
    yx_dev_status *status;
    unsigned long long *trace;       // optional: 8 timestamps / counters per CTA
    int has_prologue;
    CtaPrologue pro[MAX_PROLOGUE_CTAS];
};

__device__ __forceinline__ uint32_t field(uint32_t w, int idx) { return __shfl_sync(0xffffffffu, w, idx); }

// ---- producer: tile descriptors -> bulk copies ----------------------------------------------
// One tile: wait for a free stage, zero what a ragged copy leaves alone, start the four copies.
// Returns false when the CTA has given up.
__device__ __forceinline__ bool issue_tile(const Params &P, const Shared &S, Pipe &pipe, uint32_t block, uint32_t info,
                                           uint64_t policy, int lane) {
    const uint32_t half = info & 1u, r0 = (info >> 1) & 127u, n = (info >> 8) & 255u;
    int stop = 0;
    if (lane == 0) {
        mbar_wait(S.empty + 8 * pipe.stage, pipe.phase ^ 1u, S.abort_flag, P.status, 1);
        stop = *S.abort_flag;
    }
    if (__shfl_sync(0xffffffffu, stop, 0)) return false;
    const uint32_t sb = S.stages + pipe.stage * STAGE_BYTES;
    if (n < (uint32_t)TILE_KEYS) {
        // A ragged tile: the V rows the copy leaves alone meet zero probabilities, so they must
        // hold finite numbers, whatever the stage held before.
        for (uint32_t i = lane; i < 2u * TILE_KEYS * 8u; i += 32) {
            const uint32_t row = (i >> 3) & (TILE_KEYS - 1), sub = i >> 9;
            if (row < r0 || row >= r0 + n)
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(sb + (2 + sub) * SUB_BYTES + row * 128 + (i & 7) * 16), "r"(0u) : "memory");
        }
        __syncwarp();
    }
    if (lane == 0) {
        const uint32_t bar = S.full + 8 * pipe.stage;
        if (block >= P.n_blocks || r0 + n > (uint32_t)TILE_KEYS || n == 0) {
            // Recorded; the copy is skipped and the consumers see stale data.
            if (atomicCAS(&P.status->code, 0, 1) == 0) {
                P.status->where = 200;
                P.status->a = (int)block;
                P.status->b = (int)info;
            }
            mbar_expect_tx(bar, 0);
        } else {
            const uint32_t bytes = n * 128;
            const size_t off = (size_t)block * (PAGE * D * 2) + (size_t)(half * TILE_KEYS + r0) * 128;
            const uint32_t dst = sb + r0 * 128;
            mbar_expect_tx(bar, 4 * bytes);
            if (P.single_use) {
                bulk_g2s_hint(dst, P.k_arena + off, bytes, bar, policy);
                bulk_g2s_hint(dst + SUB_BYTES, P.k_arena + off + PAGE * 128, bytes, bar, policy);
                bulk_g2s_hint(dst + 2 * SUB_BYTES, P.v_arena + off, bytes, bar, policy);
                bulk_g2s_hint(dst + 3 * SUB_BYTES, P.v_arena + off + PAGE * 128, bytes, bar, policy);
            } else {
                bulk_g2s(dst, P.k_arena + off, bytes, bar);
                bulk_g2s(dst + SUB_BYTES, P.k_arena + off + PAGE * 128, bytes, bar);
                bulk_g2s(dst + 2 * SUB_BYTES, P.v_arena + off, bytes, bar);
                bulk_g2s(dst + 3 * SUB_BYTES, P.v_arena + off + PAGE * 128, bytes, bar);
            }
        }
    }
    pipe.advance(STAGES);
    return true;
}

__device__ void produce(const Params &P, const Shared &S, const CtaHdr hdr, int lane) {
    Pipe pipe{0, 0};
    const uint64_t policy = policy_evict_first();
    uint32_t c = hdr.tile_begin;
    // The descriptors of every later tile are on their way while the first two copies start.
    uint2 d = make_uint2(0u, 0u);
    const uint32_t skip = P.has_prologue ? min(2u, hdr.tile_end - hdr.tile_begin) : 0u;
    if (c + skip + lane < hdr.tile_end) d = *(const uint2 *)(P.tiles + c + skip + lane);
    for (uint32_t j = 0; j < skip; j++) {
        const TileDesc t = P.pro[blockIdx.x].first[j];
        if (!issue_tile(P, S, pipe, t.block, t.info, policy, lane)) return;
    }
    c += skip;
    while (c < hdr.tile_end) {
        const int n_tiles = (int)min(32u, hdr.tile_end - c);
        uint2 next = make_uint2(0u, 0u);
        if (c + 32 + lane < hdr.tile_end) next = *(const uint2 *)(P.tiles + c + 32 + lane);
        for (int j = 0; j < n_tiles; j++) {
            const uint32_t block = __shfl_sync(0xffffffffu, d.x, j), info = __shfl_sync(0xffffffffu, d.y, j);
            if (!issue_tile(P, S, pipe, block, info, policy, lane)) return;
        }
        d = next;
        c += 32;
    }
}

// ---- query staging ---------------------------------------------------------------------------
// Row r of a slot is 256 bytes (128 16-bit elements); its sixteen 16-byte chunks are stored at
// (chunk & 8) | ((chunk ^ r) & 7), which lets ldmatrix read A fragments without bank conflicts.
__device__ __forceinline__ uint32_t q_chunk_off(int row, int chunk) {
    return (uint32_t)row * 256u + (uint32_t)(((chunk & 8) | ((chunk ^ row) & 7)) << 4);
}

template <bool BF16>
__device__ __noinline__ void stage_queries(const Params &P, const Shared &S, const CtaHdr hdr, int lane) {
    Pipe pipe{0, 0};
    const bool exact = (P.q_dtype == YX_BF16 && BF16) || (P.q_dtype == YX_F16 && !BF16);
    const int chunk = lane >> 1;
    const uint32_t sub = (lane & 1) * 8;
    for (uint32_t ii = hdr.item_begin; ii < hdr.item_end; ii++) {
        // Lane r < 16 holds pass row r of the item; the first item's come with the parameters.
        uint32_t head_rows, mt, my_row = 0;
        if (ii == hdr.item_begin && P.has_prologue) {
            const CtaPrologue &pr = P.pro[blockIdx.x];
            head_rows = pr.head_rows;
            mt = pr.mt;
            my_row = pr.rows[lane & (MAX_ITEM_ROWS - 1)];
        } else {
            const uint32_t *rec = P.recs[ii].w;
            my_row = rec[IR_ROW0 + IR_ROW_WORDS * (lane & (MAX_ITEM_ROWS - 1)) + IRR_ROW];
            head_rows = rec[IR_HEAD_ROWS];
            mt = rec[IR_MT];
        }
        const int kvh = (int)(head_rows & 0xffffu), n_rows = (int)(head_rows >> 16);
        const int q_rows = n_rows * P.group;
        int stop = 0;
        if (lane == 0) {
            mbar_wait(S.qempty + 8 * pipe.stage, pipe.phase ^ 1u, S.abort_flag, P.status, 3);
            stop = *S.abort_flag;
        }
        if (__shfl_sync(0xffffffffu, stop, 0)) return;
        const uint32_t slot = S.q + pipe.stage * Q_SLOT_BYTES;
        const bool low = mt != 64 && !exact;
        for (int r0 = 0; r0 < (int)mt; r0 += 32) {
            float4 v[32];
#pragma unroll
            for (int k = 0; k < 32; k++) {
                const int qr = r0 + k;
                v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
                const uint32_t row = __shfl_sync(0xffffffffu, my_row, min(qr / P.group, MAX_ITEM_ROWS - 1));
                if (qr < q_rows)
                    v[k] = load4_as_f32(P.q, P.q_dtype, ((size_t)row * P.hq + (size_t)kvh * P.group + qr % P.group) * D + lane * 4);
            }
#pragma unroll
            for (int k = 0; k < 32; k++) {
                const int qr = r0 + k;
                if (qr >= (int)mt) break;
                const uint32_t h0 = pack2<BF16>(v[k].x, v[k].y), h1 = pack2<BF16>(v[k].z, v[k].w);
                const uint32_t addr = slot + q_chunk_off(qr, chunk) + sub;
                asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(h0), "r"(h1) : "memory");
                if (low) {
                    const float2 f0 = unpack2<BF16>(h0), f1 = unpack2<BF16>(h1);
                    const uint32_t l0 = pack2<BF16>(v[k].x - f0.x, v[k].y - f0.y), l1 = pack2<BF16>(v[k].z - f1.x, v[k].w - f1.y);
                    asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr + Q_LOW_OFFSET), "r"(l0), "r"(l1) : "memory");
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(S.qfull + 8 * pipe.stage);
        pipe.advance(Q_SLOTS);
    }
}

// ---- consumers ---------------------------------------------------------------------------------
// Word `idx` (32..127) of an item record held as three lane-indexed registers.
__device__ __forceinline__ uint32_t rec_word(uint32_t w1, uint32_t w2, uint32_t w3, int idx) {
    const uint32_t a = __shfl_sync(0xffffffffu, w1, idx & 31), b = __shfl_sync(0xffffffffu, w2, idx & 31),
                   c = __shfl_sync(0xffffffffu, w3, idx & 31);
    return idx < 64 ? a : (idx < 96 ? b : c);
}

// Merges every (row, KV head) of an item that the arrival counters found complete.  The
// completed (row, head) pairs are dealt to the warps, four at a time per warp, so that their
// loads overlap: a merge is two dependent round trips to L2, whatever it merges.
__device__ __noinline__ void merge_completed(const Params &P, const int *flags, uint32_t w1, uint32_t w2, uint32_t w3,
                                             int n_rows, int kvh, int warp, int lane) {
    const int group = P.group;
    int n_done = 0;
    uint32_t done_mask = 0;
    for (int r = 0; r < n_rows; r++)
        if (flags[r]) {
            done_mask |= 1u << r;
            n_done++;
        }
    if (n_done) {
        __threadfence();
        const int n_tasks = n_done * group;
        for (int t0 = warp * 4; t0 < n_tasks; t0 += CONSUMERS * 4) {
            uint32_t rows_[4], first_[4], count_[4];
            int hg_[4];
            bool on_[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int t = t0 + k;
                on_[k] = t < n_tasks;
                const int which = on_[k] ? t / group : 0;   // which completed row
                hg_[k] = on_[k] ? t % group : 0;
                // the which-th set bit of done_mask
                uint32_t mk = done_mask;
                for (int x = 0; x < which; x++) mk &= mk - 1;
                const int r = __ffs(mk) - 1;
                const int base = IR_ROW0 + IR_ROW_WORDS * r;
                rows_[k] = rec_word(w1, w2, w3, base + IRR_ROW);
                first_[k] = rec_word(w1, w2, w3, base + IRR_FIRST);
                count_[k] = rec_word(w1, w2, w3, base + IRR_COUNT);
            }
            float mx[4], ls[4];
            float4 acc[4];
            merge_parts4(P.part_o, P.part_ml, first_, count_, on_, group, hg_, lane, mx, ls, acc);
#pragma unroll
            for (int k = 0; k < 4; k++) {
                if (!on_[k]) continue;
                const size_t idx = (size_t)rows_[k] * P.hq + (size_t)kvh * group + hg_[k];
                if (P.out) {
                    const float inv = 1.0f / ls[k];   // a row always sees its own key: > 0 for whole attention
                    store4(P.out, P.out_dtype, idx * D + lane * 4,
                           make_float4(acc[k].x * inv, acc[k].y * inv, acc[k].z * inv, acc[k].w * inv));
                }
                if (P.o_out) {
                    *(float4 *)(P.o_out + idx * D + lane * 4) = acc[k];
                    if (lane == 0) {
                        P.m_out[idx] = mx[k];
                        P.l_out[idx] = ls[k];
                    }
                }
            }
        }
    }
}

template <int MT, bool BF16>
__device__ void consume_item(const Params &P, const Shared &S, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3,
                             Pipe &pipe, Pipe &qpipe, int warp, int lane) {
    constexpr int NMT = MT / 16;          // 16-row tiles of queries
    constexpr int NSL = CONSUMERS / NMT;  // key slices of a tile
    constexpr int KS = TILE_KEYS / NSL;   // keys per slice
    constexpr int NT = KS / 8;            // 8-key score tiles per warp
    constexpr bool LOW = MT != 64;        // f32 queries carry a low part (not for 64-row items)
    const int mi = warp % NMT, sl = warp / NMT;
    const int g = lane >> 2, t4 = lane & 3;
    const int group = P.group;
    const uint32_t n_tiles = field(w0, IR_TILES), key_base = field(w0, IR_KEY0);
    const uint32_t head_rows = field(w0, IR_HEAD_ROWS);
    const int kvh = (int)(head_rows & 0xffffu), n_rows = (int)(head_rows >> 16);
    const int q_rows = n_rows * group;
    const float sl2 = 0.08838834764831845f * 1.4426950408889634f;   // log2(e) / sqrt(128)
    const bool exact_q = !LOW || (P.q_dtype == YX_BF16 && BF16) || (P.q_dtype == YX_F16 && !BF16);

    // The two query rows this thread owns in the accumulator fragments.
    uint32_t klo[2], khi[2], part[2];
    bool valid[2];
#pragma unroll
    for (int rs = 0; rs < 2; rs++) {
        const int qr = mi * 16 + g + rs * 8;
        valid[rs] = qr < q_rows;
        const int base = IR_ROW0 + IR_ROW_WORDS * (valid[rs] ? qr / group : 0);
        const uint32_t a = rec_word(w1, w2, w3, base + IRR_KLO), b = rec_word(w1, w2, w3, base + IRR_KHI);
        part[rs] = rec_word(w1, w2, w3, base + IRR_PART);
        klo[rs] = valid[rs] ? a : 0u;            // padded rows: zero queries, nothing masked
        khi[rs] = valid[rs] ? b : 0xffffffffu;
    }

    // Query fragments from the staged slot.
    uint32_t qh[8][4], ql[LOW ? 8 : 1][4];
    {
        mbar_wait(S.qfull + 8 * qpipe.stage, qpipe.phase, S.abort_flag, P.status, 4);
        const uint32_t slot = S.q + qpipe.stage * Q_SLOT_BYTES;
        const int row = mi * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
            const uint32_t a = slot + q_chunk_off(row, 2 * ks + (lane >> 4));
            ldsm4(a, qh[ks][0], qh[ks][1], qh[ks][2], qh[ks][3]);
            if constexpr (LOW) {
                if (!exact_q) ldsm4(a + Q_LOW_OFFSET, ql[ks][0], ql[ks][1], ql[ks][2], ql[ks][3]);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(S.qempty + 8 * qpipe.stage);
        qpipe.advance(Q_SLOTS);
    }

    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    const int lm = lane >> 3, lr = lane & 7;
    for (uint32_t ti = 0; ti < n_tiles; ti++) {
        mbar_wait(S.full + 8 * pipe.stage, pipe.phase, S.abort_flag, P.status, 2);
        if (P.trace && threadIdx.x == 0 && P.trace[8 * blockIdx.x + 3] == 0) P.trace[8 * blockIdx.x + 3] = gtime();
        const uint32_t sb = S.stages + pipe.stage * STAGE_BYTES;

        // S = Q K^T over this warp's KS keys.  The low parts of the queries accumulate on their
        // own, so that no MMA waits on more than the eight before it in its chain.
        float s[NT][4], s2[LOW ? NT : 1][4];
#pragma unroll
        for (int j = 0; j < NT; j++) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        if constexpr (LOW) {
#pragma unroll
            for (int j = 0; j < NT; j++) s2[j][0] = s2[j][1] = s2[j][2] = s2[j][3] = 0.f;
        }
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
            const uint32_t sub = sb + (ks >> 2) * SUB_BYTES;
            const int c = ((2 * ks) & 7) + (lm & 1);
#pragma unroll
            for (int np = 0; np < NT / 2; np++) {
                const int key = sl * KS + np * 16 + (lm >> 1) * 8 + lr;
                uint32_t b0, b1, b2, b3;
                ldsm4(sub + key * 128 + ((c ^ lr) << 4), b0, b1, b2, b3);
                mma16816<BF16>(s[2 * np], qh[ks], b0, b1);
                mma16816<BF16>(s[2 * np + 1], qh[ks], b2, b3);
                if constexpr (LOW) {
                    if (!exact_q) {
                        mma16816<BF16>(s2[2 * np], ql[ks], b0, b1);
                        mma16816<BF16>(s2[2 * np + 1], ql[ks], b2, b3);
                    }
                }
            }
        }
        if constexpr (LOW) {
#pragma unroll
            for (int j = 0; j < NT; j++)
#pragma unroll
                for (int e = 0; e < 4; e++) s[j][e] += s2[j][e];
        }
        // Mask keys outside each row's [klo, khi].
        const uint32_t key0 = key_base + ti * TILE_KEYS + sl * KS + 2 * t4;
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const uint32_t key = key0 + j * 8 + (e & 1);
                const int rs = e >> 1;
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
            const float mn = fmaxf(m[rs], mx);
            const float mu = mn == -INFINITY ? 0.f : mn;
            const float alpha = exp2f((m[rs] - mu) * sl2);
            m[rs] = mn;
            float sum = 0.f;
            const float ms = mu * sl2;
#pragma unroll
            for (int j = 0; j < NT; j++) {
                const float p0 = exp2f(s[j][2 * rs] * sl2 - ms), p1 = exp2f(s[j][2 * rs + 1] * sl2 - ms);
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
                    const float2 hf = unpack2<BF16>(a[r]);
                    al[r] = pack2<BF16>(p0 - hf.x, p1 - hf.y);
                }
            }
            const int key = sl * KS + kk * 16 + (lm & 1) * 8 + lr;
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
        pipe.advance(STAGES);
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
                const int r = g + rs * 8;
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
                const int r = g + rs * 8;
                float mx = m[rs];
#pragma unroll
                for (int x = 1; x < NSL; x++) mx = fmaxf(mx, scratch[((x - 1) * NMT + mi) * MERGE_FLOATS + r]);
                const float mu = mx == -INFINITY ? 0.f : mx;
                const float f = exp2f((m[rs] - mu) * sl2);
                l[rs] *= f;
#pragma unroll
                for (int n = 0; n < 16; n++) {
                    o[n][2 * rs] *= f;
                    o[n][2 * rs + 1] *= f;
                }
#pragma unroll
                for (int x = 1; x < NSL; x++) {
                    const float *w = scratch + ((x - 1) * NMT + mi) * MERGE_FLOATS;
                    const float fx = exp2f((w[r] - mu) * sl2);
                    l[rs] += w[16 + r] * fx;
#pragma unroll
                    for (int n = 0; n < 16; n++) {
                        const float2 v = *(const float2 *)(w + 32 + r * D + n * 8 + 2 * t4);
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
            const int qr = mi * 16 + g + rs * 8;
            const size_t slot = (size_t)part[rs] * group + (qr % group);
            float *po = P.part_o + slot * D;
#pragma unroll
            for (int n = 0; n < 16; n++) __stcg((float2 *)(po + n * 8 + 2 * t4), make_float2(o[n][2 * rs], o[n][2 * rs + 1]));
            if (t4 == 0) {
                const bool none = m[rs] == -INFINITY;
                __stcg((float2 *)(P.part_ml + slot * 2), make_float2(none ? -1e30f : m[rs] * 0.08838834764831845f, none ? 0.f : l[rs]));
            }
        }
        __threadfence();   // the triples are visible device-wide before this item is counted
    }
    asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory");

    // Fused merge: count this item in for each of its (row, KV head); whoever completes one
    // merges all of its triples and writes the result.
    int *flags = (int *)__cvta_shared_to_generic((size_t)S.flags);
    if (warp == 0) {
        // every lane takes part in the shuffles of rec_word; lanes beyond n_rows ignore theirs
        const int base = IR_ROW0 + IR_ROW_WORDS * min(lane, MAX_ITEM_ROWS - 1);
        const uint32_t row = rec_word(w1, w2, w3, base + IRR_ROW), count = rec_word(w1, w2, w3, base + IRR_COUNT);
        if (lane < n_rows) {
            uint32_t *ctr = P.counters + (size_t)row * P.hkv + kvh;
            const uint32_t old = atomicAdd(ctr, 1u);
            const bool last = old + 1 == count;
            if (last) *ctr = 0u;   // nobody else touches it in this launch: left clean for the next
            flags[lane] = last ? 1 : 0;
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory");
    merge_completed(P, flags, w1, w2, w3, n_rows, kvh, warp, lane);
    // `flags` and the merge scratch are rewritten only after the next item's barriers.
}

template <bool BF16>
__global__ void __launch_bounds__(THREADS, 1) attend_mma_kernel(const __grid_constant__ Params P) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ int abort_flag;
    Shared S;
    S.stages = smem_u32(smem);
    S.q = S.stages + STAGES * STAGE_BYTES;
    S.merge = S.q + Q_SLOTS * Q_SLOT_BYTES;
    S.flags = S.merge + MERGE_BYTES;
    S.full = S.flags + 128;
    S.empty = S.full + 8 * STAGES;
    S.qfull = S.empty + 8 * STAGES;
    S.qempty = S.qfull + 8 * Q_SLOTS;
    S.abort_flag = &abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned long long *tr = P.trace ? P.trace + 8 * blockIdx.x : nullptr;
    if (tr && threadIdx.x == 0) tr[0] = gtime();
    const CtaHdr hdr = P.has_prologue ? P.pro[blockIdx.x].hdr : *(const CtaHdr *)(P.cta_hdr + blockIdx.x);
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; s++) {
            mbar_init(S.full + 8 * s, 1);
            mbar_init(S.empty + 8 * s, CONSUMERS);
        }
        for (int s = 0; s < Q_SLOTS; s++) {
            mbar_init(S.qfull + 8 * s, 1);
            mbar_init(S.qempty + 8 * s, CONSUMERS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (tr && threadIdx.x == 0) {
        tr[1] = gtime();
        tr[7] = hdr.item_end - hdr.item_begin;
    }

    if (warp == PRODUCER) {
        produce(P, S, hdr, lane);
        if (tr && lane == 0) tr[6] = gtime();
        return;
    }
    if (warp == QWARP) {
        stage_queries<BF16>(P, S, hdr, lane);
        return;
    }
    Pipe pipe{0, 0}, qpipe{0, 0};
    uint32_t n0 = 0, n1 = 0, n2 = 0, n3 = 0;
    if (hdr.item_begin < hdr.item_end) {
        const uint32_t *r = P.recs[hdr.item_begin].w;
        n0 = r[lane], n1 = r[32 + lane], n2 = r[64 + lane], n3 = r[96 + lane];
    }
    for (uint32_t ii = hdr.item_begin; ii < hdr.item_end; ii++) {
        const uint32_t w0 = n0, w1 = n1, w2 = n2, w3 = n3;
        if (ii + 1 < hdr.item_end) {   // in flight while this item runs
            const uint32_t *r = P.recs[ii + 1].w;
            n0 = r[lane], n1 = r[32 + lane], n2 = r[64 + lane], n3 = r[96 + lane];
        }
        if (tr && threadIdx.x == 0 && ii == hdr.item_begin) tr[2] = gtime();
        switch (field(w0, IR_MT)) {
            case 16: consume_item<16, BF16>(P, S, w0, w1, w2, w3, pipe, qpipe, warp, lane); break;
            case 32: consume_item<32, BF16>(P, S, w0, w1, w2, w3, pipe, qpipe, warp, lane); break;
            default: consume_item<64, BF16>(P, S, w0, w1, w2, w3, pipe, qpipe, warp, lane); break;
        }
        if (tr && threadIdx.x == 0 && ii == hdr.item_begin) tr[4] = gtime();
    }
    if (tr && threadIdx.x == 0) tr[5] = gtime();
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
    P.n_blocks = a.kv_pages * (uint32_t)a.hkv;
    P.cta_hdr = a.cta_hdr;
    P.tiles = a.tiles;
    P.recs = a.recs;
    P.single_use = a.single_use ? 1 : 0;
    P.part_o = a.part_o;
    P.part_ml = a.part_ml;
    P.counters = a.counters;
    P.out = a.out;
    P.out_dtype = a.out_dtype;
    P.m_out = a.m_out;
    P.l_out = a.l_out;
    P.o_out = a.o_out;
    P.status = ctx->dev_status;
    P.trace = (unsigned long long *)ctx->trace_buf;
    P.has_prologue = 0;
    if (a.plan && a.n_ctas <= MAX_PROLOGUE_CTAS) {
        const Plan &pl = *a.plan;
        P.has_prologue = 1;
        for (int c = 0; c < a.n_ctas; c++) {
            CtaPrologue &pr = P.pro[c];
            pr.hdr = pl.cta_hdr[c];
            for (uint32_t j = 0; j < 2 && pr.hdr.tile_begin + j < pr.hdr.tile_end; j++) pr.first[j] = pl.tiles[pr.hdr.tile_begin + j];
            if (pr.hdr.item_begin < pr.hdr.item_end) {
                const Item &it = pl.items[pr.hdr.item_begin];
                pr.head_rows = (uint32_t)it.kv_head | ((uint32_t)it.n_rows << 16);
                pr.mt = it.mt;
                for (int r = 0; r < MAX_ITEM_ROWS; r++) pr.rows[r] = it.rows[r];
            }
        }
    }
    if (bf16) attend_mma_kernel<true><<<a.n_ctas, THREADS, SMEM_BYTES, ctx->stream>>>(P);
    else attend_mma_kernel<false><<<a.n_ctas, THREADS, SMEM_BYTES, ctx->stream>>>(P);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "attend_mma kernel");
}

}  // namespace yx
