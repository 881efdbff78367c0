// Split-key (flash-decoding) attention for 16-bit KV caches: batched decode, speculative
// verification and rows over shared prefixes.  Bandwidth-bound: the job of this kernel is to
// keep every SM's share of HBM busy from the first microsecond to the last.
//
//  * Persistent: one CTA to an SM (by default one SM is left without, for the call behind),
//    eleven warps (eight consumers, a producer, a query stager, an epilogue warp); a CTA walks
//    the span of 64-key tiles the planner cut for it.
//  * Nothing on the device walks a page table.  The host planner resolves every tile to its
//    (page, KV head) block; the producer warp reads 32 tile descriptors with one coalesced
//    load and feeds the copy engine from them, across item boundaries, never draining.
//  * K and V tiles come in by bulk asynchronous copies (`cp.async.bulk`, the TMA engine's
//    untiled form) that complete on mbarriers.  The cache layout (yx_internal.h) makes a tile
//    four contiguous runs that land already 128-byte swizzled, so no tensor map is needed and
//    the copy of a ragged tile is simply shorter.  Tiles that no other item reads are copied
//    with an L2 evict-first hint, so that the stream does not push the plan, the queries and
//    the partial results out of L2.
//  * The CTA's first tiles and the rows of its first item ride in kernel-parameter space, and the
//    producer warp sets up the barriers and starts those copies before the CTA's first
//    __syncthreads: nothing on the way to the first byte waits on a global load.
//  * The kernel is launched as a programmatic dependent of the kernel before it.  K/V tiles
//    that kernel cannot have written (everything but the tiles holding this pass's new rows,
//    which the planner marks) are copied before the grid dependency is waited for, so a CTA
//    that starts while the previous kernel's last CTAs still run has its ring full when the
//    wait returns.  Queries, partial results and marked tiles are touched only after the wait.
//  * Queries come in by bulk copies too: the stager warp issues one copy per query row of the
//    next item (raw, in the caller's type) plus one for the item's record; the consumer warps
//    build their MMA fragments from the raw rows (f32 queries as a high and a low 16-bit part).
//  * Eight consumer warps share each tile.  All query heads of the KV head's group, and all
//    rows of an item, are columns of `mma.sync` tiles, so a K or V byte is read once per item
//    however many heads and rows use it.  Scores and softmax stay in f32 registers.
//  * Each item ends in an (m, l, o) triple per query row, the format of the reference's
//    split attention (crates/yaxus-backend-gpu/src/shaders.rs:1466-1579).  The epilogue warp
//    writes the triples while the consumers are already in the next item.  The merge of the
//    triples (the reference's `attn_combine`, shaders.rs:1581-1637) is the combine kernel's,
//    or, when asked for, this kernel's own: the CTA that delivers the last triple of a
//    (row, KV head) merges them and writes the output, found by an arrival counter in global
//    scratch that the merging CTA resets.
//  * When the kernels ahead on the stream are another split-key call of the same context and its
//    merge (a decode loop over layers with nothing between the calls), keys, values, queries
//    and the plan are all long written: the kernel then reads at once and waits for the grid
//    dependency only before its first write, of the partial buffers the merge ahead still
//    reads.  Calls then overlap SM by SM: a CTA starts when the CTA of the call before leaves
//    its SM, and the merge runs beside it.  A kernel says "launch my dependents" only once
//    everything ahead of it is complete (at its top in this mode, after its wait otherwise), which
//    is what makes the early reads of the call behind it safe.
//  * 152 registers per thread and eleven warps.  The register file is four partitions of 16384;
//    a partition holds three of this CTA's warps (3 x 152 x 32 = 14592), which leaves 1792: one
//    warp of the merge kernel (48 x 32 = 1536).  So a CTA of the merge kernel (four warps, one per
//    partition) is resident beside this one, and the merge kernel and, behind it, the next
//    attention call are resident before this call has finished.  At 168 registers the sum over the
//    SM still fits but no partition has room, and the merge CTAs then wait for these CTAs to leave
//    and keep the next call's CTAs out in their turn (measured: 23.3 us a call against 20.1).
//
// Every wait on an mbarrier is bounded: on expiry the CTA records the failure in the
// context's status word, stops waiting anywhere, waits (bounded) for the copies it has in
// flight, and returns.
#include <stddef.h>
#include <string.h>

#include "yx_device.cuh"

namespace yx {
namespace {

using namespace dev;

constexpr int STAGES = 5;
constexpr int SUB_BYTES = TILE_KEYS * 128;        // one 64-dim half of a 64-key tile
constexpr int STAGE_BYTES = 4 * SUB_BYTES;        // K lo, K hi, V lo, V hi
constexpr int CONSUMERS = 8;                      // warps 0..7, two per scheduler
constexpr int PRODUCER = CONSUMERS;               // warp 8
constexpr int QWARP = CONSUMERS + 1;              // warp 9
constexpr int EWARP = CONSUMERS + 2;              // warp 10
constexpr int EWARPS = 1;
constexpr int THREADS = (CONSUMERS + 2 + EWARPS) * 32;
constexpr int CONSUMER_BARRIER = 1;               // named barriers (0 is __syncthreads')
constexpr int SETUP_BARRIER = 2;
constexpr int Q_SLOTS = 2;
// A slot holds the item's query rows as they are in global memory, one bulk copy per row, each
// row padded so that the fragment loads of a warp fall in different banks: 32 rows of 128 f32
// (512 + 32 bytes) or 64 rows of 128 16-bit elements (256 + 16 bytes).
constexpr int Q_STRIDE_F32 = 512 + 32;
constexpr int Q_STRIDE_16 = 256 + 16;
constexpr int Q_ROWS_BYTES = 32 * Q_STRIDE_F32;
static_assert(Q_ROWS_BYTES == 64 * Q_STRIDE_16, "both query forms fill the slot");
// The query rows have one buffer: the consumer warps turn them into MMA fragments in registers at
// the start of an item and hand the buffer back at once, so the next item's rows are copied while
// this item's tiles stream.  The items' records, which are read to the end of an item, have two
// slots.  (Two full query slots cost a fifth copy stage; one slot held for the whole item cost a
// bubble at every item change.)
constexpr int REC_BYTES = 512;
constexpr int MERGE_ROW = D + 4;                  // one row's o, then m and l, padded
constexpr int MERGE_FLOATS = 8 * MERGE_ROW;       // one warp's 8 queries
constexpr int MERGE_BYTES = CONSUMERS * MERGE_FLOATS * 4;   // one buffer: every consumer warp's rows
constexpr int MERGE_BUFS = 1;
constexpr int N_BARRIERS = 2 * STAGES + 2 * Q_SLOTS + 2 * MERGE_BUFS + 1;
constexpr int MLBUF_BYTES = EWARPS * 8 * 32 * 8;  // per epilogue warp: (m, l) of 32 parts for each of 8 merges in flight
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + Q_ROWS_BYTES + Q_SLOTS * REC_BYTES + MERGE_BUFS * MERGE_BYTES + N_BARRIERS * 8 + MLBUF_BYTES;
static_assert(SMEM_BYTES + 1024 <= 227 * 1024, "the CTA's shared memory");

struct Shared {
    uint32_t stages, q, rec, merge;     // shared-space addresses
    uint32_t full, empty, qfull, qempty, qrows_free, efull, eempty, mlbuf;
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

constexpr int MAX_PROLOGUE_CTAS = 160;
#ifndef YX_FAST_TILES
#define YX_FAST_TILES 2   // tiles of a CTA issued by the short way (a call with its merge: 19.7 us with one, 19.5 with two, 20.5 with three, 22.1 with four)
#endif

struct Params {
    const void *q;
    int q_dtype, hq, group, hkv;
    const char *k_arena, *v_arena;
    uint32_t n_blocks;               // (page, kv head) blocks in an arena
    const CtaHdr *cta_hdr;
    const TileDesc *tiles;
    const char *recs;                // item records, rec_stride bytes apart
    uint32_t rec_stride;
    int single_use;
    float *part_o, *part_ml;
    uint32_t *counters;
    void *out;
    int out_dtype;
    float *m_out, *l_out, *o_out;
    yx_dev_status *status;
    unsigned long long *trace;       // optional: 16 timestamps / counters per CTA
    int fused;                       // merge in this kernel (arrival counters) or leave it to the combine kernel
    int n_stages;                    // stages of the ring in use (2..STAGES): bytes in flight per SM
    int early_kv;                    // tiles not marked TILE_FRESH may be copied before the grid dependency wait
    int late_wait;                   // nothing this kernel reads can still be written: only its writers wait
    int wait_at_end;                 // ... and they do so before the CTA leaves, not before its first write
    uint32_t n_items, n_tiles, n_parts;   // sizes of the plan's arrays and of the partial buffers, for the kernel's own checks
    unsigned long long q_bytes;      // size of the query tensor
    int has_prologue;
    CtaPrologue pro[MAX_PROLOGUE_CTAS];
};

// ---- producer: tile descriptors -> bulk copies ----------------------------------------------
// A failed check of the kernel's own index arithmetic: recorded (first one wins), the access skipped.
__device__ __noinline__ void record_bad_index(yx_dev_status *status, int where, unsigned long long a, unsigned long long b) {
    if (atomicCAS(&status->code, 0, 3) == 0) {
        status->where = where;
        status->a = (int)a;
        status->b = (int)b;
    }
}

__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// After a wait has run out: the copies already issued into this CTA's shared memory must have
// landed before the CTA may leave.  `full` are the barriers they complete on; the stages before
// `pipe.stage` were last issued in phase `pipe.phase`, the others one phase earlier.
__device__ __noinline__ void drain_copies(uint32_t full, int n, Pipe pipe) {
    for (int s = 0; s < n; s++) {
        // (a barrier never used reads as complete for the phase before its first)
        const uint32_t parity = s < pipe.stage ? pipe.phase : (pipe.phase ^ 1u);
        const long long t0 = clock64();
        while (!mbar_try(full + 8 * s, parity) && clock64() - t0 < 4000000ll) {
        }
    }
}

// One tile: wait for a free stage, zero what a ragged copy leaves alone, start the four copies.
// Returns false when the CTA has given up.
struct Issue {
    const char *k_arena, *v_arena;
    yx_dev_status *status;
    volatile int *abort_flag;
    uint64_t policy;
    uint32_t n_blocks, stages, full, empty;
    int single_use, n_stages;
};
// (By value: a reference would turn every field access of this out-of-line routine into a load.)
__device__ __noinline__ bool issue_tile(const Issue P, Pipe &pipe, uint32_t block, uint32_t info, int lane) {
    const uint32_t half = info & 1u, r0 = (info >> 1) & 127u, n = (info >> 8) & 255u;
    int stop = 0;
    if (lane == 0) {
        mbar_wait(P.empty + 8 * pipe.stage, pipe.phase ^ 1u, P.abort_flag, P.status, 1);
        stop = *P.abort_flag;
    }
    if (__shfl_sync(0xffffffffu, stop, 0)) return false;
    const uint32_t sb = P.stages + pipe.stage * STAGE_BYTES;
    if (n < (uint32_t)TILE_KEYS) {
        // A ragged tile: the V rows the copy leaves alone meet zero probabilities, so they must
        // hold finite numbers, whatever the stage held before.
        for (uint32_t i = lane; i < 2u * TILE_KEYS * 8u; i += 32) {
            const uint32_t row = (i >> 3) & (TILE_KEYS - 1), sub = i >> 9;
            if (row < r0 || row >= r0 + n)
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(sb + (2 + sub) * SUB_BYTES + row * 128 + (i & 7) * 16), "r"(0u) : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
    }
    if (lane == 0) {
        const uint32_t bar = P.full + 8 * pipe.stage;
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
            if (P.single_use && !(info & TILE_REUSED)) {
                bulk_g2s_hint(dst, P.k_arena + off, bytes, bar, P.policy);
                bulk_g2s_hint(dst + SUB_BYTES, P.k_arena + off + PAGE * 128, bytes, bar, P.policy);
                bulk_g2s_hint(dst + 2 * SUB_BYTES, P.v_arena + off, bytes, bar, P.policy);
                bulk_g2s_hint(dst + 3 * SUB_BYTES, P.v_arena + off + PAGE * 128, bytes, bar, P.policy);
            } else {
                bulk_g2s(dst, P.k_arena + off, bytes, bar);
                bulk_g2s(dst + SUB_BYTES, P.k_arena + off + PAGE * 128, bytes, bar);
                bulk_g2s(dst + 2 * SUB_BYTES, P.v_arena + off, bytes, bar);
                bulk_g2s(dst + 3 * SUB_BYTES, P.v_arena + off + PAGE * 128, bytes, bar);
            }
        }
    }
    pipe.advance(P.n_stages);
    return true;
}

// The producer warp's life after it has set the barriers up: the first tiles out of parameter
// space, then the rest of the span from the descriptor array.
__device__ void produce(const Params &P, const Shared &S, const CtaHdr hdr, int lane) {
    Pipe pipe{0, 0};
    Issue I;
    I.k_arena = P.k_arena;
    I.v_arena = P.v_arena;
    I.status = P.status;
    I.abort_flag = S.abort_flag;
    I.policy = policy_evict_first();
    I.n_blocks = P.n_blocks;
    I.stages = S.stages;
    I.full = S.full;
    I.empty = S.empty;
    I.single_use = P.single_use;
    I.n_stages = P.n_stages;
    // Until the grid dependency has been waited for, only tiles that the kernel ahead of this one
    // cannot have written are copied; the first marked tile makes the warp wait.
    bool waited = P.late_wait != 0;
    if (!P.early_kv && !waited) {
        grid_dependency_wait();
        waited = true;
    }
    auto gate = [&](uint32_t info) {
        if (!waited && (info & TILE_FRESH)) {
            grid_dependency_wait();
            waited = true;
        }
    };
    bool alive = true;
    uint32_t c = hdr.tile_begin;
    const uint32_t skip = P.has_prologue ? min(min((uint32_t)PROLOGUE_TILES, (uint32_t)P.n_stages), hdr.tile_end - hdr.tile_begin) : 0u;
    for (uint32_t j = 0; j < skip && alive; j++) {
        const TileDesc t = P.pro[blockIdx.x].first[j];
        if (YX_TR(P.trace != nullptr) && lane == 0 && j == 0) P.trace[16 * blockIdx.x + 15] = gtime() + (t.block & 1u);
        gate(t.info);
        // The CTA's very first tiles go out by the shortest way there is: their stages have never
        // been used (nothing to wait for) and a whole tile needs no zeroing.
        const uint32_t half = t.info & 1u, r0 = (t.info >> 1) & 127u, n = (t.info >> 8) & 255u;
        if (j < YX_FAST_TILES && n == (uint32_t)TILE_KEYS && r0 == 0u && t.block < P.n_blocks && pipe.phase == 0u) {
            if (lane == 0) {
                const uint32_t bar = S.full + 8 * pipe.stage, dst = S.stages + pipe.stage * STAGE_BYTES;
                const size_t off = (size_t)t.block * (PAGE * D * 2) + (size_t)(half * TILE_KEYS) * 128;
                mbar_expect_tx(bar, 4 * SUB_BYTES);
                if (P.single_use && !(t.info & TILE_REUSED)) {
                    bulk_g2s_hint(dst, P.k_arena + off, SUB_BYTES, bar, I.policy);
                    bulk_g2s_hint(dst + SUB_BYTES, P.k_arena + off + PAGE * 128, SUB_BYTES, bar, I.policy);
                    bulk_g2s_hint(dst + 2 * SUB_BYTES, P.v_arena + off, SUB_BYTES, bar, I.policy);
                    bulk_g2s_hint(dst + 3 * SUB_BYTES, P.v_arena + off + PAGE * 128, SUB_BYTES, bar, I.policy);
                } else {
                    bulk_g2s(dst, P.k_arena + off, SUB_BYTES, bar);
                    bulk_g2s(dst + SUB_BYTES, P.k_arena + off + PAGE * 128, SUB_BYTES, bar);
                    bulk_g2s(dst + 2 * SUB_BYTES, P.v_arena + off, SUB_BYTES, bar);
                    bulk_g2s(dst + 3 * SUB_BYTES, P.v_arena + off + PAGE * 128, SUB_BYTES, bar);
                }
            }
            pipe.advance(P.n_stages);
        } else {
            alive = issue_tile(I, pipe, t.block, t.info, lane);
        }
        if (YX_TR(P.trace != nullptr) && lane == 0 && j == 0) P.trace[16 * blockIdx.x + 2] = gtime();
    }
    c += skip;
    // The descriptors of every later tile.
    uint2 d = make_uint2(0u, 0u);
    if (hdr.tile_end > P.n_tiles) {   // the kernel's own check of its span
        if (lane == 0) record_bad_index(P.status, 305, hdr.tile_end, P.n_tiles);
        alive = false;
    }
    if (alive && c + lane < hdr.tile_end) d = *(const uint2 *)(P.tiles + c + lane);
    while (alive && c < hdr.tile_end) {
        const int n_tiles = (int)min(32u, hdr.tile_end - c);
        uint2 next = make_uint2(0u, 0u);
        if (c + 32 + lane < hdr.tile_end) next = *(const uint2 *)(P.tiles + c + 32 + lane);
        for (int j = 0; j < n_tiles && alive; j++) {
            const uint32_t block = __shfl_sync(0xffffffffu, d.x, j), info = __shfl_sync(0xffffffffu, d.y, j);
            gate(info);
            alive = issue_tile(I, pipe, block, info, lane);
        }
        d = next;
        c += 32;
    }
    if (!alive && lane == 0) drain_copies(S.full, P.n_stages, pipe);
}

// ---- query staging ---------------------------------------------------------------------------
// (Inlined into the kernel.  As an out-of-line routine that took this structure by value, the way
// issue_tile and epilogue_loop take theirs, it was never entered by the stager warp on sm_100a
// with CUDA 12.9 - the time stamps of a diagnostic build showed the warp reach the call and
// nothing after it - and the consumers waited for their queries until the wait ran out.)
struct QStage {
    const char *q;
    const char *recs;
    uint32_t rec_stride;
    yx_dev_status *status;
    int hq, group;
    uint32_t row_bytes, stride;           // of one query row in global and in shared memory
    uint32_t item_begin, item_end;
    int have_first;                       // the first item's header came with the parameters
    uint32_t first_head_rows, first_row0, first_row1;   // first_row<h>: the pass row of query row 32 h + lane
    uint32_t qbase, recbase, qfull, qempty, qrows_free;   // shared-space addresses
    volatile int *abort_flag;
    uint32_t n_items;                     // records in `recs`
    unsigned long long q_bytes;           // bytes in `q`
    unsigned long long *trace;            // this CTA's time stamps (diagnostic build), or null
};

// One bulk copy per query row, issued by the lane of the same index (and the lane again for
// rows 32..63), plus one for the item's record.  The rows and the head of the next item are
// fetched into registers as soon as the current item's copies are on their way, so that when
// its slot comes free only the copies remain to be started.
__device__ __forceinline__ void stage_queries(const QStage &A, int lane) {
    Pipe pipe{0, 0};
    uint32_t head_rows = 0, prow[2] = {0, 0};
    auto fetch = [&](uint32_t ii) {
        if (ii == A.item_begin && A.have_first) {
            head_rows = A.first_head_rows;
            prow[0] = A.first_row0;
            prow[1] = A.first_row1;
            return;
        }
        if (ii >= A.n_items) {
            head_rows = 0;
            return;
        }
        const uint32_t *rec = (const uint32_t *)(A.recs + (size_t)ii * A.rec_stride);
        head_rows = __ldg(rec + IR_HEAD_ROWS);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int r = min((32 * h + lane) / A.group, MAX_ITEM_ROWS - 1);
            prow[h] = __ldg(rec + IR_ROW0 + IR_ROW_WORDS * r + IRR_ROW);
        }
    };
    if (A.item_begin < A.item_end) fetch(A.item_begin);
    if (YX_TR(A.trace != nullptr) && lane == 0) A.trace[8] = gtime();
    bool alive = true;
#pragma unroll 1
    for (uint32_t ii = A.item_begin; ii < A.item_end; ii++) {
        int stop = 0;
        if (lane == 0) {
            mbar_wait(A.qempty + 8 * pipe.stage, pipe.phase ^ 1u, A.abort_flag, A.status, 3);
            // ... and the rows buffer: the consumers have built the fragments of the item before
            // (one phase an item; a barrier never used reads as complete for the phase before its first)
            mbar_wait(A.qrows_free, ((ii - A.item_begin) & 1u) ^ 1u, A.abort_flag, A.status, 7);
            stop = *A.abort_flag;
        }
        if (__shfl_sync(0xffffffffu, stop, 0)) {
            alive = false;
            break;
        }
        if (YX_TR(A.trace != nullptr) && lane == 0 && ii == A.item_begin) A.trace[9] = gtime();
        const uint32_t slot = A.qbase, rec_slot = A.recbase + pipe.stage * REC_BYTES, bar = A.qfull + 8 * pipe.stage;
        const int kvh = (int)(head_rows & 0xffffu);
        int q_rows = (int)(head_rows >> 16) * A.group;
        // The kernel's own checks: a record outside the array, more query rows than a slot holds, a
        // query row outside the tensor.  Recorded; the copy is left out (the barrier still completes).
        const bool rec_ok = ii < A.n_items;
        if (q_rows > 64 || (A.row_bytes == 512u && q_rows > 32)) {
            if (lane == 0) record_bad_index(A.status, 301, (unsigned long long)q_rows, ii);
            q_rows = 0;
        }
        size_t elem[2] = {0, 0};
        bool ok[2] = {false, false};
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int qr = 32 * h + lane;
            if (qr < q_rows) {
                const int r = qr / A.group, g = qr - r * A.group;
                elem[h] = (size_t)prow[h] * (size_t)A.hq + (size_t)(kvh * A.group + g);
                ok[h] = (elem[h] + 1) * A.row_bytes <= A.q_bytes;
                if (!ok[h]) record_bad_index(A.status, 302, elem[h], ii);
            }
        }
        const uint32_t n_ok = __popc(__ballot_sync(0xffffffffu, ok[0])) + __popc(__ballot_sync(0xffffffffu, ok[1]));
        if (!rec_ok && lane == 0) record_bad_index(A.status, 303, ii, A.n_items);
        if (lane == 0) mbar_expect_tx(bar, n_ok * A.row_bytes + (rec_ok ? A.rec_stride : 0u));
        __syncwarp();
#pragma unroll
        for (int h = 0; h < 2; h++)
            if (ok[h]) bulk_g2s(slot + (uint32_t)(32 * h + lane) * A.stride, A.q + elem[h] * A.row_bytes, A.row_bytes, bar);
        if (lane == 0 && rec_ok) bulk_g2s(rec_slot, A.recs + (size_t)ii * A.rec_stride, A.rec_stride, bar);
        if (YX_TR(A.trace != nullptr) && lane == 0 && ii == A.item_begin) {
            A.trace[10] = gtime();
            A.trace[11] = ((unsigned long long)n_ok << 32) | (unsigned long long)(n_ok * A.row_bytes + (rec_ok ? A.rec_stride : 0u));
            A.trace[12] = ((unsigned long long)head_rows << 32) | bar;
            A.trace[13] = (unsigned long long)(uintptr_t)(A.q + elem[0] * A.row_bytes);
        }
        pipe.advance(Q_SLOTS);
        if (ii + 1 < A.item_end) fetch(ii + 1);
    }
    if (!alive && lane == 0) drain_copies(A.qfull, Q_SLOTS, pipe);
}

// ---- consumers ---------------------------------------------------------------------------------

// ---- epilogue warp ---------------------------------------------------------------------------
// The end of an item costs latency, not work: a device-wide fence, an atomic round trip and,
// for whoever completes a (row, KV head), two dependent reads of other CTAs' triples.  The
// consumer warps do not wait for any of it.  They leave their rows' (o, m, l) in one of two
// shared-memory buffers and move on to the next item; this warp
//  1. merges the key slices of every valid query row and writes the row's triple to the
//     partial buffer (a lane holds four of the 128 dims, stores coalesced);
//  2. counts the item in for each of its (row, KV head) with an arrival counter in global
//     scratch; where it completes one, it merges all of that pair's triples (the reference's
//     `attn_combine`, crates/yaxus-backend-gpu/src/shaders.rs:1581-1637), writes the output
//     and resets the counter.
struct Epilogue {
    float *part_o, *part_ml;
    uint32_t *counters;
    void *out;
    float *m_out, *l_out, *o_out;
    yx_dev_status *status;
    volatile int *abort_flag;
    int out_dtype, hq, hkv, group;
    int fused;               // count items in and merge here (else a separate combine kernel merges)
    int late_wait;           // 1: the grid dependency has not been waited for yet, do so before the first store; 2: the kernel waits at its end
    uint32_t n_parts;        // slots in the partial buffers
    uint32_t n_items, first_item;    // this warp takes items first_item, first_item + EWARPS, ...
    uint32_t recbase, qempty, merge, efull, eempty, mlbuf;   // shared-space addresses
};

// Eight (row, head) pairs at a time, four lanes each: two round trips to L2 per round (the
// maxima, then weights and vectors with independent loads).  Parts with l <= 0 are dropped by
// value: their o was never written (shaders.rs:1597-1598).  Loads bypass L1: other SMs wrote
// these triples during this very kernel.
__device__ __forceinline__ void merge_completed(const Epilogue &E, const uint32_t *rec, uint32_t done_mask, int kvh,
                                                int lane) {
    const int group = E.group;
    const int n_tasks = __popc(done_mask) * group;
    const int sub = lane >> 2, l4 = lane & 3;
    const uint32_t gmask = 0xfu << (sub * 4);
#pragma unroll 1
    for (int t0 = 0; t0 < n_tasks; t0 += 8) {
        const int t = t0 + sub;
        if (t >= n_tasks) continue;   // a whole four-lane group leaves; shuffles below stay inside a group
        const int which = t / group, hg = t - which * group;
        uint32_t mk = done_mask;
        for (int x = 0; x < which; x++) mk &= mk - 1;
        const int base = IR_ROW0 + IR_ROW_WORDS * (__ffs(mk) - 1);
        const uint32_t row = rec[base + IRR_ROW], first = rec[base + IRR_FIRST], count = rec[base + IRR_COUNT];
        const float *ml = E.part_ml + ((size_t)first * group + hg) * 2;
        const float *po = E.part_o + ((size_t)first * group + hg) * D + l4 * 32;
        // Round trip one: every part's (m, l), parked in shared memory.  Round trip two: the
        // vectors, their loads independent of one another because the weights no longer come
        // from global memory.  Chunks of 32 parts, a running maximum between chunks.
        float2 *mls = (float2 *)__cvta_shared_to_generic((size_t)E.mlbuf) + sub * 32;
        float mx = -1e30f, ls = 0.0f;
        float4 acc[8];
#pragma unroll
        for (int k = 0; k < 8; k++) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
        for (uint32_t c0 = 0; c0 < count; c0 += 32) {
            const uint32_t nc = min(32u, count - c0);
            float cm = -1e30f;
#pragma unroll 1
            for (uint32_t c = l4; c < nc; c += 4) {
                const float2 v = __ldcg((const float2 *)(ml + (size_t)(c0 + c) * group * 2));
                mls[c] = v;
                if (v.y > 0.0f) cm = fmaxf(cm, v.x);
            }
            cm = fmaxf(cm, __shfl_xor_sync(gmask, cm, 1));
            cm = fmaxf(cm, __shfl_xor_sync(gmask, cm, 2));
            __syncwarp(gmask);   // the parked values are visible to the group
            const float nm = fmaxf(mx, cm), r = __expf(mx - nm);
            ls *= r;
#pragma unroll
            for (int k = 0; k < 8; k++) {
                acc[k].x *= r;
                acc[k].y *= r;
                acc[k].z *= r;
                acc[k].w *= r;
            }
            mx = nm;
#pragma unroll 2
            for (uint32_t c = 0; c < nc; c++) {
                const float2 v = mls[c];
                if (!(v.y > 0.0f)) continue;
                const float w = __expf(v.x - mx);
                ls += v.y * w;
                const float4 *src = (const float4 *)(po + (size_t)(c0 + c) * group * D);
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const float4 x = __ldcg(src + k);
                    acc[k].x += x.x * w;
                    acc[k].y += x.y * w;
                    acc[k].z += x.z * w;
                    acc[k].w += x.w * w;
                }
            }
            __syncwarp(gmask);   // the next chunk reuses the parking space
        }
        const size_t idx = (size_t)row * E.hq + (size_t)kvh * group + hg;
        if (E.out) {
            const float inv = 1.0f / ls;   // a row always sees its own key: > 0 for whole attention
#pragma unroll
            for (int k = 0; k < 8; k++)
                store4(E.out, E.out_dtype, idx * D + l4 * 32 + k * 4,
                       make_float4(acc[k].x * inv, acc[k].y * inv, acc[k].z * inv, acc[k].w * inv));
        }
        if (E.o_out) {
#pragma unroll
            for (int k = 0; k < 8; k++) *(float4 *)(E.o_out + idx * D + l4 * 32 + k * 4) = acc[k];
            if (l4 == 0) {
                E.m_out[idx] = mx;
                E.l_out[idx] = ls;
            }
        }
    }
}

// The item's triples: for each of its queries first_q, first_q + q_step, ... the slices its
// consumer warps left in shared memory are merged and written to the partial buffer (a lane
// holds four of the 128 dims, stores coalesced).  Which warps hold slices of column tile jq
// follows the kernel's dispatch table: warp w0 + x * wstep, x < nsl.
__device__ __forceinline__ void merge_queries(const float *scratch, const uint32_t *rec, float *part_o, float *part_ml,
                                              int group, int first_q, int q_step, int lane, uint32_t n_parts,
                                              yx_dev_status *status) {
    const float sl2 = 0.08838834764831845f * 1.4426950408889634f;
    const int n_rows = (int)(rec[IR_HEAD_ROWS] >> 16);
    const int mt = (int)rec[IR_MT];
    const int q_rows = n_rows * group;
    const bool narrow = mt == 16 && q_rows <= 8;
    const int nsl = narrow ? 8 : (mt == 16 ? 4 : (mt == 32 ? 2 : 1));
#pragma unroll 1
    for (int qr = first_q; qr < q_rows; qr += q_step) {
        const int r = qr / group, gq = qr - r * group;
        const uint32_t part = rec[IR_ROW0 + IR_ROW_WORDS * r + IRR_PART];
        const int jq = qr >> 3;
        const int w0 = narrow ? 0 : (mt == 16 ? jq * 4 : jq), wstep = (narrow || mt == 16) ? 1 : 4;
        const float *base = scratch + w0 * MERGE_FLOATS + (qr & 7) * MERGE_ROW;
        // all slices' loads are independent of one another
        float2 ml[8];
        float4 v[8];
#pragma unroll
        for (int x = 0; x < 8; x++) {
            ml[x] = make_float2(-INFINITY, 0.f);
            v[x] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (x < nsl) {
                const float *w = base + x * wstep * MERGE_FLOATS;
                ml[x] = *(const float2 *)(w + D);
                v[x] = *(const float4 *)(w + 4 * lane);
            }
        }
        float mx = -INFINITY;
#pragma unroll
        for (int x = 0; x < 8; x++) mx = fmaxf(mx, ml[x].x);
        const float mu = mx == -INFINITY ? 0.f : mx;
        float ls = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int x = 0; x < 8; x++) {
            const float f = fast_exp2((ml[x].x - mu) * sl2);   // 0 for a slice that saw no key (and for x >= nsl)
            ls += ml[x].y * f;
            acc.x += v[x].x * f;
            acc.y += v[x].y * f;
            acc.z += v[x].z * f;
            acc.w += v[x].w * f;
        }
        if (part >= n_parts) {   // the kernel's own check: recorded, the store left out
            if (lane == 0) record_bad_index(status, 304, part, n_parts);
            continue;
        }
        const size_t slot = (size_t)part * group + gq;
        __stcg((float4 *)(part_o + slot * D + 4 * lane), acc);
        if (lane == 0) {
            const bool none = mx == -INFINITY;
            __stcg((float2 *)(part_ml + slot * 2), make_float2(none ? -1e30f : mx * 0.08838834764831845f, none ? 0.f : ls));
        }
    }
}

__device__ __noinline__ void epilogue_loop(const Epilogue E, int lane) {
    // One merge buffer, handed back and forth between the consumer warps and this warp; the
    // item's record sits in the query slot of the item's parity.
    static_assert(MERGE_BUFS == 1 && EWARPS == 1 && Q_SLOTS == 2, "one buffer, one epilogue warp, two query slots");
    uint32_t phase = 0;
    const int group = E.group;
#pragma unroll 1
    for (uint32_t ii = 0; ii < E.n_items; ii++, phase ^= 1u) {
        const uint32_t qslot = ii & 1u;
        mbar_wait(E.efull, phase, E.abort_flag, E.status, 5);
        if (ii == 0 && E.late_wait == 1) grid_dependency_wait();   // the merge ahead has read the partial buffers
        const float *scratch = (const float *)__cvta_shared_to_generic((size_t)E.merge);
        const uint32_t *rec = (const uint32_t *)__cvta_shared_to_generic((size_t)(E.recbase + qslot * REC_BYTES));
        const uint32_t head_rows = rec[IR_HEAD_ROWS];
        const int kvh = (int)(head_rows & 0xffffu), n_rows = (int)(head_rows >> 16);
        // 1. the item's triples
        merge_queries(scratch, rec, E.part_o, E.part_ml, group, 0, 1, lane, E.n_parts, E.status);
        __syncwarp();
        if (lane == 0) mbar_arrive(E.eempty);   // the buffer is the consumers' again
        if (!E.fused) {
            if (lane == 0) mbar_arrive(E.qempty + 8 * qslot);
            continue;
        }
        // 2. count the item in; merge what it completes
        __threadfence();   // the triples are visible device-wide before the item is counted
        bool last = false;
        if (lane < n_rows) {
            const int base = IR_ROW0 + IR_ROW_WORDS * lane;
            uint32_t *ctr = E.counters + (size_t)rec[base + IRR_ROW] * E.hkv + kvh;
            last = atomicAdd(ctr, 1u) + 1 == rec[base + IRR_COUNT];
            if (last) *ctr = 0u;   // nobody else touches it in this launch: left clean for the next
        }
        const uint32_t done_mask = __ballot_sync(0xffffffffu, last);
        if (done_mask) {
            __threadfence();
            merge_completed(E, rec, done_mask, kvh, lane);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(E.qempty + 8 * qslot);   // done with the record too
    }
}

// One item on one consumer warp.  The product is taken transposed, S^T = K Q^T and
// O^T = V^T P^T: the 16-row side of the MMA holds keys (or dims), which are always full, and
// the 8-column side holds queries, of which a decode row has only its group's few.  A warp owns
// one column tile (8 queries, index j) and KBW 16-key blocks of a tile starting at key k0; with
// `turn` >= 0 it takes every other tile only (two tiles are then in work at a time).  Eight such
// warps, two per scheduler, keep the issue slots busy where one warp per scheduler left them
// waiting on its own dependent instructions.
template <int KBW, bool BF16>
__device__ void consume_item(const Params &P, const Shared &S, Pipe &pipe, Pipe &qpipe, Pipe &epipe, int warp,
                             int lane, int j, int k0, int turn, bool low_ok, bool last) {
    constexpr int PARTS = KBW == 1 ? 4 : (KBW == 2 ? 2 : 1);   // partial sums per key block: short MMA chains
    const int g = lane >> 2, t4 = lane & 3;
    const int group = P.group;
    const uint32_t slot = S.q;
    const uint32_t *rec = (const uint32_t *)__cvta_shared_to_generic((size_t)(S.rec + qpipe.stage * REC_BYTES));
    const uint32_t n_tiles = rec[IR_TILES], key_base = rec[IR_KEY0];
    const int n_rows = (int)(rec[IR_HEAD_ROWS] >> 16);
    const int q_rows = n_rows * group;
    const float sl2 = 0.08838834764831845f * 1.4426950408889634f;   // log2(e) / sqrt(128)
    const bool exact_q = (P.q_dtype == YX_BF16 && BF16) || (P.q_dtype == YX_F16 && !BF16);
    // Queries that are not already of the cache's type carry a low part on bf16 caches (8 bits of
    // mantissa would not do); on f16 caches the high part's 11 bits are within the bound by a wide
    // margin, and leaving the low part out takes a third off the tensor work of an item.
    const bool low = low_ok && !exact_q && BF16;

    // The two queries this thread meets in the accumulator fragments: columns 2 t4 and 2 t4 + 1.
    uint32_t klo[2], khi[2];
#pragma unroll
    for (int c = 0; c < 2; c++) {
        const int qr = j * 8 + 2 * t4 + c;
        const bool valid = qr < q_rows;
        const int base = IR_ROW0 + IR_ROW_WORDS * (valid ? qr / group : 0);
        klo[c] = valid ? rec[base + IRR_KLO] : 0u;            // padded queries are zero: nothing to mask
        khi[c] = valid ? rec[base + IRR_KHI] : 0xffffffffu;
    }
    const int lm = lane >> 3, lr = lane & 7;
    // (32-row items only: for the others the test is dropped at compile time)
    const bool idle = KBW >= 2 && j * 8 >= q_rows;   // this warp's eight columns are all padding: its (o, m, l) stay (0, -inf, 0)
    // Query fragments (the column operand), held for the whole item, built from the raw rows the
    // stager's copies left in the slot: this thread holds dims 16 ks + 2 t4 (+1) and + 8 of query
    // j * 8 + g.  f32 queries (and 16-bit ones of the other type) become a high part in the cache's
    // type and, where there is room for it, a low part.
    uint32_t qh[8][2], ql[8][2];
    {
        const int qr = j * 8 + g;
        const bool valid = qr < q_rows;   // rows past the item's queries were not copied: zeros instead
        if (P.q_dtype == YX_F32) {
            const uint32_t a = slot + (uint32_t)qr * Q_STRIDE_F32 + 8u * t4;
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    float2 v = make_float2(0.f, 0.f);
                    if (valid) asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a + 64u * ks + 32u * h));
                    const uint32_t hi = pack2<BF16>(v.x, v.y);
                    qh[ks][h] = hi;
                    ql[ks][h] = 0u;
                    if (low) {
                        const float2 f = unpack2<BF16>(hi);
                        ql[ks][h] = pack2<BF16>(v.x - f.x, v.y - f.y);
                    }
                }
            }
        } else {
            const uint32_t a = slot + (uint32_t)qr * Q_STRIDE_16 + 4u * t4;
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    uint32_t raw = 0u;
                    if (valid) asm volatile("ld.shared.b32 %0, [%1];" : "=r"(raw) : "r"(a + 32u * ks + 16u * h));
                    qh[ks][h] = raw;
                    ql[ks][h] = 0u;
                    if (!exact_q) {
                        const float2 v = P.q_dtype == YX_BF16 ? unpack2<true>(raw) : unpack2<false>(raw);
                        const uint32_t hi = pack2<BF16>(v.x, v.y);
                        qh[ks][h] = hi;
                        if (low) {
                            const float2 f = unpack2<BF16>(hi);
                            ql[ks][h] = pack2<BF16>(v.x - f.x, v.y - f.y);
                        }
                    }
                }
            }
        }
    }

    // The rows buffer is the stager's again (the fragments are in registers).
    __syncwarp();
    if (lane == 0) mbar_arrive(S.qrows_free);

    float o[8][4];   // O^T: dims 16 n + g (+8), queries 2 t4 (+1)
#pragma unroll
    for (int n = 0; n < 8; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (uint32_t ti = 0; ti < n_tiles; ti++) {
        const long long w0 = (YX_TR(P.trace != nullptr) && threadIdx.x == 0) ? clock64() : 0;
        mbar_wait(S.full + 8 * pipe.stage, pipe.phase, S.abort_flag, P.status, 2);
        if (idle || (turn >= 0 && (int)(ti & 1u) != turn)) {
            // The other warps' tile, or a column tile without a query (20 or 24 query rows in a
            // 32-row item leave the fourth one empty: its warps' share of the tensor work goes
            // to the other six).  The tile is still waited for and released: a warp that skipped
            // ahead without looking could meet a barrier two phases on, which a parity wait
            // cannot tell from the phase it expects.
            if (lane == 0) mbar_arrive(S.empty + 8 * pipe.stage);
            pipe.advance(P.n_stages);
            continue;
        }
        if (YX_TR(P.trace != nullptr) && threadIdx.x == 0) P.trace[16 * blockIdx.x + 7] += (unsigned long long)(clock64() - w0);
        if (YX_TR(P.trace != nullptr) && threadIdx.x == 0 && ti == 0 && P.trace[16 * blockIdx.x + 4] == 0) P.trace[16 * blockIdx.x + 4] = gtime();
        const uint32_t sb = S.stages + pipe.stage * STAGE_BYTES;

        // S^T = K Q^T over this warp's keys.
        float sp[KBW][PARTS][4];
#pragma unroll
        for (int kb = 0; kb < KBW; kb++)
#pragma unroll
            for (int p = 0; p < PARTS; p++) sp[kb][p][0] = sp[kb][p][1] = sp[kb][p][2] = sp[kb][p][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
            const uint32_t sub = sb + (ks >> 2) * SUB_BYTES;
            const int c = ((2 * ks) & 7) + (lane >> 4);
#pragma unroll
            for (int kb = 0; kb < KBW; kb++) {
                const int key = k0 + kb * 16 + (lm & 1) * 8 + lr;
                uint32_t a[4];   // keys as the row operand
                ldsm4(sub + key * 128 + ((c ^ lr) << 4), a[0], a[1], a[2], a[3]);
                // hi and lo parts, even and odd steps in different sums where there is room for them
                mma16816<BF16>(sp[kb][PARTS == 4 ? (ks & 1) * 2 : 0], a, qh[ks][0], qh[ks][1]);
                if (low) mma16816<BF16>(sp[kb][PARTS == 4 ? (ks & 1) * 2 + 1 : (PARTS == 2 ? 1 : 0)], a, ql[ks][0], ql[ks][1]);
            }
        }
        float s[KBW][4];
#pragma unroll
        for (int kb = 0; kb < KBW; kb++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float v = sp[kb][0][e];
#pragma unroll
                for (int p = 1; p < PARTS; p++) v += sp[kb][p][e];
                s[kb][e] = v;
            }
        // Mask keys outside each query's [klo, khi]: element e sits at key g + 8 (e >> 1), query 2 t4 + (e & 1).
        const uint32_t key0 = key_base + ti * TILE_KEYS + k0 + g;
#pragma unroll
        for (int kb = 0; kb < KBW; kb++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const uint32_t key = key0 + kb * 16 + (e >> 1) * 8;
                if (key < klo[e & 1] || key > khi[e & 1]) s[kb][e] = -INFINITY;
            }
        // Online softmax per query: the maximum runs over this thread's keys, then over the
        // eight lanes that hold the other keys of the same queries.
        float alpha[2];
#pragma unroll
        for (int c = 0; c < 2; c++) {
            float mx = -INFINITY;
#pragma unroll
            for (int kb = 0; kb < KBW; kb++) mx = fmaxf(mx, fmaxf(s[kb][c], s[kb][2 + c]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float mn = fmaxf(m[c], mx);
            const float mu = mn == -INFINITY ? 0.f : mn;
            alpha[c] = fast_exp2((m[c] - mu) * sl2);
            m[c] = mn;
            const float ms = mu * sl2;
            float sum = 0.f;
#pragma unroll
            for (int kb = 0; kb < KBW; kb++) {
                const float p0 = fast_exp2(s[kb][c] * sl2 - ms), p1 = fast_exp2(s[kb][2 + c] * sl2 - ms);
                s[kb][c] = p0;
                s[kb][2 + c] = p1;
                sum += p0 + p1;
            }
            l[c] = l[c] * alpha[c] + sum;   // this thread's keys only: lanes are summed at the end
        }
        // The accumulator is rescaled only when some query's maximum moved (warp-uniform).
        if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
            for (int n = 0; n < 8; n++) {
                o[n][0] *= alpha[0];
                o[n][1] *= alpha[1];
                o[n][2] *= alpha[0];
                o[n][3] *= alpha[1];
            }
        }
        // O^T += V^T P^T, 16 keys at a time.  The probabilities sit as (key row, query pair); a
        // matrix transpose across the warp turns them into the column operand (key pair, query).
#pragma unroll
        for (int kb = 0; kb < KBW; kb++) {
            uint32_t pb[2], pl[2];
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const float p0 = s[kb][2 * h], p1 = s[kb][2 * h + 1];
                const uint32_t w = pack2<BF16>(p0, p1);
                pb[h] = movmatrix_trans(w);
                if constexpr (BF16) {
                    // bf16 keeps 8 bits of a probability; its remainder goes in a second MMA.
                    const float2 hf = unpack2<BF16>(w);
                    pl[h] = movmatrix_trans(pack2<BF16>(p0 - hf.x, p1 - hf.y));
                }
            }
            const int key = k0 + kb * 16 + (lm >> 1) * 8 + lr;
#pragma unroll
            for (int n = 0; n < 8; n++) {
                const uint32_t sub = sb + 2 * SUB_BYTES + (n >> 2) * SUB_BYTES;
                const int c = ((2 * n) & 7) + (lm & 1);
                uint32_t a[4];   // dims as the row operand: V read transposed
                ldsm4t(sub + key * 128 + ((c ^ lr) << 4), a[0], a[1], a[2], a[3]);
                mma16816<BF16>(o[n], a, pb[0], pb[1]);
                if constexpr (BF16) mma16816<BF16>(o[n], a, pl[0], pl[1]);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(S.empty + 8 * pipe.stage);
        pipe.advance(P.n_stages);
    }

    // Sums of exponentials across the lanes that share a query.
#pragma unroll
    for (int c = 0; c < 2; c++) {
        l[c] += __shfl_xor_sync(0xffffffffu, l[c], 4);
        l[c] += __shfl_xor_sync(0xffffffffu, l[c], 8);
        l[c] += __shfl_xor_sync(0xffffffffu, l[c], 16);
    }
    // Every warp leaves its 8 queries' (o, m, l) in shared memory for the epilogue warp and goes
    // on to the next item.
    {
        mbar_wait(S.eempty + 8 * epipe.stage, epipe.phase ^ 1u, S.abort_flag, P.status, 6);
        float *w = (float *)__cvta_shared_to_generic((size_t)(S.merge + epipe.stage * MERGE_BYTES)) + warp * MERGE_FLOATS;
#pragma unroll
        for (int c = 0; c < 2; c++) {
            float *row = w + (2 * t4 + c) * MERGE_ROW;
            if (g == 0) *(float2 *)(row + D) = make_float2(m[c], l[c]);
#pragma unroll
            for (int n = 0; n < 8; n++) {
                row[n * 16 + g] = o[n][c];
                row[n * 16 + g + 8] = o[n][2 + c];
            }
        }
        if (last) {
            // The CTA's last item: nothing is left to stream, so the consumer warps merge it
            // themselves, a share of the queries each, instead of queueing it behind one
            // epilogue warp at the very end of the kernel.
            asm volatile("bar.sync %0, %1;" ::"n"(CONSUMER_BARRIER), "n"(CONSUMERS * 32) : "memory");
            if (P.late_wait && !P.wait_at_end) grid_dependency_wait();   // the merge ahead has read the partial buffers
            const float *scratch = (const float *)__cvta_shared_to_generic((size_t)(S.merge + epipe.stage * MERGE_BYTES));
            merge_queries(scratch, rec, P.part_o, P.part_ml, group, warp, CONSUMERS, lane, P.n_parts, P.status);
            return;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(S.efull + 8 * epipe.stage);
        epipe.advance(MERGE_BUFS);
    }
    // The slot (queries and record) is free once every consumer warp and the epilogue warp are
    // done with the item.
    if (lane == 0) mbar_arrive(S.qempty + 8 * qpipe.stage);
    qpipe.advance(Q_SLOTS);
}

template <bool BF16>
__global__ void __maxnreg__(152) attend_mma_kernel(const __grid_constant__ Params P) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ int abort_flag;
    Shared S;
    S.stages = smem_u32(smem);
    S.q = S.stages + STAGES * STAGE_BYTES;
    S.rec = S.q + Q_ROWS_BYTES;
    S.merge = S.rec + Q_SLOTS * REC_BYTES;
    S.full = S.merge + MERGE_BUFS * MERGE_BYTES;
    S.empty = S.full + 8 * STAGES;
    S.qfull = S.empty + 8 * STAGES;
    S.qempty = S.qfull + 8 * Q_SLOTS;
    S.qrows_free = S.qempty + 8 * Q_SLOTS;
    S.efull = S.qrows_free + 8;
    S.eempty = S.efull + 8 * MERGE_BUFS;
    S.mlbuf = S.eempty + 8 * MERGE_BUFS;
    S.abort_flag = &abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // The kernels behind this one in the stream (the merge, then the next attention call) may be
    // made resident once every CTA has said so.  The next call's kernel may then read keys, values
    // and queries without waiting (late_wait), so this is said only when everything ahead of this
    // kernel is complete: at once if that was true at the launch, else after the wait below.
    if (P.late_wait && threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    unsigned long long *tr = YX_TR(P.trace != nullptr) ? P.trace + 16 * blockIdx.x : nullptr;
    if (tr && threadIdx.x == 0) tr[0] = gtime();
    const CtaHdr hdr = P.has_prologue ? P.pro[blockIdx.x].hdr : *(const CtaHdr *)(P.cta_hdr + blockIdx.x);

    if (warp == PRODUCER) {
        // The producer sets the barriers up itself and starts the first copies at once.
        if (lane == 0) {
            abort_flag = 0;
            for (int s = 0; s < STAGES; s++) {
                mbar_init(S.full + 8 * s, 1);
                mbar_init(S.empty + 8 * s, CONSUMERS);
            }
            for (int s = 0; s < Q_SLOTS; s++) {
                mbar_init(S.qfull + 8 * s, 1);
                mbar_init(S.qempty + 8 * s, CONSUMERS + 1);   // the consumer warps and the epilogue warp
            }
            mbar_init(S.qrows_free, CONSUMERS);
            for (int s = 0; s < MERGE_BUFS; s++) {
                mbar_init(S.efull + 8 * s, CONSUMERS);
                mbar_init(S.eempty + 8 * s, 1);
            }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncwarp();
        // The set-up is published through a named barrier that this warp only arrives at (it has
        // nothing to wait for) and the ten other warps wait on; they then fetch queries while
        // this warp starts the first K/V copies.  (Barrier 0, the __syncthreads barrier, reached
        // from two places in the code did not hold the other warps back: they went on to use
        // mbarriers that were not yet initialised.)
        __threadfence_block();
        asm volatile("bar.arrive %0, %1;" ::"n"(SETUP_BARRIER), "n"(THREADS) : "memory");
        if (tr && lane == 0) tr[14] = gtime();
        produce(P, S, hdr, lane);
        return;
    }
    asm volatile("bar.sync %0, %1;" ::"n"(SETUP_BARRIER), "n"(THREADS) : "memory");
    // Nothing written by earlier kernels (queries, the partial buffers' previous readers) is
    // touched by these warps before this wait.  With late_wait the queries are long written, and
    // the warps that write wait before their first store instead.
    if (!P.late_wait) {
        grid_dependency_wait();
        if (threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    if (tr && threadIdx.x == 0) tr[1] = gtime();

    if (warp == QWARP) {
        QStage A;
        A.q = (const char *)P.q;
        A.recs = P.recs;
        A.rec_stride = P.rec_stride;
        A.status = P.status;
        A.hq = P.hq;
        A.group = P.group;
        A.row_bytes = P.q_dtype == YX_F32 ? 512u : 256u;
        A.stride = P.q_dtype == YX_F32 ? (uint32_t)Q_STRIDE_F32 : (uint32_t)Q_STRIDE_16;
        A.item_begin = hdr.item_begin;
        A.item_end = hdr.item_end;
        A.have_first = P.has_prologue;
        A.first_head_rows = A.first_row0 = A.first_row1 = 0;
        if (P.has_prologue) {
            A.first_head_rows = P.pro[blockIdx.x].head_rows;
            A.first_row0 = P.pro[blockIdx.x].rows[min(lane / P.group, MAX_ITEM_ROWS - 1)];
            A.first_row1 = P.pro[blockIdx.x].rows[min((32 + lane) / P.group, MAX_ITEM_ROWS - 1)];
        }
        A.qbase = S.q;
        A.recbase = S.rec;
        A.qfull = S.qfull;
        A.qempty = S.qempty;
        A.qrows_free = S.qrows_free;
        A.abort_flag = S.abort_flag;
        A.n_items = P.n_items;
        A.q_bytes = P.q_bytes;
        A.trace = tr;
        stage_queries(A, lane);
        return;
    }
    if (warp >= EWARP) {
        Epilogue E;
        E.part_o = P.part_o;
        E.part_ml = P.part_ml;
        E.counters = P.counters;
        E.out = P.out;
        E.m_out = P.m_out;
        E.l_out = P.l_out;
        E.o_out = P.o_out;
        E.status = P.status;
        E.abort_flag = S.abort_flag;
        E.out_dtype = P.out_dtype;
        E.hq = P.hq;
        E.hkv = P.hkv;
        E.group = P.group;
        E.fused = P.fused;
        E.late_wait = P.late_wait ? (P.wait_at_end ? 2 : 1) : 0;
        E.n_parts = P.n_parts;
        E.n_items = hdr.item_end - hdr.item_begin;
        if (!P.fused && E.n_items > 0) E.n_items--;   // the last item is the consumer warps' own
        E.recbase = S.rec;
        E.qempty = S.qempty;
        E.merge = S.merge;
        E.efull = S.efull;
        E.eempty = S.eempty;
        E.mlbuf = S.mlbuf;
        E.first_item = 0;
        epilogue_loop(E, lane);
        // A CTA that has not waited yet (with wait_at_end: none has; without: an empty one, or one
        // whose only item the consumer warps merged) does so here, through this warp: the kernel
        // then completes after the kernels ahead, as the stream's order says, and no CTA leaves
        // its SM to a CTA of the next call before the merge that reads the partial buffers that
        // call will write has finished.
        if (P.late_wait) grid_dependency_wait();
        return;
    }
    Pipe pipe{0, 0}, qpipe{0, 0}, epipe{0, 0};
    for (uint32_t ii = hdr.item_begin; ii < hdr.item_end; ii++) {
        // The staged slot holds the item's record and queries.
        mbar_wait(S.qfull + 8 * qpipe.stage, qpipe.phase, S.abort_flag, P.status, 4);
        if (tr && threadIdx.x == 0 && ii == hdr.item_begin) tr[3] = gtime();
        const uint32_t mt = *(const uint32_t *)__cvta_shared_to_generic((size_t)(S.rec + qpipe.stage * REC_BYTES + 4 * IR_MT));
        const bool last = !P.fused && ii + 1 == hdr.item_end;   // merged by the consumer warps themselves
        const uint32_t hr = *(const uint32_t *)__cvta_shared_to_generic((size_t)(S.rec + qpipe.stage * REC_BYTES + 4 * IR_HEAD_ROWS));
        const int q_rows = (int)(hr >> 16) * P.group;
        // Who takes what of a 64-key tile (the epilogue warp's merge knows the same table):
        //   up to 8 queries: column tile 0 everywhere, a 16-key block each, warps 0-3 even tiles and 4-7 odd ones;
        //   up to 16: column tile warp / 4, a 16-key block each;  up to 32: column tile warp % 4, 32 keys each;
        //   up to 64: column tile warp, the whole tile (16-bit queries only: 64 f32 rows do not fit a slot).
        if (mt == 16 && q_rows <= 8) consume_item<1, BF16>(P, S, pipe, qpipe, epipe, warp, lane, 0, (warp & 3) * 16, warp >> 2, true, last);
        else if (mt == 16) consume_item<1, BF16>(P, S, pipe, qpipe, epipe, warp, lane, warp >> 2, (warp & 3) * 16, -1, true, last);
        else if (mt == 32) consume_item<2, BF16>(P, S, pipe, qpipe, epipe, warp, lane, warp & 3, (warp >> 2) * 32, -1, true, last);
        else consume_item<4, BF16>(P, S, pipe, qpipe, epipe, warp, lane, warp, 0, -1, false, last);
        if (tr && threadIdx.x == 0 && ii == hdr.item_begin) tr[6] = gtime();
    }
    if (tr && threadIdx.x == 0) tr[5] = gtime();
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
    // The bulk copies of the query rows need 16-byte aligned sources.
    if (((uintptr_t)a.q & 15u) != 0) return fail(ctx, YX_ERR_INVALID, "attention: the query tensor must be 16-byte aligned");
    if (a.q_dtype == YX_F32 && a.plan) {
        for (const Item &it : a.plan->items)
            if (it.mt > 32) return fail(ctx, YX_ERR_INVALID, "attention: an item of more than 32 f32 query rows (planner bug)");
    }
    static thread_local Params P;   // 13 KB: kept off the stack
    memset(&P, 0, offsetof(Params, pro));
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
    P.rec_stride = a.rec_stride;
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
    P.fused = a.fused ? 1 : 0;
    P.n_stages = a.n_stages >= 2 && a.n_stages <= STAGES ? a.n_stages : STAGES;
    P.early_kv = a.early_kv ? 1 : 0;
    P.late_wait = a.late_wait ? 1 : 0;
    P.wait_at_end = a.wait_at_end ? 1 : 0;
    P.n_items = a.plan ? (uint32_t)a.plan->items.size() : 0u;
    P.n_tiles = a.plan ? (uint32_t)a.plan->tiles.size() : 0u;
    P.n_parts = a.plan ? a.plan->n_parts : 0u;
    P.q_bytes = (unsigned long long)a.rows * (unsigned long long)a.hq * D * (a.q_dtype == YX_F32 ? 4u : 2u);
    if (a.plan && a.n_ctas <= MAX_PROLOGUE_CTAS && (int)a.plan->prologue.size() == a.n_ctas) {
        P.has_prologue = 1;
        memcpy(P.pro, a.plan->prologue.data(), sizeof(CtaPrologue) * (size_t)a.n_ctas);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)a.n_ctas);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t le = bf16 ? cudaLaunchKernelEx(&cfg, attend_mma_kernel<true>, P) : cudaLaunchKernelEx(&cfg, attend_mma_kernel<false>, P);
    if (int rc = check_cuda(ctx, le, "attend_mma kernel launch")) return rc;
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "attend_mma kernel");
}

}  // namespace yx
