// Host-side planner of the split-key attention kernels: the counterpart of the reference's
// `AttentionCase::plan` (crates/yaxus-backend-gpu/src/plan.rs:275-309), re-thought for a
// persistent kernel on 148 SMs.
//
// The reference cuts every row's context into fixed chunks of 16/32 keys and launches one
// workgroup per (row, KV head, chunk).  Here the keys of all rows are laid end to end as one
// sequence of 64-key tiles and that sequence is cut into one equal span per persistent CTA
// ("stream-K"), so every CTA streams the same number of bytes whatever the mix of context
// lengths, and a (row, head) gets as many partial triples as CTAs touched it.
//
// Rows whose page tables name the same physical pages over a common prefix (what
// `KvCache::fork` shares, crates/yaxus-model/src/kv.rs:277-295) are put in one item over that
// prefix, so the shared pages are read once for all of them.
#include <string.h>

#include <algorithm>
#include <functional>
#include <queue>
#include <string>
#include <unordered_map>

#include "yx_internal.h"

namespace yx {
namespace {

struct Group {          // consecutive rows of one sequence
    uint32_t row0, n;
    uint32_t pt_off;
    uint32_t lo, hi;    // keys any of its rows may see, inclusive (after the range restriction)
    bool live;
};

struct Unit {           // rows x one key range, before it is cut across CTAs (all KV heads)
    std::vector<uint16_t> rows;
    uint32_t pt_off;
    uint32_t lo, hi;    // inclusive
    bool reused = false;   // other units read the same pages: keep them in L2
    uint32_t fresh_from = 0;   // first position its sequence(s) append in this pass: keys from here on may be new
};

inline uint32_t row_lo(uint32_t pos, int64_t window) {
    // cpu lib.rs:402-405: (p + 1).saturating_sub(w)
    if (window <= 0) return 0;
    uint64_t p1 = (uint64_t)pos + 1;
    return p1 > (uint64_t)window ? (uint32_t)(p1 - (uint64_t)window) : 0u;
}

int padded_rows(int q_rows) { return q_rows <= 16 ? 16 : (q_rows <= 32 ? 32 : 64); }

}  // namespace

void build_split_plan(const PassHost &pass, const PlanParams &pp, Plan &out) {
    const uint32_t T = pass.rows;
    if (pp.hkv <= 0 || pp.group <= 0) throw std::string("bad head counts");
    if (pp.max_rows < 1 || pp.max_rows > MAX_ITEM_ROWS) throw std::string("bad rows per item");
    if (T > 65535) throw std::string("a pass holds at most 65535 rows");
    // The plan object is reused from call to call: its arrays keep their capacity, and what the
    // last plan was built from is remembered (see `try_patch` below).
    out.tile_items.clear();
    out.tile_cta_begin.clear();
    out.patched = false;

    // Dense ids of the physical pages named in this pass (page-table entry -> id), so that
    // per-page bookkeeping below is a flat array.  Found with a small open-addressing table:
    // sorting the entries cost more than the rest of the plan of a decode pass.
    std::vector<uint32_t> &dense = out.scratch_dense;
    dense.resize(pass.pages.size());
    uint32_t n_dense = 0;
    {
        size_t cap = 64;
        while (cap < 2 * pass.pages.size()) cap <<= 1;
        std::vector<uint64_t> &table = out.scratch_table;   // (page + 1) << 32 | id; 0 = empty
        table.assign(cap, 0);
        for (size_t i = 0; i < pass.pages.size(); i++) {
            const uint64_t key = (uint64_t)pass.pages[i] + 1;
            size_t h = (size_t)((key * 0x9E3779B97F4A7C15ull) >> 32) & (cap - 1);
            while (table[h] != 0 && (table[h] >> 32) != key) h = (h + 1) & (cap - 1);
            if (table[h] == 0) table[h] = (key << 32) | n_dense++;
            dense[i] = (uint32_t)table[h];
        }
    }

    // 1. Row groups: runs of rows with the same page table.
    std::vector<Group> groups;
    for (uint32_t i = 0; i < T;) {
        uint32_t j = i + 1;
        while (j < T && pass.pt_off[j] == pass.pt_off[i]) j++;
        groups.push_back({i, j - i, pass.pt_off[i], 0, 0, false});
        i = j;
    }
    // Every page-table entry a row can reach must exist.
    for (const Group &g : groups) {
        for (uint32_t r = g.row0; r < g.row0 + g.n; r++) {
            uint64_t need = (uint64_t)g.pt_off + pass.pos[r] / PAGE + 1;
            if (need > pass.pages.size()) throw std::string("a row's page table runs past `pages`");
        }
    }

    // 1b. Long runs of rows (prompt chunks) go to the tiled kernel: 128 consecutive rows of one
    //     sequence and one query head per item, longest first.  Rows of one sequence have
    //     consecutive positions (PassMeta's contract, crates/yaxus-model/src/lib.rs:63-65).
    std::vector<bool> tiled(groups.size(), false);
    if (pp.tile_min_rows > 0 && pp.key_lo == 0 && pp.key_hi == UINT64_MAX) {
        for (uint32_t gi = 0; gi < groups.size(); gi++) {
            const Group &g = groups[gi];
            if (g.n < (uint32_t)pp.tile_min_rows) continue;
            bool consecutive = true;
            for (uint32_t r = 1; r < g.n && consecutive; r++) consecutive = pass.pos[g.row0 + r] == pass.pos[g.row0] + r;
            if (!consecutive) continue;
            tiled[gi] = true;
            for (uint32_t a = 0; a < g.n; a += 128) {
                const uint32_t n = std::min<uint32_t>(128, g.n - a), pos0 = pass.pos[g.row0 + a];
                for (int h = 0; h < pp.hkv * pp.group; h += pp.tile_pairs ? 2 : 1) {
                    TileItem ti{};
                    ti.row0 = g.row0 + a;
                    ti.n_rows = n;
                    ti.pos0 = pos0;
                    ti.pt_off = g.pt_off;
                    ti.head = (uint16_t)h;
                    ti.kv_head = (uint16_t)(h / pp.group);
                    ti.page_begin = row_lo(pos0, pp.window) / PAGE;
                    ti.page_end = (pos0 + n - 1) / PAGE + 1;
                    out.tile_items.push_back(ti);
                }
            }
        }
        // Deal the items to the persistent CTAs of the tiled kernel: longest first, each to the
        // CTA with the least work so far (among equals the one that has waited longest).  An item
        // costs its pages plus a fixed part (Q tile in, output tile out, pipeline fill), about
        // three pages' worth.  Costs are small integers, so "longest first" is a counting sort and
        // "least loaded" a row of FIFO buckets by load: this runs on the critical path of every
        // prompt pass, and a heap of 148 CTAs and a list per CTA cost 45 us of its 100.
        if (!out.tile_items.empty()) {
            const int n_items = (int)out.tile_items.size();
            const int G = std::max(1, std::min(n_items, pp.tile_ctas > 0 ? pp.tile_ctas : n_items));
            std::vector<TileItem> &sorted = out.scratch_tile_items;
            sorted.resize(n_items);
            uint32_t max_len = 0;
            uint64_t total_cost = 0;
            for (const TileItem &ti : out.tile_items) {
                max_len = std::max(max_len, ti.page_end - ti.page_begin);
                total_cost += ti.page_end - ti.page_begin + 3;
            }
            std::vector<uint32_t> &at = out.scratch_lengths;   // counting sort by length, longest first, stable
            at.assign((size_t)max_len + 2, 0);
            for (const TileItem &ti : out.tile_items) at[max_len - (ti.page_end - ti.page_begin) + 1]++;
            for (uint32_t l = 1; l <= max_len + 1; l++) at[l] += at[l - 1];
            for (const TileItem &ti : out.tile_items) sorted[at[max_len - (ti.page_end - ti.page_begin)]++] = ti;
            // FIFO buckets of CTAs by load; a load never exceeds the even share plus one item.
            const size_t n_loads = (size_t)(total_cost / (uint64_t)G) + max_len + 3 + 2;
            std::vector<uint32_t> &links = out.scratch_links;   // head[n_loads] | tail[n_loads] | next[G] | cta_of[n_items] | count[G + 1]
            const uint32_t NONE = UINT32_MAX;
            links.assign(2 * n_loads + (size_t)G + (size_t)n_items + (size_t)G + 1, NONE);
            uint32_t *head = links.data(), *tail = head + n_loads, *next = tail + n_loads, *cta_of = next + G, *count = cta_of + n_items;
            for (int c = 0; c < G; c++) {   // all at load 0, in order
                next[c] = c + 1 < G ? (uint32_t)c + 1 : NONE;
                count[c] = 0;
            }
            count[G] = 0;
            head[0] = 0;
            tail[0] = (uint32_t)G - 1;
            size_t lowest = 0;
            for (int i = 0; i < n_items; i++) {
                while (head[lowest] == NONE) lowest++;
                const uint32_t c = head[lowest];
                head[lowest] = next[c];
                if (head[lowest] == NONE) tail[lowest] = NONE;
                const size_t load = lowest + (sorted[i].page_end - sorted[i].page_begin) + 3;
                next[c] = NONE;
                if (head[load] == NONE) head[load] = c;
                else next[tail[load]] = c;
                tail[load] = c;
                cta_of[i] = c;
                count[c + 1]++;
            }
            for (int c = 0; c < G; c++) count[c + 1] += count[c];
            out.tile_cta_begin.assign(count, count + G + 1);
            for (int i = 0; i < n_items; i++) out.tile_items[count[cta_of[i]]++] = sorted[i];
        }
    }

    // 2. Units.  First the per-sequence ones, rows chunked to max_rows.
    std::vector<Unit> units;
    struct Solo { size_t unit; uint32_t group; };
    std::vector<Solo> solos;   // units that hold all rows of one group (candidates for sharing)
    for (uint32_t gi = 0; gi < groups.size(); gi++) {
        const Group &g = groups[gi];
        if (tiled[gi]) continue;
        for (uint32_t a = 0; a < g.n; a += pp.max_rows) {
            uint32_t b = std::min<uint32_t>(g.n, a + pp.max_rows);
            Unit u;
            u.pt_off = g.pt_off;
            u.fresh_from = pass.pos[g.row0];   // rows of a sequence are consecutive: its first row's position
            uint64_t lo = UINT64_MAX, hi = 0;
            for (uint32_t r = g.row0 + a; r < g.row0 + b; r++) {
                u.rows.push_back((uint16_t)r);
                lo = std::min<uint64_t>(lo, row_lo(pass.pos[r], pp.window));
                hi = std::max<uint64_t>(hi, pass.pos[r]);
            }
            lo = std::max<uint64_t>(lo, pp.key_lo);
            if (pp.key_hi != UINT64_MAX) {
                if (pp.key_hi == 0) continue;
                hi = std::min<uint64_t>(hi, pp.key_hi - 1);
            }
            if (lo > hi) continue;   // no live key: the rows keep zero partials
            u.lo = (uint32_t)lo;
            u.hi = (uint32_t)hi;
            if (a == 0 && b == g.n) solos.push_back({units.size(), gi});
            units.push_back(std::move(u));
        }
    }

    uint64_t logical = 0;   // keys read if every unit streamed its own copy
    for (const Unit &u : units) logical += (uint64_t)u.hi - u.lo + 1;

    // 3. Shared prefixes.  Cluster whole-group units by their first page; within a cluster
    //    the common run of identical page ids is read once for all member rows.
    // Rows a shared item may hold.  The default keeps its query rows within one 16-row MMA tile
    // (16 / group sequences of one row each): such an item costs what a private one costs, its
    // padding rows become real work, and the other sharers find the pages in L2.
    const int share_rows = std::max(1, std::min(pp.max_rows, pp.share_rows > 0 ? pp.share_rows : std::max(1, 16 / pp.group)));
    int shared_groups = 0;
    if (pp.share_prefix && pp.max_rows > 1 && share_rows > 1 && solos.size() > 1) {
        std::unordered_map<uint64_t, std::vector<size_t>> by_first;   // first page id -> solos
        std::vector<uint64_t> order;
        for (size_t si = 0; si < solos.size(); si++) {
            const Unit &u = units[solos[si].unit];
            uint32_t first_pg = u.lo / PAGE;
            uint64_t key = ((uint64_t)first_pg << 32) | pass.pages[u.pt_off + first_pg];
            auto it = by_first.find(key);
            if (it == by_first.end()) {
                order.push_back(key);
                by_first[key] = {si};
            } else {
                it->second.push_back(si);
            }
        }
        std::vector<Unit> shared_units;
        for (uint64_t key : order) {
            const std::vector<size_t> &members = by_first[key];
            if (members.size() < 2) continue;
            // Pack members into clusters of at most max_rows rows.
            size_t at = 0;
            while (at < members.size()) {
                size_t end = at;
                size_t rows = 0;
                while (end < members.size() && rows + units[solos[members[end]].unit].rows.size() <= (size_t)share_rows) {
                    rows += units[solos[members[end]].unit].rows.size();
                    end++;
                }
                if (end - at < 2) {
                    at = std::max(end, at + 1);
                    continue;
                }
                // Common run of pages, starting at the first page of the latest-starting member.
                uint32_t pg0 = 0, pg_end = UINT32_MAX;
                for (size_t k = at; k < end; k++) {
                    const Unit &u = units[solos[members[k]].unit];
                    pg0 = std::max(pg0, u.lo / PAGE);
                    pg_end = std::min(pg_end, u.hi / PAGE + 1);   // pages this member has at all
                }
                const Unit &u0 = units[solos[members[at]].unit];
                uint32_t common = pg0;
                while (common < pg_end) {
                    uint32_t id = pass.pages[u0.pt_off + common];
                    bool same = true;
                    for (size_t k = at + 1; k < end && same; k++)
                        same = pass.pages[units[solos[members[k]].unit].pt_off + common] == id;
                    if (!same) break;
                    common++;
                }
                // A page that some member is still writing in this pass (its last, partly
                // filled page) is never shared by construction of the page tables: a shared
                // page is copied before it is written (kv.rs:299-326).
                if (common > pg0) {
                    Unit su;
                    su.pt_off = u0.pt_off;
                    su.fresh_from = UINT32_MAX;
                    for (size_t k = at; k < end; k++) su.fresh_from = std::min(su.fresh_from, units[solos[members[k]].unit].fresh_from);
                    su.reused = members.size() > end - at;   // other clusters read these pages too
                    uint32_t lo = UINT32_MAX, hi = 0;
                    for (size_t k = at; k < end; k++) {
                        Unit &u = units[solos[members[k]].unit];
                        for (uint16_t r : u.rows) su.rows.push_back(r);
                        lo = std::min(lo, u.lo);
                        // keys of the shared run this member can see
                        uint32_t h = std::min<uint32_t>(u.hi, common * PAGE - 1);
                        hi = std::max(hi, h);
                    }
                    su.lo = std::max<uint32_t>(lo, pg0 * PAGE);
                    su.hi = hi;
                    if (su.lo <= su.hi) {
                        // Members start after the shared run (or before it, for the keys in
                        // front of pg0, which stay private).
                        bool ok = true;
                        for (size_t k = at; k < end; k++)
                            if (units[solos[members[k]].unit].lo < pg0 * PAGE) ok = false;
                        if (ok) {
                            for (size_t k = at; k < end; k++) {
                                Unit &u = units[solos[members[k]].unit];
                                if (u.hi < common * PAGE) {
                                    u.rows.clear();   // wholly inside the shared run
                                } else {
                                    u.lo = std::max<uint32_t>(u.lo, common * PAGE);
                                }
                            }
                            shared_units.push_back(std::move(su));
                            shared_groups++;
                        }
                    }
                }
                at = end;
            }
        }
        // Shared units first: they are the long-running items.
        std::vector<Unit> all;
        for (Unit &u : shared_units) all.push_back(std::move(u));
        for (Unit &u : units)
            if (!u.rows.empty()) all.push_back(std::move(u));
        units.swap(all);
    }

    // Keys streamed and distinct keys streamed (for the plan's byte counts).
    std::vector<uint32_t> &seen = out.scratch_seen;   // (physical page, half) -> most keys read
    seen.assign(2 * (size_t)n_dense, 0);
    for (const Unit &u : units)
        for (uint32_t t = u.lo / TILE_KEYS; t <= u.hi / TILE_KEYS; t++) {
            const uint32_t a = std::max(u.lo, t * TILE_KEYS), b = std::min(u.hi, t * TILE_KEYS + TILE_KEYS - 1);
            uint32_t &sn = seen[((size_t)dense[u.pt_off + t * TILE_KEYS / PAGE] << 1) | (t & 1)];
            sn = std::max(sn, b - a + 1);
        }
    uint64_t uniq = 0;
    for (uint32_t v : seen) uniq += v;
    const int64_t per_key = (int64_t)2 * D * pp.esize * pp.hkv;   // K and V of every KV head

    // 3b. The short way.  The next decode step has the shape of the last one: the same rows over
    //     the same page tables, every row a key or so further, no run a tile longer.  Then the
    //     cut into spans, the partial slots and all but the two end tiles of every item stand as
    //     they are; only the key ranges move.  Building a plan from scratch costs several times
    //     what the rest of a decode step's host work does.
    const int params[10] = {pp.hkv, pp.group, pp.max_rows, pp.n_ctas, pp.share_prefix ? 1 : 0, pp.esize, pp.w32, pp.w64,
                            pp.item_cost, pp.min_piece};
    auto same_shape = [&]() -> bool {
        if (!out.sig_valid || !pp.resolve || !out.tile_items.empty()) return false;
        if (out.sig_rows_in_pass != T || out.sig_window != pp.window || pp.key_lo != 0 || pp.key_hi != UINT64_MAX) return false;
        if (memcmp(params, out.sig_params, sizeof params) != 0 || pp.share_rows != 0) return false;
        if (out.sig_units.size() != units.size() || out.sig_pages.size() != pass.pages.size()) return false;
        if (!pass.pages.empty() && memcmp(out.sig_pages.data(), pass.pages.data(), pass.pages.size() * 4) != 0) return false;
        size_t at = 0;
        for (size_t ui = 0; ui < units.size(); ui++) {
            const Unit &u = units[ui];
            const Plan::UnitSig &g = out.sig_units[ui];
            if (g.pt_off != u.pt_off || g.t0 != u.lo / TILE_KEYS || g.n != u.hi / TILE_KEYS - u.lo / TILE_KEYS + 1 ||
                g.n_rows != u.rows.size() || g.reused != (u.reused ? 1u : 0u) || g.fresh_tile != u.fresh_from / TILE_KEYS)
                return false;
            if (at + u.rows.size() > out.sig_unit_rows.size() ||
                memcmp(out.sig_unit_rows.data() + at, u.rows.data(), u.rows.size() * sizeof(uint16_t)) != 0)
                return false;
            at += u.rows.size();
        }
        return true;
    };
    if (same_shape()) {
        const uint32_t hkv = (uint32_t)pp.hkv;
        TileDesc *td = out.tiles.data();
        for (size_t i = 0; i < out.items.size(); i++) {
            Item &it = out.items[i];
            const Unit &u = units[out.item_unit[i]];
            it.key_lo = u.lo;
            it.key_hi = u.hi;
            it.flags = (u.reused ? 1u : 0u) | (u.fresh_from << 1);
            const uint32_t flags = u.reused ? TILE_REUSED : 0u;
            const uint32_t ends[2] = {it.tile_begin, it.tile_end - 1};
            for (int e = 0; e < 2; e++) {
                const uint32_t t = ends[e], k0 = t * TILE_KEYS;
                const uint32_t a = std::max(it.key_lo, k0), b = std::min(it.key_hi, k0 + TILE_KEYS - 1);
                TileDesc &d = td[out.item_tile0[i] + (t - it.tile_begin)];
                d.info = (t & 1u) | ((a - k0) << 1) | ((b - a + 1) << 8) | flags | (b >= u.fresh_from ? TILE_FRESH : 0u);
            }
            uint32_t *w = out.recs[i].w;
            for (int k = 0; k < it.n_rows; k++) {
                const uint32_t p = pass.pos[it.rows[k]];
                uint32_t *rw = w + IR_ROW0 + IR_ROW_WORDS * k;
                rw[IRR_KLO] = std::max(row_lo(p, pp.window), it.key_lo);
                rw[IRR_KHI] = std::min(p, it.key_hi);
            }
        }
        for (int c = 0; c < out.n_ctas; c++) {
            CtaPrologue &pr = out.prologue[c];
            for (uint32_t j = 0; j < (uint32_t)PROLOGUE_TILES && pr.hdr.tile_begin + j < pr.hdr.tile_end; j++)
                pr.first[j] = td[pr.hdr.tile_begin + j];
        }
        (void)hkv;
        out.info.unique_kv_bytes = (int64_t)uniq * per_key;
        out.info.logical_kv_bytes = (int64_t)logical * per_key;
        out.patched = true;
        return;
    }
    out.sig_valid = false;
    out.path = 0;
    out.n_ctas = 0;
    out.items.clear();
    out.item_unit.clear();
    out.cta_begin.clear();
    out.merges.clear();
    out.n_parts = 0;
    out.cta_hdr.clear();
    out.tiles.clear();
    out.prologue.clear();   // (recs keeps its records: every word that is read is rewritten below)
    out.single_use = false;
    out.has_empty_rows = false;
    out.info = yx_plan_info{};

    // 4. Cut the tile sequence (units x KV heads) into one contiguous span per CTA so that the
    //    most loaded CTA is as light as can be.  A CTA's load is what it was measured to be: a
    //    weight per tile (a tile of an item with many query rows costs more tensor work than its
    //    bytes alone) plus a fixed amount per item (queries in, triples merged and written).  The
    //    smallest limit under which the spans fit the CTAs is found by bisection; under a given
    //    limit every CTA is simply filled as far as the limit allows.  A piece of a run is at
    //    least `min_piece` tiles: a shorter one is not worth an item of its own.
    auto weight = [&](const Unit &u) -> uint64_t {
        int mt = padded_rows((int)u.rows.size() * pp.group);
        return mt == 16 ? 16u : (mt == 32 ? (uint64_t)std::max(pp.w32, 1) : (uint64_t)std::max(pp.w64, 1));
    };
    const uint64_t item_cost = (uint64_t)std::max(pp.item_cost, 0);
    const uint32_t min_piece = (uint32_t)std::max(pp.min_piece, 1);
    struct Run { uint32_t unit, t0, n; uint64_t w; };   // n tiles from t0, for each KV head
    std::vector<Run> runs;
    runs.reserve(units.size());
    uint64_t total_tiles = 0, total_cost = 0, floor_cost = 0;
    for (size_t ui = 0; ui < units.size(); ui++) {
        const Unit &u = units[ui];
        Run r{(uint32_t)ui, u.lo / TILE_KEYS, u.hi / TILE_KEYS - u.lo / TILE_KEYS + 1, weight(u)};
        // An item of one or two tiles is over before its successor's queries have arrived (1.8 us):
        // a run of them costs that per item, not its tiles' streaming time.
        if (r.n <= 2 && pp.resolve) r.w = r.n == 1 ? 42u : 29u;
        runs.push_back(r);
        total_tiles += (uint64_t)r.n * pp.hkv;
        total_cost += ((uint64_t)r.n * r.w + item_cost) * pp.hkv;
        floor_cost = std::max(floor_cost, item_cost + (uint64_t)std::min(r.n, min_piece) * r.w);
    }
    int n_ctas = (int)std::min<uint64_t>((uint64_t)std::max(1, pp.n_ctas), std::max<uint64_t>(total_tiles, 1));
    out.n_ctas = n_ctas;
    out.cta_begin.assign(n_ctas + 1, 0);
    // (a pass that the tiled kernel takes whole has nothing to merge)
    const bool merges_needed = !units.empty() || out.tile_items.empty();
    if (merges_needed) out.merges.assign((size_t)T * pp.hkv, Merge{0, 0});

    // How much of a run of `left` tiles goes into a CTA that holds `load` already, under `lim`:
    // 0 = none (close the CTA first, unless it is empty: then the limit is too small).
    auto take_under = [&](uint64_t lim, uint64_t load, uint64_t w, uint32_t left) -> uint32_t {
        if (load + item_cost + w > lim) return 0;
        uint64_t room = (lim - load - item_cost) / w;
        if (room >= left) return left;
        if (room < min_piece) return 0;
        if (left - room < min_piece) {           // the rest would be a crumb: leave it min_piece tiles
            if (left < 2 * min_piece) return 0;  // cannot be cut at all: all of it or none
            room = left - min_piece;
        }
        return (uint32_t)room;
    };
    // CTAs needed under `lim`, or n_ctas + 1 if some piece cannot be placed at all.
    auto ctas_under = [&](uint64_t lim) -> int {
        int used = 1;
        uint64_t load = 0;
        for (const Run &r : runs)
            for (int kh = 0; kh < pp.hkv; kh++) {
                uint32_t left = r.n;
                while (left > 0) {
                    const uint32_t take = take_under(lim, load, r.w, left);
                    if (take == 0) {
                        if (load == 0) return n_ctas + 1;
                        load = 0;
                        if (++used > n_ctas) return used;
                        continue;
                    }
                    load += item_cost + (uint64_t)take * r.w;
                    left -= take;
                }
            }
        return used;
    };
    // The smallest limit that fits, among the multiples of a tile's weight (so that the answer
    // does not depend on where the search starts).  The limit the plan object found last time is
    // tried first: a decode pass differs from the one before it by a key per row, and its answer
    // is the same or a step away, so the search is two or three passes over the runs instead of
    // a bisection from scratch.
    const uint64_t step = 16;
    auto up16 = [&](uint64_t x) { return (x + step - 1) / step * step; };
    const uint64_t lo_lim = up16(std::max<uint64_t>(floor_cost, (total_cost + n_ctas - 1) / n_ctas));
    uint64_t hi_lim = std::max<uint64_t>(total_cost, floor_cost);
    for (const Run &r : runs) hi_lim = std::max<uint64_t>(hi_lim, item_cost + (uint64_t)r.n * r.w);   // admits any run whole
    hi_lim = up16(hi_lim);
    uint64_t good, bad;   // a limit known to fit, and one known not to (both multiples of `step`)
    const uint64_t guess = out.last_limit >= lo_lim && out.last_limit <= hi_lim && out.last_limit % step == 0
                               ? out.last_limit : std::min(hi_lim, up16(lo_lim + lo_lim / 16));
    if (ctas_under(guess) <= n_ctas) {
        good = guess;
        bad = lo_lim - step;
        while (good > lo_lim) {             // walk down a tile at a time while it still fits
            if (ctas_under(good - step) > n_ctas) {
                bad = good - step;
                break;
            }
            good -= step;
        }
    } else {
        bad = guess;
        good = hi_lim;
        for (uint64_t up = step; bad + up < hi_lim; up *= 2) {   // gallop up to a limit that fits
            if (ctas_under(bad + up) <= n_ctas) {
                good = bad + up;
                break;
            }
            bad += up;
        }
        while (good - bad > step) {          // and close in
            const uint64_t mid = bad + (good - bad) / (2 * step) * step;
            if (ctas_under(mid) <= n_ctas) good = mid;
            else bad = mid;
        }
    }
    hi_lim = good;
    out.last_limit = good;
    const uint64_t lim = hi_lim;

    int cta = 0;
    uint64_t load = 0;
    for (const Run &r : runs) {
        const Unit &u = units[r.unit];
        const uint32_t t0 = r.t0, t1 = r.t0 + r.n;
        Item proto{};
        proto.key_lo = u.lo;
        proto.key_hi = u.hi;
        proto.pt_off = u.pt_off;
        proto.n_rows = (uint16_t)u.rows.size();
        proto.mt = (uint32_t)padded_rows((int)u.rows.size() * pp.group);
        proto.flags = (u.reused ? 1u : 0u) | (u.fresh_from << 1);   // bit 0: reused; the rest: fresh_from (positions < 2^31)
        for (size_t k = 0; k < u.rows.size(); k++) proto.rows[k] = u.rows[k];
        for (int kh = 0; kh < pp.hkv; kh++) {
            uint32_t t = t0;
            while (t < t1) {
                uint32_t take = take_under(lim, load, r.w, t1 - t);
                if (take == 0) {
                    if (load > 0 && cta < n_ctas - 1) {
                        cta++;
                        out.cta_begin[cta] = (uint32_t)out.items.size();
                        load = 0;
                        continue;
                    }
                    take = t1 - t;   // cannot happen under a feasible limit; never lose tiles
                }
                Item it = proto;
                it.tile_begin = t;
                it.tile_end = t + take;
                it.kv_head = (uint16_t)kh;
                for (size_t k = 0; k < u.rows.size(); k++) out.merges[(size_t)u.rows[k] * pp.hkv + kh].count++;
                out.items.push_back(it);
                out.item_unit.push_back(r.unit);
                load += item_cost + (uint64_t)take * r.w;
                t += take;
            }
        }
    }
    for (int c = cta + 1; c <= n_ctas; c++) out.cta_begin[c] = (uint32_t)out.items.size();

    // 5. Partial slots: contiguous per (row, kv head).
    uint32_t next = 0;
    for (Merge &m : out.merges) {
        m.first = next;
        next += m.count;
        m.count = 0;
    }
    out.n_parts = next;
    for (Item &it : out.items)
        for (int r = 0; r < it.n_rows; r++) {
            Merge &m = out.merges[(size_t)it.rows[r] * pp.hkv + it.kv_head];
            it.part[r] = m.first + m.count++;
        }
    for (const Merge &m : out.merges)
        if (m.count == 0) out.has_empty_rows = true;
    if (!merges_needed) out.has_empty_rows = false;

    // 6. The resolved form: page tables walked here, once, instead of by every CTA.  (Plain
    //    pointers into arrays sized up front: this loop is most of the cost of planning a decode
    //    pass, and it runs on the critical path of every pass.)
    if (pp.resolve) {
        out.cta_hdr.resize(n_ctas);
        if (out.recs.size() < out.items.size()) out.recs.resize(out.items.size());   // words a record does not use keep old values
        out.tiles.resize((size_t)total_tiles);
        out.item_tile0.resize(out.items.size());
        TileDesc *td = out.tiles.data();
        const uint32_t *pages = pass.pages.data(), *pos = pass.pos.data();
        const Item *items = out.items.data();
        const Merge *merges = out.merges.data();
        ItemRec *recs = out.recs.data();
        const uint32_t hkv = (uint32_t)pp.hkv;
        size_t n_tiles = 0;
        for (int c = 0; c < n_ctas; c++) {
            CtaHdr &h = out.cta_hdr[c];
            h.item_begin = out.cta_begin[c];
            h.item_end = out.cta_begin[c + 1];
            h.tile_begin = (uint32_t)n_tiles;
            for (uint32_t i = h.item_begin; i < h.item_end; i++) {
                const Item &it = items[i];
                out.item_tile0[i] = (uint32_t)n_tiles;
                const uint32_t *pt = pages + it.pt_off;
                const uint32_t flags = (it.flags & 1u) ? TILE_REUSED : 0u, fresh_from = it.flags >> 1;
                for (uint32_t t = it.tile_begin; t < it.tile_end; t++) {
                    const uint32_t k0 = t * TILE_KEYS;
                    const uint32_t a = std::max(it.key_lo, k0), b = std::min(it.key_hi, k0 + TILE_KEYS - 1);
                    TileDesc &d = td[n_tiles++];
                    d.block = pt[t >> 1] * hkv + it.kv_head;
                    d.info = (t & 1u) | ((a - k0) << 1) | ((b - a + 1) << 8) | flags | (b >= fresh_from ? TILE_FRESH : 0u);
                }
                uint32_t *w = recs[i].w;
                w[IR_TILES] = it.tile_end - it.tile_begin;
                w[IR_KEY0] = it.tile_begin * TILE_KEYS;
                w[IR_HEAD_ROWS] = (uint32_t)it.kv_head | ((uint32_t)it.n_rows << 16);
                w[IR_MT] = it.mt;
                for (int k = 0; k < it.n_rows; k++) {
                    const uint32_t row = it.rows[k], p = pos[row];
                    const Merge &m = merges[(size_t)row * hkv + it.kv_head];
                    uint32_t *rw = w + IR_ROW0 + IR_ROW_WORDS * k;
                    rw[IRR_KLO] = std::max(row_lo(p, pp.window), it.key_lo);
                    rw[IRR_KHI] = std::min(p, it.key_hi);
                    rw[IRR_PART] = it.part[k];
                    rw[IRR_ROW] = row;
                    rw[IRR_FIRST] = m.first;
                    rw[IRR_COUNT] = m.count;
                }
            }
            h.tile_end = (uint32_t)n_tiles;
        }
        out.tiles.resize(n_tiles);
        out.prologue.assign(n_ctas, CtaPrologue{});
        for (int c = 0; c < n_ctas; c++) {
            CtaPrologue &pr = out.prologue[c];
            pr.hdr = out.cta_hdr[c];
            for (uint32_t j = 0; j < (uint32_t)PROLOGUE_TILES && pr.hdr.tile_begin + j < pr.hdr.tile_end; j++)
                pr.first[j] = out.tiles[pr.hdr.tile_begin + j];
            if (pr.hdr.item_begin < pr.hdr.item_end) {
                const Item &it = out.items[pr.hdr.item_begin];
                pr.head_rows = (uint32_t)it.kv_head | ((uint32_t)it.n_rows << 16);
                pr.mt = it.mt;
                for (int r = 0; r < MAX_ITEM_ROWS; r++) pr.rows[r] = it.rows[r];
            }
        }
    }

    out.info.n_ctas = n_ctas;
    out.info.n_items = (int)out.items.size();
    out.info.n_parts = (int)out.n_parts;
    out.info.tiles = (int64_t)total_tiles;
    out.info.unique_kv_bytes = (int64_t)uniq * per_key;
    out.info.logical_kv_bytes = (int64_t)logical * per_key;
    out.info.shared_groups = shared_groups;
    // Tiles not marked as reused are copied with an evict-first hint when each of them is read
    // by one item only: nothing is gained by keeping those K/V lines in L2.
    {
        std::vector<uint32_t> once(2 * (size_t)n_dense, 0);   // (physical page, half) -> most keys read by unmarked items
        uint64_t streamed = 0;
        for (const Item &it : out.items) {
            if ((it.flags & 1u) || it.kv_head != 0) continue;
            for (uint32_t t = it.tile_begin; t < it.tile_end; t++) {
                uint32_t n = std::min(it.key_hi, t * TILE_KEYS + TILE_KEYS - 1) - std::max(it.key_lo, t * TILE_KEYS) + 1;
                streamed += n;
                uint32_t &m = once[((size_t)dense[it.pt_off + t * TILE_KEYS / PAGE] << 1) | (t & 1)];
                m = std::max(m, n);
            }
        }
        uint64_t distinct = 0;
        for (uint32_t v : once) distinct += v;
        out.single_use = streamed <= distinct;
    }
    // What this plan was built from, for the short way next time.
    if (pp.resolve && out.tile_items.empty()) {
        out.sig_rows_in_pass = T;
        out.sig_window = pp.window;
        memcpy(out.sig_params, params, sizeof params);
        out.sig_pages.assign(pass.pages.begin(), pass.pages.end());
        out.sig_units.clear();
        out.sig_unit_rows.clear();
        for (const Unit &u : units) {
            out.sig_units.push_back({u.pt_off, u.lo / TILE_KEYS, u.hi / TILE_KEYS - u.lo / TILE_KEYS + 1, (uint32_t)u.rows.size(),
                                     u.reused ? 1u : 0u, u.fresh_from / TILE_KEYS});
            out.sig_unit_rows.insert(out.sig_unit_rows.end(), u.rows.begin(), u.rows.end());
        }
        out.sig_valid = pp.share_rows == 0;
    }
}

}  // namespace yx
