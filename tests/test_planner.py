"""The split-key planner (host side of the attention kernels): every (row, KV head, visible
key) is covered by exactly one item, CTA spans are balanced, partial slots are contiguous.
Expectations on *when* to split come from the reference's planner test
(crates/yaxus-backend-gpu/src/plan.rs:427-443): decode passes are split across keys."""
import ctypes

import numpy as np
import pytest

from yaxus_b200 import _lib
from yaxus_b200 import workloads as W
from yaxus_b200.kvcache import PassMeta

U64_MAX = (1 << 64) - 1


def probe(meta, hkv, group, window=0, key_lo=0, key_hi=U64_MAX, max_rows=16, n_ctas=148, share=1, esize=2, cost32=16,
          cost64=32, item_cost=0, min_piece=1):
    L = _lib.cuda_lib()
    info = _lib.PlanInfo()
    cap = 200000
    buf = np.zeros(cap * _lib.PROBE_ITEM_WORDS, np.uint32)
    p = lambda a: np.ascontiguousarray(a, np.uint32).ctypes.data_as(ctypes.POINTER(ctypes.c_uint32))
    pos, off, pages = (np.ascontiguousarray(x, np.uint32) for x in (meta.pos, meta.pt_off, meta.pages))
    rc = L.yx_plan_probe(len(pos), p(pos), p(off), p(pages), len(pages), hkv, group, window or 0, key_lo, key_hi,
                         max_rows, n_ctas, share, esize, cost32, cost64, item_cost, min_piece, ctypes.byref(info), p(buf), cap)
    assert rc == 0
    items = buf[: info.n_items * _lib.PROBE_ITEM_WORDS].reshape(info.n_items, _lib.PROBE_ITEM_WORDS)
    return info, items


def check_cover(meta, items, hkv, window, key_lo=0, key_hi=U64_MAX):
    T = meta.rows
    seen = {}
    for it in items:
        tb, te, klo, khi, pt, kvh, nr = (int(x) for x in it[:7])
        for r in range(nr):
            row = int(it[9 + r])
            p = int(meta.pos[row])
            lo = max(0, p + 1 - window) if window else 0
            a = max(lo, klo, tb * 64, key_lo)
            b = min(p, khi, te * 64 - 1, key_hi - 1)
            # the item's page table must agree with the row's over the keys it reads for it
            for key in range(a, b + 1, 64):
                assert meta.pages[pt + key // 128] == meta.pages[int(meta.pt_off[row]) + key // 128]
            if a <= b:
                seen.setdefault((row, kvh), []).append((a, b))
    for row in range(T):
        p = int(meta.pos[row])
        lo = max(0, p + 1 - window) if window else 0
        lo, hi = max(lo, key_lo), min(p, key_hi - 1)
        for kvh in range(hkv):
            spans = sorted(seen.get((row, kvh), []))
            if lo > hi:
                assert not spans
                continue
            assert spans and spans[0][0] == lo and spans[-1][1] == hi, (row, kvh, spans, lo, hi)
            for (a0, b0), (a1, b1) in zip(spans[:-1], spans[1:]):
                assert a1 == b0 + 1   # no gap, no overlap


def check_slots(items, info, group_rows):
    used = set()
    for it in items:
        nr, kvh = int(it[6]), int(it[5])
        for r in range(nr):
            s = int(it[9 + 16 + r])
            assert s < info.n_parts and s not in used
            used.add(s)
    assert len(used) == info.n_parts


def check_balance(items, info, cost32=16, cost64=32, item_cost=0, min_piece=1):
    """The most loaded CTA (tiles weighted by the item's padded rows, plus a fixed cost per item)
    carries at most a few tiles more than an even share: the planner minimises the maximum, and
    what that leaves over makes the last CTAs lighter, never heavier."""
    w = {16: 16, 32: cost32, 64: cost64}
    per = np.zeros(info.n_ctas, np.int64)
    per_items = np.zeros(info.n_ctas, np.int64)
    tiles = 0
    for it in items:
        n = int(it[1]) - int(it[0])
        tiles += n
        per[int(it[8])] += n * w[int(it[7])] + item_cost
        per_items[int(it[8])] += 1
    assert tiles == info.tiles
    if info.tiles >= info.n_ctas:
        share = -(-int(per.sum()) // info.n_ctas)
        assert per.max() <= share + (min_piece + 2) * max(w.values()) + 2 * item_cost, (per.max(), share)
    return per_items


@pytest.mark.parametrize("share", [0, 1, 16])
def test_batched_decode_plan(share):
    # share: 0 off, 1 the default (a shared item holds 16 / group = 4 one-row sequences, one
    # 16-row MMA tile), 16: all sixteen sequences in one item of 64 padded rows.
    s = W.batched_decode(fill=False)
    info, items = probe(s.meta, s.hkv, s.hq // s.hkv, share=share)
    check_cover(s.meta, items, s.hkv, None)
    check_slots(items, info, 1)
    check_balance(items, info)
    assert info.n_ctas == 148
    assert info.logical_kv_bytes == s.logical_kv_bytes()
    assert info.unique_kv_bytes == s.unique_kv_bytes()
    tile_bytes = 64 * 2 * 128 * 2
    prefix_tiles = 1536 // 64 * s.hkv
    if share == 16:
        assert info.shared_groups == 1
        # the shared prefix is streamed once: tiles ~ unique tokens / 64 per KV head
        assert info.tiles * tile_bytes < 1.02 * s.unique_kv_bytes() + 16 * 8 * tile_bytes
        assert any(int(it[6]) == 16 and int(it[7]) == 64 for it in items)
    elif share == 1:
        assert info.shared_groups == 4
        # ... four times, by items that each fill one 16-row tile
        assert all(int(it[7]) == 16 for it in items)
        assert any(int(it[6]) == 4 for it in items)
        assert info.tiles * tile_bytes < 1.02 * s.unique_kv_bytes() + (16 * 8 + 3 * prefix_tiles) * tile_bytes
    else:
        assert info.shared_groups == 0
        assert all(int(it[6]) == 1 and int(it[7]) == 16 for it in items)


def test_verify_plan_groups_rows_of_a_sequence():
    s = W.verify(fill=False)
    info, items = probe(s.meta, s.hkv, 4)
    check_cover(s.meta, items, s.hkv, None)
    check_slots(items, info, 5)
    check_balance(items, info)
    assert all(int(it[6]) == 5 and int(it[7]) == 32 for it in items)   # 5 rows x 4 heads -> 32 padded rows


@pytest.mark.parametrize("window", [None, 100, 2048])
def test_windows_and_ragged_passes(window):
    rows = [(0, p) for p in range(300, 340)] + [(1, 5)] + [(2, 4095)] + [(3, 0)]
    tables = [np.arange(10, 13), np.array([40]), np.arange(50, 82), np.array([7])]
    meta = PassMeta.from_rows(rows, tables)
    for max_rows in (1, 4, 16):
        info, items = probe(meta, 2, 4, window=window, max_rows=max_rows, n_ctas=37)
        check_cover(meta, items, 2, window)
        check_slots(items, info, max_rows)
        check_balance(items, info)


def test_key_range_restriction():
    s = W.long_decode(ctx=8192, fill=False)
    for world in (1, 2, 4, 8):
        for rank in range(world):
            _, _, klo, khi = W.partition_pages(64, world, rank)
            for window in (None, 2048):
                info, items = probe(s.meta, 8, 4, window=window, key_lo=klo, key_hi=khi)
                check_cover(s.meta, items, 8, window, klo, khi)
                check_balance(items, info)
                if window and khi <= 8192 - 2048:
                    assert info.n_items == 0 and info.n_parts == 0   # a rank with no live key


@pytest.mark.parametrize("item_cost,min_piece", [(48, 4), (0, 8), (200, 1)])
def test_item_cost_and_minimum_piece(item_cost, min_piece):
    # The production settings: a fixed cost per item and no pieces of fewer than min_piece
    # tiles (unless a whole run is that short).  Coverage stays exact; balance is looser.
    for s in (W.batched_decode(fill=False), W.verify(fill=False)):
        info, items = probe(s.meta, s.hkv, s.hq // s.hkv, item_cost=item_cost, min_piece=min_piece)
        check_cover(s.meta, items, s.hkv, None)
        check_slots(items, info, 1)
        runs = {}
        for it in items:
            runs.setdefault((int(it[4]), int(it[5]), int(it[2])), []).append(int(it[1]) - int(it[0]))
        for pieces in runs.values():
            if sum(pieces) >= min_piece:
                assert min(pieces) >= min_piece
        per = np.zeros(info.n_ctas, np.int64)
        for it in items:
            per[int(it[8])] += int(it[1]) - int(it[0])
        assert per.max() <= info.tiles / info.n_ctas + 2 * min_piece + item_cost / 16 * 3 + 2


def test_decode_is_split_across_keys():
    # plan.rs:432-434: a single decode row over a long context is cut into many pieces.
    meta = PassMeta.from_rows([(0, 1000)], [np.arange(8)])
    info, items = probe(meta, 8, 2)
    assert info.n_items == info.tiles == 8 * 16 and info.n_ctas == 128


def test_empty_pass():
    meta = PassMeta()
    info, items = probe(meta, 8, 4)
    assert info.n_items == 0 and info.tiles == 0


@pytest.mark.parametrize("window", [0, 2048, 100])
def test_patched_plans_equal_plans_built_from_scratch(window):
    # A decode loop: every step each row is one key further.  Most steps have the shape of the step
    # before (no run a tile longer) and the plan is patched in place; it must be, word for word, the
    # plan a fresh planner builds for the same pass.  The page tables have room for the steps.
    rng = np.random.default_rng(3)
    ctx_len = [1536 + int(x) for x in rng.integers(0, 2561, 16)]
    tables, nxt = [], 12
    for c in ctx_len:
        n = (c + 200) // 128 + 1
        tables.append(np.array(list(range(12)) + list(range(nxt, nxt + n - 12)), np.uint32))
        nxt += n - 12
    from yaxus_b200.kvcache import PassMeta
    meta = PassMeta.from_rows([(sq, ctx_len[sq]) for sq in range(16)], tables)
    L = _lib.cuda_lib()
    p = lambda a: np.ascontiguousarray(a, np.uint32).ctypes.data_as(ctypes.POINTER(ctypes.c_uint32))
    pos, off, pages = (np.ascontiguousarray(x, np.uint32) for x in (meta.pos, meta.pt_off, meta.pages))
    patched = ctypes.c_int(0)
    differing = L.yx_hook_plan_steps(len(pos), p(pos), p(off), p(pages), len(pages), 8, 4, window, 8, 148, 150, ctypes.byref(patched))
    assert differing == 0
    assert 75 <= patched.value < 150      # a row crosses a tile every 64 steps: most steps are patched, not all
