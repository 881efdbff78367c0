"""The host-side KvCache restatement against the reference's own expectations
(crates/yaxus-model/src/kv.rs:365-403, crates/yaxus-model/src/lib.rs:725-775)."""
import numpy as np
import pytest

from yaxus_b200.kvcache import PAGE, KvCache, KvCacheError, slot


def run(kv, seq, toks):
    kv.append([(seq, list(toks))])
    return kv.take_copies()


def test_a_shared_page_is_copied_before_it_is_written():
    # kv.rs:366-383
    kv = KvCache(4, 1024)
    a = kv.new_seq()
    assert run(kv, a, range(150)) == []
    b = kv.fork(a, 140)
    copies = kv.take_copies()
    assert len(copies) == 1                       # page 0 shared, page 1 (partly used) copied
    assert (kv.seq_len(b), kv.free_pages()) == (140, 1)
    c = kv.fork(a, PAGE)
    assert kv.take_copies() == []
    kv.truncate(c, 100)
    copies = run(kv, c, [7])
    assert len(copies) == 1 and copies[0][0] != copies[0][1]
    assert len(kv.seq_tokens(c)) == 101


def test_kept_sequences_are_evicted_least_recent_first():
    # kv.rs:385-403
    kv = KvCache(3, 1024)
    a, b = kv.new_seq(), kv.new_seq()
    run(kv, a, [1] * 20)
    run(kv, b, [2] * 20)
    kv.finish(a)
    kv.finish(b)
    assert kv.free_pages() == 1
    c, reused = kv.begin([1] * 30)
    assert reused == 20
    kv.free_seq(c)
    d = kv.new_seq()
    run(kv, d, [3] * (2 * PAGE))
    assert kv.seq_len(b) == 0
    assert kv.seq_len(a) == 20


def test_reuse_falls_back_when_the_arena_is_full():
    # lib.rs:725-743: two pages, both held by a finished sequence of 130 tokens.
    kv = KvCache(2, 8192)
    a = list(range(130))
    s = kv.new_seq()
    run(kv, s, a)
    kv.finish(s)
    assert kv.free_pages() == 0
    b = a[:129] + [500, 501]
    s2, reused = kv.begin(b)
    assert reused == PAGE       # the whole first page is shared, the rest computed
    run(kv, s2, b[reused:])
    assert kv.seq_len(s2) == len(b)
    assert list(kv.seq_tokens(s2)) == b


def test_reuse_shares_whole_pages_without_a_free_page():
    # lib.rs:745-758
    kv = KvCache(2, 8192)
    a = list(range(200))
    s = kv.new_seq()
    run(kv, s, a)
    kv.finish(s)
    b = a[:PAGE] + [999]
    s2, reused = kv.begin(b)
    assert reused == PAGE
    assert kv.take_copies() == []
    run(kv, s2, b[reused:])
    assert list(kv.seq_tokens(s2)) == b


def test_a_pass_beyond_max_pos_keeps_the_prefix_cache():
    # lib.rs:760-775
    kv = KvCache(2, 200)
    s = kv.new_seq()
    run(kv, s, range(100))
    kv.finish(s)
    free = kv.free_pages()
    s2, _ = kv.begin([7] * 20)
    with pytest.raises(KvCacheError):
        kv.append([(s2, [7] * 300)])
    assert kv.free_pages() == free


def test_pass_meta_and_allocation_order():
    # Pages are handed out in ascending order first, then last-freed-first (kv.rs:55-71);
    # kv_slot is slot(pages, pos) (kv.rs:343); rows of an item are consecutive.
    kv = KvCache(6, 4096)
    a, b = kv.new_seq(), kv.new_seq()
    m = kv.append([(a, list(range(130))), (b, [9, 9, 9])])
    assert list(kv.seq_pages(a)) == [0, 1] and list(kv.seq_pages(b)) == [2]
    assert m.rows == 133 and list(m.last) == [129, 132]
    assert list(m.pt_off[:130]) == [0] * 130 and list(m.pt_off[130:]) == [2] * 3
    assert list(m.pages) == [0, 1, 2]
    for r in range(m.rows):
        assert m.kv_slot[r] == m.slot(r, int(m.pos[r]))
    assert m.kv_slot[129] == slot([0, 1], 129) == 128 + 1
    kv.free_seq(a)                       # frees 0 then 1: the free list pops 1 first
    c = kv.new_seq()
    kv.append([(c, [1])])
    assert list(kv.seq_pages(c)) == [1]


def test_refcounts_stay_consistent_under_random_traffic():
    rng = np.random.default_rng(0)
    kv = KvCache(24, 2048)
    kv.set_prefix_reuse(False)
    live = []
    for _ in range(300):
        op = rng.integers(0, 5)
        try:
            if op == 0 or not live:
                s = kv.new_seq()
                live.append(s)   # a failed append still leaves the sequence (and pages it got)
                kv.append([(s, list(rng.integers(0, 50, rng.integers(1, 200))))])
            elif op == 1:
                s = live[rng.integers(len(live))]
                kv.append([(s, list(rng.integers(0, 50, rng.integers(1, 40))))])
            elif op == 2:
                s = live[rng.integers(len(live))]
                live.append(kv.fork(s, int(rng.integers(0, kv.seq_len(s) + 1))))
            elif op == 3:
                s = live[rng.integers(len(live))]
                kv.truncate(s, int(rng.integers(0, kv.seq_len(s) + 1)))
            else:
                s = live.pop(rng.integers(len(live)))
                kv.free_seq(s)
        except KvCacheError:
            pass
        for src, dst in kv.take_copies():
            assert src != dst
        # every page's reference count equals the number of sequences naming it
        counts = np.zeros(kv.total_pages(), np.int64)
        for s in live:
            for p in kv.seq_pages(s):
                counts[p] += 1
        for p in range(kv.total_pages()):
            assert kv.page_refs(p) == counts[p]
        assert kv.free_pages() == int((counts == 0).sum())
    for s in live:
        kv.free_seq(s)
    assert kv.free_pages() == kv.total_pages()
