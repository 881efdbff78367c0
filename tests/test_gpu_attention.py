"""Attention on the GPU against the CPU oracle on the same seeded inputs."""
import os

import numpy as np
import pytest
import torch

from oracle.check import ABS_TOL, assert_close, dev, layers_for, load, oracle_arenas, oracle_step, run_step
from yaxus_b200 import workloads as W
from yaxus_b200._lib import BF16, F16, F32, PAGE
from yaxus_b200.backend import LayerMeta, Rope
from yaxus_b200.kvcache import PassMeta

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kv_dtype,tol", [(F32, 2e-5), (F16, ABS_TOL), (BF16, ABS_TOL)])
@pytest.mark.parametrize("window", [None, 16])
def test_reference_attention_test_shape(backend, oracle, kv_dtype, tol, window):
    # paged_attention_matches_dense_attention (crates/yaxus-backend-cpu/src/lib.rs:676-714)
    # through Backend::attention, at head_dim 128: two sequences on pages [[3,1],[0]], lengths
    # 140 and 9, two passes (100+4 rows, then 40+5) so the second reads keys the first wrote
    # across a page boundary; inputs from the reference's own value generator.
    hq, hkv, d, eps = 4, 2, 128, 1e-6
    cols = (hq + 2 * hkv) * d
    rope = Rope(np.resize(np.array([1.0, 0.3, 0.05, 0.01], np.float32), 64), 1.1)
    layer = LayerMeta(index=0, window=window, rope=rope)
    kv = backend.new_kv(hkv, [layer], 4, 1024, kv_dtype)
    tables = [np.array([3, 1], np.uint32), np.array([0], np.uint32)]
    lens = [140, 9]
    qkv = [[oracle.values(cols, s * 1000 + p) for p in range(n)] for s, n in enumerate(lens)]
    K = np.zeros((4 * PAGE, hkv * d), np.float32)
    V = np.zeros_like(K)
    norm = np.zeros(d, np.float32)
    first = [(0, p) for p in range(100)] + [(1, p) for p in range(4)]
    second = [(0, p) for p in range(100, 140)] + [(1, p) for p in range(4, 9)]
    for rows in (first, second):
        meta = PassMeta.from_rows(rows, tables)
        x = np.stack([qkv[s][p] for s, p in rows])
        backend.begin_pass(meta)
        got = backend.to_host(backend.attention(dev(backend, x), dev(backend, norm), dev(backend, norm), kv, hq, eps, layer))
        q = oracle.write_rows(x, meta.pos, meta.kv_slot, norm, norm, hq, hkv, d, eps, rope.inv_freq, rope.concentration,
                              K, V, store_dtype=kv_dtype)
        want = oracle.attend(q, meta.pos, meta.pt_off, meta.pages, hq, hkv, d, window, K, V)
        assert_close(got, want, abs_tol=tol, what=f"window {window}")
    # the cache holds what write_rows wrote, at the slots PassMeta named
    k_dev, v_dev = backend.read_pages(kv, 0, 0, 4)
    assert np.abs(W.from_bits(k_dev, kv_dtype) - K).max() <= (1e-6 if kv_dtype == F32 else 2e-2)
    assert np.array_equal(W.from_bits(v_dev, kv_dtype), V)   # v is copied, not transformed
    kv.close()


@pytest.mark.parametrize("kv_dtype,tol", [(F32, 2e-5), (F16, ABS_TOL), (BF16, ABS_TOL)])
def test_golden_fixture(backend, kv_dtype, tol):
    # tests/golden/attention_small.npz: a 30-row chunk across a page boundary, a decode row and
    # five verification rows in one pass, with nonzero norm weights and standard RoPE.
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "attention_small.npz"))
    hq, hkv, eps = int(g["hq"]), int(g["hkv"]), float(g["eps"])
    meta = PassMeta(np.zeros(len(g["pos"]), np.uint32), g["pos"], g["kv_slot"], g["pt_off"], g["pages"])
    for tag in ("full", "win"):
        window = None if tag == "full" else int(g["window"])
        layer = LayerMeta(index=0, window=window, rope=Rope(g["inv_freq"], float(g["conc"])))
        kv = backend.new_kv(hkv, [layer], 5, 1024, kv_dtype)
        backend.write_pages(kv, 0, 0, W.to_bits(g["K0"], kv_dtype), W.to_bits(g["V0"], kv_dtype))
        backend.begin_pass(meta)
        got = backend.to_host(backend.attention(dev(backend, g["qkv"]), dev(backend, g["q_norm"]),
                                                dev(backend, g["k_norm"]), kv, hq, eps, layer))
        # 16-bit caches round K and V on the way in: the fixture holds the reference algorithm's
        # result on the rounded cache for each storage type
        want = g[f"out_{tag}"] if kv_dtype == F32 else g[f"out_{tag}_{'f16' if kv_dtype == F16 else 'bf16'}"]
        assert_close(got, want, abs_tol=tol, what=tag)
        kv.close()


def test_single_sequence_decode_f32(backend, oracle):
    # 1 query token, 16 query / 4 KV heads, 1024 keys in an f32 cache on permuted pages.
    s = W.single_decode()
    kv = load(backend, s)
    got = run_step(backend, kv, s)
    assert backend.last_plan().path == 1
    assert_close(got, oracle_step(oracle, s), abs_tol=2e-5, what="single decode")
    kv.close()


@pytest.mark.parametrize("share,share_rows,groups,q16", [(1, 0, 4, False), (1, 16, 2, False), (1, 16, 1, True),
                                                       (1, 8, 2, False), (2, 0, 0, False)])
@pytest.mark.parametrize("kv_dtype", [F16, BF16])
def test_batched_decode_shared_prefix(backend, oracle, share, share_rows, groups, q16, kv_dtype):
    # 16 sequences over a shared 1536-token prefix (same physical pages) with private
    # suffixes of 0..2560 tokens; 32 query / 8 KV heads.  The prefix is read by items of 4
    # sequences (the default), of 8 (the most f32 query rows an item holds: 32), of all 16
    # (16-bit queries: 64 rows), or by every sequence on its own.
    s = W.batched_decode(kv_dtype=kv_dtype)
    kv = load(backend, s)
    backend.set_tuning(share_prefix=share, share_rows=share_rows)
    qt = (torch.float16 if kv_dtype == F16 else torch.bfloat16) if q16 else torch.float32
    got = run_step(backend, kv, s, q_dtype=qt)
    info = backend.last_plan()
    backend.set_tuning()
    assert info.path == 2 and info.shared_groups == groups
    assert info.unique_kv_bytes == s.unique_kv_bytes()
    q = W.round_through(s.q, kv_dtype) if q16 else None
    assert_close(got, oracle_step(oracle, s, q=q), what=f"batched decode share={share}")
    kv.close()


def test_tensor_and_simt_kernels_agree(backend, oracle):
    s = W.batched_decode(seed=77, n_seq=7, prefix=256, max_suffix=700, hq=16, hkv=4)
    kv = load(backend, s)
    a = run_step(backend, kv, s)
    backend.set_tuning(force_path=1)
    b = run_step(backend, kv, s)
    assert backend.last_plan().path == 1
    backend.set_tuning()
    ref = oracle_step(oracle, s)
    assert_close(b, ref, abs_tol=5e-5, what="simt")
    assert_close(a, ref, what="tensor")
    kv.close()


@pytest.mark.parametrize("kv_dtype", [F16, BF16])
def test_speculative_verification(backend, oracle, kv_dtype):
    # 16 sequences x 5 rows (1 accepted + 4 drafts) after 2048 cached tokens: all rows' K/V
    # are appended first, then each row attends to keys <= its own position.
    s = W.verify(kv_dtype=kv_dtype)
    kv = load(backend, s)
    got = run_step(backend, kv, s)
    k_dev, v_dev = backend.read_pages(kv, 0, 0, s.arena_pages)
    K, V = oracle_arenas(oracle, s)
    assert np.array_equal(W.from_bits(k_dev, kv_dtype), K) and np.array_equal(W.from_bits(v_dev, kv_dtype), V)
    assert_close(got, oracle_step(oracle, s), what="verify")
    kv.close()


@pytest.mark.parametrize("rows", [17, 40, 130])
def test_many_rows_per_sequence(backend, oracle, rows):
    # Prompt-like passes (more rows than one item holds) through the split-key kernel.
    s = W.build("chunk", 5, 8, 2, BF16, [200, 0, 513], [rows, rows // 2, 3])
    kv = load(backend, s)
    got = run_step(backend, kv, s, q_dtype=torch.bfloat16)
    q = W.round_through(s.q, BF16)
    assert_close(got, oracle_step(oracle, s, q=q), what=f"{rows} rows")
    kv.close()


@pytest.mark.parametrize("hq,hkv", [(4, 4), (8, 1), (16, 1), (24, 4), (32, 4)])
def test_head_groupings(backend, oracle, hq, hkv):
    # group sizes 1, 8, 16, 6, 8 (the reference compiles split kernels for groups up to 16,
    # crates/yaxus-backend-gpu/src/plan.rs:240).
    s = W.build("heads", 13, hq, hkv, F16, [300, 129, 5], [1, 2, 1])
    kv = load(backend, s)
    got = run_step(backend, kv, s)
    assert_close(got, oracle_step(oracle, s), what=f"hq {hq} hkv {hkv}")
    kv.close()


@pytest.mark.parametrize("kv_dtype", [F32, F16])
@pytest.mark.parametrize("window", [1, 64, 100, 2048])
def test_sliding_window(backend, oracle, kv_dtype, window):
    # LayerMeta.window: the query at p sees keys in (p - window, p] (config.rs:167).
    s = W.build("win", 17, 8, 2, kv_dtype, [700, 63, 0, 128], [4, 1, 1, 2], window=window)
    kv = load(backend, s)
    got = run_step(backend, kv, s)            # window = -1: the layer's own
    assert_close(got, oracle_step(oracle, s), abs_tol=2e-5 if kv_dtype == F32 else ABS_TOL, what=f"window {window}")
    got = run_step(backend, kv, s, window=0)  # explicit override: no window
    assert_close(got, oracle_step(oracle, s, window=None), abs_tol=2e-5 if kv_dtype == F32 else ABS_TOL, what="override")
    kv.close()


def test_first_token_and_page_edges(backend, oracle):
    # Positions 0, 127, 128 and 255: one key, a full page, the first key of the next page.
    for ctx in (0, 127, 128, 255, 256):
        s = W.build("edge", 100 + ctx, 8, 2, F16, [ctx], [1])
        kv = load(backend, s)
        got = run_step(backend, kv, s)
        assert_close(got, oracle_step(oracle, s), what=f"ctx {ctx}")
        kv.close()


def test_poisoned_unused_slots_are_never_read(backend, oracle):
    # Slots past a sequence's length hold NaN here; the reference never reads keys > pos
    # (cpu lib.rs:399-406), so the result must not change.
    s = W.batched_decode(seed=31, n_seq=5, prefix=256, max_suffix=300, hq=8, hkv=2)
    nan16 = np.uint16(0x7E00)
    used = np.zeros(s.arena_pages * PAGE, bool)
    for i, tab in enumerate(s.tables):
        n = s.ctx_len[i] + s.new_rows[i]
        for p in range(n):
            used[int(tab[p // PAGE]) * PAGE + p % PAGE] = True
    s.k_bits[~used] = nan16
    s.v_bits[~used] = nan16
    kv = load(backend, s)
    got = run_step(backend, kv, s)
    s.k_bits[~used] = 0
    s.v_bits[~used] = 0
    assert_close(got, oracle_step(oracle, s), what="poisoned")
    kv.close()


def test_output_dtypes(backend, oracle):
    s = W.build("out", 3, 8, 2, BF16, [333], [6])
    kv = load(backend, s)
    ref = oracle_step(oracle, s)
    for dt, tol in ((torch.float32, ABS_TOL), (torch.bfloat16, 2e-2), (torch.float16, 4e-3)):
        got = run_step(backend, kv, s, out_dtype=dt)
        assert_close(got, ref, abs_tol=tol, what=str(dt))
    kv.close()


@pytest.mark.parametrize("window", [None, 2048])
def test_partials_over_key_ranges_merge_to_whole(backend, oracle, window):
    # Long-context decode with the keys in contiguous page ranges, as each GPU of a split-KV
    # run sees them: the triples of every range, merged by lse_combine, equal whole attention;
    # ranges outside the window are marked (-1e30, 0).
    s = W.long_decode(ctx=16384, window=window)
    kv = load(backend, s, max_pos=16384)
    backend.begin_pass(s.meta)
    backend.kv_append(kv, 0, dev(backend, s.k_new), dev(backend, s.v_new))
    q = dev(backend, s.q)
    whole = backend.to_host(backend.attend(kv, 0, q, s.hq))
    ref = oracle_step(oracle, s)
    assert_close(whole, ref, what="whole")
    world = 4
    ms, ls, os_ = [], [], []
    for rank in range(world):
        _, _, klo, khi = W.partition_pages(s.arena_pages, world, rank)
        m, l, o = backend.attend_partial(kv, 0, q, s.hq, window, klo, khi)
        ms.append(m), ls.append(l), os_.append(o)
        if window and khi <= 16384 - window:
            backend.sync()
            assert torch.all(m == -1e30) and torch.all(l == 0)
        Km, Lm, Om = oracle.attend_partial(s.q, s.meta.pos, s.meta.pt_off, s.meta.pages, s.hq, s.hkv, 128, window, klo,
                                           khi, *oracle_arenas(oracle, s))
        backend.sync()
        live = Lm > 0
        # compare normalised partial outputs where the range has live keys
        if live.any():
            got_n = (o / l.unsqueeze(-1)).cpu().numpy()[live]
            ref_n = (Om / Lm[..., None])[live]
            assert_close(got_n, ref_n, what=f"partial rank {rank}")
    merged = backend.to_host(backend.lse_combine(torch.stack(ms), torch.stack(ls), torch.stack(os_)))
    assert_close(merged.reshape(ref.shape), ref, what="merged")
    # single-rank all-gather path = partial + combine
    backend.comm_create(1, 0)
    one = backend.to_host(backend.attend_allgather(kv, 0, q, s.hq, window, 0, 1 << 40))
    assert_close(one, ref, what="allgather n=1")
    kv.close()


@pytest.mark.parametrize("window", [None, 2048])
def test_long_context_decode_at_full_size(backend, oracle, window):
    # One sequence, one query token, 131072 keys in an f16 cache (1024 pages, 512 MiB of K and V),
    # 32 query / 8 KV heads; the keys in eight contiguous page ranges as eight GPUs would hold
    # them, every range's triple from yx_attend_partial, merged by yx_lse_combine.  With the
    # 2048-key window only the last range has live keys; the others report (-1e30, 0).
    s = W.long_decode(window=window)
    assert s.arena_pages == 1024 and int(s.meta.pos[0]) == 131071
    kv = load(backend, s, max_pos=131072)
    backend.begin_pass(s.meta)
    backend.kv_append(kv, 0, dev(backend, s.k_new), dev(backend, s.v_new))
    q = dev(backend, s.q)
    ref = oracle_step(oracle, s)
    whole = backend.to_host(backend.attend(kv, 0, q, s.hq))
    assert_close(whole, ref, what="whole")
    world = 8
    ms, ls, os_ = [], [], []
    for rank in range(world):
        _, _, klo, khi = W.partition_pages(s.arena_pages, world, rank)
        m, l, o = backend.attend_partial(kv, 0, q, s.hq, window, klo, khi)
        ms.append(m), ls.append(l), os_.append(o)
        if window and khi <= 131072 - window:
            backend.sync()
            assert torch.all(m == -1e30) and torch.all(l == 0)
    merged = backend.to_host(backend.lse_combine(torch.stack(ms), torch.stack(ls), torch.stack(os_)))
    assert_close(merged.reshape(ref.shape), ref, what="merged over 8 ranges")
    kv.close()


@pytest.mark.parametrize("shape", ["default", "small", "every_sm", "verify"])
@pytest.mark.parametrize("kv_dtype", [F16, BF16])
def test_back_to_back_calls_each_get_their_own_answer(backend, oracle, kv_dtype, shape):
    # An attention call that directly follows another one starts reading before the one ahead has
    # finished and waits only before it writes.  Forty calls in a row, alternating between two
    # layers (the second holds the first's values negated), two query tensors and four output
    # buffers: every buffer must hold the answer of the last call that wrote it, and the same bits
    # as with the overlap switched off.  The default plan leaves one SM spare and `small` has far
    # fewer CTAs than SMs: the overlapping call waits before its first write.  `every_sm` asks for
    # a CTA on every SM, after which the call behind waits only before its CTAs leave.  `verify`:
    # five rows a sequence, whose merge kernel in such a run takes several (row, head) pairs a warp.
    small = shape == "small"
    per_sm = 1 if shape == "every_sm" else 0
    s = W.batched_decode(seed=3, n_seq=4, prefix=256, max_suffix=300, kv_dtype=kv_dtype) if small else W.batched_decode(kv_dtype=kv_dtype)
    if shape == "verify":
        s = W.verify(kv_dtype=kv_dtype)
    kv = load(backend, s, n_layers=2)
    backend.write_pages(kv, 1, 0, s.k_bits, s.v_bits ^ np.uint16(0x8000))
    rng = np.random.default_rng(5)
    qs = [s.q, rng.standard_normal(s.q.shape).astype(np.float32)]
    refs = [oracle_step(oracle, s, q=q) for q in qs]
    results = []
    for overlap in (0, 2):
        backend.set_tuning(overlap_calls=overlap, ctas_per_sm=per_sm)
        backend.begin_pass(s.meta)
        backend.kv_append(kv, 0, dev(backend, s.k_new), dev(backend, s.v_new))
        backend.kv_append(kv, 1, dev(backend, s.k_new), dev(backend, -s.v_new))
        q_dev = [dev(backend, q) for q in qs]
        outs = [torch.zeros(s.meta.rows, s.hq * 128, device=backend.device) for _ in range(4)]
        for i in range(40):
            backend.attend(kv, i % 2, q_dev[(i // 2) % 2], s.hq, out=outs[i % 4])
        results.append([backend.to_host(o) for o in outs])
        if not small:
            sms = torch.cuda.get_device_properties(backend.device).multi_processor_count
            assert backend.last_plan().n_ctas == sms - (0 if per_sm else 1)
    backend.set_tuning()
    for i, got in enumerate(results[0]):      # buffer i was last written by call 36 + i
        sign = -1.0 if i % 2 else 1.0
        assert_close(got, sign * refs[(i // 2) % 2], what=f"call {36 + i}")
        assert np.array_equal(got, results[1][i])
    kv.close()


def test_a_call_fed_by_the_call_before_waits_for_it(backend, oracle):
    # Back-to-back calls overlap only when the second one's queries cannot be the first one's
    # output.  Here they are: the second call must see the finished result of the first.
    s = W.batched_decode(seed=9)
    kv = load(backend, s, n_layers=2)
    backend.begin_pass(s.meta)
    for l in range(2):
        backend.kv_append(kv, l, dev(backend, s.k_new), dev(backend, s.v_new))
    q = dev(backend, s.q)
    warm = torch.empty_like(q)
    backend.attend(kv, 0, q, s.hq, out=warm)          # so that the next two calls follow an attention call
    mid = torch.zeros_like(q)
    backend.attend(kv, 0, q, s.hq, out=mid)
    out = backend.attend(kv, 1, mid, s.hq)            # reads what the call before wrote
    ref_mid = oracle_step(oracle, s)
    ref = oracle_step(oracle, s, q=ref_mid)
    assert_close(backend.to_host(mid), ref_mid, what="first call")
    assert_close(backend.to_host(out), ref, what="second call")
    kv.close()


def test_empty_pass(backend):
    s = W.build("e", 1, 8, 2, F16, [10], [1])
    kv = load(backend, s)
    backend.begin_pass(PassMeta())
    out = backend.attend(kv, 0, torch.zeros(0, 8 * 128, device=backend.device), 8)
    backend.sync()
    assert out.shape == (0, 1024)
    kv.close()
