"""The CPU oracle against the pins the reference offers for this path."""
import numpy as np
import pytest

from yaxus_b200 import workloads as W
from yaxus_b200._lib import BF16, F16, F32


def test_reference_known_answer(oracle):
    # paged_attention_matches_dense_attention (crates/yaxus-backend-cpu/src/lib.rs:676-714):
    # same shapes, page tables, PRNG and tolerance.
    worst = oracle.selftest()
    assert 0.0 <= worst < 1e-5


def test_values_generator(oracle):
    # xorshift64 of cpu lib.rs:572-582, recomputed independently in Python.
    def values(n, seed):
        s = ((seed * 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF) | 1
        out = []
        for _ in range(n):
            s ^= (s << 13) & 0xFFFFFFFFFFFFFFFF
            s ^= s >> 7
            s ^= (s << 17) & 0xFFFFFFFFFFFFFFFF
            out.append(np.float32(np.float32(s >> 40) / np.float32(1 << 23)) - np.float32(1.0))
        return np.array(out, np.float32)

    for seed in (0, 1, 7, 1003):
        got = oracle.values(64, seed)
        assert np.array_equal(got, values(64, seed))
        assert got.min() >= -1.0 and got.max() < 1.0


def test_slot(oracle):
    # kv::slot (crates/yaxus-model/src/kv.rs:20-22)
    pages = [3, 1, 7]
    assert oracle.slot(pages, 0) == 3 * 128
    assert oracle.slot(pages, 127) == 3 * 128 + 127
    assert oracle.slot(pages, 128) == 1 * 128
    assert oracle.slot(pages, 300) == 7 * 128 + 44


def test_dot_is_sixteen_lane(oracle):
    # cpu lib.rs:280-294: 16 partial sums, summed left to right, then the tail.
    rng = np.random.default_rng(5)
    a = rng.standard_normal(150).astype(np.float32)
    b = rng.standard_normal(150).astype(np.float32)
    acc = np.zeros(16, np.float32)
    for c in range(0, 144, 16):
        acc += a[c:c + 16] * b[c:c + 16]
    s = np.float32(0)
    for x in acc:
        s = np.float32(s + x)
    for i in range(144, 150):
        s = np.float32(s + np.float32(a[i] * b[i]))
    import ctypes
    got = oracle.L.yxref_dot(a.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
                             b.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), 150)
    assert np.float32(got) == s


def test_storage_rounding(oracle):
    rng = np.random.default_rng(11)
    x = np.concatenate([rng.standard_normal(4096), rng.standard_normal(512) * 1e-6, rng.standard_normal(512) * 3e4,
                        [0.0, -0.0, 65504.0, 65519.9, 65520.0, 6e-8, 2.98e-8, 2.99e-8, 1e-10]]).astype(np.float32)
    with np.errstate(over="ignore"):
        assert np.array_equal(oracle.round_through(x, F16), x.astype(np.float16).astype(np.float32))
    # bf16 as crates/yaxus-model/src/weights.rs:100-111
    assert np.array_equal(oracle.round_through(x, BF16), W.round_through(x, BF16))
    assert np.array_equal(oracle.round_through(x, F32), x)
    for v in x[:200]:
        assert oracle.L.yxref_f32_to_bf16(float(v)) == int(W.to_bits(np.array([v]), BF16)[0])


def test_rope_default_matches_numpy(oracle):
    from yaxus_b200.backend import Rope
    assert np.allclose(oracle.rope_default(128, 10000.0), Rope.default(10000.0).inv_freq, rtol=3e-7, atol=0)


@pytest.mark.parametrize("window", [None, 48])
def test_partials_merge_to_whole(oracle, window):
    # Split-key triples over disjoint key ranges, merged by the combine rule
    # (crates/yaxus-backend-gpu/src/shaders.rs:1581-1637), equal whole attention.
    s = W.build("t", 3, 8, 2, F32, [200, 37], [3, 2], window=window)
    K, V = s.k_f32(), s.v_f32()
    oracle.append_rows(s.k_new, s.v_new, s.meta.kv_slot, K, V)
    want = oracle.attend(s.q, s.meta.pos, s.meta.pt_off, s.meta.pages, s.hq, s.hkv, 128, window, K, V)
    cuts = [0, 64, 130, 131, 1 << 40]
    ms, ls, os_ = [], [], []
    for a, b in zip(cuts[:-1], cuts[1:]):
        m, l, o = oracle.attend_partial(s.q, s.meta.pos, s.meta.pt_off, s.meta.pages, s.hq, s.hkv, 128, window, a, b,
                                        K, V)
        ms.append(m), ls.append(l), os_.append(o)
    got = oracle.combine(np.stack(ms), np.stack(ls), np.stack(os_)).reshape(want.shape)
    assert np.abs(got - want).max() < 2e-6
    # an empty range marks itself (-1e30, 0)
    m, l, _ = oracle.attend_partial(s.q, s.meta.pos, s.meta.pt_off, s.meta.pages, s.hq, s.hkv, 128, window, 5000, 6000,
                                    K, V)
    assert np.all(m == np.float32(-1e30)) and np.all(l == 0)


def test_copy_page(oracle):
    kvd = 256
    K = np.arange(4 * 128 * kvd, dtype=np.float32).reshape(-1, kvd).copy()
    V = -K.copy()
    oracle.copy_page(K, V, kvd, 2, 0)
    assert np.array_equal(K[:128], K[256:384]) and np.array_equal(V[:128], V[256:384])


def test_golden_fixture(oracle):
    # Small fixtures made by tests/golden/make_golden.py from the pinned oracle.
    import os
    path = os.path.join(os.path.dirname(__file__), "golden", "attention_small.npz")
    g = np.load(path)
    for tag in ("full", "win"):
        window = None if tag == "full" else int(g["window"])
        K, V = g["K0"].copy(), g["V0"].copy()
        q = oracle.write_rows(g["qkv"], g["pos"], g["kv_slot"], g["q_norm"], g["k_norm"], int(g["hq"]), int(g["hkv"]),
                              128, float(g["eps"]), g["inv_freq"], float(g["conc"]), K, V)
        out = oracle.attend(q, g["pos"], g["pt_off"], g["pages"], int(g["hq"]), int(g["hkv"]), 128, window, K, V)
        assert np.array_equal(out, g[f"out_{tag}"])
        assert np.array_equal(q, g["q_rot"])


# ---- the operators either side of attention ------------------------------------------------

def test_bf16_rounding_matches_the_reference_formula(oracle):
    # f32_to_bf16 (crates/yaxus-model/src/weights.rs:100-106): round to nearest even, NaN stays NaN.
    x = np.array([0.0, 1.0, -1.0, 1.00390625, 1.01171875, 3.14159274, 65504.0, 1e-40, np.inf, -np.inf], np.float32)
    bits = oracle.to_bf16(x)
    assert [int(oracle.L.yxref_f32_to_bf16(float(v))) for v in x] == [int(b) for b in bits]
    assert bits[3] == 0x3F80 and bits[4] == 0x3F82      # ties go to the even mantissa
    assert oracle.to_bf16(np.array([np.nan], np.float32))[0] & 0x7FC0 == 0x7FC0


def test_matmul_matches_a_plain_loop(oracle):
    # matmul_matches_a_plain_loop (cpu lib.rs:716-744), bf16 arm: n, k = 40, 64; t in 1, 3, 9;
    # values(n*k, 7) for the weights, values(t*k, t) for the rows; tolerance 1e-4 x the sum of |terms|.
    n, k = 40, 64
    w_bits = oracle.to_bf16(oracle.values(n * k, 7)).reshape(n, k)
    w = (w_bits.astype(np.uint32) << 16).view(np.float32)
    for t in (1, 3, 9):
        x = oracle.values(t * k, t).reshape(t, k)
        y = oracle.matmul(x, w_bits)
        assert y.shape == (t, n)
        terms = w[None, :, :] * x[:, None, :]
        want = np.zeros((t, n), np.float32)
        scale = np.zeros((t, n), np.float32)
        for c in range(k):          # the reference folds left to right
            want = (want + terms[:, :, c]).astype(np.float32)
            scale = (scale + np.abs(terms[:, :, c])).astype(np.float32)
        assert (np.abs(y - want) <= 1e-4 * np.maximum(scale, 1.0)).all()


def test_argmax_takes_the_first_maximum_and_skips_nans(oracle):
    # argmax_takes_the_first_maximum_and_skips_nans (cpu lib.rs:746-752)
    nan = np.nan
    rows = [([1.0, 3.0, 3.0, 2.0], 1), ([nan, 1.0, 2.0], 2), ([0.5, nan, 0.2], 0), ([nan, nan], 0)]
    for row, want in rows:
        assert int(oracle.argmax_rows(np.array([row], np.float32))[0]) == want


def test_elementwise_operators_against_numpy(oracle):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((5, 96)).astype(np.float32)
    w = rng.standard_normal(96).astype(np.float32)
    # rmsnorm_row (cpu lib.rs:296-302)
    got = oracle.rmsnorm(x, w, 1.0, 1e-6)
    ref = (1.0 + w) * (x / np.sqrt((x.astype(np.float64) ** 2).mean(1, keepdims=True) + 1e-6))
    assert np.abs(got - ref).max() < 1e-5
    # swiglu (cpu lib.rs:532-542)
    g, u = x[:, :48].astype(np.float64), x[:, 48:].astype(np.float64)
    assert np.abs(oracle.swiglu(x) - g / (1 + np.exp(-g)) * u).max() < 1e-6
    # add_norm (crates/yaxus-model/src/lib.rs:149-162) is the three calls of the default method
    d = rng.standard_normal((5, 96)).astype(np.float32)
    w2 = rng.standard_normal(96).astype(np.float32)
    x2, out = oracle.add_norm(x, d, w, 0.0, w2, 1.0, 1e-6)
    step = x + oracle.rmsnorm(d, w, 0.0, 1e-6)
    assert np.array_equal(x2, step) and np.array_equal(out, oracle.rmsnorm(step, w2, 1.0, 1e-6))
    # embed (cpu lib.rs:485-497)
    table = oracle.to_bf16(rng.standard_normal((10, 32)).astype(np.float32))
    e = oracle.embed(table, [3, 3, 9, 0])
    assert np.array_equal(e, (table[[3, 3, 9, 0]].astype(np.uint32) << 16).view(np.float32))


def _tiny_model(oracle):
    from tests.test_gpu_forward import TinyWeights
    from yaxus_b200.backend import LayerMeta, Rope
    metas = [LayerMeta(index=0, window=None, rope=Rope.default()), LayerMeta(index=1, window=48, rope=Rope.default(theta=5000.0))]
    return TinyWeights(oracle, len(metas), seed=11), metas


def _arenas(metas, pages):
    from tests.test_gpu_forward import D, HKV
    from yaxus_b200._lib import PAGE
    return [(np.zeros((pages * PAGE, HKV * D), np.float32), np.zeros((pages * PAGE, HKV * D), np.float32)) for _ in metas]


def test_a_prompt_in_chunks_gives_the_logits_of_the_prompt_at_once(oracle):
    # The property chunked prefill rests on (crates/yaxus-model/src/lib.rs:475-482): feeding a prompt
    # in chunks leaves the same cache and the same last-row logits as feeding it whole.  Here on the
    # oracle's own operators composed in Model::forward's order, over the host-side page bookkeeping.
    from tests.test_gpu_forward import VOCAB, forward_oracle
    from yaxus_b200.kvcache import KvCache
    w, metas = _tiny_model(oracle)
    prompt = np.random.default_rng(3).integers(0, VOCAB, 150)
    results = []
    for chunks in ((150,), (100, 50), (128, 1, 21)):
        cache, arenas = KvCache(4, 1024), _arenas(metas, 4)
        seq, at = cache.new_seq(), 0
        for n in chunks:
            logits = forward_oracle(oracle, w, arenas, metas, cache.append([(seq, prompt[at:at + n])]), F32)
            at += n
        results.append((logits, arenas))
    for logits, arenas in results[1:]:
        assert np.abs(logits - results[0][0]).max() <= 2e-5
        for (K, V), (K0, V0) in zip(arenas, results[0][1]):
            assert np.abs(K - K0).max() <= 2e-6 and np.abs(V - V0).max() <= 2e-6


def test_a_fork_continues_like_the_sequence_it_came_from(oracle):
    # KvCache::fork (crates/yaxus-model/src/kv.rs:277-295): the fork shares the full pages, gets a copy
    # of the half-filled one, and the same next token gives it the same logits as its parent.
    from tests.test_gpu_forward import D, HKV, VOCAB, forward_oracle
    from yaxus_b200.kvcache import KvCache
    w, metas = _tiny_model(oracle)
    cache, arenas = KvCache(6, 1024), _arenas(metas, 6)
    prompt = np.random.default_rng(4).integers(0, VOCAB, 140)
    a = cache.new_seq()
    forward_oracle(oracle, w, arenas, metas, cache.append([(a, prompt)]), BF16)
    b = cache.fork(a, 140)
    meta = cache.append([(a, [7]), (b, [7])])
    copies = cache.take_copies()
    assert len(copies) == 1 and cache.page_refs(int(cache.seq_pages(a)[0])) == 2
    for src, dst in copies:
        for K, V in arenas:
            oracle.copy_page(K, V, HKV * D, src, dst)
    logits = forward_oracle(oracle, w, arenas, metas, meta, BF16)
    assert logits.shape == (2, VOCAB) and np.array_equal(logits[0], logits[1])
