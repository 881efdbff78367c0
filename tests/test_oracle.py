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
