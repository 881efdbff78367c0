"""KV page writes on the GPU: byte-exact against the oracle's arenas."""
import numpy as np
import pytest
import torch

from oracle.check import dev, layers_for, load
from yaxus_b200 import workloads as W
from yaxus_b200._lib import BF16, F16, F32, PAGE
from yaxus_b200.backend import LayerMeta
from yaxus_b200.kvcache import KvCache, PassMeta

pytestmark = pytest.mark.gpu

TORCH = {F32: torch.float32, F16: torch.float16, BF16: torch.bfloat16}


@pytest.mark.parametrize("kv_dtype", [F32, F16, BF16])
@pytest.mark.parametrize("native_src", [False, True])
def test_plain_append_is_byte_exact(backend, oracle, kv_dtype, native_src):
    # 80 rows (16 sequences x 5) scattered to their slots, as in speculative verification.
    s = W.verify(seed=21, n_seq=16, ctx=300, rows=5, kv_dtype=kv_dtype, hq=8, hkv=2)
    kv = load(backend, s)
    backend.begin_pass(s.meta)
    src = TORCH[kv_dtype] if native_src else torch.float32
    backend.kv_append(kv, 0, dev(backend, s.k_new, src), dev(backend, s.v_new, src))
    k_dev, v_dev = backend.read_pages(kv, 0, 0, s.arena_pages)
    k_ref, v_ref = s.k_bits.copy(), s.v_bits.copy()
    k_ref[s.meta.kv_slot] = W.to_bits(s.k_new, kv_dtype)
    v_ref[s.meta.kv_slot] = W.to_bits(s.v_new, kv_dtype)
    assert np.array_equal(k_dev, k_ref) and np.array_equal(v_dev, v_ref)
    # and the oracle's own append agrees slot for slot
    K, V = s.k_f32(), s.v_f32()
    oracle.append_rows(W.round_through(s.k_new, kv_dtype), W.round_through(s.v_new, kv_dtype), s.meta.kv_slot, K, V)
    assert np.array_equal(W.from_bits(k_dev, kv_dtype), K) and np.array_equal(W.from_bits(v_dev, kv_dtype), V)
    kv.close()


def test_new_kv_is_zeroed_and_pages_round_trip(backend):
    # cpu lib.rs:466-468: arenas start at zero.
    layers = [LayerMeta(index=i) for i in range(3)]
    kv = backend.new_kv(2, layers, 5, 1024, F16)
    for l in range(3):
        k, v = backend.read_pages(kv, l, 0, 5)
        assert not k.any() and not v.any()
    rng = np.random.default_rng(1)
    k = rng.integers(0, 65535, (2 * PAGE, 256)).astype(np.uint16)
    v = rng.integers(0, 65535, (2 * PAGE, 256)).astype(np.uint16)
    backend.write_pages(kv, 1, 2, k, v)
    k2, v2 = backend.read_pages(kv, 1, 2, 2)
    assert np.array_equal(k, k2) and np.array_equal(v, v2)
    k0, _ = backend.read_pages(kv, 0, 0, 5)
    assert not k0.any()
    kv.close()


@pytest.mark.parametrize("kv_dtype", [F32, BF16])
def test_copy_page_every_layer(backend, oracle, kv_dtype):
    # Backend::copy_page (crates/yaxus-model/src/lib.rs:120; cpu lib.rs:472-479).
    n_layers, hkv, pages = 3, 2, 6
    kv = backend.new_kv(hkv, [LayerMeta(index=i) for i in range(n_layers)], pages, 1024, kv_dtype)
    rng = np.random.default_rng(3)
    ref = []
    for l in range(n_layers):
        k = W.to_bits(rng.standard_normal((pages * PAGE, hkv * 128)).astype(np.float32), kv_dtype)
        v = W.to_bits(rng.standard_normal((pages * PAGE, hkv * 128)).astype(np.float32), kv_dtype)
        backend.write_pages(kv, l, 0, k, v)
        ref.append((k.copy(), v.copy()))
    for src, dst in [(4, 1), (1, 5), (2, 2)]:
        backend.copy_page(kv, src, dst)
        for k, v in ref:
            k[dst * PAGE:(dst + 1) * PAGE] = k[src * PAGE:(src + 1) * PAGE]
            v[dst * PAGE:(dst + 1) * PAGE] = v[src * PAGE:(src + 1) * PAGE]
    for l in range(n_layers):
        k, v = backend.read_pages(kv, l, 0, pages)
        assert np.array_equal(k, ref[l][0]) and np.array_equal(v, ref[l][1])
    kv.close()


def test_fork_copy_on_write_through_the_host_cache(backend, oracle):
    # The scenario of kv.rs:366-383 with real data: a sequence of 150 tokens, a fork at 140
    # (page 0 shared, page 1 copied), then both grow; the copies come from the host cache and
    # are made in order before the pass, as crates/yaxus-model/src/lib.rs:438-444 does.
    hq, hkv, kvd = 8, 2, 256
    cache = KvCache(6, 1024)
    kv = backend.new_kv(hkv, [LayerMeta(index=0)], 6, 1024, F16)
    K = np.zeros((6 * PAGE, kvd), np.float32)
    V = np.zeros((6 * PAGE, kvd), np.float32)
    rng = np.random.default_rng(9)

    def step(items):
        meta = cache.append(items)
        for src, dst in cache.take_copies():
            backend.copy_page(kv, src, dst)
            oracle.copy_page(K, V, kvd, src, dst)
        T = meta.rows
        q = rng.standard_normal((T, hq * 128)).astype(np.float32)
        k = rng.standard_normal((T, kvd)).astype(np.float32)
        v = rng.standard_normal((T, kvd)).astype(np.float32)
        backend.begin_pass(meta)
        backend.kv_append(kv, 0, dev(backend, k), dev(backend, v))
        out = backend.to_host(backend.attend(kv, 0, dev(backend, q), hq))
        oracle.append_rows(W.round_through(k, F16), W.round_through(v, F16), meta.kv_slot, K, V)
        ref = oracle.attend(q, meta.pos, meta.pt_off, meta.pages, hq, hkv, 128, None, K, V)
        from oracle.check import assert_close
        assert_close(out, ref, what="fork step")

    a = cache.new_seq()
    for lo in range(0, 150, 50):
        step([(a, list(range(lo, lo + 50)))])
    b = cache.fork(a, 140)
    copies = cache.take_copies()
    assert len(copies) == 1
    for src, dst in copies:
        backend.copy_page(kv, src, dst)
        oracle.copy_page(K, V, kvd, src, dst)
    step([(a, [1]), (b, [2, 3, 4])])
    c = cache.fork(a, PAGE)
    cache.truncate(c, 100)
    step([(c, [7]), (a, [5]), (b, [6])])     # writing into c's shared first page copies it
    k_dev, v_dev = backend.read_pages(kv, 0, 0, 6)
    assert np.array_equal(W.from_bits(k_dev, F16), K) and np.array_equal(W.from_bits(v_dev, F16), V)
    kv.close()
