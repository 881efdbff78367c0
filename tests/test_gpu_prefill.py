"""Chunked causal prefill on the tcgen05 tile kernel against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle.check import assert_close, dev, load, oracle_step, run_step
from yaxus_b200 import workloads as W
from yaxus_b200._lib import BF16, F16

pytestmark = pytest.mark.gpu


def q_rounded(s):
    return W.round_through(s.q, s.kv_dtype)


@pytest.mark.parametrize("kv_dtype,qt", [(BF16, torch.bfloat16), (F16, torch.float16)])
@pytest.mark.parametrize("done", [0, 512, 1000])
def test_prefill_chunks(backend, oracle, kv_dtype, qt, done):
    # Two sequences, one 512-row chunk each after `done` cached tokens: every row attends to
    # the cached pages plus the chunk's own rows up to itself (chunk c of the chunked prefill).
    s = W.prefill_chunk(seed=11 + done, n_seq=2, done=done, chunk=512, kv_dtype=kv_dtype, hq=8, hkv=2, total=2048)
    kv = load(backend, s)
    got = run_step(backend, kv, s, q_dtype=qt)
    info = backend.last_plan()
    assert info.path == 3     # all rows on the tile kernel
    assert_close(got, oracle_step(oracle, s, q=q_rounded(s)), what=f"prefill done={done}")
    kv.close()


@pytest.mark.parametrize("rows", [64, 129, 200])
@pytest.mark.parametrize("window", [None, 100])
def test_ragged_tiles_and_windows(backend, oracle, rows, window):
    # Tiles that are not full, a chunk that starts inside a page, a sliding window narrower
    # than a tile, and decode rows of other sequences in the same pass (split-key kernel).
    s = W.build("ragged", 21 + rows, 8, 2, BF16, [77, 300, 5], [rows, 1, 2], window=window)
    kv = load(backend, s)
    got = run_step(backend, kv, s, q_dtype=torch.bfloat16)
    assert backend.last_plan().path == 5     # both kernels
    assert_close(got, oracle_step(oracle, s, q=q_rounded(s)), what=f"rows {rows} window {window}")
    kv.close()


def test_one_head_per_cta_variant(backend, oracle):
    # The tile kernel normally takes two query heads of a KV head per CTA; one head per CTA is
    # used for odd groups and for f32 queries on bf16 caches (they carry a low part).
    s = W.prefill_chunk(seed=9, n_seq=2, done=300, chunk=200, kv_dtype=BF16, hq=6, hkv=2, total=1024)   # group 3
    kv = load(backend, s)
    got = run_step(backend, kv, s, q_dtype=torch.bfloat16)
    assert backend.last_plan().path == 3
    assert_close(got, oracle_step(oracle, s, q=q_rounded(s)), what="odd group")
    kv.close()
    s = W.prefill_chunk(seed=10, n_seq=1, done=128, chunk=256, kv_dtype=F16, hq=8, hkv=2, total=512)
    kv = load(backend, s)
    backend.set_tuning(tile_single=1)
    got = run_step(backend, kv, s, q_dtype=torch.float16)
    backend.set_tuning()
    assert_close(got, oracle_step(oracle, s, q=q_rounded(s)), what="forced single")
    kv.close()


def test_forced_tile_path_on_short_rows(backend, oracle):
    s = W.build("short", 5, 8, 2, F16, [130, 0], [7, 1])
    kv = load(backend, s)
    backend.set_tuning(force_path=3)
    got = run_step(backend, kv, s)
    assert backend.last_plan().path == 3
    backend.set_tuning()
    assert_close(got, oracle_step(oracle, s), what="forced tiles")
    kv.close()


def test_output_dtypes_and_f32_queries(backend, oracle):
    s = W.prefill_chunk(seed=3, n_seq=1, done=256, chunk=256, kv_dtype=BF16, hq=4, hkv=1, total=512)
    kv = load(backend, s)
    ref = oracle_step(oracle, s, q=q_rounded(s))
    for qt, ot, tol in ((torch.bfloat16, torch.bfloat16, 2e-2), (torch.bfloat16, torch.float32, 2e-3)):
        got = run_step(backend, kv, s, q_dtype=qt, out_dtype=ot)
        assert_close(got, ref, abs_tol=tol, what=f"{qt} -> {ot}")
    # f32 queries keep their low part on a bf16 cache: the reference is fed the unrounded queries
    got = run_step(backend, kv, s, q_dtype=torch.float32)
    assert_close(got, oracle_step(oracle, s), what="f32 q")
    kv.close()


def test_last_chunk_of_the_full_configuration(backend, oracle):
    # Chunked prefill at its benchmark shape: 8 sequences x 4096 tokens, 32 query / 8 KV heads,
    # bf16 Q/K/V.  The cache holds the first seven chunks (3584 tokens per sequence); the pass is
    # the eighth chunk, 512 rows per sequence: the most pages per item, 512 items dealt over the
    # persistent CTAs.  The appended rows are checked byte-exact at their slots, the output
    # against the oracle on every eighth row of every sequence.
    s = W.prefill_chunk(seed=W.SEED0 + 3, n_seq=8, done=3584, chunk=512, kv_dtype=BF16, hq=32, hkv=8, total=4096)
    assert s.meta.rows == 4096
    kv = load(backend, s)
    got = run_step(backend, kv, s, q_dtype=torch.bfloat16, src_dtype=torch.float32)
    assert backend.last_plan().path == 3
    K = s.k_f32()
    V = s.v_f32()
    oracle.append_rows(W.round_through(s.k_new, BF16), W.round_through(s.v_new, BF16), s.meta.kv_slot, K, V)
    k_dev, v_dev = backend.read_pages(kv, 0, 0, s.arena_pages)
    assert np.array_equal(W.from_bits(k_dev, BF16), K) and np.array_equal(W.from_bits(v_dev, BF16), V)
    sample = np.concatenate([np.arange(sq * 512, (sq + 1) * 512)[::8] for sq in range(8)])
    ref = oracle.attend(q_rounded(s)[sample], s.meta.pos[sample], s.meta.pt_off[sample], s.meta.pages, s.hq, s.hkv, 128,
                        None, K, V)
    assert_close(got[sample], ref, what="chunk 7 of 8 x 4096")
    kv.close()


def test_bf16_values_beyond_f16_take_the_two_part_path(backend, oracle):
    # On a bf16 cache the tile kernel turns V pages into f16 in shared memory and multiplies once;
    # that is exact unless the cache holds a V value of magnitude 65536 or more, which the kernels
    # that write V record.  Here one appended value and, in a second cache, one imported value are
    # that large: the kernel's two-part variant must do the work, with the same result as ever.
    for where in ("appended", "imported"):
        s = W.prefill_chunk(seed=31, n_seq=2, done=256, chunk=256, kv_dtype=BF16, hq=8, hkv=2, total=512)
        if where == "appended":
            s.v_new[5, 17] = 1.0e5
            s.v_new[300, 200] = -3.0e6
        else:
            big = W.to_bits(np.array([2.5e5], np.float32), BF16)[0]
            s.v_bits[int(s.tables[0][1]) * 128 + 3, 77] = big
        kv = load(backend, s)
        got = run_step(backend, kv, s, q_dtype=torch.bfloat16)
        assert backend.last_plan().path == 3
        assert_close(got, oracle_step(oracle, s, q=q_rounded(s)), what=f"large V value {where}")
        kv.close()
