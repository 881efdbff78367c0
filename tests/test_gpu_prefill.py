"""Chunked causal prefill on the tcgen05 tile kernel against the CPU oracle."""
import numpy as np
import pytest
import torch

from tests.gpu_util import assert_close, dev, load, oracle_step, run_step
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
    # f32 queries are rounded to the cache's type by the kernel: same reference
    got = run_step(backend, kv, s, q_dtype=torch.float32)
    assert_close(got, ref, abs_tol=4e-3, what="f32 q")
    kv.close()
