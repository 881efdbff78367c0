"""Seeded random passes against the oracle: mixed decode rows, draft rows and prompt chunks in
one pass, random head groupings, windows, shared prefixes, cache and tensor types.  The shapes
are small enough for the oracle to finish in a moment; every kernel path of the library is
reached (the plan's path is printed on failure)."""
import numpy as np
import pytest
import torch

from oracle.check import ABS_TOL, assert_close, dev, load, oracle_step
from yaxus_b200 import workloads as W
from yaxus_b200._lib import BF16, F16, F32

pytestmark = pytest.mark.gpu

TORCH = {F16: torch.float16, BF16: torch.bfloat16}


def random_case(seed):
    rng = np.random.default_rng(1000 + seed)
    hkv = int(rng.choice([1, 2, 4, 8]))
    group = int(rng.choice([1, 2, 4, 8]))
    kv_dtype = int(rng.choice([F16, F16, F16, BF16, BF16, F32]))
    n_seq = int(rng.integers(1, 9))
    shared = int(rng.choice([0, 0, 128, 384])) if n_seq > 1 else 0
    ctx, rows = [], []
    for _ in range(n_seq):
        kind = rng.choice(["decode", "decode", "draft", "chunk"])
        c = shared + int(rng.integers(0, 900))
        r = 1 if kind == "decode" else (int(rng.integers(2, 9)) if kind == "draft" else int(rng.integers(60, 300)))
        ctx.append(c)
        rows.append(r)
    window = int(rng.choice([0, 0, 0, 50, 200, 1000])) or None
    q_same = bool(rng.integers(0, 2)) and kv_dtype != F32
    return dict(hq=hkv * group, hkv=hkv, kv_dtype=kv_dtype, ctx=ctx, rows=rows, shared=shared, window=window, q_same=q_same)


@pytest.mark.parametrize("seed", range(40))
def test_random_pass(backend, oracle, seed):
    c = random_case(seed)
    s = W.build(f"fuzz{seed}", 7000 + seed, c["hq"], c["hkv"], c["kv_dtype"], c["ctx"], c["rows"],
                shared_prefix=c["shared"], window=c["window"])
    kv = load(backend, s)
    backend.begin_pass(s.meta)
    backend.kv_append(kv, 0, dev(backend, s.k_new), dev(backend, s.v_new))
    if c["q_same"]:
        # queries in the cache's own type: the oracle sees the same rounded values
        qdt = TORCH[c["kv_dtype"]]
        q_dev = dev(backend, s.q, qdt)
        q_ref = q_dev.float().cpu().numpy()
    else:
        q_dev, q_ref = dev(backend, s.q), s.q
    got = backend.to_host(backend.attend(kv, 0, q_dev, s.hq))
    want = oracle_step(oracle, s, q=q_ref)
    info = backend.last_plan()
    assert_close(got, want, abs_tol=2e-5 if c["kv_dtype"] == F32 else ABS_TOL, what=f"{c} path {info.path}")
    kv.close()
