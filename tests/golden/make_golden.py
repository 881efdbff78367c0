"""Writes tests/golden/attention_small.npz from the CPU oracle.

The reference stores no numeric vectors for attention (its only model-free attention test is
a self-consistency check, which the oracle restates and passes), and its Rust code cannot be
run where this repository is built, so these fixtures are the pinned oracle's own outputs:
they freeze its arithmetic, and they give the GPU tests a case that needs no oracle library.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle.binding import Oracle  # noqa: E402
from yaxus_b200 import workloads as W  # noqa: E402
from yaxus_b200._lib import BF16, F16  # noqa: E402
from yaxus_b200.kvcache import PassMeta  # noqa: E402


def main():
    o = Oracle()
    assert o.selftest() < 1e-5
    hq, hkv, d, eps = 4, 2, 128, 1e-6
    rng = np.random.default_rng(20260101)
    tables = [np.array([3, 0], np.uint32), np.array([1], np.uint32), np.array([4, 2], np.uint32)]
    # A pass mixing a 30-row chunk that crosses a page boundary, a decode row and 5 verify rows.
    pages_total = 5
    kvd = hkv * d
    K0 = np.zeros((pages_total * 128, kvd), np.float32)
    V0 = np.zeros((pages_total * 128, kvd), np.float32)
    ctx = [100, 20, 130]
    for s, n in enumerate(ctx):
        for p in range(n):
            sl = int(tables[s][p // 128]) * 128 + p % 128
            K0[sl] = rng.standard_normal(kvd).astype(np.float32)
            V0[sl] = rng.standard_normal(kvd).astype(np.float32)
    rows = [(0, p) for p in range(100, 130)] + [(1, 20)] + [(2, p) for p in range(130, 135)]
    meta = PassMeta.from_rows(rows, tables)
    T = meta.rows
    qkv = rng.standard_normal((T, (hq + 2 * hkv) * d)).astype(np.float32)
    q_norm = (rng.standard_normal(d) * 0.1).astype(np.float32)
    k_norm = (rng.standard_normal(d) * 0.1).astype(np.float32)
    inv_freq = o.rope_default(d, 10000.0)
    conc = 1.0
    window = 64
    out = {}
    for tag, w in (("full", None), ("win", window)):
        K, V = K0.copy(), V0.copy()
        q = o.write_rows(qkv, meta.pos, meta.kv_slot, q_norm, k_norm, hq, hkv, d, eps, inv_freq, conc, K, V)
        out[f"out_{tag}"] = o.attend(q, meta.pos, meta.pt_off, meta.pages, hq, hkv, d, w, K, V, threads=1)
        out["q_rot"] = q
        # 16-bit caches: the cached context and the rows write_rows stores are rounded to the
        # storage type (round to nearest even), everything else is the f32 algorithm.
        for name, dt in (("f16", F16), ("bf16", BF16)):
            K, V = W.round_through(K0, dt), W.round_through(V0, dt)
            q = o.write_rows(qkv, meta.pos, meta.kv_slot, q_norm, k_norm, hq, hkv, d, eps, inv_freq, conc, K, V,
                             store_dtype=dt)
            out[f"out_{tag}_{name}"] = o.attend(q, meta.pos, meta.pt_off, meta.pages, hq, hkv, d, w, K, V, threads=1)
    np.savez_compressed(
        os.path.join(os.path.dirname(os.path.abspath(__file__)), "attention_small.npz"), hq=hq, hkv=hkv, eps=eps,
        window=window, conc=conc, inv_freq=inv_freq, qkv=qkv, q_norm=q_norm, k_norm=k_norm, pos=meta.pos,
        kv_slot=meta.kv_slot, pt_off=meta.pt_off, pages=meta.pages, K0=K0, V0=V0, **out)
    print("wrote attention_small.npz", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
