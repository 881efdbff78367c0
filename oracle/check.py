"""The checker side of a parity comparison: load a workload into the CUDA backend, run the
same step through the CPU oracle, compare within the path's tolerance.  Test infrastructure,
like everything in this directory: used by the tests, the smoke check and the benchmark's
parity and CPU-baseline legs, never by the CUDA library."""
import numpy as np
import torch

from yaxus_b200 import workloads as W
from yaxus_b200._lib import F32
from yaxus_b200.backend import LayerMeta, Rope

ABS_TOL, REL_TOL = 2e-3, 1e-2   # |gpu - ref| <= 2e-3 + 1e-2 |ref| for f32-accumulated outputs


def layers_for(s, n_layers=1):
    return [LayerMeta(index=i, window=s.window, rope=Rope.default()) for i in range(n_layers)]


def load(backend, s, n_layers=1, max_pos=None):
    if max_pos is None:
        max_pos = max(int(s.meta.pos.max()) + 1 if s.meta.rows else 1, max(s.ctx_len) + 1, 8192)
    kv = backend.new_kv(s.hkv, layers_for(s, n_layers), s.arena_pages, max_pos, s.kv_dtype)
    for l in range(n_layers):
        backend.write_pages(kv, l, 0, s.k_bits, s.v_bits)
    return kv


def dev(backend, x, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(x)).to(backend.device).to(dtype).contiguous()


def run_step(backend, kv, s, layer=0, window=-1, q_dtype=torch.float32, out_dtype=torch.float32, src_dtype=torch.float32):
    backend.begin_pass(s.meta)
    backend.kv_append(kv, layer, dev(backend, s.k_new, src_dtype), dev(backend, s.v_new, src_dtype))
    out = backend.attend(kv, layer, dev(backend, s.q, q_dtype), s.hq, window=window, out_dtype=out_dtype)
    return backend.to_host(out)


def oracle_arenas(oracle, s):
    """The oracle's K, V after the step's append: cached context plus the new rows rounded to
    the storage type."""
    K, V = s.k_f32(), s.v_f32()
    oracle.append_rows(W.round_through(s.k_new, s.kv_dtype), W.round_through(s.v_new, s.kv_dtype), s.meta.kv_slot, K, V)
    return K, V


def oracle_step(oracle, s, q=None, window="own"):
    K, V = oracle_arenas(oracle, s)
    w = s.window if window == "own" else window
    return oracle.attend(s.q if q is None else q, s.meta.pos, s.meta.pt_off, s.meta.pages, s.hq, s.hkv, 128, w, K, V)


def assert_close(got, ref, abs_tol=ABS_TOL, rel_tol=REL_TOL, what=""):
    got, ref = np.asarray(got, np.float32), np.asarray(ref, np.float32)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    err = np.abs(got - ref)
    bound = abs_tol + rel_tol * np.abs(ref)
    worst = int(np.argmax(err - bound))
    assert (err <= bound).all(), (
        f"{what}: max-abs {err.max():.3e}, worst at flat index {worst}: got {got.flat[worst]} ref {ref.flat[worst]}")
    return float(err.max())
