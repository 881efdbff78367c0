"""ctypes face of the CPU oracle (yx_ref.cpp beside this file).  Test infrastructure: only the
tests, the smoke check and the benchmark's CPU-baseline and reference legs may use it; the
CUDA library never does."""
import ctypes
import os
from ctypes import POINTER, c_double, c_float, c_int, c_int64, c_size_t, c_uint16, c_uint32, c_uint64

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "oracle", "libyx_oracle.so")

_F = POINTER(c_float)
_U = POINTER(c_uint32)


def _f(a):
    return a.ctypes.data_as(_F)


def _u(a):
    return a.ctypes.data_as(_U)


def _f32(a):
    return np.ascontiguousarray(a, np.float32)


def _u32(a):
    return np.ascontiguousarray(a, np.uint32)


class Oracle:
    def __init__(self):
        if not os.path.exists(LIB):
            from . import build
            build.build()
        L = ctypes.CDLL(LIB)
        L.yxref_selftest.restype = c_double
        L.yxref_slot.restype = c_uint64
        L.yxref_slot.argtypes = [_U, c_uint64]
        L.yxref_dot.restype = c_float
        L.yxref_dot.argtypes = [_F, _F, c_size_t]
        L.yxref_f32_to_f16.restype = c_uint16
        L.yxref_f32_to_f16.argtypes = [c_float]
        L.yxref_f32_to_bf16.restype = c_uint16
        L.yxref_f32_to_bf16.argtypes = [c_float]
        L.yxref_round_through.argtypes = [_F, _F, c_size_t, c_int]
        L.yxref_rope_default.argtypes = [c_size_t, c_double, _F]
        L.yxref_cos_sin.argtypes = [_F, c_size_t, c_float, c_uint64, _F, _F]
        L.yxref_values.argtypes = [_F, c_size_t, c_uint64]
        L.yxref_write_rows.argtypes = [_F, c_size_t, _U, _U, _F, _F, c_size_t, c_size_t, c_size_t, c_float, _F,
                                       c_float, c_int, _F, _F, _F]
        L.yxref_append_rows.argtypes = [_F, _F, c_size_t, _U, c_size_t, _F, _F]
        L.yxref_attend.argtypes = [_F, c_size_t, _U, _U, _U, c_size_t, c_size_t, c_size_t, c_int64, _F, _F, _F, c_int]
        L.yxref_attend_partial.argtypes = [_F, c_size_t, _U, _U, _U, c_size_t, c_size_t, c_size_t, c_int64, c_uint64,
                                           c_uint64, _F, _F, _F, _F, _F, c_int]
        L.yxref_combine.argtypes = [_F, _F, _F, c_size_t, c_size_t, c_size_t, _F]
        L.yxref_copy_page.argtypes = [_F, _F, c_size_t, c_uint32, c_uint32]
        L.yxref_max_threads.restype = c_int
        _H = POINTER(c_uint16)
        L.yxref_dot_bf16.restype = c_float
        L.yxref_dot_bf16.argtypes = [_H, _F, c_size_t]
        L.yxref_matmul_bf16.argtypes = [_F, _H, c_size_t, c_size_t, c_size_t, _F, c_int]
        L.yxref_swiglu.argtypes = [_F, c_size_t, c_size_t, _F]
        L.yxref_embed.argtypes = [_H, c_size_t, _U, c_size_t, _F]
        L.yxref_rmsnorm.argtypes = [_F, _F, c_size_t, c_size_t, c_float, c_float, _F]
        L.yxref_add_norm.argtypes = [_F, _F, _F, c_float, _F, c_float, c_float, c_size_t, c_size_t, _F]
        L.yxref_argmax.restype = c_uint32
        L.yxref_argmax.argtypes = [_F, c_size_t]
        self.L = L

    def selftest(self) -> float:
        return self.L.yxref_selftest()

    def max_threads(self) -> int:
        return self.L.yxref_max_threads()

    def slot(self, pages, pos: int) -> int:
        return self.L.yxref_slot(_u(_u32(pages)), pos)

    def values(self, n: int, seed: int) -> np.ndarray:
        out = np.zeros(n, np.float32)
        self.L.yxref_values(_f(out), n, seed)
        return out

    def round_through(self, x, dtype: int) -> np.ndarray:
        x = _f32(x)
        out = np.empty_like(x)
        self.L.yxref_round_through(_f(x), _f(out), x.size, dtype)
        return out

    def rope_default(self, dim: int = 128, theta: float = 10000.0) -> np.ndarray:
        out = np.zeros(dim // 2, np.float32)
        self.L.yxref_rope_default(dim, theta, _f(out))
        return out

    def write_rows(self, qkv, pos, kv_slot, q_norm, k_norm, hq, hkv, d, eps, inv_freq, conc, K, V, store_dtype=0):
        """Writes k, v into K, V in place (reference layout `[slots][hkv*d]`), returns q."""
        qkv = _f32(qkv)
        T = qkv.shape[0]
        q = np.zeros((T, hq * d), np.float32)
        assert K.dtype == np.float32 and K.flags.c_contiguous and V.flags.c_contiguous
        self.L.yxref_write_rows(_f(qkv), T, _u(_u32(pos)), _u(_u32(kv_slot)), _f(_f32(q_norm)), _f(_f32(k_norm)), hq,
                                hkv, d, eps, _f(_f32(inv_freq)), conc, store_dtype, _f(K), _f(V), _f(q))
        return q

    def append_rows(self, k_rows, v_rows, kv_slot, K, V):
        k_rows, v_rows = _f32(k_rows), _f32(v_rows)
        self.L.yxref_append_rows(_f(k_rows), _f(v_rows), k_rows.shape[0], _u(_u32(kv_slot)), k_rows.shape[1], _f(K),
                                 _f(V))

    def attend(self, q, pos, pt_off, pages, hq, hkv, d, window, K, V, threads=0) -> np.ndarray:
        q = _f32(q)
        T = q.shape[0]
        out = np.zeros((T, hq * d), np.float32)
        self.L.yxref_attend(_f(q), T, _u(_u32(pos)), _u(_u32(pt_off)), _u(_u32(pages)), hq, hkv, d,
                            -1 if not window else int(window), _f(K), _f(V), _f(out), threads)
        return out

    def attend_partial(self, q, pos, pt_off, pages, hq, hkv, d, window, key_lo, key_hi, K, V, threads=0):
        q = _f32(q)
        T = q.shape[0]
        m = np.zeros((T, hq), np.float32)
        l = np.zeros((T, hq), np.float32)
        o = np.zeros((T, hq, d), np.float32)
        self.L.yxref_attend_partial(_f(q), T, _u(_u32(pos)), _u(_u32(pt_off)), _u(_u32(pages)), hq, hkv, d,
                                    -1 if not window else int(window), key_lo, key_hi, _f(K), _f(V), _f(m), _f(l),
                                    _f(o), threads)
        return m, l, o

    def combine(self, m, l, o) -> np.ndarray:
        m, l, o = _f32(m), _f32(l), _f32(o)
        parts = m.shape[0]
        n = m[0].size
        d = o.shape[-1]
        out = np.zeros((n, d), np.float32)
        self.L.yxref_combine(_f(m), _f(l), _f(o), parts, n, d, _f(out))
        return out

    def copy_page(self, K, V, kvd, src, dst):
        self.L.yxref_copy_page(_f(K), _f(V), kvd, src, dst)

    # ---- the other Backend operators ----

    def to_bf16(self, x) -> np.ndarray:
        """f32 -> bf16 bits, round to nearest even (crates/yaxus-model/src/weights.rs:100-111)."""
        return _bf16_bits(_f32(x))

    def matmul(self, x, w_bits, threads=0) -> np.ndarray:
        x, w_bits = _f32(x), np.ascontiguousarray(w_bits, np.uint16)
        (T, K), (N, K2) = x.shape, w_bits.shape
        assert K == K2
        out = np.zeros((T, N), np.float32)
        self.L.yxref_matmul_bf16(_f(x), w_bits.ctypes.data_as(POINTER(c_uint16)), T, N, K, _f(out), threads)
        return out

    def swiglu(self, x) -> np.ndarray:
        x = _f32(x)
        T, two_i = x.shape
        out = np.zeros((T, two_i // 2), np.float32)
        self.L.yxref_swiglu(_f(x), T, two_i // 2, _f(out))
        return out

    def embed(self, table_bits, ids) -> np.ndarray:
        table_bits, ids = np.ascontiguousarray(table_bits, np.uint16), _u32(ids)
        out = np.zeros((len(ids), table_bits.shape[1]), np.float32)
        self.L.yxref_embed(table_bits.ctypes.data_as(POINTER(c_uint16)), table_bits.shape[1], _u(ids), len(ids), _f(out))
        return out

    def rmsnorm(self, x, w, offset, eps) -> np.ndarray:
        x = _f32(x)
        out = np.zeros_like(x)
        self.L.yxref_rmsnorm(_f(x), _f(_f32(w)), x.shape[0], x.shape[1], offset, eps, _f(out))
        return out

    def add_norm(self, x, delta, post_w, post_offset, pre_w, pre_offset, eps):
        """Returns (x after the add, the normalised output); `x` itself is left alone."""
        x, delta = _f32(x).copy(), _f32(delta)
        out = np.zeros_like(x)
        self.L.yxref_add_norm(_f(x), _f(delta), _f(_f32(post_w)), post_offset, _f(_f32(pre_w)), pre_offset, eps,
                              x.shape[0], x.shape[1], _f(out))
        return x, out

    def argmax_rows(self, x) -> np.ndarray:
        x = _f32(x)
        return np.array([self.L.yxref_argmax(_f(x[r]), x.shape[1]) for r in range(x.shape[0])], np.uint32)


def _bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even bf16 bits of an f32 array, NaNs quieted (weights.rs:100-111), vectorised."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    nan = (u & 0x7fffffff) > 0x7f800000
    r = (u + 0x7fff + ((u >> 16) & 1)) >> 16
    r = np.where(nan, (u >> 16) | 0x40, r)
    return r.astype(np.uint16).reshape(x.shape)
