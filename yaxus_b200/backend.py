"""`CudaBackend`: the hot-path half of yaxus's `trait Backend`
(crates/yaxus-model/src/lib.rs:95-171) over libyaxus_cuda's C ABI.

Method names, argument meaning and error behaviour follow the trait: `new_kv`, `copy_page`,
`begin_pass`, `attention`, and `to_host` from `SyncReadback` (lib.rs:177-185).  As in the
reference, `attention`, `copy_page` and `begin_pass` do not return errors; a failure sticks to
the backend and is raised by the next read-back (`to_host`, `sync`).  PyTorch is used only to
own device memory and the stream; every computation is a kernel of the C library.
"""
import ctypes
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import _lib
from ._lib import BF16, F16, F32, HEAD_DIM, PAGE
from .kvcache import PassMeta

_TORCH_DTYPE = {F32: torch.float32, F16: torch.float16, BF16: torch.bfloat16}
_YX_DTYPE = {v: k for k, v in _TORCH_DTYPE.items()}


class BackendError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"yaxus_cuda error {code}: {message}")
        self.code = code


@dataclass
class Rope:
    """Rope (crates/yaxus-model/src/config.rs:174-179)."""
    inv_freq: np.ndarray
    concentration: float = 1.0

    @staticmethod
    def default(theta: float = 10000.0, dim: int = HEAD_DIM) -> "Rope":
        # Rope::new without scaling (config.rs:185-188), in f32 like the reference.
        i = np.arange(0, dim, 2, dtype=np.float32)
        freq = np.power(np.float32(theta), i / np.float32(dim)).astype(np.float32)
        return Rope((np.float32(1.0) / freq).astype(np.float32), 1.0)


@dataclass
class LayerMeta:
    """LayerMeta (crates/yaxus-model/src/config.rs:163-170)."""
    index: int = 0
    window: Optional[int] = None
    rope: Rope = field(default_factory=Rope.default)

    @property
    def full_attn(self) -> bool:
        return self.window is None


class Kv:
    """Opaque paged K/V storage of all layers of one model (`Backend::Kv`)."""

    def __init__(self, backend: "CudaBackend", handle, layers: List[LayerMeta], pages: int, hkv: int, dtype: int,
                 max_pos: int):
        self._backend, self._h = backend, handle
        self.layers, self.pages, self.hkv, self.dtype, self.max_pos = layers, pages, hkv, dtype, max_pos
        self.kv_dim = hkv * HEAD_DIM

    def close(self):
        if self._h:
            self._backend._L.yx_kv_destroy(self._backend._ctx, self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _u32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint32)


def _u32p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32))


class CudaBackend:
    def __init__(self, device: int = 0, stream: Optional[torch.cuda.Stream] = None):
        self._L = _lib.cuda_lib()
        if not torch.cuda.is_available():
            raise BackendError(_lib.YX_ERR_CUDA, "no CUDA device: yaxus_b200 has no CPU fallback")
        self.device = torch.device("cuda", device)
        torch.cuda.set_device(self.device)
        self.stream = stream if stream is not None else torch.cuda.current_stream(self.device)
        ctx = ctypes.c_void_p()
        # torch's default stream has handle 0, which the C ABI reads as "make a private stream":
        # name the legacy default stream explicitly (cudaStreamLegacy == 1).
        handle = self.stream.cuda_stream or 1
        rc = self._L.yx_ctx_create(device, ctypes.c_void_p(handle), ctypes.byref(ctx))
        if rc != _lib.YX_OK:
            raise BackendError(rc, "yx_ctx_create failed (is this an sm_100 GPU?)")
        self._ctx = ctx
        self._rows = 0
        self._ids = None
        self.world_size, self.rank = 1, 0

    def close(self):
        if getattr(self, "_ctx", None):
            self._L.yx_ctx_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- trait plumbing ----------------------------------------------------------------
    def name(self) -> str:
        return f"cuda:{self.device.index} (sm_100a)"

    def status(self) -> int:
        return self._L.yx_status(self._ctx)

    def last_error(self) -> str:
        return self._L.yx_last_error(self._ctx).decode()

    def clear_error(self) -> None:
        self._L.yx_clear_error(self._ctx)

    def _raise_if_failed(self) -> None:
        rc = self.status()
        if rc != _lib.YX_OK:
            raise BackendError(rc, self.last_error())

    def sync(self) -> None:
        """Waits for the device and raises the sticky error, if any (the read-back check)."""
        rc = self._L.yx_sync(self._ctx)
        if rc != _lib.YX_OK:
            raise BackendError(rc, self.last_error())

    def to_host(self, x: torch.Tensor) -> np.ndarray:
        """SyncReadback::to_host (lib.rs:184)."""
        self.sync()
        return x.detach().float().cpu().numpy()

    def set_tuning(self, force_path: int = 0, ctas_per_sm: int = 0, share_prefix: int = 0, tile_min_rows: int = 0,
                   cost32: int = 0, cost64: int = 0, stages: int = 0, share_rows: int = 0,
                   item_cost: int = 0, fused_merge: int = 0, tile_single: int = 0, min_piece: int = 0, overlap_calls: int = 0):
        t = _lib.Tuning(force_path, ctas_per_sm, share_prefix, tile_min_rows, cost32, cost64, stages, share_rows, item_cost,
                        fused_merge, tile_single, min_piece, overlap_calls)
        self._L.yx_set_tuning(self._ctx, ctypes.byref(t))

    def hook_skip_merge(self, on: bool) -> None:
        """Measurement hook (csrc/yx_hooks.h): attention calls leave the merge out."""
        self._L.yx_hook_skip_merge(self._ctx, 1 if on else 0)

    def last_plan(self) -> _lib.PlanInfo:
        info = _lib.PlanInfo()
        self._L.yx_last_plan(self._ctx, ctypes.byref(info))
        return info

    def launch_count(self) -> int:
        return self._L.yx_launch_count(self._ctx)

    def profile_begin(self) -> None:
        self._L.yx_profile_begin(self._ctx)

    def profile_end(self):
        """(split-key kernel ms, combine kernel ms, attention calls) since profile_begin."""
        a, b, n = ctypes.c_float(0), ctypes.c_float(0), ctypes.c_int(0)
        rc = self._L.yx_profile_end(self._ctx, ctypes.byref(a), ctypes.byref(b), ctypes.byref(n))
        if rc != _lib.YX_OK:
            raise BackendError(rc, self.last_error())
        return a.value, b.value, n.value

    # ---- Backend::new_kv / copy_page / begin_pass / attention ---------------------------
    def new_kv(self, hkv: int, layers: Sequence[LayerMeta], pages: int, max_pos: int, dtype: int = F32,
               head_dim: int = HEAD_DIM) -> Kv:
        """Backend::new_kv (lib.rs:118).  Fallible, like the reference's `Result<Kv>`."""
        arr = (_lib.Layer * len(layers))()
        for i, lm in enumerate(layers):
            arr[i].window = int(lm.window) if lm.window else 0
            inv = np.asarray(lm.rope.inv_freq, np.float32)
            if inv.shape != (HEAD_DIM // 2,):
                raise BackendError(_lib.YX_ERR_INVALID, "rope.inv_freq must have head_dim/2 entries")
            for j in range(HEAD_DIM // 2):
                arr[i].rope.inv_freq[j] = float(inv[j])
            arr[i].rope.concentration = float(lm.rope.concentration)
        h = ctypes.c_void_p()
        rc = self._L.yx_kv_create(self._ctx, len(layers), arr, pages, hkv, head_dim, dtype, max_pos, ctypes.byref(h))
        if rc != _lib.YX_OK:
            msg = self.last_error()
            self.clear_error()
            raise BackendError(rc, msg)
        return Kv(self, h, list(layers), pages, hkv, dtype, max_pos)

    def copy_page(self, kv: Kv, src: int, dst: int) -> None:
        """Backend::copy_page (lib.rs:120)."""
        self._L.yx_kv_copy_page(self._ctx, kv._h, src, dst)

    def begin_pass(self, meta: PassMeta) -> None:
        """Backend::begin_pass (lib.rs:123)."""
        pos, slot, off, pages = _u32(meta.pos), _u32(meta.kv_slot), _u32(meta.pt_off), _u32(meta.pages)
        self._rows = len(pos)
        self._ids = _u32(meta.ids) if len(meta.ids) == len(pos) else None
        self._L.yx_begin_pass(self._ctx, len(pos), _u32p(pos), _u32p(slot), _u32p(off), _u32p(pages), len(pages))

    # ---- the operators either side of attention (lib.rs:124-171) --------------------------
    def load_weight(self, values, shape=None) -> torch.Tensor:
        """Backend::load_weight with Quant::Bf16 (lib.rs:104-106; cpu :455-462).  `values`: bf16 bit
        patterns (uint16 array) or a tensor.  Matrices and the embedding table stay bf16 on the
        device; vectors are widened to f32, as the reference's `vector_f32` does (cpu :200-202)."""
        if isinstance(values, np.ndarray) and values.dtype == np.uint16:
            t = torch.from_numpy(np.ascontiguousarray(values).view(np.int16)).view(torch.bfloat16)
        else:
            t = torch.as_tensor(values).to(torch.bfloat16)
        if shape is not None:
            t = t.reshape(tuple(shape))
        t = t.to(self.device).contiguous()
        self._weight_bytes = getattr(self, "_weight_bytes", 0) + t.numel() * 2
        return t.float() if t.dim() == 1 else t

    def weight_bytes(self) -> int:
        return getattr(self, "_weight_bytes", 0)

    def _f32(self, rows: int, cols: int) -> torch.Tensor:
        return torch.empty(rows, cols, dtype=torch.float32, device=self.device)

    def embed(self, table: torch.Tensor) -> torch.Tensor:
        """Backend::embed (lib.rs:125): the embedding rows of the pass's token ids."""
        assert table.dtype == torch.bfloat16 and table.dim() == 2 and table.is_contiguous()
        if self._ids is None:
            raise AssertionError("the pass carries no token ids")
        out = self._f32(len(self._ids), table.shape[1])
        self._L.yx_embed(self._ctx, _ptr(table), table.shape[0], table.shape[1], _u32p(self._ids), len(self._ids), _ptr(out))
        return out

    def rmsnorm(self, x: torch.Tensor, w: torch.Tensor, offset: float, eps: float) -> torch.Tensor:
        assert x.dtype == torch.float32 and x.is_contiguous() and w.dtype == torch.float32 and w.numel() == x.shape[1]
        out = torch.empty_like(x)
        self._L.yx_rmsnorm(self._ctx, _ptr(x), _ptr(w), x.shape[0], x.shape[1], offset, eps, _ptr(out))
        return out

    def add_norm(self, x: torch.Tensor, delta: torch.Tensor, post_w: torch.Tensor, post_offset: float,
                 pre_w: torch.Tensor, pre_offset: float, eps: float) -> torch.Tensor:
        """Backend::add_norm (lib.rs:149-162): `x` is updated in place, the return is pre_norm(x)."""
        assert x.shape == delta.shape and x.dtype == delta.dtype == torch.float32 and x.is_contiguous() and delta.is_contiguous()
        out = torch.empty_like(x)
        self._L.yx_add_norm(self._ctx, _ptr(x), _ptr(delta), _ptr(post_w), post_offset, _ptr(pre_w), pre_offset, eps,
                            x.shape[0], x.shape[1], _ptr(out))
        return out

    def matmul(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """Backend::matmul (lib.rs:128): `x [T, K] . w[N, K]^T -> [T, N]`, w a bf16 matrix."""
        assert x.dtype == torch.float32 and x.is_contiguous() and w.dtype == torch.bfloat16 and w.is_contiguous()
        assert x.shape[1] == w.shape[1], "matmul inner dim"
        out = self._f32(x.shape[0], w.shape[0])
        self._L.yx_matmul(self._ctx, _ptr(x), _ptr(w), x.shape[0], w.shape[0], w.shape[1], _ptr(out))
        return out

    def matmul_glu(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """Backend::matmul_glu (lib.rs:164-168): swiglu(x . w^T) for w = [gate; up]."""
        assert x.dtype == torch.float32 and x.is_contiguous() and w.dtype == torch.bfloat16 and w.is_contiguous()
        assert x.shape[1] == w.shape[1], "matmul inner dim"
        out = self._f32(x.shape[0], w.shape[0] // 2)
        self._L.yx_matmul_glu(self._ctx, _ptr(x), _ptr(w), x.shape[0], w.shape[0], w.shape[1], _ptr(out))
        return out

    def swiglu(self, x: torch.Tensor) -> torch.Tensor:
        assert x.dtype == torch.float32 and x.is_contiguous() and x.shape[1] % 2 == 0
        out = self._f32(x.shape[0], x.shape[1] // 2)
        self._L.yx_swiglu(self._ctx, _ptr(x), x.shape[0], x.shape[1] // 2, _ptr(out))
        return out

    def add_assign(self, a: torch.Tensor, b: torch.Tensor) -> None:
        assert a.numel() == b.numel() and a.dtype == b.dtype == torch.float32 and a.is_contiguous() and b.is_contiguous()
        self._L.yx_add_assign(self._ctx, _ptr(a), _ptr(b), a.numel())

    def select_rows(self, x: torch.Tensor, rows) -> torch.Tensor:
        assert x.dtype == torch.float32 and x.is_contiguous()
        idx = _u32(np.asarray(rows))
        out = self._f32(len(idx), x.shape[1])
        self._L.yx_select_rows(self._ctx, _ptr(x), x.shape[0], x.shape[1], _u32p(idx), len(idx), _ptr(out))
        return out

    def argmax_rows(self, logits: torch.Tensor) -> np.ndarray:
        """SyncReadback::argmax_rows (lib.rs:177-185): waits for the device; raises its sticky error."""
        assert logits.dtype == torch.float32 and logits.is_contiguous()
        out = np.zeros(logits.shape[0], np.uint32)
        rc = self._L.yx_argmax_rows(self._ctx, _ptr(logits), logits.shape[0], logits.shape[1], _u32p(out))
        if rc != _lib.YX_OK:
            raise BackendError(rc, self.last_error())
        return out

    def attention(self, qkv: torch.Tensor, q_norm: torch.Tensor, k_norm: torch.Tensor, kv: Kv, hq: int, eps: float,
                  layer: LayerMeta) -> torch.Tensor:
        """Backend::attention (lib.rs:132-140): `[T, (Hq+2Hkv)*D]` f32 -> `[T, Hq*D]` f32."""
        assert qkv.dtype == torch.float32 and qkv.is_contiguous() and qkv.is_cuda
        rows = qkv.shape[0]
        if rows != self._rows:   # the reference asserts this (cpu lib.rs:525)
            raise AssertionError("attention rows differ from the pass")
        out = torch.empty(rows, hq * HEAD_DIM, dtype=torch.float32, device=self.device)
        self._L.yx_attention(self._ctx, kv._h, layer.index, _ptr(qkv), _ptr(q_norm.float().contiguous()),
                             _ptr(k_norm.float().contiguous()), hq, eps, _ptr(out))
        return out

    # ---- the two halves of attention, for callers that hold final q, k, v ----------------
    def kv_append(self, kv: Kv, layer: int, k_rows: torch.Tensor, v_rows: torch.Tensor) -> None:
        assert k_rows.is_contiguous() and v_rows.is_contiguous() and k_rows.dtype == v_rows.dtype
        self._L.yx_kv_append(self._ctx, kv._h, layer, _ptr(k_rows), _ptr(v_rows), _YX_DTYPE[k_rows.dtype])

    def attend(self, kv: Kv, layer: int, q: torch.Tensor, hq: int, window: Optional[int] = -1,
               out_dtype: torch.dtype = torch.float32, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """window: -1 the layer's own, None or 0 none, > 0 that many keys."""
        assert q.is_contiguous() and q.is_cuda
        if out is None:
            out = torch.empty(q.shape[0], hq * HEAD_DIM, dtype=out_dtype, device=self.device)
        w = 0 if window is None else int(window)
        self._L.yx_attend(self._ctx, kv._h, layer, _ptr(q), _YX_DTYPE[q.dtype], hq, w, _ptr(out), _YX_DTYPE[out.dtype])
        return out

    def attend_partial(self, kv: Kv, layer: int, q: torch.Tensor, hq: int, window, key_lo: int, key_hi: int):
        rows = q.shape[0]
        m = torch.empty(rows, hq, dtype=torch.float32, device=self.device)
        l = torch.empty(rows, hq, dtype=torch.float32, device=self.device)
        o = torch.zeros(rows, hq, HEAD_DIM, dtype=torch.float32, device=self.device)
        w = 0 if window is None else int(window)
        self._L.yx_attend_partial(self._ctx, kv._h, layer, _ptr(q), _YX_DTYPE[q.dtype], hq, w, key_lo, key_hi, _ptr(m),
                                  _ptr(l), _ptr(o))
        return m, l, o

    def lse_combine(self, m: torch.Tensor, l: torch.Tensor, o: torch.Tensor,
                    out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """m, l `[parts, n]`, o `[parts, n, 128]` -> `[n, 128]`."""
        parts, n = m.shape[0], m[0].numel()
        out = torch.empty(n, HEAD_DIM, dtype=out_dtype, device=self.device)
        self._L.yx_lse_combine(self._ctx, parts, _ptr(m.contiguous()), _ptr(l.contiguous()), _ptr(o.contiguous()), n,
                               _ptr(out), _YX_DTYPE[out_dtype])
        return out

    # ---- keys split across GPUs --------------------------------------------------------
    def comm_create(self, world_size: int, rank: int, broadcast_bytes=None) -> None:
        """One process per GPU.  `broadcast_bytes(buf: bytearray) -> bytes` must return rank
        0's buffer on every rank; by default torch.distributed does it."""
        ident = (ctypes.c_ubyte * 128)()
        if world_size > 1:
            if rank == 0:
                rc = self._L.yx_comm_unique_id(ident)
                if rc != _lib.YX_OK:
                    raise BackendError(rc, "yx_comm_unique_id failed")
            if broadcast_bytes is None:
                import torch.distributed as dist
                t = torch.tensor(list(bytes(ident)), dtype=torch.uint8, device=self.device)
                dist.broadcast(t, src=0)
                data = bytes(t.cpu().tolist())
            else:
                data = broadcast_bytes(bytes(ident))
            ident = (ctypes.c_ubyte * 128).from_buffer_copy(data)
        rc = self._L.yx_comm_create(self._ctx, world_size, rank, ident)
        if rc != _lib.YX_OK:
            raise BackendError(rc, self.last_error())
        self.world_size, self.rank = world_size, rank

    def attend_allgather(self, kv: Kv, layer: int, q: torch.Tensor, hq: int, window, key_lo: int, key_hi: int,
                         out_dtype: torch.dtype = torch.float32, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty(q.shape[0], hq * HEAD_DIM, dtype=out_dtype, device=self.device)
        w = 0 if window is None else int(window)
        self._L.yx_attend_allgather(self._ctx, kv._h, layer, _ptr(q), _YX_DTYPE[q.dtype], hq, w, key_lo, key_hi,
                                    _ptr(out), _YX_DTYPE[out.dtype])
        return out

    # ---- page import / export (tests, cache migration) -----------------------------------
    def read_pages(self, kv: Kv, layer: int, first_page: int, n_pages: int = 1):
        """(K, V) of consecutive pages in the reference's layout `[n_pages*128, hkv*128]`, as
        raw storage elements (float32, or uint16 bit patterns for 16-bit caches)."""
        np_dtype = np.float32 if kv.dtype == F32 else np.uint16
        k = np.zeros((n_pages * PAGE, kv.kv_dim), np_dtype)
        v = np.zeros((n_pages * PAGE, kv.kv_dim), np_dtype)
        rc = self._L.yx_kv_read_pages(self._ctx, kv._h, layer, first_page, n_pages, k.ctypes.data_as(ctypes.c_void_p),
                                      v.ctypes.data_as(ctypes.c_void_p))
        if rc != _lib.YX_OK:
            raise BackendError(rc, self.last_error())
        return k, v

    def write_pages(self, kv: Kv, layer: int, first_page: int, k: np.ndarray, v: np.ndarray) -> None:
        np_dtype = np.float32 if kv.dtype == F32 else np.uint16
        k = np.ascontiguousarray(k, np_dtype)
        v = np.ascontiguousarray(v, np_dtype)
        assert k.shape == v.shape and k.shape[1] == kv.kv_dim and k.shape[0] % PAGE == 0
        rc = self._L.yx_kv_write_pages(self._ctx, kv._h, layer, first_page, k.shape[0] // PAGE,
                                       k.ctypes.data_as(ctypes.c_void_p), v.ctypes.data_as(ctypes.c_void_p))
        if rc != _lib.YX_OK:
            raise BackendError(rc, self.last_error())
