"""Python face of the host-side KvCache restatement (csrc/host/kv_cache.hpp), which mirrors
yaxus-model's `KvCache` (crates/yaxus-model/src/kv.rs:110-353): same method names, same
results.  Used by tests and benchmarks to produce the PassMeta arrays and PageCopy lists the
reference would hand a backend."""
import ctypes
from dataclasses import dataclass, field
from typing import List, Sequence, Tuple

import numpy as np

from . import _lib

PAGE = _lib.PAGE
MIN_REUSE = 16
MAX_CACHED = 32


def slot(pages: Sequence[int], pos: int) -> int:
    """kv::slot (crates/yaxus-model/src/kv.rs:20-22)."""
    return int(pages[pos // PAGE]) * PAGE + pos % PAGE


@dataclass
class PassMeta:
    """PassMeta (crates/yaxus-model/src/lib.rs:63-75) plus PassRows::last."""
    ids: np.ndarray = field(default_factory=lambda: np.zeros(0, np.uint32))
    pos: np.ndarray = field(default_factory=lambda: np.zeros(0, np.uint32))
    kv_slot: np.ndarray = field(default_factory=lambda: np.zeros(0, np.uint32))
    pt_off: np.ndarray = field(default_factory=lambda: np.zeros(0, np.uint32))
    pages: np.ndarray = field(default_factory=lambda: np.zeros(0, np.uint32))
    last: np.ndarray = field(default_factory=lambda: np.zeros(0, np.uint32))

    @property
    def rows(self) -> int:
        return len(self.pos)

    def page_table(self, row: int) -> np.ndarray:
        return self.pages[int(self.pt_off[row]):]

    def slot(self, row: int, pos: int) -> int:
        return slot(self.page_table(row), pos)

    @staticmethod
    def from_rows(rows: Sequence[Tuple[int, int]], page_tables: Sequence[Sequence[int]]) -> "PassMeta":
        """Rows `(sequence, position)` over explicit page tables, as the reference's attention
        test builds its pass (crates/yaxus-backend-cpu/src/lib.rs:645-662)."""
        meta = PassMeta()
        ids, pos, kv_slot, pt_off, pages = [], [], [], [], []
        off = {}
        for sq, p in rows:
            if sq not in off:
                off[sq] = len(pages)
                pages.extend(int(x) for x in page_tables[sq])
            ids.append(0)
            pos.append(p)
            kv_slot.append(slot(page_tables[sq], p))
            pt_off.append(off[sq])
        meta.ids = np.array(ids, np.uint32)
        meta.pos = np.array(pos, np.uint32)
        meta.kv_slot = np.array(kv_slot, np.uint32)
        meta.pt_off = np.array(pt_off, np.uint32)
        meta.pages = np.array(pages, np.uint32)
        return meta


def _u32p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32))


class KvCacheError(RuntimeError):
    pass


class KvCache:
    def __init__(self, pages: int, max_pos: int):
        self._L = _lib.host_lib()
        self._h = ctypes.c_void_p(self._L.yxh_kvcache_new(pages, max_pos))

    def __del__(self):
        if getattr(self, "_h", None):
            self._L.yxh_kvcache_free(self._h)
            self._h = None

    def _check(self, rc: int) -> int:
        if rc < 0:
            raise KvCacheError(self._L.yxh_last_error().decode())
        return rc

    def set_prefix_reuse(self, on: bool) -> None:
        self._L.yxh_set_prefix_reuse(self._h, int(on))

    def new_seq(self) -> int:
        return self._L.yxh_new_seq(self._h)

    def free_seq(self, seq: int) -> None:
        self._L.yxh_free_seq(self._h, seq)

    def finish(self, seq: int) -> None:
        self._L.yxh_finish(self._h, seq)

    def seq_len(self, seq: int) -> int:
        return self._L.yxh_seq_len(self._h, seq)

    def free_pages(self) -> int:
        return self._L.yxh_free_pages(self._h)

    def total_pages(self) -> int:
        return self._L.yxh_total_pages(self._h)

    def page_refs(self, page: int) -> int:
        return self._L.yxh_page_refs(self._h, page)

    def seq_pages(self, seq: int) -> np.ndarray:
        n = self._L.yxh_seq_pages(self._h, seq, None, 0)
        out = np.zeros(max(n, 1), np.uint32)
        self._L.yxh_seq_pages(self._h, seq, _u32p(out), n)
        return out[:n]

    def seq_tokens(self, seq: int) -> np.ndarray:
        n = self._L.yxh_seq_tokens(self._h, seq, None, 0)
        out = np.zeros(max(n, 1), np.uint32)
        self._L.yxh_seq_tokens(self._h, seq, _u32p(out), n)
        return out[:n]

    def begin(self, prompt: Sequence[int]) -> Tuple[int, int]:
        """(sequence, prompt tokens already in it); page copies it needs are left pending."""
        p = np.ascontiguousarray(prompt, np.uint32)
        reused = ctypes.c_uint64(0)
        seq = self._check(self._L.yxh_begin(self._h, _u32p(p), len(p), ctypes.byref(reused)))
        return seq, reused.value

    def fork(self, seq: int, length: int) -> int:
        return self._check(self._L.yxh_fork(self._h, seq, length))

    def truncate(self, seq: int, length: int) -> None:
        self._check(self._L.yxh_truncate(self._h, seq, length))

    def append(self, items: Sequence[Tuple[int, Sequence[int]]]) -> PassMeta:
        ids = np.array([s for s, _ in items], np.uint64)
        counts = np.array([len(t) for _, t in items], np.uint64)
        toks = np.ascontiguousarray(np.concatenate([np.asarray(t, np.uint32) for _, t in items])
                                    if items else np.zeros(0, np.uint32), np.uint32)
        rows = self._check(self._L.yxh_append(
            self._h, len(items), ids.ctypes.data_as(ctypes.POINTER(ctypes.c_uint64)),
            counts.ctypes.data_as(ctypes.POINTER(ctypes.c_uint64)), _u32p(toks)))
        n_pages = self._L.yxh_meta_pages(self._h)
        n_items = self._L.yxh_meta_items(self._h)
        m = PassMeta(*(np.zeros(max(n, 1), np.uint32) for n in (rows, rows, rows, rows, n_pages, n_items)))
        self._L.yxh_meta_get(self._h, _u32p(m.ids), _u32p(m.pos), _u32p(m.kv_slot), _u32p(m.pt_off), _u32p(m.pages),
                             _u32p(m.last))
        m.ids, m.pos, m.kv_slot, m.pt_off = m.ids[:rows], m.pos[:rows], m.kv_slot[:rows], m.pt_off[:rows]
        m.pages, m.last = m.pages[:n_pages], m.last[:n_items]
        return m

    def take_copies(self) -> List[Tuple[int, int]]:
        """The pending PageCopy list, in the order the copies must be made."""
        n = self._L.yxh_copies_pending(self._h)
        src, dst = np.zeros(max(n, 1), np.uint32), np.zeros(max(n, 1), np.uint32)
        self._L.yxh_copies_take(self._h, _u32p(src), _u32p(dst), n)
        return [(int(src[i]), int(dst[i])) for i in range(n)]
