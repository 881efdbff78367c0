"""Seeded synthetic workloads with the shapes of the benchmark configurations: single-sequence
decode, batched decode over a shared prefix, speculative verification, chunked prefill and
long-context decode with the keys split across GPUs.  Everything is generated on the host
from a seed, so the CUDA library and the CPU oracle see identical inputs.

Page tables are built the way yaxus-model's KvCache would hand them out (shared whole pages
for a common prefix, private pages after it) but with the physical page order shuffled by a
seeded permutation, as nothing in the reference guarantees contiguity
(crates/yaxus-model/src/kv.rs:55-71).
"""
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

from ._lib import BF16, F16, F32, HEAD_DIM, PAGE
from .kvcache import PassMeta, slot

D = HEAD_DIM


def to_bits(x: np.ndarray, dtype: int) -> np.ndarray:
    """f32 -> raw storage elements, round to nearest even (uint16 for 16-bit types)."""
    x = np.ascontiguousarray(x, np.float32)
    if dtype == F32:
        return x
    if dtype == F16:
        return x.astype(np.float16).view(np.uint16)
    b = x.view(np.uint32)
    r = (b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)
    return r.astype(np.uint16)


def from_bits(bits: np.ndarray, dtype: int) -> np.ndarray:
    """Raw storage elements -> f32 (exact)."""
    if dtype == F32:
        return np.ascontiguousarray(bits, np.float32)
    if dtype == F16:
        return bits.view(np.float16).astype(np.float32)
    return (bits.astype(np.uint32) << np.uint32(16)).view(np.float32)


def round_through(x: np.ndarray, dtype: int) -> np.ndarray:
    return from_bits(to_bits(x, dtype), dtype)


@dataclass
class Scenario:
    name: str
    hq: int
    hkv: int
    kv_dtype: int
    window: Optional[int]
    arena_pages: int
    tables: List[np.ndarray]          # page table of every sequence
    ctx_len: List[int]                # tokens already cached per sequence
    new_rows: List[int]               # rows of the step per sequence
    meta: PassMeta                    # the step
    q: np.ndarray                     # [T, hq*128] f32
    k_new: np.ndarray                 # [T, hkv*128] f32, not yet rounded
    v_new: np.ndarray
    k_bits: np.ndarray                # [arena_pages*128, hkv*128] cached context, storage elements
    v_bits: np.ndarray
    seed: int = 0
    extra: dict = field(default_factory=dict)

    @property
    def kvd(self) -> int:
        return self.hkv * D

    @property
    def esize(self) -> int:
        return 4 if self.kv_dtype == F32 else 2

    def k_f32(self) -> np.ndarray:
        return from_bits(self.k_bits, self.kv_dtype)

    def v_f32(self) -> np.ndarray:
        return from_bits(self.v_bits, self.kv_dtype)

    def unique_kv_bytes(self) -> int:
        """K+V bytes of the distinct cached tokens the step reads (own new rows included)."""
        seen = set()
        total = 0
        for s, tab in enumerate(self.tables):
            n = self.ctx_len[s] + self.new_rows[s]
            lo = 0
            if self.window:
                lo = max(0, self.ctx_len[s] + 1 - self.window)   # first row's window start
            for pi in range(lo // PAGE, (n + PAGE - 1) // PAGE):
                a, b = max(lo, pi * PAGE), min(n, (pi + 1) * PAGE)
                key = int(tab[pi])
                if key in seen:
                    continue
                seen.add(key)
                total += b - a
        return total * 2 * self.kvd * self.esize

    def logical_kv_bytes(self) -> int:
        total = 0
        for s in range(len(self.tables)):
            n = self.ctx_len[s] + self.new_rows[s]
            lo = max(0, self.ctx_len[s] + 1 - self.window) if self.window else 0
            total += n - lo
        return total * 2 * self.kvd * self.esize

    def flops(self) -> float:
        """Causal-exact attention FLOPs of the step: 4*D per (query row, head, visible key)."""
        keys = 0
        for r in range(self.meta.rows):
            p = int(self.meta.pos[r])
            lo = max(0, p + 1 - self.window) if self.window else 0
            keys += p + 1 - lo
        return 4.0 * D * keys * self.hq


def _normal(rng: np.random.Generator, shape) -> np.ndarray:
    return rng.standard_normal(shape, dtype=np.float32)


def build(name: str, seed: int, hq: int, hkv: int, kv_dtype: int, ctx_len: List[int], new_rows: List[int],
          shared_prefix: int = 0, window: Optional[int] = None, arena_pages: Optional[int] = None,
          fill: bool = True) -> Scenario:
    """Sequences with `ctx_len[s]` cached tokens each, the first `shared_prefix` tokens of all
    of them in the same physical pages (a multiple of the page size), and `new_rows[s]` rows in
    the step at the next positions."""
    assert shared_prefix % PAGE == 0 and all(c >= shared_prefix for c in ctx_len)
    rng = np.random.default_rng(seed)
    n_seq = len(ctx_len)
    shared_pages = shared_prefix // PAGE
    need = [(ctx_len[s] + new_rows[s] + PAGE - 1) // PAGE for s in range(n_seq)]
    total = shared_pages + sum(n - shared_pages for n in need)
    if arena_pages is None:
        arena_pages = total + 3
    assert arena_pages >= total
    perm = rng.permutation(arena_pages).astype(np.uint32)
    tables, at = [], shared_pages
    for s in range(n_seq):
        priv = need[s] - shared_pages
        tables.append(np.concatenate([perm[:shared_pages], perm[at:at + priv]]).astype(np.uint32))
        at += priv
    kvd = hkv * D
    esz_dtype = np.float32 if kv_dtype == F32 else np.uint16
    k_bits = np.zeros((arena_pages * PAGE, kvd), esz_dtype)
    v_bits = np.zeros((arena_pages * PAGE, kvd), esz_dtype)
    if fill:
        done = set()
        for s in range(n_seq):
            for pi in range((ctx_len[s] + PAGE - 1) // PAGE):
                pg = int(tables[s][pi])
                if pg in done:
                    continue
                done.add(pg)
                n = min(PAGE, ctx_len[s] - pi * PAGE)
                k_bits[pg * PAGE:pg * PAGE + n] = to_bits(_normal(rng, (n, kvd)), kv_dtype)
                v_bits[pg * PAGE:pg * PAGE + n] = to_bits(_normal(rng, (n, kvd)), kv_dtype)
    rows = [(s, ctx_len[s] + j) for s in range(n_seq) for j in range(new_rows[s])]
    meta = PassMeta.from_rows(rows, tables)
    T = len(rows)
    q = _normal(rng, (T, hq * D))
    k_new = _normal(rng, (T, kvd))
    v_new = _normal(rng, (T, kvd))
    return Scenario(name, hq, hkv, kv_dtype, window, arena_pages, tables, list(ctx_len), list(new_rows), meta, q,
                    k_new, v_new, k_bits, v_bits, seed)


SEED0 = 0x59415801


def single_decode(seed: int = SEED0 + 0, ctx: int = 1024) -> Scenario:
    """One query token, 16 query / 4 KV heads, f32 cache, `ctx` keys including its own."""
    return build("single_decode", seed, 16, 4, F32, [ctx - 1], [1], arena_pages=64)


def batched_decode(seed: int = SEED0 + 1, n_seq: int = 16, prefix: int = 1536, max_suffix: int = 2560,
                   kv_dtype: int = F16, hq: int = 32, hkv: int = 8, fill: bool = True,
                   length_seed: Optional[int] = None, rotate: int = 0) -> Scenario:
    """`n_seq` sequences sharing a `prefix`-token prefix through the same physical pages, each
    with a private suffix of seeded uniform length in [0, max_suffix], one query token each.
    `length_seed` draws the lengths from another seed than the pages and values (shards of equal
    work: every shard the same lengths, rotated by `rotate` sequences, over its own data)."""
    rng = np.random.default_rng((seed if length_seed is None else length_seed) ^ 0xABCDEF)
    suffix = [int(x) for x in rng.integers(0, max_suffix + 1, n_seq)]
    suffix = suffix[rotate % n_seq:] + suffix[:rotate % n_seq]
    return build("batched_decode", seed, hq, hkv, kv_dtype, [prefix + s for s in suffix], [1] * n_seq,
                 shared_prefix=prefix, fill=fill)


def verify(seed: int = SEED0 + 2, n_seq: int = 16, ctx: int = 2048, rows: int = 5, kv_dtype: int = F16,
           hq: int = 32, hkv: int = 8, fill: bool = True) -> Scenario:
    """Speculative verification: `rows` query tokens per sequence (one accepted + drafts) at
    consecutive positions after a private `ctx`-token context."""
    return build("verify", seed, hq, hkv, kv_dtype, [ctx] * n_seq, [rows] * n_seq, fill=fill)


def prefill_chunk(seed: int = SEED0 + 3, n_seq: int = 8, done: int = 0, chunk: int = 512, kv_dtype: int = BF16,
                  hq: int = 32, hkv: int = 8, total: int = 4096, fill: bool = True) -> Scenario:
    """One 512-row chunk per sequence after `done` cached tokens."""
    s = build("prefill_chunk", seed, hq, hkv, kv_dtype, [done] * n_seq, [chunk] * n_seq,
              arena_pages=n_seq * ((total + PAGE - 1) // PAGE) + 3, fill=fill)
    return s


def prefill_passes(seed: int = SEED0 + 3, n_seq: int = 8, total: int = 4096, chunk: int = 512, kv_dtype: int = BF16,
                   hq: int = 32, hkv: int = 8, chunks: Optional[range] = None) -> List[Scenario]:
    """Chunked prefill of `n_seq` sequences of `total` tokens: one Scenario per chunk index, all
    over the same page tables; chunk c holds rows [c*chunk, (c+1)*chunk) of every sequence.
    Each scenario carries the chunk's q and the k, v rows it appends; its cached context is
    left empty (the passes are meant to be run in order on one cache)."""
    rng = np.random.default_rng(seed)
    pages_per_seq = (total + PAGE - 1) // PAGE
    arena_pages = n_seq * pages_per_seq + 3
    perm = rng.permutation(arena_pages).astype(np.uint32)
    tables = [perm[s * pages_per_seq:(s + 1) * pages_per_seq].copy() for s in range(n_seq)]
    kvd = hkv * D
    out = []
    empty = np.zeros((0, kvd), np.float32 if kv_dtype == F32 else np.uint16)
    for c in (chunks if chunks is not None else range(total // chunk)):
        rows = [(s, c * chunk + j) for s in range(n_seq) for j in range(chunk)]
        meta = PassMeta.from_rows(rows, tables)
        T = len(rows)
        crng = np.random.default_rng(seed * 1000 + c)
        q = round_through(_normal(crng, (T, hq * D)), kv_dtype)
        k_new = _normal(crng, (T, kvd))
        v_new = _normal(crng, (T, kvd))
        out.append(Scenario(f"prefill_chunk_{c}", hq, hkv, kv_dtype, None, arena_pages, tables, [c * chunk] * n_seq,
                            [chunk] * n_seq, meta, q, k_new, v_new, empty, empty, seed))
    return out


def long_decode(seed: int = SEED0 + 4, ctx: int = 131072, window: Optional[int] = None, kv_dtype: int = F16,
                hq: int = 32, hkv: int = 8, fill: bool = True) -> Scenario:
    """One sequence, one query token, `ctx` keys including its own."""
    return build("long_decode", seed, hq, hkv, kv_dtype, [ctx - 1], [1], window=window,
                 arena_pages=(ctx + PAGE - 1) // PAGE, fill=fill)


def partition_pages(n_pages: int, world: int, rank: int):
    """Contiguous page range `[first, last)` of `rank` when `n_pages` pages are split across
    `world` GPUs, and the matching key range."""
    first = n_pages * rank // world
    last = n_pages * (rank + 1) // world
    return first, last, first * PAGE, last * PAGE
