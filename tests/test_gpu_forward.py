"""A whole forward pass through the Backend operators in the reference's order
(Model::forward, crates/yaxus-model/src/lib.rs:434-471) on a small random model, against the
same pass composed from the CPU oracle's operators: prompt chunk, fork over shared pages with a
page copy, a pass that mixes one decode row with three rows of another sequence, greedy decode."""
import numpy as np
import pytest

from oracle.check import ABS_TOL, REL_TOL, assert_close
from yaxus_b200._lib import BF16, F16, F32, PAGE
from yaxus_b200.backend import LayerMeta, Rope
from yaxus_b200.kvcache import KvCache

pytestmark = pytest.mark.gpu

# crates/yaxus-model/src/lib.rs:24-27
PRE_NORM_OFFSET, POST_MIXER_NORM_OFFSET, POST_MLP_NORM_OFFSET = 1.0, 0.2, 0.08944272
VOCAB, HIDDEN, INNER, HQ, HKV, D, EPS = 333, 256, 384, 4, 2, 128, 1e-6


def bf16_to_f32(bits):
    return (np.asarray(bits).astype(np.uint32) << 16).view(np.float32)


class TinyWeights:
    """bf16 matrices as bit patterns, vectors as the f32 values of their bf16 roundings."""

    def __init__(self, oracle, n_layers, seed):
        rng = np.random.default_rng(seed)
        mat = lambda n, k: oracle.to_bf16((rng.standard_normal((n, k)) / np.sqrt(k)).astype(np.float32))
        vec = lambda n: bf16_to_f32(oracle.to_bf16((0.1 * rng.standard_normal(n)).astype(np.float32)))
        self.embed = oracle.to_bf16(rng.standard_normal((VOCAB, HIDDEN)).astype(np.float32))
        self.norm = vec(HIDDEN)
        self.lm_head = mat(VOCAB, HIDDEN)
        self.layers = []
        for _ in range(n_layers):
            self.layers.append(dict(
                pre_mixer_norm=vec(HIDDEN), qkv_proj=mat((HQ + 2 * HKV) * D, HIDDEN), q_norm=vec(D), k_norm=vec(D),
                o_proj=mat(HIDDEN, HQ * D), post_mixer_norm=vec(HIDDEN), pre_mlp_norm=vec(HIDDEN),
                gate_up_proj=mat(2 * INNER, HIDDEN), down_proj=mat(HIDDEN, INNER), post_mlp_norm=vec(HIDDEN)))


def on_device(backend, w):
    # (the vectors hold bf16-representable values: their upper halves are their bf16 bit patterns)
    put = lambda a: backend.load_weight(a if a.dtype == np.uint16 else (a.view(np.uint32) >> 16).astype(np.uint16))
    out = TinyWeights.__new__(TinyWeights)
    out.embed, out.norm, out.lm_head = put(w.embed), put(w.norm), put(w.lm_head)
    out.layers = [{k: put(v) for k, v in l.items()} for l in w.layers]
    return out


def forward_cuda(b, w, kv, metas, meta):
    b.begin_pass(meta)
    x = b.embed(w.embed)
    h = b.rmsnorm(x, w.layers[0]["pre_mixer_norm"], PRE_NORM_OFFSET, EPS)
    for i, l in enumerate(w.layers):
        qkv = b.matmul(h, l["qkv_proj"])
        a = b.attention(qkv, l["q_norm"], l["k_norm"], kv, HQ, EPS, metas[i])
        o = b.matmul(a, l["o_proj"])
        hm = b.add_norm(x, o, l["post_mixer_norm"], POST_MIXER_NORM_OFFSET, l["pre_mlp_norm"], PRE_NORM_OFFSET, EPS)
        m = b.matmul(b.matmul_glu(hm, l["gate_up_proj"]), l["down_proj"])
        nxt = w.layers[i + 1]["pre_mixer_norm"] if i + 1 < len(w.layers) else w.norm
        h = b.add_norm(x, m, l["post_mlp_norm"], POST_MLP_NORM_OFFSET, nxt, PRE_NORM_OFFSET, EPS)
    sel = h if len(meta.last) == meta.rows else b.select_rows(h, meta.last)
    return b.matmul(sel, w.lm_head)


def forward_oracle(o, w, arenas, metas, meta, kv_dtype):
    x = o.embed(w.embed, meta.ids)
    h = o.rmsnorm(x, w.layers[0]["pre_mixer_norm"], PRE_NORM_OFFSET, EPS)
    for i, l in enumerate(w.layers):
        K, V = arenas[i]
        qkv = o.matmul(h, l["qkv_proj"])
        q = o.write_rows(qkv, meta.pos, meta.kv_slot, l["q_norm"], l["k_norm"], HQ, HKV, D, EPS, metas[i].rope.inv_freq,
                         metas[i].rope.concentration, K, V, store_dtype=kv_dtype)
        a = o.attend(q, meta.pos, meta.pt_off, meta.pages, HQ, HKV, D, metas[i].window, K, V)
        x, hm = o.add_norm(x, o.matmul(a, l["o_proj"]), l["post_mixer_norm"], POST_MIXER_NORM_OFFSET, l["pre_mlp_norm"],
                           PRE_NORM_OFFSET, EPS)
        m = o.matmul(o.swiglu(o.matmul(hm, l["gate_up_proj"])), l["down_proj"])
        nxt = w.layers[i + 1]["pre_mixer_norm"] if i + 1 < len(w.layers) else w.norm
        x, h = o.add_norm(x, m, l["post_mlp_norm"], POST_MLP_NORM_OFFSET, nxt, PRE_NORM_OFFSET, EPS)
    sel = h if len(meta.last) == meta.rows else h[meta.last]
    return o.matmul(sel, w.lm_head)


@pytest.mark.parametrize("kv_dtype,abs_tol", [(F32, 3e-4), (F16, ABS_TOL), (BF16, 2 * ABS_TOL)])
def test_forward_passes_match_the_oracle(backend, oracle, kv_dtype, abs_tol):
    pages, max_pos = 8, 1024
    metas = [LayerMeta(index=0, window=None, rope=Rope.default()), LayerMeta(index=1, window=48, rope=Rope.default(theta=5000.0))]
    w = TinyWeights(oracle, len(metas), seed=11)
    wd = on_device(backend, w)
    kv = backend.new_kv(HKV, metas, pages, max_pos, kv_dtype)
    arenas = [(np.zeros((pages * PAGE, HKV * D), np.float32), np.zeros((pages * PAGE, HKV * D), np.float32)) for _ in metas]
    cache = KvCache(pages, max_pos)
    rng = np.random.default_rng(12)

    def both(items):
        meta = cache.append(items)
        for src, dst in cache.take_copies():     # Model::copy_pages before the pass (lib.rs:438-440)
            backend.copy_page(kv, src, dst)
            for K, V in arenas:
                oracle.copy_page(K, V, HKV * D, src, dst)
        got = backend.to_host(forward_cuda(backend, wd, kv, metas, meta))
        want = forward_oracle(oracle, w, arenas, metas, meta, kv_dtype)
        assert_close(got, want, abs_tol=abs_tol, rel_tol=REL_TOL, what=f"logits of a {meta.rows}-row pass")
        return got, want

    # a 150-token prompt (crosses a page boundary), logits of its last row
    a = cache.new_seq()
    prompt = rng.integers(0, VOCAB, 150)
    got, want = both([(a, prompt)])
    assert got.shape == (1, VOCAB)
    tok_a = int(oracle.argmax_rows(want)[0])
    # a second sequence forks off after 140 tokens: page 0 shared, the half-filled page copied
    b2 = cache.fork(a, 140)
    assert cache.page_refs(int(cache.seq_pages(a)[0])) == 2
    # one decode row of the first sequence and three rows of the fork in one pass
    got, want = both([(a, [tok_a]), (b2, rng.integers(0, VOCAB, 3))])
    assert got.shape == (2, VOCAB)
    toks = oracle.argmax_rows(want)
    # greedy decode of both, the device picking the tokens
    for _ in range(4):
        meta = cache.append([(a, [int(toks[0])]), (b2, [int(toks[1])])])
        assert not cache.take_copies()
        logits = forward_cuda(backend, wd, kv, metas, meta)
        picked = backend.argmax_rows(logits)
        got = backend.to_host(logits)
        want = forward_oracle(oracle, w, arenas, metas, meta, kv_dtype)
        assert_close(got, want, abs_tol=abs_tol, rel_tol=REL_TOL, what="decode logits")
        assert np.array_equal(picked, oracle.argmax_rows(got))      # the device's pick over its own logits
        top2 = np.sort(want, axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 4 * (abs_tol + REL_TOL * np.abs(top2[:, 1]))
        toks = oracle.argmax_rows(want)
        assert np.array_equal(picked[clear], toks[clear])           # and the oracle's, where the lead is clear
    assert cache.seq_len(a) == 150 + 5 and cache.seq_len(b2) == 140 + 3 + 4
    kv.close()
