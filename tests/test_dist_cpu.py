"""The two ways the path spreads over GPUs, run as two `gloo` ranks on CPU with the oracle as
the compute (host-side protocol only; the GPU versions are in test_gpu_dist.py):

* by sequence: every rank attends its own sequences, nothing is exchanged, and the union of
  the ranks' outputs is the single-process result;
* one long sequence split by pages: every rank computes the triples (m, l, o) of its key range,
  the triples are all-gathered in rank order, and every rank merges them
  (crates/yaxus-backend-gpu/src/shaders.rs:1581-1637) to the whole attention.
"""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, case, results):
    sys.path.insert(0, ROOT)
    from oracle.binding import Oracle
    from yaxus_b200 import workloads as W
    from yaxus_b200._lib import F16
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        o = Oracle()
        if case == "by_sequence":
            # four sequences with ragged contexts, one decode row each; rank r owns sequences r, r + world, ...
            ctx = [300, 5, 127, 1000]
            whole = W.build("seq", 21, 8, 2, F16, ctx, [1] * 4)
            K, V = whole.k_f32(), whole.v_f32()
            o.append_rows(W.round_through(whole.k_new, F16), W.round_through(whole.v_new, F16), whole.meta.kv_slot, K, V)
            ref = o.attend(whole.q, whole.meta.pos, whole.meta.pt_off, whole.meta.pages, 8, 2, 128, None, K, V)
            mine = [s for s in range(4) if s % world == rank]
            rows = np.array(mine)   # one row per sequence, in sequence order
            got = o.attend(whole.q[rows], whole.meta.pos[rows], whole.meta.pt_off[rows], whole.meta.pages, 8, 2, 128, None, K, V)
            # no collective on the data path; the check itself gathers
            parts = [None] * world
            dist.all_gather_object(parts, (mine, got))
            out = np.zeros_like(ref)
            for seqs, g in parts:
                out[np.array(seqs)] = g
            ok = np.array_equal(out, ref)
        else:
            window = 700 if case == "split_keys_window" else None
            s = W.long_decode(ctx=2048 + 77, window=window, hq=8, hkv=2)
            K, V = s.k_f32(), s.v_f32()
            o.append_rows(W.round_through(s.k_new, F16), W.round_through(s.v_new, F16), s.meta.kv_slot, K, V)
            ref = o.attend(s.q, s.meta.pos, s.meta.pt_off, s.meta.pages, 8, 2, 128, window, K, V)
            _, _, klo, khi = W.partition_pages(s.arena_pages, world, rank)
            m, l, acc = o.attend_partial(s.q, s.meta.pos, s.meta.pt_off, s.meta.pages, 8, 2, 128, window, klo, khi, K, V)
            # the exchange: triples of every rank, in rank order (what yx_attend_allgather does over NCCL)
            mine = torch.from_numpy(np.concatenate([m.ravel(), l.ravel(), acc.ravel()]))
            gathered = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(gathered, mine)
            n = m.size
            ms = np.stack([g.numpy()[:n].reshape(m.shape) for g in gathered])
            ls = np.stack([g.numpy()[n:2 * n].reshape(l.shape) for g in gathered])
            accs = np.stack([g.numpy()[2 * n:].reshape(acc.shape) for g in gathered])
            out = o.combine(ms, ls, accs).reshape(ref.shape)
            ok = bool(np.abs(out - ref).max() <= 2e-6)
            if window:
                # a rank whose pages lie wholly below the window contributes the empty mark
                lo_key = s.meta.pos[0] + 1 - window
                if khi <= lo_key:
                    ok = ok and bool((l == 0).all() and (m == -1e30).all())
        results[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case", ["by_sequence", "split_keys", "split_keys_window"])
def test_two_ranks(case):
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, port, case, results)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0, f"rank exited with {p.exitcode}"
        assert dict(results) == {0: True, 1: True}
