"""Two GPUs, one process each: one long sequence split by pages, partial triples all-gathered
over NCCL inside yx_attend_allgather and merged on every rank; and the by-sequence split, which
exchanges nothing.  Needs two devices; skipped on one."""
import os
import socket
import sys
import time

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    from oracle.check import assert_close, dev, load, oracle_step
    from oracle.binding import Oracle
    from yaxus_b200 import CudaBackend
    from yaxus_b200 import workloads as W
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ok = False
    try:
        b = CudaBackend(rank)
        o = Oracle()
        b.comm_create(world, rank)
        # Every collective first, every comparison afterwards: a rank whose check fails must not
        # leave its peer alone inside the next all-gather, which has no bound of its own.
        pending = []
        for window in (None, 3000):
            # every rank holds the whole cache here (the test is about the exchange); it reads its pages only
            s = W.long_decode(ctx=8192 + 33, window=window, hq=8, hkv=2)
            kv = load(b, s)
            b.begin_pass(s.meta)
            b.kv_append(kv, 0, dev(b, s.k_new), dev(b, s.v_new))
            _, _, klo, khi = W.partition_pages(s.arena_pages, world, rank)
            out = b.attend_allgather(kv, 0, dev(b, s.q), s.hq, -1, klo, khi)
            pending.append((b.to_host(out), s, f"rank {rank} window {window}"))
            kv.close()
        dist.barrier()    # the last collective of this test: nothing below waits for a peer
        for got, s, what in pending:
            assert_close(got, oracle_step(o, s), what=what)
        # by sequence: each rank its own sequences, no exchange
        whole = W.build("seq", 21, 8, 2, 1, [300, 5, 127, 1000], [1] * 4)
        ref = oracle_step(o, whole)
        mine = [q for q in range(4) if q % world == rank]
        part = W.build("seq", 21, 8, 2, 1, [300, 5, 127, 1000], [1] * 4)   # same seed: same data
        kv = load(b, part)
        b.begin_pass(part.meta)
        b.kv_append(kv, 0, dev(b, part.k_new), dev(b, part.v_new))
        got = b.to_host(b.attend(kv, 0, dev(b, part.q), part.hq))
        assert_close(got[mine], ref[mine], what=f"rank {rank} by sequence")
        kv.close()
        b.sync()
        b.close()
        ok = True
    finally:
        results[rank] = ok
        # No destroy_process_group here: it is a collective, and a rank that failed must not make
        # its peer wait.  The process ends right after this.


def test_two_gpus_split_keys_and_sequences():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
        for p in procs:
            p.start()
        try:
            deadline = time.time() + 300
            for p in procs:
                p.join(max(1.0, deadline - time.time()))
        finally:
            # A rank still alive here is stuck (its peer died inside a collective): it is ended, not
            # left spinning on a GPU.
            for p in procs:
                if p.is_alive():
                    p.terminate()
                    p.join(10)
                if p.is_alive():
                    p.kill()
                    p.join(10)
        assert [p.exitcode for p in procs] == [0] * world, [p.exitcode for p in procs]
        assert dict(results) == {0: True, 1: True}
