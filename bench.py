#!/usr/bin/env python
"""Benchmark of the paged-attention hot path on B200.

Default line: batched paged decode attention, 16 sequences sharing a 1536-token prefix
through the same physical pages with private suffixes of 0..2560 tokens, 32 query / 8 KV
heads, head_dim 128, f16 cache, f32 accumulation.  A step is one attention call over the
batch (one layer); steps rotate over several layers' arenas, so the pages of a step are not in
L2 from the step before.  The metric is HBM GB/s over the step's unique K+V bytes.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

With N > 1 (torchrun) every rank runs its own batch of 16 sequences: sequences never interact
inside attention, so there is no data-path collective (weak scaling); `--workload long_decode`
instead splits one sequence's keys across ranks and merges with an NCCL all-gather.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from yaxus_b200 import workloads as W  # noqa: E402
from yaxus_b200._lib import BF16, F16, F32  # noqa: E402

METRIC = "paged decode-attn HBM GB/s @B=16"
N_LAYERS = 6   # arenas rotated over; 6 x ~91 MB >> the 126 MB L2


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            t0 = time.time()
            while not self.rows and time.time() - t0 < 3.0:   # a very short run: wait for one sample
                time.sleep(0.05)
            self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_scenario(name, rank):
    if name == "batched_decode":
        return W.batched_decode(seed=W.SEED0 + 1 + 1000 * rank)
    if name == "verify":
        return W.verify(seed=W.SEED0 + 2 + 1000 * rank)
    if name == "single_decode":
        return W.single_decode(seed=W.SEED0 + 1000 * rank)
    if name == "long_decode":
        return W.long_decode()
    if name == "long_decode_window":
        return W.long_decode(window=2048)
    raise SystemExit(f"unknown workload {name}")


def workload_config(name, s, n_gpus):
    cfg = {"workload": name, "sequences": len(s.tables), "rows_per_step": int(s.meta.rows), "hq": s.hq, "hkv": s.hkv,
           "head_dim": 128, "kv_dtype": {F32: "f32", F16: "f16", BF16: "bf16"}[s.kv_dtype],
           "context_tokens": [int(c) for c in s.ctx_len] if len(s.ctx_len) <= 16 else "…",
           "unique_kv_bytes_per_step": int(s.unique_kv_bytes()), "logical_kv_bytes_per_step": int(s.logical_kv_bytes()),
           "l2": f"steps rotate over {N_LAYERS} layer arenas ({N_LAYERS} x working set > L2)",
           "parallelism": f"by sequence, {n_gpus} GPU(s), no collective"}
    if s.window:
        cfg["window"] = s.window
    return cfg


def run_reference(args):
    """The reference's CPU implementation of the path (its restated CPU backend, all host
    threads) on the same workload.  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from tests.oracle import Oracle
    o = Oracle()
    s = make_scenario(args.workload, 0)
    K, V = s.k_f32(), s.v_f32()
    o.append_rows(W.round_through(s.k_new, s.kv_dtype), W.round_through(s.v_new, s.kv_dtype), s.meta.kv_slot, K, V)
    cores = o.max_threads()

    def step():
        return o.attend(s.q, s.meta.pos, s.meta.pt_off, s.meta.pages, s.hq, s.hkv, 128, s.window, K, V, threads=cores)

    # Bounded: the CPU takes tens of milliseconds per step, and K may be a GPU-sized count.  At most
    # about a minute of timed CPU work; the per-step time is what is reported.
    t0 = time.perf_counter()
    step()
    est = time.perf_counter() - t0
    n_warm = max(0, min(args.warmup, int(10.0 / est)) - 1)
    n_timed = max(1, min(args.steps, int(60.0 / est)))
    for _ in range(n_warm):
        step()
    t0 = time.perf_counter()
    for _ in range(n_timed):
        step()
    dt = (time.perf_counter() - t0) / n_timed
    value = s.unique_kv_bytes() / dt / 1e9
    sample = f"the whole step ({s.meta.rows} rows x {s.hq} heads), {n_timed} of the {args.steps} steps timed"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": workload_config(args.workload, s, args.gpus),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def run_prefill(args):
    """Chunked causal prefill: 8 sequences x 4096 tokens in 512-row chunks, 16-bit Q/K/V (f16 or bf16), f32
    softmax and accumulation.  A step is the whole prefill of the batch (eight passes, each
    appending its 4096 K/V rows and attending); the metric is causal-exact TFLOP/s."""
    import torch
    import torch.distributed as dist
    from yaxus_b200 import CudaBackend
    from yaxus_b200.backend import LayerMeta, Rope

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    b = CudaBackend(local)
    dev = b.device
    n_seq, total, chunk, hq, hkv = 8, 4096, 512, 32, 8
    kvt = F16 if args.kv_dtype == "f16" else BF16   # bf16 Q/K/V is the configuration the metric is quoted on
    tdt = torch.bfloat16 if kvt == BF16 else torch.float16
    kv_name = "bf16" if kvt == BF16 else "f16"
    n_layers = 2   # 2 x 134 MB of K+V: a step does not find its pages in L2 from the step before
    passes = W.prefill_passes(seed=W.SEED0 + 3 + 1000 * rank, n_seq=n_seq, total=total, chunk=chunk, hq=hq, hkv=hkv)
    s0 = passes[0]
    layers = [LayerMeta(index=i, rope=Rope.default()) for i in range(n_layers)]
    kv = b.new_kv(hkv, layers, s0.arena_pages, 8192, kvt)
    g = torch.Generator(device=dev).manual_seed(7 + rank)
    T = s0.meta.rows
    q = torch.randn(T, hq * 128, device=dev, generator=g).to(tdt)
    k_rows = torch.randn(T, hkv * 128, device=dev, generator=g).to(tdt)
    v_rows = torch.randn(T, hkv * 128, device=dev, generator=g).to(tdt)
    out = torch.empty(T, hq * 128, dtype=tdt, device=dev)
    flops = sum(p.flops() for p in passes)

    def step(i):
        layer = i % n_layers
        for p in passes:
            b.begin_pass(p.meta)
            b.kv_append(kv, layer, k_rows, v_rows)
            b.attend(kv, layer, q, hq, out=out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # parity of the same kernels on a bounded sample: chunks 0 and 1 of the first two sequences
    max_err = None
    if rank == 0 and not args.no_check:
        from tests.gpu_util import assert_close, load
        from tests.oracle import Oracle
        o = Oracle()
        small = W.prefill_passes(seed=5, n_seq=2, total=1024, chunk=512, hq=hq, hkv=hkv)
        kvs = b.new_kv(hkv, [LayerMeta(index=0, rope=Rope.default())], small[0].arena_pages, 8192, kvt)
        K = np.zeros((small[0].arena_pages * 128, hkv * 128), np.float32)
        V = np.zeros_like(K)
        t = lambda x, dt: torch.from_numpy(np.ascontiguousarray(x)).to(dev).to(dt)
        for p in small:
            b.begin_pass(p.meta)
            b.kv_append(kvs, 0, t(p.k_new, torch.float32), t(p.v_new, torch.float32))
            got = b.to_host(b.attend(kvs, 0, t(p.q, tdt), hq))
            o.append_rows(W.round_through(p.k_new, kvt), W.round_through(p.v_new, kvt), p.meta.kv_slot, K, V)
            ref = o.attend(p.q, p.meta.pos, p.meta.pt_off, p.meta.pages, hq, hkv, 128, None, K, V)
            e = assert_close(got, ref, what=p.name)
            max_err = e if max_err is None else max(max_err, e)
        kvs.close()

    sampler = ClockSampler(local)
    sampler.start()
    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    launches0 = b.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    launches = b.launch_count() - launches0
    info = b.last_plan()
    clocks = sampler.stop()
    # the tile kernel alone (CUDA events around every attention call)
    b.profile_begin()
    for i in range(min(args.steps, 64)):
        step(i)
    split_ms, combine_ms, calls = b.profile_end()
    kernel_ms_per_step = split_ms / max(calls, 1) * len(passes)

    # end to end: metadata, 16-bit q/k/v rows from pinned host memory, result read back, per pass
    qh = torch.empty(T, hq * 128, dtype=tdt).pin_memory()
    kh = torch.empty(T, hkv * 128, dtype=tdt).pin_memory()
    vh = torch.empty(T, hkv * 128, dtype=tdt).pin_memory()
    oh = torch.empty(T, hq * 128, dtype=tdt).pin_memory()
    # Two sets of device buffers and two copy streams: the rows of pass p + 1 go up and the
    # result of pass p - 1 comes down while pass p computes (what a serving loop does with host
    # buffers); every buffer's reuse is ordered by events.
    qd = [torch.empty_like(qh, device=dev) for _ in range(2)]
    kd = [torch.empty_like(kh, device=dev) for _ in range(2)]
    vd = [torch.empty_like(vh, device=dev) for _ in range(2)]
    od = [torch.empty(T, hq * 128, dtype=tdt, device=dev) for _ in range(2)]
    up, down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    main = torch.cuda.current_stream(dev)
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_ready = [torch.cuda.Event() for _ in range(2)]
    out_free = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(i):
        for n, p in enumerate(passes):
            x = n & 1
            with torch.cuda.stream(up):
                up.wait_event(in_free[x])            # the pass that last read this set is done
                qd[x].copy_(qh, non_blocking=True)
                kd[x].copy_(kh, non_blocking=True)
                vd[x].copy_(vh, non_blocking=True)
                in_ready[x].record(up)
            b.begin_pass(p.meta)
            main.wait_event(in_ready[x])
            main.wait_event(out_free[x])             # the download that last read this output is done
            b.kv_append(kv, i % n_layers, kd[x], vd[x])
            b.attend(kv, i % n_layers, qd[x], hq, out=od[x])
            in_free[x].record(main)
            out_ready[x].record(main)
            with torch.cuda.stream(down):
                down.wait_event(out_ready[x])
                oh.copy_(od[x], non_blocking=True)
                out_free[x].record(down)
        main.wait_stream(down)
        b.sync()
    for x in range(2):
        in_free[x].record(main)
        out_free[x].record(main)
    e2e_step(0)
    barrier()
    e2e_n = max(1, min(args.steps, 10))
    e0.record()
    for i in range(e2e_n):
        e2e_step(i)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_n

    if world > 1:
        tt = torch.tensor([ms, e2e_ms, kernel_ms_per_step], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, e2e_ms, kernel_ms_per_step = (float(x) for x in tt.tolist())
    if rank == 0:
        peak = 1377.6
        ppath = os.path.join(ROOT, "MEASURED_PEAKS.json")
        which = "fallback"
        if os.path.exists(ppath):
            with open(ppath) as f:
                peak = float(json.load(f)["bf16_tflops_sustained"])
            which = "measured (sustained)"
        achieved = flops / (kernel_ms_per_step * 1e-3) / 1e12
        bytes_in = (qh.numel() + kh.numel() + vh.numel()) * 2 * len(passes)
        line = {
            "metric": "prefill-attn TFLOPS", "value": world * flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": kv_name, "data": "synthetic",
            "config": {"workload": "chunked causal prefill", "sequences": n_seq, "tokens_per_sequence": total,
                       "chunk": chunk, "hq": hq, "hkv": hkv, "head_dim": 128, "kv_dtype": kv_name,
                       "flops_per_step": flops, "passes_per_step": len(passes),
                       "l2": f"steps alternate over {n_layers} layer arenas of 134 MB",
                       "parallelism": f"by sequence, {world} GPU(s), no collective"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": which, "kernel": "prefill_tc2_kernel",
                         "kernel_ms_per_step": kernel_ms_per_step},
            "clocks": clocks, "gpu_launches": int(launches),
            "plan": {"path": info.path, "tile_items_last_pass": None},
            "parity_max_abs": max_err,
            "e2e": {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(bytes_in), "d2h_bytes_per_step": int(oh.numel() * 2 * len(passes))},
        }
        print(json.dumps(line))
    kv.close()
    b.close()
    if world > 1:
        dist.destroy_process_group()


def run_cuda(args):
    import torch
    import torch.distributed as dist
    from yaxus_b200 import CudaBackend
    from yaxus_b200.backend import LayerMeta, Rope

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    b = CudaBackend(local)
    dev = b.device
    split_kv = args.workload.startswith("long_decode")
    s = make_scenario(args.workload, 0 if split_kv else rank)
    layers = [LayerMeta(index=i, window=s.window, rope=Rope.default()) for i in range(N_LAYERS)]
    max_pos = max(int(s.meta.pos.max()) + 1, 8192)
    kv = b.new_kv(s.hkv, layers, s.arena_pages, max_pos, s.kv_dtype)
    key_lo, key_hi = 0, (1 << 62)
    if split_kv and world > 1:
        b.comm_create(world, rank)
        first, last, key_lo, key_hi = W.partition_pages(s.arena_pages, world, rank)
    for l in range(N_LAYERS):
        # distinct contents per layer without regenerating: rotate the rows
        b.write_pages(kv, l, 0, np.roll(s.k_bits, 977 * l, axis=1), np.roll(s.v_bits, 977 * l, axis=1))
    t = lambda x, dt=torch.float32: torch.from_numpy(np.ascontiguousarray(x)).to(dev).to(dt)
    q, k_new, v_new = t(s.q), t(s.k_new), t(s.v_new)
    b.begin_pass(s.meta)
    for l in range(N_LAYERS):
        b.kv_append(kv, l, k_new, v_new)
    out = torch.empty(s.meta.rows, s.hq * 128, dtype=torch.float32, device=dev)

    def step(i):
        if split_kv:
            b.attend_allgather(kv, i % N_LAYERS, q, s.hq, -1, key_lo, key_hi, out=out)
        else:
            b.attend(kv, i % N_LAYERS, q, s.hq, out=out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # parity of what is about to be timed (layer 0 holds the unrotated data)
    max_err = None
    if not args.no_check and (rank == 0 or (split_kv and world > 1)):
        # with the keys split over ranks the step is a collective: every rank takes it, rank 0 checks
        from tests.gpu_util import assert_close, oracle_step
        from tests.oracle import Oracle
        step(0)
        if rank == 0:
            max_err = assert_close(b.to_host(out), oracle_step(Oracle(), s), what="bench parity")
    sampler = ClockSampler(local)
    sampler.start()
    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    launches0 = b.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    launches = b.launch_count() - launches0
    info = b.last_plan()

    # per-kernel time of the dominant kernel, measured live with CUDA events
    clocks = sampler.stop()
    b.profile_begin()
    for i in range(min(args.steps, 4096)):
        step(i)
    split_ms, combine_ms, calls = b.profile_end()
    kernel_ms = split_ms / max(calls, 1)
    if not split_kv:
        # The dominant kernel by itself, as it runs in the stream: back-to-back launches between
        # two events (events around every single launch add the launch latency that chained
        # launches hide, and read higher than the whole step).
        b.set_tuning(skip_merge=1)
        b.begin_pass(s.meta)
        for i in range(20):
            step(i)
        n_k = min(args.steps, 4096)
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        k0.record()
        for i in range(n_k):
            step(i)
        k1.record()
        torch.cuda.synchronize()
        kernel_ms = k0.elapsed_time(k1) / n_k
        b.set_tuning()
        b.begin_pass(s.meta)

    # end to end through the boundary call: pass metadata and qkv rows from pinned host
    # memory, fused norm + RoPE + append + attention, result read back to the host.
    qkv_host = torch.empty(s.meta.rows, (s.hq + 2 * s.hkv) * 128, dtype=torch.float32).pin_memory()
    qkv_host.normal_(generator=torch.Generator().manual_seed(5 + rank))
    out_host = torch.empty(s.meta.rows, s.hq * 128, dtype=torch.float32).pin_memory()
    qkv_dev = torch.empty_like(qkv_host, device=dev)
    w = torch.zeros(128, device=dev)
    e2e_ms = None
    if not split_kv:
        def e2e_step(i):
            b.begin_pass(s.meta)
            qkv_dev.copy_(qkv_host, non_blocking=True)
            o = b.attention(qkv_dev, w, w, kv, s.hq, 1e-6, layers[i % N_LAYERS])
            out_host.copy_(o, non_blocking=True)
            b.sync()
        for i in range(3):
            e2e_step(i)
        barrier()
        e0.record()
        for i in range(args.steps):
            e2e_step(i)
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1) / args.steps

    if world > 1:
        tt = torch.tensor([ms, e2e_ms or 0.0, kernel_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, e2e_max, kernel_ms = (float(x) for x in tt.tolist())
        e2e_ms = e2e_max if e2e_ms is not None else None
        ub = torch.tensor([float(s.unique_kv_bytes())], device=dev, dtype=torch.float64)
        if not split_kv:
            dist.all_reduce(ub, op=dist.ReduceOp.SUM)
        total_bytes = float(ub.item())
    else:
        total_bytes = float(s.unique_kv_bytes())

    if rank == 0:
        peak, which = measured_peaks()
        per_gpu_bytes = float(s.unique_kv_bytes()) / (world if split_kv else 1)
        achieved = per_gpu_bytes / (kernel_ms * 1e-3) / 1e9 if kernel_ms > 0 else None
        line = {
            "metric": METRIC, "value": total_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong" if split_kv else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args.workload, s, world),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak if achieved else None,
                         # dram__bytes_read.sum + dram__bytes_write.sum of one launch of the split-key kernel on
                         # this very workload, from the ncu capture summarised under profiles/
                         "traffic": 95.9e6 if (args.workload == "batched_decode" and world == 1) else None,
                         "peak_source": which,
                         "kernel": "attend_mma_kernel" if info.path == 2 else "attend_simt_kernel",
                         "kernel_ms": kernel_ms, "combine_ms": combine_ms / max(calls, 1),
                         "algorithmic_bytes": per_gpu_bytes},
            "clocks": clocks, "gpu_launches": int(launches),
            "plan": {"path": info.path, "ctas": info.n_ctas, "items": info.n_items, "parts": info.n_parts,
                     "tiles": int(info.tiles), "shared_groups": info.shared_groups},
            "parity_max_abs": max_err,
        }
        if e2e_ms is not None:
            h2d = qkv_host.numel() * 4 + (3 * s.meta.rows + len(s.meta.pages)) * 4
            line["e2e"] = {"value": total_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
                           "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(out_host.numel() * 4)}
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(s)
        print(json.dumps(line))
    kv.close()
    b.close()
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline(s):
    """The CPU oracle on the same step, all host threads, best of three."""
    from tests.oracle import Oracle
    o = Oracle()
    K, V = s.k_f32(), s.v_f32()
    o.append_rows(W.round_through(s.k_new, s.kv_dtype), W.round_through(s.v_new, s.kv_dtype), s.meta.kv_slot, K, V)
    cores = o.max_threads()
    best = None
    for _ in range(3):
        t0 = time.perf_counter()
        o.attend(s.q, s.meta.pos, s.meta.pt_off, s.meta.pages, s.hq, s.hkv, 128, s.window, K, V, threads=cores)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": s.unique_kv_bytes() / best / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"the whole step ({s.meta.rows} rows x {s.hq} heads), best of 3", "ms_per_step": best * 1e3}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20000)
    ap.add_argument("--warmup", type=int, default=200)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--workload", default="batched_decode")
    ap.add_argument("--kv-dtype", default=None, choices=["f16", "bf16"],
                    help="cache storage type of the prefill workload (default bf16; f16 needs one P V MMA instead of two)")
    ap.add_argument("--no-check", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "prefill":
        run_prefill(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
