#!/usr/bin/env python
"""Benchmark of the paged-attention hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

The line it prints is headed by batched paged decode attention: 16 sequences sharing a
1536-token prefix through the same physical pages with private suffixes of 0..2560 tokens,
32 query / 8 KV heads, head_dim 128, f16 cache, f32 accumulation.  A step is one attention
call over the batch (one layer); steps rotate over several layers' arenas, so the pages of a
step are not in L2 from the step before.  The metric is HBM GB/s over the step's unique K+V
bytes.  At least 10000 calls are timed whatever K is (`config.timed_calls`).

Under `workloads` the same line carries the other configurations of the path, each with its
own value, roofline and parity: chunked causal prefill (bf16, 8 x 4096 tokens in 512-row
chunks, TFLOP/s), speculative verification (16 x 5 rows), single-sequence decode (f32 cache),
and long-context decode over 131072 keys with and without a 2048-key window.

With N > 1 (torchrun, one rank per GPU) decode, verification and prefill shard by sequence:
every rank runs its own batch and there is no data-path collective (weak scaling).  The
long-context workloads split the one sequence's pages across the N ranks and merge the
partial (m, l, o) triples with an NCCL all-gather (strong scaling).

`--workload NAME` prints one workload as the whole line (for profiler captures).
"""
import argparse
import dataclasses
import json
import math
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
MIN_TIMED_CALLS = 10000   # 0.2 s of device time: the clock sampler (one line per 100 ms) sees the timed region
DTYPE_NAME = {F32: "f32", F16: "f16", BF16: "bf16"}
L2_BYTES = 126e6


def host_cores():
    """Cores this process may run on.  Not omp_get_max_threads(): torchrun exports
    OMP_NUM_THREADS=1, which would shrink the CPU baseline to one thread."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm": float(p["hbm_gbs"]), "bf16": float(p["bf16_tflops_sustained"]),
                "bf16_burst": float(p["bf16_tflops"]), "source": "measured"}
    return {"hbm": 6650.0, "bf16": 1400.0, "bf16_burst": 1590.0, "source": "fallback"}


def captured_traffic(name):
    """DRAM bytes of one launch from the committed profiler summary of this kernel and workload
    (profiles/<name>.json).  Not measured by this run: the source is named beside it."""
    path = os.path.join(ROOT, "profiles", name + ".json")
    if not os.path.exists(path):
        return None, None
    with open(path) as f:
        p = json.load(f)
    return float(p["dram_bytes_read"]) + float(p["dram_bytes_write"]), f"profiles/{name}.json ({p.get('captured', '')})"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of every GPU of the node, sampled by one process
    per node while the timed regions run."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
            return
        # NVML initialisation enumerates every GPU and holds a driver lock while it does: it must
        # be over before anything is timed.
        t0 = time.time()
        while not self.rows and time.time() - t0 < 10.0:
            time.sleep(0.02)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def summary(self, t0, t1, index):
        """Samples of GPU `index` taken between t0 and t1 (all of its samples if none fall inside)."""
        mine = [r for t, r in self.rows if r and r[0] == str(index)]
        inside = [r for t, r in self.rows if r and r[0] == str(index) and t0 <= t <= t1]
        sm, mx, reasons = [], [], set()
        for r in inside or mine:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "samples_in_timed_region": len(inside)}

    def stop(self):
        if self.proc:
            self.proc.terminate()


class Env:
    """One rank of the run: its GPU, its backend context, the process group if any."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        from yaxus_b200 import CudaBackend
        self.torch, self.dist = torch, dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
        self.b = CudaBackend(self.local)
        self.dev = self.b.device
        self.comm = False
        self.sampler = None
        if self.local == 0:
            self.sampler = ClockSampler()
            self.sampler.start()
        self.barrier()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        if self.world == 1:
            return [float(v) for v in values]
        t = self.torch.tensor([float(v) for v in values], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t.tolist()]

    def sum_over_ranks(self, value):
        if self.world == 1:
            return float(value)
        t = self.torch.tensor([float(value)], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t.item())

    def ensure_comm(self):
        if not self.comm and self.world > 1:
            self.b.comm_create(self.world, self.rank)
            self.comm = True

    def timed(self, fn, calls, warm):
        """`calls` calls of fn(i) between two CUDA events on the launching stream, after `warm`
        untimed ones, barriers and device synchronisation on both sides.  Returns (device ms per
        call as the max over ranks, host microseconds per call spent issuing, clock summary)."""
        torch = self.torch
        for i in range(warm):
            fn(i)
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        w0 = time.time()
        e0.record()
        h0 = time.perf_counter()
        for i in range(calls):
            fn(i)
        h1 = time.perf_counter()
        e1.record()
        self.barrier()
        w1 = time.time()
        ms = e0.elapsed_time(e1) / calls
        ms, host_us = self.max_over_ranks([ms, (h1 - h0) / calls * 1e6])
        clocks = self.sampler.summary(w0, w1, self.local) if self.sampler else None
        return ms, host_us, clocks

    def close(self):
        if self.sampler:
            self.sampler.stop()
        self.b.close()
        if self.world > 1:
            self.dist.destroy_process_group()


def make_scenario(name, rank):
    if name == "batched_decode":
        # Weak scaling: every rank the same work (rank 0's sequence lengths, in another order) over
        # its own pages and values.
        return W.batched_decode(seed=W.SEED0 + 1 + 1000 * rank, length_seed=W.SEED0 + 1, rotate=3 * rank)
    if name == "verify":
        return W.verify(seed=W.SEED0 + 2 + 1000 * rank)
    if name == "single_decode":
        return W.single_decode(seed=W.SEED0 + 1000 * rank)
    if name == "long_decode":
        return W.long_decode()
    if name == "long_decode_window":
        return W.long_decode(window=2048)
    raise SystemExit(f"unknown workload {name}")


def layers_needed(bytes_per_call):
    """Arenas to rotate over so that a call does not find its pages in L2 from an earlier call (at least
    two, also where one arena is several times L2: consecutive calls overlap on the device)."""
    return max(2, min(48, int(math.ceil(4.0 * L2_BYTES / max(bytes_per_call, 1)))))


def workload_config(name, s, n_gpus, n_layers, split_kv):
    cfg = {"workload": name, "sequences": len(s.tables), "rows_per_step": int(s.meta.rows), "hq": s.hq, "hkv": s.hkv,
           "head_dim": 128, "kv_dtype": DTYPE_NAME[s.kv_dtype],
           "context_tokens": [int(c) for c in s.ctx_len] if len(s.ctx_len) <= 16 else "…",
           "unique_kv_bytes_per_step": int(s.unique_kv_bytes()), "logical_kv_bytes_per_step": int(s.logical_kv_bytes()),
           "l2": (f"steps rotate over {n_layers} layer arenas ({n_layers} x working set > L2)" if n_layers > 1
                  else "one arena: the working set of a step is larger than L2"),
           "parallelism": (f"keys split over {n_gpus} GPU(s), NCCL all-gather of the (m, l, o) triples" if split_kv
                           else f"by sequence, {n_gpus} GPU(s), no collective"
                                + ("; every rank its own pages and values with rank 0's sequence lengths in another order"
                                   if name == "batched_decode" and n_gpus > 1 else ""))}
    if s.window:
        cfg["window"] = s.window
    return cfg


def oracle_reference(s, threads):
    """The CPU oracle's output for the step, and how long its attend took (one run)."""
    from oracle.binding import Oracle
    from oracle.check import oracle_arenas
    o = Oracle()
    K, V = oracle_arenas(o, s)
    t0 = time.perf_counter()
    ref = o.attend(s.q, s.meta.pos, s.meta.pt_off, s.meta.pages, s.hq, s.hkv, 128, s.window, K, V, threads=threads)
    return ref, time.perf_counter() - t0, (o, K, V)


def run_split_key(env, name, s, calls, warm, check=True, e2e=False, cpu=False, kernel_only=False):
    """Decode-like workloads (everything but prefill).  Returns the record on rank 0."""
    torch, b, dev = env.torch, env.b, env.dev
    from yaxus_b200.backend import LayerMeta, Rope
    world, rank = env.world, env.rank
    split_kv = name.startswith("long_decode")
    per_rank_bytes = float(s.unique_kv_bytes()) / (world if split_kv else 1)
    # A windowed run reads a few megabytes: it rotates over the arenas of the full run.
    n_layers = layers_needed(float(dataclasses.replace(s, window=None).unique_kv_bytes()) / (world if split_kv else 1))
    layers = [LayerMeta(index=i, window=s.window, rope=Rope.default()) for i in range(n_layers)]
    max_pos = max(int(s.meta.pos.max()) + 1, 8192)
    kv = b.new_kv(s.hkv, layers, s.arena_pages, max_pos, s.kv_dtype)
    key_lo, key_hi = 0, (1 << 62)
    first, last = 0, s.arena_pages
    if split_kv and world > 1:
        env.ensure_comm()
        # the one sequence's page table covers the arena in order: page ranges are key ranges
        assert (np.sort(s.tables[0]) == np.arange(s.arena_pages)).all()
        first, last, key_lo, key_hi = W.partition_pages(s.arena_pages, world, rank)
    own = np.zeros(s.arena_pages, bool)
    if split_kv and world > 1:
        own[s.tables[0][first:last]] = True      # physical pages of this rank's key range
    else:
        own[:] = True
    for l in range(n_layers):
        # distinct contents per layer without regenerating: rotate the rows' elements
        kb, vb = s.k_bits, s.v_bits
        if l:
            kb, vb = np.roll(kb, 977 * l, axis=1), np.roll(vb, 977 * l, axis=1)
        if own.all():
            b.write_pages(kv, l, 0, kb, vb)
        else:
            for pg in np.nonzero(own)[0]:
                b.write_pages(kv, l, int(pg), kb[pg * 128:(pg + 1) * 128], vb[pg * 128:(pg + 1) * 128])
    t = lambda x, dt=torch.float32: torch.from_numpy(np.ascontiguousarray(x)).to(dev).to(dt)
    q, k_new, v_new = t(s.q), t(s.k_new), t(s.v_new)
    b.begin_pass(s.meta)
    if all(own[int(sl) // 128] for sl in s.meta.kv_slot):
        for l in range(n_layers):
            b.kv_append(kv, l, k_new, v_new)
    out = torch.empty(s.meta.rows, s.hq * 128, dtype=torch.float32, device=dev)

    # The timed call is the C entry point itself (through ctypes, arguments prepared once): the
    # Python wrapper's checks and conversions would be half of the host time of a 20 us call.
    import ctypes
    vp = ctypes.c_void_p
    q_p, out_p = vp(q.data_ptr()), vp(out.data_ptr())
    yx_attend, ctx_p, kv_p, hq = b._L.yx_attend, b._ctx, kv._h, s.hq

    def step(i):
        if split_kv:
            b.attend_allgather(kv, i % n_layers, q, s.hq, -1, key_lo, key_hi, out=out)
        else:
            yx_attend(ctx_p, kv_p, i % n_layers, q_p, 0, hq, -1, out_p, 0)

    # parity of what is about to be timed (layer 0 holds the unrotated data)
    max_err, cpu_s, oracle_state = None, None, None
    if check and (rank == 0 or (split_kv and world > 1)):
        from oracle.check import assert_close
        step(0)   # with the keys split over ranks the step is a collective: every rank takes it
        if rank == 0:
            ref, cpu_s, oracle_state = oracle_reference(s, host_cores())
            max_err = assert_close(b.to_host(out), ref, what=f"{name} parity")
    env.barrier()

    ms, host_us, clocks = env.timed(step, calls, warm)
    launches0 = b.launch_count()
    step(0)
    launches_per_call = b.launch_count() - launches0
    info = b.last_plan()

    # the dominant kernel alone, events around every launch (adds the launch latency that chained
    # launches hide)
    b.profile_begin()
    for i in range(min(calls, 512)):
        step(i)
    split_ms, combine_ms, n_prof = b.profile_end()
    bracketed_ms = split_ms / max(n_prof, 1)
    (bracketed_ms,) = env.max_over_ranks([bracketed_ms])
    kernel_ms = bracketed_ms
    chain_timed = kernel_only and (not split_kv or world == 1)
    if chain_timed:
        # ... and as it runs in the stream: back-to-back launches of that kernel between two events
        b.hook_skip_merge(True)
        kernel_ms, _, _ = env.timed(step, calls, 20)
        b.hook_skip_merge(False)

    rec_e2e = e2e_decode(env, s, kv, layers, calls) if (e2e and not split_kv) else None

    total_bytes = float(s.unique_kv_bytes()) if split_kv else env.sum_over_ranks(s.unique_kv_bytes())
    rec = None
    if rank == 0:
        peaks = measured_peaks()
        achieved = per_rank_bytes / (kernel_ms * 1e-3) / 1e9 if kernel_ms > 0 else None
        kernel = "attend_mma_kernel" if info.path == 2 else "attend_simt_kernel"
        traffic, traffic_source = captured_traffic(f"{kernel}_{name}") if world == 1 else (None, None)
        rec = {
            "metric": METRIC if name == "batched_decode" else f"{name} HBM GB/s", "value": total_bytes / (ms * 1e-3) / 1e9,
            "unit": "GB/s", "ms_per_step": ms, "scaling": "strong" if split_kv else "weak",
            "dtype": DTYPE_NAME[s.kv_dtype], "accum": "f32",
            "config": dict(workload_config(name, s, world, n_layers, split_kv), timed_calls=calls),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm"] if achieved else None, "traffic": traffic,
                         "traffic_source": traffic_source, "peak_source": peaks["source"], "kernel": kernel,
                         "kernel_ms": kernel_ms, "kernel_ms_bracketed": bracketed_ms,
                         "how": ("kernel_ms: back-to-back launches of the kernel alone between two CUDA events (its "
                                 "issue interval in the stream, programmatic dependent launch in effect); "
                                 "kernel_ms_bracketed: events around every single launch"
                                 if chain_timed else "kernel_ms: events around every single launch"),
                         "combine_ms": combine_ms / max(n_prof, 1), "algorithmic_bytes": per_rank_bytes},
            "host_us_per_call": host_us, "clocks": clocks, "gpu_launches": int(launches_per_call * calls),
            "plan": {"path": info.path, "ctas": info.n_ctas, "items": info.n_items, "parts": info.n_parts,
                     "tiles": int(info.tiles), "shared_groups": info.shared_groups},
            "parity_max_abs": max_err,
        }
        if cpu_s is not None:
            rec["cpu_ms_per_step"] = cpu_s * 1e3
        if rec_e2e:
            rec["e2e"] = rec_e2e
        if cpu:
            rec["cpu_baseline"] = cpu_baseline(s, oracle_state)
    kv.close()
    return rec


def e2e_decode(env, s, kv, layers, calls):
    """The same step through the boundary calls with HOST buffers: pass metadata (begin_pass),
    the step's qkv rows uploaded from pinned host memory, yx_attention (norm, RoPE, append,
    split-key attention, merge), the result downloaded to pinned host memory and waited for,
    every step.  Plain C-ABI calls through ctypes, nothing else on the path."""
    import ctypes
    torch, b = env.torch, env.b
    L, ctx = b._L, b._ctx
    rows, hq, hkv = s.meta.rows, s.hq, s.hkv
    qkv_host = torch.empty(rows, (hq + 2 * hkv) * 128, dtype=torch.float32).pin_memory()
    qkv_host.normal_(generator=torch.Generator().manual_seed(5 + env.rank))
    out_host = torch.empty(rows, hq * 128, dtype=torch.float32).pin_memory()
    qkv_dev = torch.empty_like(qkv_host, device=env.dev)
    out_dev = torch.empty(rows, hq * 128, dtype=torch.float32, device=env.dev)
    w = torch.zeros(128, device=env.dev)
    u32p = ctypes.POINTER(ctypes.c_uint32)
    arr = [np.ascontiguousarray(a, np.uint32) for a in (s.meta.pos, s.meta.kv_slot, s.meta.pt_off, s.meta.pages)]
    p_pos, p_slot, p_off, p_pages = (a.ctypes.data_as(u32p) for a in arr)
    n_pages = len(arr[3])
    vp = ctypes.c_void_p
    qh, qd, oh, od, wp = (vp(x.data_ptr()) for x in (qkv_host, qkv_dev, out_host, out_dev, w))
    in_bytes, out_bytes = qkv_host.numel() * 4, out_host.numel() * 4
    n_layers = len(layers)
    acc = [0.0, 0.0, 0.0, 0.0]
    pc = time.perf_counter

    # In a decode loop some row's keys grow into a new 64-key tile on about one step in four at
    # this batch size, and the attention plan is then built from scratch instead of patched; this
    # loop repeats one pass, so it asks for that on every fourth step.
    full_plan_every = 4

    def step(i):
        if i % full_plan_every == 0:
            L.yx_hook_forget_plan_shape(ctx)
        t0 = pc()
        L.yx_begin_pass(ctx, rows, p_pos, p_slot, p_off, p_pages, n_pages)
        t1 = pc()
        L.yx_upload(ctx, qd, qh, in_bytes)
        t2 = pc()
        L.yx_attention(ctx, kv._h, i % n_layers, qd, wp, wp, hq, 1e-6, od)
        t3 = pc()
        rc = L.yx_download(ctx, oh, od, out_bytes, 1)
        t4 = pc()
        if rc:
            raise RuntimeError(b.last_error())
        acc[0] += t1 - t0
        acc[1] += t2 - t1
        acc[2] += t3 - t2
        acc[3] += t4 - t3

    for i in range(5):
        step(i)
    acc[:] = [0.0, 0.0, 0.0, 0.0]
    ms, _, _ = env.timed(step, calls, 0)
    total = env.sum_over_ranks(s.unique_kv_bytes())
    h2d = in_bytes + (3 * rows + n_pages) * 4
    return {"value": total / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms,
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(out_bytes),
            "host_us": {"begin_pass": acc[0] / calls * 1e6, "upload_call": acc[1] / calls * 1e6,
                        "attention_call_plan_and_launches": acc[2] / calls * 1e6,
                        "download_and_wait_for_device": acc[3] / calls * 1e6},
            "plan": f"built from scratch on every {full_plan_every}th step, patched in place on the others",
            "note": "the library's own upload of the attention plan built from the metadata is not counted in h2d_bytes_per_step"}


def cpu_baseline(s, oracle_state=None):
    """The CPU oracle on the same step, every host core, best of three."""
    from oracle.binding import Oracle
    from oracle.check import oracle_arenas
    if oracle_state is None:
        o = Oracle()
        K, V = oracle_arenas(o, s)
    else:
        o, K, V = oracle_state
    cores = host_cores()
    best = None
    for _ in range(3):
        t0 = time.perf_counter()
        o.attend(s.q, s.meta.pos, s.meta.pt_off, s.meta.pages, s.hq, s.hkv, 128, s.window, K, V, threads=cores)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": s.unique_kv_bytes() / best / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"the whole step ({s.meta.rows} rows x {s.hq} heads), best of 3", "ms_per_step": best * 1e3}


def run_matmul(env, calls, warm, check=True):
    """The decode step's largest operator outside attention (Backend::matmul_glu, the fused gate/up
    projection of a layer with hidden 4096 and intermediate 14336): 16 pass rows against a bf16
    weight of [28672, 4096].  Bandwidth-bound on the weights, which is what the record counts."""
    torch, b, dev = env.torch, env.b, env.dev
    T, N, K = 16, 28672, 4096
    w_bytes = N * K * 2
    n_w = max(2, int(math.ceil(4.0 * L2_BYTES / w_bytes)))
    g = torch.Generator(device="cpu").manual_seed(77 + env.rank)
    ws = [(torch.randn(N, K, generator=g) * (1.0 / math.sqrt(K))).to(torch.bfloat16).to(dev) for _ in range(n_w)]
    x = torch.randn(T, K, generator=g).to(dev)
    max_err = None
    if check and env.rank == 0:
        from oracle.binding import Oracle
        o = Oracle()
        rows = slice(0, 2048)        # the oracle on the first 2048 gate rows and their up rows
        sub = torch.cat([ws[0][:2048], ws[0][N // 2:N // 2 + 2048]]).contiguous()
        got = b.to_host(b.matmul_glu(x, sub))
        w_bits = sub.view(torch.int16).cpu().numpy().view(np.uint16)
        ref = o.swiglu(o.matmul(x.cpu().numpy(), w_bits, threads=host_cores()))
        max_err = float(np.abs(got - ref).max())
        assert max_err <= 2e-5 * max(1.0, float(np.abs(ref).max())), f"matmul_glu parity: {max_err}"
        full = b.to_host(b.matmul_glu(x, ws[0]))      # and the full weight agrees with its slice
        assert np.array_equal(full[:, rows], got), "matmul_glu: the full weight differs from its slice"
    env.barrier()
    out = torch.empty(T, N // 2, dtype=torch.float32, device=dev)

    def step(i):
        b._L.yx_matmul_glu(b._ctx, x.data_ptr(), ws[i % n_w].data_ptr(), T, N, K, out.data_ptr())

    launches0 = b.launch_count()
    step(0)
    launches_per_call = b.launch_count() - launches0
    ms, host_us, clocks = env.timed(step, calls, warm)
    rec = None
    if env.rank == 0:
        peaks = measured_peaks()
        achieved = w_bytes / (ms * 1e-3) / 1e9
        rec = {"metric": "decode matmul_glu weight GB/s", "value": env.world * achieved, "unit": "GB/s", "ms_per_step": ms,
               "scaling": "weak", "dtype": "bf16 weights, f32 activations (as two bf16 parts), f32 sums",
               "config": {"workload": "decode_matmul_glu", "rows": T, "n": N, "k": K, "timed_calls": calls,
                          "l2": f"calls rotate over {n_w} weights ({n_w} x {w_bytes >> 20} MiB > L2)"},
               "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                            "frac": achieved / peaks["hbm"], "traffic": captured_traffic("matmul_rows_kernel_decode_matmul_glu")[0],
                            "traffic_source": captured_traffic("matmul_rows_kernel_decode_matmul_glu")[1], "peak_source": peaks["source"],
                            "kernel": "matmul_rows_kernel", "algorithmic_bytes": float(w_bytes),
                            "how": "the whole call (packing, the matmul kernel, the finishing kernel) between two CUDA events"},
               "host_us_per_call": host_us, "clocks": clocks, "gpu_launches": int(launches_per_call * calls),
               "parity_max_abs": max_err}
    del ws
    return rec


def run_prefill(env, steps, warm, kv_name="bf16", check=True, e2e=False):
    """Chunked causal prefill: 8 sequences x 4096 tokens in 512-row chunks, 16-bit Q/K/V, f32
    softmax and accumulation.  A step is the whole prefill of the batch (eight passes, each
    appending its 4096 K/V rows and attending); the metric is causal-exact TFLOP/s."""
    torch, b, dev = env.torch, env.b, env.dev
    from yaxus_b200.backend import LayerMeta, Rope
    world, rank = env.world, env.rank
    n_seq, total, chunk, hq, hkv = 8, 4096, 512, 32, 8
    kvt = F16 if kv_name == "f16" else BF16
    tdt = torch.bfloat16 if kvt == BF16 else torch.float16
    n_layers = 2   # 2 x 134 MB of K+V: a step does not find its pages in L2 from the step before
    passes = W.prefill_passes(seed=W.SEED0 + 3 + 1000 * rank, n_seq=n_seq, total=total, chunk=chunk, kv_dtype=kvt,
                              hq=hq, hkv=hkv)
    s0 = passes[0]
    layers = [LayerMeta(index=i, rope=Rope.default()) for i in range(n_layers)]
    kv = b.new_kv(hkv, layers, s0.arena_pages, 8192, kvt)
    T = s0.meta.rows
    up = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(dev).to(tdt)
    qs = [up(p.q) for p in passes]
    ks = [up(p.k_new) for p in passes]
    vs = [up(p.v_new) for p in passes]
    out = torch.empty(T, hq * 128, dtype=tdt, device=dev)
    flops = sum(p.flops() for p in passes)

    def step(i):
        layer = i % n_layers
        for n, p in enumerate(passes):
            b.begin_pass(p.meta)
            b.kv_append(kv, layer, ks[n], vs[n])
            b.attend(kv, layer, qs[n], hq, out=out)

    # Parity at the configuration's own shape: the whole prefill once, then the last chunk's
    # output (context 3584 + 512, all eight sequences) against the oracle on a sample of its rows.
    max_err, cpu_s, rows_checked, sample_flops = None, None, 0, 0.0
    if check and rank == 0:
        from oracle.binding import Oracle
        from oracle.check import assert_close
        o = Oracle()
        step(0)
        got = b.to_host(out)
        K = np.zeros((s0.arena_pages * 128, hkv * 128), np.float32)
        V = np.zeros_like(K)
        for p in passes:
            o.append_rows(W.round_through(p.k_new, kvt), W.round_through(p.v_new, kvt), p.meta.kv_slot, K, V)
        p = passes[-1]
        sample = np.concatenate([np.arange(sq * chunk, (sq + 1) * chunk)[::8] for sq in range(n_seq)])
        t0 = time.perf_counter()
        ref = o.attend(p.q[sample], p.meta.pos[sample], p.meta.pt_off[sample], p.meta.pages, hq, hkv, 128, None, K, V,
                       threads=host_cores())
        cpu_s = time.perf_counter() - t0
        rows_checked = len(sample)
        # outputs are stored in the 16-bit type: half a unit in the last place on top of the bound
        max_err = assert_close(got[sample], ref, abs_tol=2e-3, rel_tol=1e-2 + (2.0 ** -8 if kvt == BF16 else 2.0 ** -11),
                               what="prefill parity (last chunk)")
        sample_flops = 4.0 * 128 * hq * float((p.meta.pos[sample].astype(np.int64) + 1).sum())
    env.barrier()

    ms, host_us, clocks = env.timed(step, steps, max(warm, 3))
    launches0 = b.launch_count()
    step(0)
    launches_per_step = b.launch_count() - launches0
    info = b.last_plan()
    # the tile kernel alone (CUDA events around every attention call)
    b.profile_begin()
    for i in range(min(steps, 16)):
        step(i)
    split_ms, _, n_prof = b.profile_end()
    kernel_ms_per_step = split_ms / max(n_prof, 1) * len(passes)
    (kernel_ms_per_step,) = env.max_over_ranks([kernel_ms_per_step])

    rec_e2e = prefill_e2e(env, passes, kv, n_layers, hq, hkv, tdt, flops, min(steps, 5)) if e2e else None
    rec = None
    if rank == 0:
        peaks = measured_peaks()
        achieved = flops / (kernel_ms_per_step * 1e-3) / 1e12
        traffic, traffic_source = captured_traffic("prefill_tc2_kernel_chunked_prefill") if world == 1 else (None, None)
        rec = {
            "metric": "prefill-attn TFLOPS", "value": world * flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "ms_per_step": ms, "scaling": "weak", "dtype": kv_name, "accum": "f32",
            "config": {"workload": "chunked causal prefill", "sequences": n_seq, "tokens_per_sequence": total,
                       "chunk": chunk, "hq": hq, "hkv": hkv, "head_dim": 128, "kv_dtype": kv_name,
                       "flops_per_step": flops, "passes_per_step": len(passes), "timed_steps": steps,
                       "l2": f"steps alternate over {n_layers} layer arenas of 134 MB",
                       "parallelism": f"by sequence, {world} GPU(s), no collective"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["bf16"], "frac_of_burst_peak": achieved / peaks["bf16_burst"],
                         "traffic": traffic, "traffic_source": traffic_source,
                         "peak_source": peaks["source"] + " (sustained)", "kernel": f"prefill_tc2_{kv_name}_kernel",
                         "kernel_ms_per_step": kernel_ms_per_step,
                         "how": "events around every launch of the tile kernel, summed over the step's eight passes"},
            "host_us_per_call": host_us, "clocks": clocks, "gpu_launches": int(launches_per_step * steps),
            "plan": {"path": info.path}, "parity_max_abs": max_err, "parity_rows_checked": rows_checked,
        }
        if cpu_s is not None:
            rec["cpu_baseline"] = {"value": sample_flops / cpu_s / 1e12, "unit": "TFLOP/s", "cores": host_cores(),
                                   "kind": "port",
                                   "sample": f"{rows_checked} rows of the last chunk (every 8th row of each sequence), one run",
                                   "ms_per_step_extrapolated": cpu_s * flops / sample_flops * 1e3}
        if rec_e2e:
            rec["e2e"] = rec_e2e
    kv.close()
    return rec


def prefill_e2e(env, passes, kv, n_layers, hq, hkv, tdt, flops, steps):
    """Prefill with host buffers: per pass the metadata, the 16-bit q/k/v rows from pinned host
    memory and the result read back.  Two sets of device buffers and two copy streams: the rows
    of pass p + 1 go up and the result of pass p - 1 comes down while pass p computes (what a
    serving loop does with host buffers); every buffer's reuse is ordered by events."""
    torch, b, dev = env.torch, env.b, env.dev
    T = passes[0].meta.rows
    qh = torch.empty(T, hq * 128, dtype=tdt).pin_memory()
    kh = torch.empty(T, hkv * 128, dtype=tdt).pin_memory()
    vh = torch.empty(T, hkv * 128, dtype=tdt).pin_memory()
    oh = torch.empty(T, hq * 128, dtype=tdt).pin_memory()
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
    ms, _, _ = env.timed(e2e_step, steps, 1)
    bytes_in = (qh.numel() + kh.numel() + vh.numel()) * 2 * len(passes)
    return {"value": env.world * flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms,
            "h2d_bytes_per_step": int(bytes_in), "d2h_bytes_per_step": int(oh.numel() * 2 * len(passes))}


def run_reference(args):
    """The reference's CPU implementation of the path (its restated CPU backend, every host
    core) on the headline workload.  Rank 0 only; other ranks leave at once."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle.binding import Oracle
    from oracle.check import oracle_arenas
    o = Oracle()
    name = args.workload or "batched_decode"
    s = make_scenario(name, 0)
    K, V = oracle_arenas(o, s)
    cores = host_cores()

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
        "dtype": DTYPE_NAME[s.kv_dtype], "data": "synthetic",
        "config": dict(workload_config(name, s, args.gpus, layers_needed(s.unique_kv_bytes()), False), timed_calls=n_timed),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


SUB_WORKLOADS = ("prefill", "verify", "single_decode", "long_decode", "long_decode_window", "decode_matmul_glu")


def run_cuda(args):
    env = Env()
    warm = max(args.warmup, 3)
    calls = args.calls if args.calls > 0 else max(args.steps, MIN_TIMED_CALLS)
    head_name = args.workload or "batched_decode"
    if head_name == "prefill":
        head = run_prefill(env, max(1, min(args.steps, 50)), warm, args.kv_dtype or "bf16", check=not args.no_check, e2e=True)
    elif head_name == "decode_matmul_glu":
        head = run_matmul(env, args.calls if args.calls > 0 else 2000, warm, check=not args.no_check)
    else:
        head = run_split_key(env, head_name, make_scenario(head_name, env.rank), calls, warm, check=not args.no_check,
                             e2e=True, cpu=not args.no_cpu, kernel_only=True)
    subs = {}
    if not args.workload and not args.headline_only:
        long_s = None
        for name in SUB_WORKLOADS:
            t0 = time.time()
            try:
                if name == "prefill":
                    rec = run_prefill(env, 5, 3, "bf16", check=not args.no_check)
                elif name == "decode_matmul_glu":
                    rec = run_matmul(env, 2000, warm, check=not args.no_check)
                elif name.startswith("long_decode"):
                    if long_s is None:
                        long_s = make_scenario("long_decode", 0)
                    s = long_s if name == "long_decode" else dataclasses.replace(long_s, window=2048)
                    rec = run_split_key(env, name, s, 3000, warm, check=not args.no_check, kernel_only=True)
                else:
                    rec = run_split_key(env, name, make_scenario(name, env.rank), 3000, warm, check=not args.no_check, kernel_only=True)
            except AssertionError as e:     # a parity failure is reported, not hidden
                rec = {"error": str(e)[:300]} if env.rank == 0 else None
            if rec is not None:
                rec["wall_s"] = round(time.time() - t0, 1)
                subs[name] = rec
    if env.rank == 0:
        line = {"metric": head.pop("metric"), "value": head.pop("value"), "unit": head.pop("unit"), "n_gpus": env.world,
                "steps": args.steps, "warmup": warm, "ms_per_step": head.pop("ms_per_step"), "higher_is_better": True,
                "scaling": head.pop("scaling"), "vs_baseline": None, "dtype": head.pop("dtype"), "data": "synthetic"}
        line.update(head)
        if subs:
            line["workloads"] = subs
        print(json.dumps(line))
    env.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--workload", default=None, help="print this workload alone as the whole line")
    ap.add_argument("--kv-dtype", default=None, choices=["f16", "bf16"],
                    help="cache storage type of the prefill workload (default bf16)")
    ap.add_argument("--headline-only", action="store_true", help="leave the other workloads' records out")
    ap.add_argument("--calls", type=int, default=0,
                    help="time exactly this many calls of the headline workload (for profiler captures; default: at least 10000)")
    ap.add_argument("--no-check", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
