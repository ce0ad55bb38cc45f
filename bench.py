#!/usr/bin/env python
"""Benchmark of the Q8_0 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload (the lm_head shape the bandwidth target is quoted on):
the lm_head GEMV, 151936 rows x K=2560, Q8_0 weights ~N(0, 0.02), fp32
activation ~N(0, 1), batch 1.  A step is one full matvec.  The metric is
weight-GB/s: rows * (K/32) * 34 bytes per step, over the device time of the
step.  With N > 1 the rows are split evenly over the ranks (fixed total work:
strong scaling) and every step ends with the all-gather of the fp32 logits.

One JSON line is printed by rank 0.  Beside the contract keys it carries
`roofline` (the GEMV kernel against measured HBM bandwidth), `cpu_baseline` (the
reference's own CPU matvec on this host), `e2e` (the same step through the
host-buffer entry point with pinned buffers) and `mmq` (the batched prefill
product at M=512, K=2560, N=9728 in int8 TOPS).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ROWS, WIDTH = 151936, 2560
BLOCKS = WIDTH // 32
WEIGHT_BYTES = ROWS * BLOCKS * 34
MMQ_M, MMQ_K, MMQ_N = 512, 2560, 9728
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the register-pipelined GEMV
# kernel over 65536 rows x 2560 (one ncu capture, 181.95 MB); DRAM traffic grows in
# proportion to the rows, so a launch's traffic is this figure scaled by its row count.  It
# describes that kernel only: `roofline.traffic_source` names it in the JSON line.
GEMV_DRAM_TRAFFIC_CAPTURE = {"kernel": "q8_gemv_pipelined_kernel", "rows": 65536, "width": 2560,
                             "bytes": 181.95e6}
GEMV_DRAM_TRAFFIC_PER_ROW = GEMV_DRAM_TRAFFIC_CAPTURE["bytes"] / GEMV_DRAM_TRAFFIC_CAPTURE["rows"]


def set_rows(rows: int) -> None:
    global ROWS, WEIGHT_BYTES
    ROWS = int(rows)
    WEIGHT_BYTES = ROWS * BLOCKS * 34


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": FALLBACK_HBM_GBS}, "fallback"


# ------------------------------------------------------------------------------ clocks
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.samples = []
        self.proc = None
        self.device_index = device_index
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.device_index), "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0: float, t1: float, busy0: float = None, busy1: float = None):
        """Samples taken inside the timed region [t0, t1]; when the region is shorter than the
        sampling period, the samples of the busy period around it (the same loop, untimed:
        [busy0, busy1]).  `window` says which."""
        window = "timed region"
        rows = [s for (t, s) in self.samples if t0 <= t <= t1]
        if not rows and busy0 is not None:
            window = "same loop continued around the timed region"
            rows = [s for (t, s) in self.samples if busy0 <= t <= busy1]
        if not rows:
            window = "whole run"
            rows = [s for (_, s) in self.samples]
        sm, smax, reasons = [], [], set()
        for row in rows:
            parts = [p.strip() for p in row.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                    "sw_power_cap"), parts[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0,
                    "window": window}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(smax)),
                "reasons": sorted(reasons), "samples": len(sm), "window": window}


# ------------------------------------------------------------------------------ reference arm
def reference_library():
    """The reference's CPU matvec, on every core this process may use.  The reference's own
    policy is OMP_NUM_THREADS=$(nproc) (tools/build_native.sh:7-9); a launcher that exports
    OMP_NUM_THREADS=1 to its children (torch.distributed.run does) must not turn the
    baseline into a one-thread run, so the count is set through the OpenMP API."""
    from oracle import q8_oracle as o
    o.build()
    threads = int(os.environ.get("FORTAI_BENCH_CPU_THREADS", "0")) or o.host_threads()
    o.set_threads(threads)
    if o.Reference.available(fast=True):
        ref = o.Reference(fast=True)
        ref.set_threads(threads)
        return o, ref, "reference"
    return o, None, "port"


def time_cpu_matvec(o, ref, weights, rows, x, repeats):
    """Seconds for `repeats` matvecs of the first `rows` rows on all host threads."""
    if ref is not None:
        t = time.perf_counter()
        ref.matvec_repeat(weights, rows, WIDTH, x, repeats)
        return time.perf_counter() - t
    t = time.perf_counter()
    for _ in range(repeats):
        o.matvec(weights, rows, WIDTH, x)
    return time.perf_counter() - t


def cpu_baseline_block(weights_host, x, budget_s=12.0):
    """The reference's CPU matvec (oracle/_ref, its own C arithmetic compiled with its
    native-profile flags) on a bounded sample of the same workload."""
    o, ref, kind = reference_library()
    threads = ref.thread_count() if ref is not None else o.thread_count()
    w = np.ascontiguousarray(weights_host).view(np.int8).reshape(-1)
    time_cpu_matvec(o, ref, w, ROWS, x, 1)                       # warm
    once = time_cpu_matvec(o, ref, w, ROWS, x, 2) / 2
    repeats = int(max(3, min(2000, budget_s / max(once, 1e-6))))
    seconds = time_cpu_matvec(o, ref, w, ROWS, x, repeats)
    value = WEIGHT_BYTES * repeats / seconds / 1e9
    return {"value": value, "unit": "GB/s", "cores": threads, "kind": kind,
            "sample": f"{repeats} repeats of the full {ROWS}x{WIDTH} matvec, "
                      f"{seconds:.1f} s, OMP threads={threads}, "
                      f"avx2={'yes' if (ref is None or ref.uses_avx2()) else 'no'}",
            "ms_per_matvec": seconds / repeats * 1e3}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    o, ref, kind = reference_library()
    threads = ref.thread_count() if ref is not None else o.thread_count()
    weights = o.make_weights(ROWS, WIDTH, seed=0, sigma=0.02)
    x = o.normal(WIDTH, seed=1)
    time_cpu_matvec(o, ref, weights, ROWS, x, 1)
    full = time_cpu_matvec(o, ref, weights, ROWS, x, 2) / 2
    # bound the whole run to about two minutes: a step is the matvec of the first
    # `rows` rows (all of them when that fits)
    budget = 120.0
    total_steps = max(1, args.steps + args.warmup)
    rows = ROWS
    if full * total_steps > budget:
        rows = int(max(1024, min(ROWS, ROWS * budget / (full * total_steps))))
    time_cpu_matvec(o, ref, weights, rows, x, max(1, args.warmup))
    seconds = time_cpu_matvec(o, ref, weights, rows, x, args.steps)
    sample_bytes = rows * BLOCKS * 34
    value = sample_bytes * args.steps / seconds / 1e9
    sample = (f"each step = matvec of the first {rows} of {ROWS} rows x {WIDTH} "
              f"({sample_bytes} weight bytes), OMP threads={threads} of {os.cpu_count()} host "
              f"cpus (OMP_NUM_THREADS in the environment: "
              f"{os.environ.get('OMP_NUM_THREADS', 'unset')})")
    line = {
        "impl": "reference", "metric": "q8_0_gemv_weight_bandwidth", "value": value,
        "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": seconds / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8 x int8 -> int32, fp32 scales",
        "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": kind,
                         "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


L2_BYTES = 126 * 1000 * 1000


def shard_copies(n_gpus):
    """How many copies of a rank's shard the steps go round: one when the shard is at least
    twice the L2, else enough for three L2 sizes."""
    shard = -(-ROWS // n_gpus) * BLOCKS * 34
    return 1 if shard >= 2 * L2_BYTES else int(min(12, 3 * L2_BYTES // shard + 1))


def workload_config(n_gpus, copies=None):
    copies = shard_copies(n_gpus) if copies is None else copies
    cache = "inputs larger than L2 (413 MB of weights per step, L2 is 126 MB)"
    if copies > 1:
        cache += (f"; a rank's shard is smaller than twice the L2, so the steps go round "
                  f"{copies} copies of it and every step reads from HBM")
    return {
        "workload": f"lm_head Q8_0 GEMV {ROWS}x{WIDTH} batch 1 (headline configuration)",
        "rows": ROWS, "width": WIDTH, "weight_bytes": WEIGHT_BYTES,
        "sharding": "none" if n_gpus == 1 else f"rows/{n_gpus} per rank, fp32 logits reassembled on every rank",
        "cache": cache,
        "inputs": "weights ~N(0,0.02) quantized to Q8_0 on the device, activation ~N(0,1), seed 0",
    }


# ------------------------------------------------------------------------------ GPU arm
def make_device_weights(torch, backend, ctx, first_row, rows, width, seed):
    """Q8_0 bytes (GGUF order, host numpy) of rows [first_row, first_row+rows) of a
    seeded N(0, 0.02) matrix; sampled and quantized on the device."""
    out = np.empty(rows * (width // 32) * 34, dtype=np.int8)
    chunk = 16384
    done = 0
    while done < rows:
        n = min(chunk, rows - done)
        gen = torch.Generator(device="cuda")
        gen.manual_seed(seed * 1000003 + first_row + done)
        values = torch.randn(n, width, generator=gen, device="cuda", dtype=torch.float32) * 0.02
        q = torch.empty(n * (width // 32) * 34, dtype=torch.int8, device="cuda")
        torch.cuda.current_stream().synchronize()
        stat = backend.cuda_q8_quantize_device(ctx, values.data_ptr(), values.numel(),
                                               q.data_ptr(), q.numel())
        if not stat.is_ok():
            raise RuntimeError(f"device quantize failed: {stat}")
        ctx.synchronize()
        out[done * (width // 32) * 34:(done + n) * (width // 32) * 34] = q.cpu().numpy()
        done += n
    return out


def run_gpu_arm(args):
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    from fortai_b200 import backend_cuda as backend

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world,
                                device_id=torch.device("cuda", local_rank))
    torch.cuda.set_device(local_rank)
    stream = torch.cuda.current_stream()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()         # nvidia-smi needs a moment before its first sample

    ctx = backend.cuda_q8_context_t()
    stat = ctx.create(local_rank, stream=stream.cuda_stream)
    if not stat.is_ok():
        raise SystemExit(f"context creation failed: {stat}")

    # ---- this rank's shard of the lm_head
    from fortai_b200 import sharded
    ranges = sharded.partition(ROWS, world)
    counts = [c for _, c in ranges]
    first_row, my_rows = ranges[rank]
    host_weights = make_device_weights(torch, backend, ctx, first_row, my_rows, WIDTH, seed=0)
    # A shard smaller than twice the L2 would be served from L2 when the same bytes are read
    # step after step (a quarter of the lm_head is 103 MB, L2 is 126 MB): such shards are
    # uploaded several times and the steps go round the copies, so that every step streams
    # its weights from HBM, as the single-GPU step does.
    copies = shard_copies(world)
    ring = []
    for _ in range(copies):
        handle = backend.cuda_q8_weights_t()
        stat = handle.upload(ctx, host_weights, host_weights.size, my_rows, WIDTH)
        if not stat.is_ok():
            raise SystemExit(f"weight upload failed: {stat}")
        ring.append(handle)
    weights = ring[0]
    turn = [0]

    def next_weights():
        turn[0] = (turn[0] + 1) % copies
        return ring[turn[0]]

    gen = torch.Generator(device="cuda")
    gen.manual_seed(1)
    x = torch.randn(WIDTH, generator=gen, device="cuda", dtype=torch.float32)

    # The logits vector lives in symmetric memory when there are peers, so that the GEMV
    # epilogue can store this rank's slice straight into every rank's copy.
    peer_ptrs, symm_handle, flag_ptrs = None, None, None
    logits = None
    if world > 1 and args.exchange in ("auto", "peers", "fused", "pairs"):
        try:
            import torch.distributed._symmetric_memory as symm
            logits = symm.empty(ROWS, dtype=torch.float32, device=torch.device("cuda", local_rank))
            symm_handle = symm.rendezvous(logits, dist.group.WORLD)
            peer_ptrs = backend.pointer_array([int(p) for p in symm_handle.buffer_ptrs])
            flags = symm.empty(world, dtype=torch.int32, device=torch.device("cuda", local_rank))
            flags.zero_()
            flag_handle = symm.rendezvous(flags, dist.group.WORLD)
            flag_ptrs = backend.pointer_array([int(p) for p in flag_handle.buffer_ptrs])
            pair_buffer = symm.empty(4 * ROWS, dtype=torch.int32, device=torch.device("cuda", local_rank))
            pair_buffer.zero_()
            pair_handle = symm.rendezvous(pair_buffer, dist.group.WORLD)
            pair_ptrs = backend.pointer_array([int(p) for p in pair_handle.buffer_ptrs])
            torch.cuda.synchronize()
            dist.barrier()
        except Exception as error:  # no peer access on this box: fall back to NCCL
            if args.exchange in ("peers", "fused", "pairs"):
                raise SystemExit(f"symmetric memory unavailable: {error}")
            peer_ptrs, symm_handle, logits = None, None, None
    if logits is None:
        logits = torch.empty(ROWS, device="cuda", dtype=torch.float32)
    my_slice = logits[first_row:first_row + my_rows]

    def step_allgather(x=x):
        stat = backend.cuda_q8_matvec_device_f32(ctx, next_weights(), x.data_ptr(), WIDTH,
                                                 my_slice.data_ptr(), my_rows)
        if not stat.is_ok():
            raise RuntimeError(f"matvec failed: {stat}")
        if world > 1:
            sharded.all_gather_rows(dist, my_slice, counts, logits)

    def step_peers(x=x):
        stat = backend.cuda_q8_matvec_device_f32_peers(ctx, next_weights(), x.data_ptr(), WIDTH,
                                                       peer_ptrs, first_row, ROWS)
        if not stat.is_ok():
            raise RuntimeError(f"peer matvec failed: {stat}")
        symm_handle.barrier(channel=0)

    def step_fused(x=x):
        stat = backend.cuda_q8_matvec_device_f32_allgather(ctx, next_weights(), x.data_ptr(), WIDTH,
                                                           peer_ptrs, flag_ptrs, rank, first_row,
                                                           ROWS)
        if not stat.is_ok():
            raise RuntimeError(f"all-gather matvec failed: {stat}")

    def step_pairs(x=x):
        stat = backend.cuda_q8_matvec_device_f32_allgather_ll(ctx, next_weights(), x.data_ptr(),
                                                              WIDTH, pair_ptrs, rank, first_row,
                                                              logits.data_ptr(), ROWS)
        if not stat.is_ok():
            raise RuntimeError(f"all-gather matvec (pairs) failed: {stat}")

    def time_steps(fn, n):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(n):
            fn()
        b.record(stream)
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / n], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def verify(fn):
        """One step of `fn` on a fresh activation into zeroed logits; every rank's assembled
        vector must equal, bit for bit, the slices that each rank's own GEMV wrote into a
        private buffer, gathered by NCCL.  A store at a wrong offset, a flag raised before the
        slice is visible or a stale slice all fail this."""
        gen_v = torch.Generator(device="cuda")
        gen_v.manual_seed(12345)
        xv = torch.randn(WIDTH, generator=gen_v, device="cuda", dtype=torch.float32)
        own = torch.empty(my_rows, device="cuda", dtype=torch.float32)
        stat = backend.cuda_q8_matvec_device_f32(ctx, weights, xv.data_ptr(), WIDTH,
                                                 own.data_ptr(), my_rows)
        if not stat.is_ok():
            raise RuntimeError(f"matvec failed: {stat}")
        truth = torch.empty(ROWS, device="cuda", dtype=torch.float32)
        sharded.all_gather_rows(dist, own, counts, truth)
        logits.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        fn(xv)
        torch.cuda.synchronize()
        dist.barrier()
        same = torch.tensor([1 if torch.equal(logits, truth) else 0], device="cuda")
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        # leave the buffers as the timed loops expect them
        torch.cuda.synchronize()
        dist.barrier()
        return bool(same.item())

    exchange = "none"
    exchange_ms = {}
    exchange_verified = {}
    step = step_allgather
    if world > 1:
        exchange = "allgather"
        candidates = {"allgather": step_allgather}
        if peer_ptrs is not None:
            candidates["peers"] = step_peers
            candidates["fused"] = step_fused
            candidates["pairs"] = step_pairs
        for name, fn in candidates.items():
            exchange_verified[name] = verify(fn)
            exchange_ms[name] = time_steps(fn, 200)
        eligible = {k: v for k, v in exchange_ms.items() if exchange_verified[k]}
        if not eligible:
            raise SystemExit(f"no exchange mode reproduced the gathered logits: {exchange_verified}")
        if args.exchange in ("peers", "fused", "pairs") and args.exchange in eligible:
            exchange = args.exchange
        else:
            exchange = min(eligible, key=eligible.get)
        step = candidates[exchange]

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # The timed region of the default run is about a millisecond, far shorter than a clock
    # sample: the same loop runs untimed for a while before and after it, so that the clocks
    # reported are those of this loop under load.
    # (a step count, the same on every rank: the steps contain collectives)
    if world > 1:
        step_ms_estimate = exchange_ms[exchange]
    else:
        for _ in range(5):
            step()
        torch.cuda.synchronize()
        a0, b0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record(stream)
        for _ in range(50):
            step()
        b0.record(stream)
        torch.cuda.synchronize()
        step_ms_estimate = a0.elapsed_time(b0) / 50

    def run_for(seconds):
        count = int(min(20000, max(50, seconds * 1e3 / max(step_ms_estimate, 1e-3))))
        for _ in range(count):
            step()
        torch.cuda.synchronize()
    busy0 = time.time()
    run_for(0.25)
    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    launches_before = ctx.launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    start.record(stream)
    for _ in range(args.steps):
        step()
    stop.record(stream)
    barrier()
    t1 = time.time()
    launches = ctx.launch_count() - launches_before
    elapsed_ms = start.elapsed_time(stop)
    run_for(0.15)
    barrier()
    busy1 = time.time()
    if world > 1:
        t = torch.tensor([elapsed_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    stat = ctx.synchronize()
    if not stat.is_ok():
        raise SystemExit(f"device reported: {stat}")

    # ---- kernel alone on this rank (no collective), for the roofline
    for _ in range(3):
        backend.cuda_q8_matvec_device_f32(ctx, next_weights(), x.data_ptr(), WIDTH,
                                          my_slice.data_ptr(), my_rows)
    torch.cuda.synchronize()
    k_iters = max(20, min(args.steps, 2000))
    start.record(stream)
    for _ in range(k_iters):
        backend.cuda_q8_matvec_device_f32(ctx, next_weights(), x.data_ptr(), WIDTH,
                                          my_slice.data_ptr(), my_rows)
    stop.record(stream)
    torch.cuda.synchronize()
    kernel_ms = start.elapsed_time(stop) / k_iters

    if args.kernel_only:
        if rank == 0:
            sampler.stop()
            print(json.dumps({"kernel_only": True, "rows": ROWS, "kernel_ms": kernel_ms,
                              "weight_gbs": my_rows * BLOCKS * 34 / kernel_ms / 1e6,
                              "ms_per_step": elapsed_ms / args.steps}), flush=True)
        ctx_cleanup(ring, ctx, dist)
        return 0

    # ---- end to end through the host-buffer entry point, pinned buffers
    host_x = torch.empty(WIDTH, dtype=torch.float32).pin_memory()
    host_x.copy_(x.cpu())
    host_out = torch.empty(my_rows, dtype=torch.float32).pin_memory()
    hx, ho = host_x.numpy(), host_out.numpy()
    e2e_steps = max(10, min(args.steps, 500))
    for _ in range(3):
        backend.cuda_q8_matvec_host_f32(ctx, next_weights(), hx, ho)
    barrier()
    te = time.perf_counter()
    for _ in range(e2e_steps):
        _, stat = backend.cuda_q8_matvec_host_f32(ctx, next_weights(), hx, ho)
        if world > 1:
            my_slice.copy_(host_out, non_blocking=True)
            sharded.all_gather_rows(dist, my_slice, counts, logits)
            torch.cuda.synchronize()
    barrier()
    e2e_s = time.perf_counter() - te
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    if rank == 0:
        sampler.stop()

    # ---- prefill product at M=512 (rank 0, single GPU run only)
    mmq = None
    if world == 1:
        mmq = bench_mmq(torch, backend, ctx)

    if rank != 0:
        ctx_cleanup(ring, ctx, dist)
        return 0

    peaks, peak_kind = measured_peaks()
    hbm_peak = float(peaks.get("hbm_gbs", FALLBACK_HBM_GBS))
    ms_per_step = elapsed_ms / args.steps
    value = WEIGHT_BYTES / (ms_per_step * 1e-3) / 1e9
    shard_bytes = my_rows * BLOCKS * 34
    achieved = shard_bytes / (kernel_ms * 1e-3) / 1e9
    line = {
        "metric": "q8_0_gemv_weight_bandwidth", "value": value, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8 x int8 -> int32, fp32 scales", "data": "synthetic",
        "config": workload_config(world, copies),
        "exchange": {"used": exchange, "ms_per_step": exchange_ms, "verified": exchange_verified},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                     "frac": achieved / hbm_peak, "traffic": GEMV_DRAM_TRAFFIC_PER_ROW * my_rows,
                     "traffic_source": ("one ncu capture of %(kernel)s over %(rows)d x %(width)d "
                                        "(%(bytes).0f bytes), scaled by rows" %
                                        GEMV_DRAM_TRAFFIC_CAPTURE),
                     "peak_source": f"of {peak_kind}",
                     "kernel": "q8_gemv (quantize prologue + streaming dot), this rank's shard",
                     "kernel_ms": kernel_ms, "algorithmic_bytes": shard_bytes,
                     "frac_of_8TBs_nominal": achieved / 8000.0},
        "e2e": {"value": WEIGHT_BYTES * e2e_steps / e2e_s / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": WIDTH * 4, "d2h_bytes_per_step": my_rows * 4,
                "ms_per_step": e2e_s / e2e_steps * 1e3,
                "api": "fortai_cuda_q8_matvec_host_f32 (pinned host buffers; the activation is copied up, the kernel stores the results into the pinned output)"},
        "gpu_launches": int(launches),
        "clocks": sampler.summary(t0, t1, busy0, busy1),
    }
    if mmq is not None:
        line["mmq"] = mmq
    if world == 1:
        xs = x.cpu().numpy()
        line["cpu_baseline"] = cpu_baseline_block(host_weights, xs)
    print(json.dumps(line), flush=True)
    ctx_cleanup(ring, ctx, dist)
    return 0


def run_mmq_only(args):
    import torch
    from fortai_b200 import backend_cuda as backend
    ctx = backend.cuda_q8_context_t()
    stat = ctx.create(0, stream=torch.cuda.current_stream().cuda_stream)
    if not stat.is_ok():
        raise SystemExit(f"context creation failed: {stat}")
    apply_options(ctx, args.options)
    result = bench_mmq(torch, backend, ctx, tokens=args.tokens, iters=max(1, args.steps),
                       warmup=max(1, args.warmup), rows=args.mmq_rows, width=args.mmq_width)
    ctx.destroy()
    print(json.dumps(result), flush=True)
    return 0 if result and result.get("ok") else 1


def bench_mmq(torch, backend, ctx, tokens=MMQ_M, iters=50, warmup=3, rows=MMQ_N, width=MMQ_K):
    """Batched product; by default M=512 x K=2560 x N=9728 (the prefill configuration)."""
    MMQ_M, MMQ_N, MMQ_K = tokens, rows, width
    host_weights = make_device_weights(torch, backend, ctx, 0, MMQ_N, MMQ_K, seed=2)
    w = backend.cuda_q8_weights_t()
    if not w.upload(ctx, host_weights, host_weights.size, MMQ_N, MMQ_K).is_ok():
        return None
    gen = torch.Generator(device="cuda")
    gen.manual_seed(3)
    act = torch.randn(MMQ_M, MMQ_K, generator=gen, device="cuda", dtype=torch.float32)
    out = torch.empty(MMQ_M, MMQ_N, device="cuda", dtype=torch.float32)
    stream = torch.cuda.current_stream()

    def once():
        return backend.cuda_q8_matmul_device_f32(ctx, w, act.data_ptr(), MMQ_M, out.data_ptr(),
                                                 out.numel())
    for _ in range(warmup):
        if not once().is_ok():
            w.destroy()
            return None
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = ctx.launch_count()
    start.record(stream)
    for _ in range(iters):
        once()
    stop.record(stream)
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / iters
    launches = (ctx.launch_count() - launches) // iters
    ok = ctx.synchronize().is_ok()
    w.destroy()
    ops = 2.0 * MMQ_M * MMQ_K * MMQ_N
    achieved = ops / (ms * 1e-3) / 1e12
    # the denominators, measured here and now: a bare tcgen05.mma loop on every SM
    i8_peak, _, stat_i8 = backend.cuda_tensor_peak(ctx, 0, 4000)
    f16_peak, _, stat_f16 = backend.cuda_tensor_peak(ctx, 1, 4000)
    peaks_ok = stat_i8.is_ok() and stat_f16.is_ok() and i8_peak > 0 and f16_peak > 0
    roofline = {
        "bound": "int8 tensor", "achieved": achieved, "unit": "TOPS",
        "peak_measured": i8_peak if peaks_ok else None,
        "frac": achieved / i8_peak if peaks_ok else None,
        "peak_nominal": 4500.0, "frac_of_nominal": achieved / 4500.0,
        "peak_source": "bare tcgen05.mma.kind::i8 loop, 128x256x32 tiles resident in shared "
                       "memory, no drain, all SMs, timed in this run",
        "kernel": "q8_prefill_kernel: kind::f16 MMAs on exact binary16 operands, four per "
                  "Q8_0 block, i.e. twice the tensor time of one int8 MMA at half its rate",
        "f16_peak_measured_tflops": f16_peak if peaks_ok else None,
        # the kernel's own tensor work is 4 f16 MMAs of K=16 per block: 2*M*N*64 flops per block
        "tensor_pipe_frac_of_measured_f16": (2.0 * ops / (ms * 1e-3) / 1e12 / f16_peak)
        if peaks_ok else None,
    }
    return {"metric": "q8_0_mmq_int8_throughput", "value": achieved,
            "unit": "TOPS", "ms": ms, "m": MMQ_M, "k": MMQ_K, "n": MMQ_N,
            "includes": "activation quantization + product", "launches_per_call": int(launches),
            "frac_of_4500_TOPS_nominal": achieved / 4500.0, "roofline": roofline, "ok": ok}


def apply_options(ctx, spec):
    """--options name=value,name=value: tuning knobs of fortai_cuda_q8_context_set_option."""
    for item in filter(None, (spec or "").split(",")):
        name, value = item.split("=")
        if not ctx.set_option(name.strip(), int(value)).is_ok():
            raise SystemExit(f"unknown backend option {name}")


def decode_shapes():
    """Every named decode-step projection shape: (label, rows, width)."""
    shapes = [("config0 3072x1024", 3072, 1024)]
    for hidden in (1024, 2048, 2560):
        inner = int(round(3.8 * hidden / 256.0)) * 256
        shapes += [(f"H{hidden} qkv", 3 * hidden, hidden), (f"H{hidden} out", hidden, hidden),
                   (f"H{hidden} gate/up", inner, hidden), (f"H{hidden} down", hidden, inner)]
    shapes += [("27B gate/up", 17408, 5120), ("27B down", 5120, 17408)]
    return shapes


def graph_time_us(torch, ctx, enqueue, per_graph=20, replays=25, warm=3):
    """Average device time of one `enqueue()` when `per_graph` of them are captured into a
    CUDA graph on the context's own stream and the graph is replayed `replays` times."""
    stream = torch.cuda.ExternalStream(ctx.stream())
    for i in range(warm):
        enqueue(i)
    torch.cuda.synchronize()
    before = ctx.launch_count()
    assert ctx.capture_begin().is_ok()
    for i in range(per_graph):
        enqueue(i)
    assert ctx.capture_end().is_ok()
    launches = (ctx.launch_count() - before) // per_graph
    for _ in range(3):
        ctx.graph_launch()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(replays):
        ctx.graph_launch()
    b.record(stream)
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / (replays * per_graph), int(launches)


def sweep_batched(torch, backend, args):
    """Batched product at the token counts of the prefill configuration and the batch-8 decode of
    the 27B-class projections; weights rotate over copies that together exceed twice the L2 size."""
    l2_bytes = 126 * 1024 * 1024
    cases = [("prefill 9728x2560", 9728, 2560, (2, 4, 8, 16, 32, 64, 128, 512)),
             ("27B gate/up 17408x5120", 17408, 5120, (8,)),
             ("27B down 5120x17408", 5120, 17408, (8,))]
    for label, rows, width, token_counts in cases:
        if args.only and args.only not in label and args.only not in "batched":
            continue
        nbytes = rows * (width // 32) * 34
        copies = int(max(2, min(64, (2 * l2_bytes + nbytes - 1) // nbytes + 1)))
        for tokens in token_counts:
            # a context holds one captured graph, so every token count gets its own
            ctx = backend.cuda_q8_context_t()
            if not ctx.create(0).is_ok():
                raise SystemExit("context creation failed")
            apply_options(ctx, args.options)
            handles = []
            for c in range(copies):
                host = make_device_weights(torch, backend, ctx, 0, rows, width, seed=50 + c)
                w = backend.cuda_q8_weights_t()
                if not w.upload(ctx, host, host.size, rows, width).is_ok():
                    raise SystemExit("weight upload failed")
                handles.append(w)
            x = torch.randn(tokens, width, device="cuda", dtype=torch.float32)
            out = torch.empty(tokens, rows, device="cuda", dtype=torch.float32)

            def enqueue(i):
                stat = backend.cuda_q8_matmul_device_f32(ctx, handles[i % copies], x.data_ptr(),
                                                         tokens, out.data_ptr(), out.numel())
                assert stat.is_ok(), stat
            us, launches = graph_time_us(torch, ctx, enqueue, per_graph=max(copies, 10))
            ops = 2.0 * tokens * width * rows
            print(json.dumps({"shape": f"{label} M={tokens}", "weight_bytes": nbytes,
                              "hbm_cold_us": us, "weight_gbs": nbytes / us / 1e3,
                              "tops": ops / us / 1e6, "launches_per_call": launches,
                              "copies": copies}), flush=True)
            for w in handles:
                w.destroy()
            ctx.destroy()


def sweep_batched_ffn(torch, backend, args):
    """The 27B-class FFN at batch 8: the FFN for eight activations per call."""
    for hidden, inner, tokens in ((5120, 17408, 8), (2560, 9728, 8)):
        label = f"FFN H{hidden} F{inner} M={tokens}"
        if args.only and args.only not in label and args.only not in "batched":
            continue
        ctx = backend.cuda_q8_context_t()
        if not ctx.create(0).is_ok():
            raise SystemExit("context creation failed")
        apply_options(ctx, args.options)
        mats = []
        for seed, (r, k) in enumerate(((inner, hidden), (inner, hidden), (hidden, inner))):
            host = make_device_weights(torch, backend, ctx, 0, r, k, seed=30 + seed)
            w = backend.cuda_q8_weights_t()
            w.upload(ctx, host, host.size, r, k)
            mats.append(w)
        x = torch.randn(tokens, hidden, device="cuda", dtype=torch.float32)
        out = torch.empty(tokens, hidden, device="cuda", dtype=torch.float32)

        def enqueue(i):
            stat = backend.cuda_q8_ffn_batch_device(ctx, mats[0], mats[1], mats[2], x.data_ptr(),
                                                    tokens, out.data_ptr(), out.numel())
            assert stat.is_ok(), stat
        us, launches = graph_time_us(torch, ctx, enqueue, per_graph=10)
        nbytes = 3 * inner * (hidden // 32) * 34
        print(json.dumps({"shape": label, "weight_bytes": nbytes, "us": us,
                          "gbs": nbytes / us / 1e3, "launches_per_call": launches,
                          "note": "same matrices every call; 284 MB exceeds L2 for the 27B layer"}),
              flush=True)
        for w in mats:
            w.destroy()
        ctx.destroy()


def run_sweep(args):
    """Every named batch-1 shape, timed by replaying a CUDA graph of back-to-back launches
    (small kernels are launch-bound from Python otherwise).  Two numbers per shape: L2-warm
    (the same matrix every launch) and HBM-cold (rotating over copies that together exceed
    twice the L2 size), as one JSON line per shape."""
    import torch
    from fortai_b200 import backend_cuda as backend
    # graphs cannot be captured on the legacy default stream: each context owns its stream
    l2_bytes = 126 * 1024 * 1024
    for label, rows, width in decode_shapes():
        if args.only and args.only not in label:
            continue
        nbytes = rows * (width // 32) * 34
        copies = max(2, min(64, (2 * l2_bytes + nbytes - 1) // nbytes + 1))
        result = {"shape": label, "rows": rows, "width": width, "weight_bytes": nbytes,
                  "copies": int(copies)}
        for mode in ("l2_warm", "hbm_cold"):
            ctx = backend.cuda_q8_context_t()
            if not ctx.create(0).is_ok():
                raise SystemExit("context creation failed")
            apply_options(ctx, args.options)
            stream = torch.cuda.ExternalStream(ctx.stream())
            n = 1 if mode == "l2_warm" else int(copies)
            handles = []
            for c in range(n):
                host = make_device_weights(torch, backend, ctx, 0, rows, width, seed=10 + c)
                w = backend.cuda_q8_weights_t()
                if not w.upload(ctx, host, host.size, rows, width).is_ok():
                    raise SystemExit("weight upload failed")
                handles.append(w)
            x = torch.randn(width, device="cuda", dtype=torch.float32)
            out = torch.empty(rows, device="cuda", dtype=torch.float32)
            torch.cuda.synchronize()
            per_graph = 40
            for i in range(4):
                backend.cuda_q8_matvec_device_f32(ctx, handles[i % n], x.data_ptr(), width,
                                                  out.data_ptr(), rows)
            torch.cuda.synchronize()
            assert ctx.capture_begin().is_ok()
            for i in range(per_graph):
                backend.cuda_q8_matvec_device_f32(ctx, handles[i % n], x.data_ptr(), width,
                                                  out.data_ptr(), rows)
            assert ctx.capture_end().is_ok()
            for _ in range(3):
                ctx.graph_launch()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            replays = 25
            a.record(stream)
            for _ in range(replays):
                ctx.graph_launch()
            b.record(stream)
            torch.cuda.synchronize()
            us = a.elapsed_time(b) * 1e3 / (replays * per_graph)
            result[mode + "_us"] = us
            result[mode + "_gbs"] = nbytes / us / 1e3
            for w in handles:
                w.destroy()
            ctx.destroy()
        print(json.dumps(result), flush=True)
    # fused FFN at the three hidden sizes and the 27B-class layer
    for hidden, inner in ((1024, 3840), (2048, 7680), (2560, 9728), (5120, 17408)):
        if args.only and args.only not in "FFN":
            continue
        ctx = backend.cuda_q8_context_t()
        ctx.create(0)
        apply_options(ctx, args.options)
        stream = torch.cuda.ExternalStream(ctx.stream())
        mats = []
        for seed, (r, k) in enumerate(((inner, hidden), (inner, hidden), (hidden, inner))):
            host = make_device_weights(torch, backend, ctx, 0, r, k, seed=30 + seed)
            w = backend.cuda_q8_weights_t()
            w.upload(ctx, host, host.size, r, k)
            mats.append(w)
        x = torch.randn(hidden, device="cuda", dtype=torch.float32)
        out = torch.empty(hidden, device="cuda", dtype=torch.float32)
        torch.cuda.synchronize()
        for _ in range(3):
            backend.cuda_q8_ffn_device(ctx, mats[0], mats[1], mats[2], x.data_ptr(), hidden,
                                       out.data_ptr(), hidden)
        torch.cuda.synchronize()
        launches = ctx.launch_count()
        assert ctx.capture_begin().is_ok()
        per_graph = 20
        for _ in range(per_graph):
            backend.cuda_q8_ffn_device(ctx, mats[0], mats[1], mats[2], x.data_ptr(), hidden,
                                       out.data_ptr(), hidden)
        assert ctx.capture_end().is_ok()
        launches = (ctx.launch_count() - launches) // per_graph
        for _ in range(3):
            ctx.graph_launch()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(25):
            ctx.graph_launch()
        b.record(stream)
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / (25 * per_graph)
        nbytes = 3 * inner * (hidden // 32) * 34
        print(json.dumps({"shape": f"FFN H{hidden} F{inner}", "weight_bytes": nbytes,
                          "us": us, "gbs": nbytes / us / 1e3, "launches_per_call": int(launches),
                          "note": "same matrices every call; L2-warm when they fit"}), flush=True)
        for w in mats:
            w.destroy()
        ctx.destroy()
    sweep_batched(torch, backend, args)
    sweep_batched_ffn(torch, backend, args)
    return 0


def run_ffn(args):
    """The 27B-class FFN (hidden 5120, inner 17408, 284 MB of Q8_0 weights) sharded over the
    ranks: gate/up by rows, down by columns (each rank feeds its own slice of the hidden
    vector), partial outputs all-reduced over NCCL.  One JSON line from rank 0 with the step
    time with and without the collective; an auxiliary number, not the headline metric."""
    import torch
    from fortai_b200 import backend_cuda as backend, sharded
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world,
                                device_id=torch.device("cuda", local_rank))
    torch.cuda.set_device(local_rank)
    stream = torch.cuda.current_stream()
    ctx = backend.cuda_q8_context_t()
    if not ctx.create(local_rank, stream=stream.cuda_stream).is_ok():
        raise SystemExit("context creation failed")
    apply_options(ctx, args.options)
    hidden, inner = 5120, 17408
    gate = make_device_weights(torch, backend, ctx, 0, inner, hidden, seed=40)
    up = make_device_weights(torch, backend, ctx, 0, inner, hidden, seed=41)
    down = make_device_weights(torch, backend, ctx, 0, hidden, inner, seed=42)
    # shards that would fit in L2 are uploaded several times; the steps go round the copies
    shard_bytes = 3 * inner * (hidden // 32) * 34 // world
    copies = 1 if shard_bytes >= 2 * L2_BYTES else int(min(12, 3 * L2_BYTES // shard_bytes + 1))
    ffns = [sharded.ShardedFfn(backend, ctx, gate, up, down, hidden, inner, rank, world)
            for _ in range(copies)]
    turn = [0]

    class Rotating:
        """The next copy's method on every attribute access."""
        def __getattr__(self, name):
            turn[0] = (turn[0] + 1) % copies
            return getattr(ffns[turn[0]], name)
    ffn = Rotating()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(2)
    x = torch.randn(hidden, generator=gen, device="cuda", dtype=torch.float32)
    out = torch.empty(hidden, device="cuda", dtype=torch.float32)

    def local_only():
        one = ffns[turn[0]]
        turn[0] = (turn[0] + 1) % copies
        stat = backend.cuda_q8_ffn_device(ctx, one.gate, one.up, one.down, x.data_ptr(), hidden,
                                          out.data_ptr(), hidden)
        if not stat.is_ok():
            raise RuntimeError(f"FFN failed: {stat}")

    def timed(fn, steps):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(steps):
            fn()
        b.record(stream)
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / steps
        if dist is not None:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    steps = max(10, min(args.steps, 5000))
    with_collective = timed(lambda: ffn.forward(dist, x, out), steps)
    without = timed(local_only, steps)
    # the same with the partial vectors exchanged by the down GEMV itself (no collective call)
    fused_ms, fused_out, keep = None, None, []
    if world > 1:
        try:
            import torch.distributed._symmetric_memory as symm
            device = torch.device("cuda", local_rank)
            pairs = symm.empty(4 * world * hidden, dtype=torch.int32, device=device)
            pairs.zero_()
            pair_handle = symm.rendezvous(pairs, dist.group.WORLD)
            keep += [pairs, pair_handle]
            torch.cuda.synchronize()
            dist.barrier()
            for one in ffns:
                one.attach([int(p) for p in pair_handle.buffer_ptrs])
            fused_out = torch.empty(hidden, device="cuda", dtype=torch.float32)
            fused_ms = timed(lambda: ffn.forward_fused(x, fused_out), steps)
            stat = ctx.synchronize()
            if not stat.is_ok():
                raise RuntimeError(f"fused FFN: {stat}")
        except Exception as error:
            if rank == 0:
                print(f"fused FFN exchange unavailable: {error}", file=sys.stderr)
            fused_ms = None
    # batch 8: eight activations per call through the few-token kernels
    batch = 8
    xb = torch.randn(batch, hidden, generator=gen, device="cuda", dtype=torch.float32)
    outb = torch.empty(batch, hidden, device="cuda", dtype=torch.float32)
    batch_ms = timed(lambda: ffn.forward_batch(dist, xb, outb), steps)

    # ---- what was timed is also checked: the sharded result against the unsharded FFN of
    # the same weights on rank 0's GPU (the hidden vector is cut on block boundaries, so its
    # Q8_0 image is the same; only the fp32 sum over the K shards is ordered differently)
    verified = {}
    ffn.forward(dist, x, out)
    ffn.forward_batch(dist, xb, outb)
    if fused_ms is not None:
        ffn.forward_fused(x, fused_out)
    torch.cuda.synchronize()
    if rank == 0:
        full = [backend.cuda_q8_weights_t() for _ in range(3)]
        for handle, (data, r, k) in zip(full, ((gate, inner, hidden), (up, inner, hidden),
                                               (down, hidden, inner))):
            if not handle.upload(ctx, data, data.size, r, k).is_ok():
                raise SystemExit("full-matrix upload failed")
        ref1 = torch.empty(hidden, device="cuda", dtype=torch.float32)
        refb = torch.empty(batch, hidden, device="cuda", dtype=torch.float32)
        backend.cuda_q8_ffn_device(ctx, full[0], full[1], full[2], x.data_ptr(), hidden,
                                   ref1.data_ptr(), hidden)
        backend.cuda_q8_ffn_batch_device(ctx, full[0], full[1], full[2], xb.data_ptr(), batch,
                                         refb.data_ptr(), refb.numel())
        torch.cuda.synchronize()

        def close(a, b):
            bound = 2e-5 * float(torch.linalg.vector_norm(b.double()))
            return bool(float((a.double() - b.double()).abs().max()) <= bound)
        verified["batch1"] = close(out, ref1)
        verified["batch8"] = all(close(outb[t], refb[t]) for t in range(batch))
        if fused_ms is not None:
            verified["batch1_fused"] = close(fused_out, ref1)
        for handle in full:
            handle.destroy()
    if rank == 0:
        nbytes = 3 * inner * (hidden // 32) * 34
        print(json.dumps({"metric": "q8_0_ffn_weight_bandwidth", "unit": "GB/s", "n_gpus": world,
                          "value": nbytes / with_collective / 1e6,
                          "ms_per_step": with_collective, "ms_per_step_without_all_reduce": without,
                          "ms_per_step_fused_exchange": fused_ms,
                          "batch8_ms_per_step": batch_ms,
                          "batch8_value": nbytes / batch_ms / 1e6,
                          "verified": verified,
                          "scaling": "strong", "steps": steps,
                          "config": {"workload": "FFN hidden 5120 inner 17408, batch 1 and batch 8",
                                     "weight_bytes": nbytes,
                                     "sharding": f"gate/up rows/{world}, down columns/{world}, "
                                                 "fp32 all-reduce of 5120 floats per token",
                                     "cache": f"284 MB of weights per step in total; the steps go "
                                              f"round {copies} copies of a rank's shard"}}),
              flush=True)
    for one in ffns:
        one.destroy()
    ctx.destroy()
    if dist is not None:
        dist.destroy_process_group()
    return 0


def run_decode(args):
    """Whole decode steps through the device pipeline of the model object (embedding, layer
    objects, FFN, lm_head: every call of one token of the reference's fortai_cuda_run), with
    random-init weights of a Qwen3.5-like shape.  Tokens per second, eager launches and CUDA
    graph replay; an auxiliary number, not the headline metric."""
    import torch
    from fortai_b200 import backend_cuda as backend
    from fortai_b200.qwen35_device import qwen35_device_model_t, synthetic_model
    helper = backend.cuda_q8_context_t()
    if not helper.create(0).is_ok():
        raise SystemExit("context creation failed")
    shapes = {"0.8B-like": dict(hidden=1024, inner=3840, layer_count=24),
              "2B-like": dict(hidden=2048, inner=7680, layer_count=24),
              "4B-like": dict(hidden=2560, inner=9728, layer_count=32)}
    for label, shape in shapes.items():
        if args.only and args.only not in label:
            continue
        spec = synthetic_model(
            lambda rows, width, seed, sigma: make_device_weights(torch, backend, helper, 0, rows,
                                                                 width, seed),
            vocabulary=151936, max_context=256, **shape)
        weight_bytes = sum(v.size for v in [spec["output"]] +
                           [l[k] for l in spec["layers"] for k in ("ffn_gate", "ffn_up", "ffn_down")] +
                           [v for l in spec["layers"] for v in l["mixer"].values()
                            if isinstance(v, np.ndarray) and v.dtype == np.int8])
        result = {"shape": label, **shape, "vocabulary": 151936,
                  "weight_bytes_per_token": int(weight_bytes)}
        for mode in ("eager", "graph", "fused_eager", "fused_graph"):
            if args.modes and mode not in args.modes.split(","):
                continue
            model = qwen35_device_model_t()
            stat = model.open(spec, cuda_graph=mode.endswith("graph"),
                              fused=mode.startswith("fused"))
            if not stat.is_ok():
                raise SystemExit(f"model setup failed: {stat}")
            apply_options(model.cuda, args.options)
            token, steps = 1, max(8, min(args.steps, 200))
            for position in range(4):                       # warm-up (and graph capture)
                logits, stat = model.forward(token, position)
                assert stat.is_ok(), stat
                token = int(np.argmax(logits))
            before = model.cuda.launch_count()
            t0 = time.perf_counter()
            for position in range(4, 4 + steps):
                logits, stat = model.forward(token, position)
                token = int(np.argmax(logits))
            seconds = time.perf_counter() - t0
            result[mode + "_tokens_per_s"] = steps / seconds
            result[mode + "_ms_per_token"] = seconds / steps * 1e3
            result[mode + "_weight_gbs"] = weight_bytes * steps / seconds / 1e9
            if mode.endswith("eager"):
                result[mode.replace("eager", "launches_per_token")] = \
                    (model.cuda.launch_count() - before) // steps
            model.close()
        print(json.dumps(result), flush=True)
    helper.destroy()
    return 0


# ------------------------------------------------------------------------------ reference formats
def run_reference_format(args):
    """The reference's own micro-benchmark conventions, so that its scripts and result files
    read both implementations alike.

    `--format reference --rows R --width W --iterations I --warmup N [--seed S] [--device D]`:
    the CLI and JSON line of backend/cuda/fortai_cuda_q8_bench.cu:97-165 (same fixture:
    xorshift32 weights and activation with quants 127 / -127 planted in every block, same
    scalar oracle and gate abs <= 2e-3, rel <= 1e-4, same events-around-the-loop timing of
    the resident matvec, same GiB/s over weight + activation bytes), through this backend's
    fortai_cuda_q8_matvec_device_q8 (the resident matvec, enqueue only).  The fixture generator and the
    scalar oracle are the checker's (oracle/), used here to make inputs and to judge, never
    timed.

    `--format reference-cpu --rows R --width W --iterations I`: the CSV of
    app/fortai_bench_cpu_matvec.f90:37-40 for the Q8_0 CPU matvec (the reference's own C
    arithmetic under the restated OpenMP row loop), backend name `cpu-native-q8`."""
    from oracle import q8_oracle as o
    rows, width = args.rows, args.width
    blocks = width // 32
    if width % 32 or rows < 1 or args.iterations < 1:
        raise SystemExit("rows, width (a multiple of 32) and iterations must be positive")
    if args.format == "reference-cpu":
        o_mod, ref, _ = reference_library()
        weights = o.make_weights(rows, width, seed=0, sigma=0.02)
        x = o.normal(width, seed=1)
        time_cpu_matvec(o_mod, ref, weights, rows, x, 1)
        global WIDTH
        WIDTH = width
        seconds = time_cpu_matvec(o_mod, ref, weights, rows, x, args.iterations)
        checksum = float(np.sum(o.matvec(weights, rows, width, x)[0], dtype=np.float64))
        print("backend,operation,rows,cols,repeats,seconds,matvec_per_second,checksum")
        print(f"cpu-native-q8,matvec,{rows},{width},{args.iterations},{seconds:.8E},"
              f"{args.iterations / seconds:.8E},{checksum:.8E}")
        return 0
    import torch
    from fortai_b200 import backend_cuda as backend
    seed = args.seed & 0xffffffff
    weights = o.fixture_fill_q8(rows, blocks, seed, True)
    activation = o.fixture_fill_q8(1, blocks, seed ^ 0x9e3779b9, False)
    act = activation.view(np.int8)
    for b in range(blocks):
        act[b * 34 + 2] = 127
        act[b * 34 + 3] = -127
    expected = o.fixture_matvec(weights, activation, rows, blocks)
    torch.cuda.set_device(args.device)
    ctx = backend.cuda_q8_context_t()
    if not ctx.create(args.device).is_ok():
        raise SystemExit("context creation failed")
    apply_options(ctx, args.options)
    w = backend.cuda_q8_weights_t()
    if not w.upload(ctx, weights.view(np.int8), weights.size, rows, width).is_ok():
        raise SystemExit("weight upload failed")
    d_act = torch.from_numpy(activation.copy()).cuda(args.device)
    d_out = torch.empty(rows, dtype=torch.float32, device=f"cuda:{args.device}")
    stream = torch.cuda.ExternalStream(ctx.stream())

    def once():
        return backend.cuda_q8_matvec_device_q8(ctx, w, d_act.data_ptr(), d_out.data_ptr(), rows)
    for _ in range(args.warmup):
        once()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(args.iterations):
        once()
    b.record(stream)
    torch.cuda.synchronize()
    elapsed_ms = a.elapsed_time(b)
    if not ctx.synchronize().is_ok():
        raise SystemExit(f"device reported: {ctx.last_error()}")
    out = d_out.cpu().numpy()
    absolute = np.abs(out - expected)
    max_abs = float(absolute.max())
    max_rel = float((absolute / np.maximum(1.0, np.abs(expected))).max())
    correct = max_abs <= 2.0e-3 and max_rel <= 1.0e-4
    tokens_per_second = args.iterations / (elapsed_ms / 1000.0)
    bandwidth = (weights.size + activation.size) * tokens_per_second / (1 << 30)
    props = torch.cuda.get_device_properties(args.device)
    print(json.dumps({
        "implementation": "fortai-b200-q8", "device": args.device, "device_name": props.name,
        "compute_capability": f"{props.major}.{props.minor}", "rows": rows, "width": width,
        "blocks": blocks, "iterations": args.iterations, "warmup": args.warmup,
        "kernel_ms": elapsed_ms / args.iterations, "tokens_per_second": tokens_per_second,
        "bandwidth_gib_per_second": bandwidth, "max_abs_error": max_abs,
        "max_rel_error": max_rel, "correct": bool(correct)}, separators=(",", ":")), flush=True)
    w.destroy()
    ctx.destroy()
    return 0 if correct else 1


def ctx_cleanup(ring, ctx, dist):
    for handle in ring:
        handle.destroy()
    ctx.destroy()
    if dist is not None:
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20000)
    parser.add_argument("--warmup", type=int, default=200)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--exchange", default="auto", choices=["auto", "allgather", "peers", "fused", "pairs"],
                        help="how row shards are reassembled when --gpus > 1")
    parser.add_argument("--rows", type=int, default=ROWS,
                        help="row count of the GEMV (smaller cases are for profiler captures)")
    parser.add_argument("--mmq-only", action="store_true",
                        help="run only the batched prefill product (profiler captures)")
    parser.add_argument("--tokens", type=int, default=MMQ_M, help="token count of the prefill leg")
    parser.add_argument("--mmq-rows", type=int, default=MMQ_N, help="--mmq-only: weight rows")
    parser.add_argument("--mmq-width", type=int, default=MMQ_K, help="--mmq-only: weight width")
    parser.add_argument("--options", default="",
                        help="backend tuning knobs, name=value[,name=value...]")
    parser.add_argument("--only", default="", help="--sweep: only shapes whose label contains this")
    parser.add_argument("--sweep", action="store_true",
                        help="time every named batch-1 shape and the fused FFN (one JSON line each)")
    parser.add_argument("--ffn", action="store_true",
                        help="the 27B-class FFN sharded over --gpus ranks (rows + columns, all-reduce)")
    parser.add_argument("--modes", default="",
                        help="--decode: comma-separated subset of eager,graph,fused_eager,fused_graph")
    parser.add_argument("--decode", action="store_true",
                        help="whole decode steps of a random-init Qwen3.5-like model (tokens/s)")
    parser.add_argument("--kernel-only", action="store_true",
                        help="skip the e2e, prefill and CPU legs (profiler captures)")
    parser.add_argument("--format", default="", choices=["", "reference", "reference-cpu"],
                        help="the reference's own micro-benchmark CLI and output (see "
                             "run_reference_format); takes --rows --width --iterations --warmup "
                             "--seed --device")
    parser.add_argument("--width", type=int, default=WIDTH, help="--format: matrix width")
    parser.add_argument("--iterations", type=int, default=1000, help="--format: timed launches")
    parser.add_argument("--seed", type=lambda t: int(t, 0), default=0x6f727461,
                        help="--format reference: fixture seed")
    parser.add_argument("--device", type=int, default=0, help="--format reference: device index")
    args = parser.parse_args()
    if args.format:
        if args.warmup == 200:
            args.warmup = 100        # the reference's default (fortai_q8_bench_spec.h:107-108)
        return run_reference_format(args)
    set_rows(args.rows)
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.mmq_only:
        return run_mmq_only(args)
    if args.sweep:
        return run_sweep(args)
    if args.decode:
        return run_decode(args)
    if args.ffn:
        return run_ffn(args)
    return run_gpu_arm(args)


if __name__ == "__main__":
    sys.exit(main())
