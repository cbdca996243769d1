#!/usr/bin/env python
"""Benchmark of the Walsh-Hadamard hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  A "step" is one fused C = W.H(X) call over this run's
token batch: K=8192 (Hadamard size), M=28672 rows of W, 16384 tokens in total,
bf16 inputs, fp32 accumulation, bf16 token-major result.  With N GPUs the
tokens are split into N contiguous shards (one process per GPU, W replicated,
no collective on the data path), so total work is fixed: strong scaling.

  value     whole-job TFLOP/s = 2*M*N*K / max-over-ranks device time, inputs
            already resident in HBM
  e2e       same metric with the token shard copied from pinned host memory
            and the result copied back inside the timed region (HostPipeline:
            2048-token chunks on three streams so copies and kernels overlap)
  roofline  tensor-core bound; achieved = 2*M*(N/G)*K / device time of one
            fused call (transform kernel + GEMM kernel, so a lower bound for the
            GEMM kernel alone) against the measured sustained bf16 peak
  fwht      secondary block: standalone transform of (16384, n) bf16, n = 2^8..
            2^15, in place on >= 512 MB of rotating buffers, HBM GB/s against the
            measured copy bandwidth; roofline_fwht is the WORST n >= 512
  fwht_2p30_elements  the reference's benchmark shape: 2^30 elements per n, in place
  sustained the fused call looped for >= 2 s on every rank with the SM clock
            sampled: TFLOP/s, median MHz, TFLOP/s per MHz (scaling at equal clocks)
  host_call_cost  host microseconds per C-ABI call (enqueue only)
  gemv      secondary block: fused GEMV, W 4096 x 4096 bf16, B = 1, 4, 16, GB/s
  c3        secondary block: fused W.H(X) at K=1024, 4096 tokens, M=4096, fp32 and bf16
  k4096     secondary block: fused W.H(X) at K=4096, M=16384, 16384 tokens, bf16, TFLOP/s
  gemv_rows (N > 1 only) small-batch GEMV with the rows of W split over the GPUs and an all-gather of Y
  cpu_baseline  the reference's torch path (explicit Hadamard matmul, then
            matmul; bench/bench.py:44-59 of the reference) on the host cores,
            on a bounded slice of the same tokens

``--impl reference`` times that CPU path alone (rank 0 only).
Inputs are synthetic: seeded N(0,1) tokens times a seeded +-1 diagonal,
W ~ N(0, 1/K); there is no dataset behind this benchmark.
"""
from __future__ import annotations

import argparse
import importlib
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

K_DIM, M_DIM, N_TOKENS = 8192, 28672, 16384
CPU_SAMPLE_TOKENS = 4096  # bounded slice for the CPU legs: ~1-2 s of host work per step
GEMV_ROWS_LIMIT_S = 150   # time limit of the row-sharded GEMV block (it normally takes a few seconds)
METRIC = "fused W.H(X) TFLOP/s (K=8192, M=28672, 16384 tokens, bf16 in / fp32 acc); FWHT HBM GB/s in 'fwht'"


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock/throttle samples taken while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, period_ms: int = 20):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms),
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, reasons = [], None, set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        busy = [v for v in sm if smax and v > 0.35 * smax] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": smax,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------
# CPU reference path (the oracle port of the reference's torch expression)
# ----------------------------------------------------------------------------
def cpu_reference_step(X_tok, W, H):
    """bench/bench.py:55-59 of the reference (t @ H_scaled), then the GEMM."""
    Y = X_tok @ H
    return W @ Y.t()


def cpu_setup(tokens: int):
    import torch

    oracle = importlib.import_module("oracle.fwht_oracle")
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(4)
    d = (2 * torch.randint(0, 2, (K_DIM,), generator=g) - 1).float()
    X = torch.randn(tokens, K_DIM, generator=g) * d
    W = torch.randn(M_DIM, K_DIM, generator=g) / math.sqrt(K_DIM)
    H = torch.from_numpy(oracle.sylvester(K_DIM, dtype="float32")) * oracle.get_scale(K_DIM)
    return X, W, H


def run_reference_arm(args):
    """Times the reference's CPU torch path on a bounded token slice."""
    import torch

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tokens = CPU_SAMPLE_TOKENS
    X, W, H = cpu_setup(tokens)
    for _ in range(max(args.warmup, 1)):
        cpu_reference_step(X, W, H)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_reference_step(X, W, H)
    dt = (time.perf_counter() - t0) / args.steps
    tflops = 2.0 * M_DIM * tokens * K_DIM / dt / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "c5 fused W.H(X): K=8192, M=28672, bf16-valued inputs up-cast to fp32",
                   "tokens_per_step": tokens},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{tokens} of {N_TOKENS} tokens per step; explicit {K_DIM}x{K_DIM} Hadamard "
                                   "matmul then W matmul, fp32 torch on host cores"},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------
# DRAM read + write bytes per element of one transform launch (steady state of the rotating in-place loop below), from
# a one-pass ncu capture of `bench.py --profile-case fwht-sweep` with the caches left alone between launches
# (profiles/fwht_sweep_dram_bytes.md); the algorithmic figure is 4 bytes per element.
FWHT_DRAM_BYTES_PER_ELEMENT = {256: 3.759, 512: 3.857, 1024: 3.925, 2048: 3.958, 4096: 3.968, 8192: 3.984, 16384: 3.988,
                               32768: 3.998}


def time_fwht_sweep(pkg, torch, peaks, rows=16384, reps=10):
    """Standalone transform, (rows, n) bf16, n = 2^8..2^15, IN PLACE on rotating buffers (the reference's loop
    transforms in place too: bench/bench.py:206-238 there).  Per n at least 512 MB of distinct buffers are read and
    written between two uses of the same buffer, four times the 126 MB L2, so neither the reads nor the write-back
    of a launch are served by the cache.  H with scale 1/sqrt(n) is an involution: values stay bounded."""
    out = {}
    lib = pkg._lib.load()
    st = torch.cuda.current_stream().cuda_stream
    for logn in range(8, 16):
        n = 1 << logn
        nbytes = rows * n * 2
        nbuf = max(2, math.ceil((512 << 20) / nbytes))
        bufs = [torch.randn(rows, n, device="cuda", dtype=torch.float32).bfloat16() for _ in range(nbuf)]
        sc = float(n ** -0.5)

        def call(b):
            rc = lib.b200ht_fwht(b.data_ptr(), b.data_ptr(), rows, n, pkg._lib.BF16, sc, st)
            if rc:
                raise RuntimeError(pkg._lib.error_string(rc))

        for b in bufs:
            call(b)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            for b in bufs:
                call(b)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / (reps * nbuf)
        gbs = rows * n * 4 / (ms * 1e-3) / 1e9
        bpe = FWHT_DRAM_BYTES_PER_ELEMENT.get(n)
        out[str(n)] = {"ms": ms, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                       "traffic": None if bpe is None else bpe * rows * n, "buffers": nbuf}
        del bufs
    return out


def time_fwht_reference_shape(pkg, torch, peaks, reps=5):
    """The reference's own benchmark shape for the transform: 2^30 elements per n (rows = 2^30 / n), bf16, in place on
    one 2 GB buffer (bench/bench.py:138, 268-276 there); 4.3 GB of traffic per launch, far beyond L2."""
    out = {}
    lib = pkg._lib.load()
    st = torch.cuda.current_stream().cuda_stream
    total = 1 << 30
    buf = torch.randn(total // 2, device="cuda", dtype=torch.float32).bfloat16()
    buf = torch.cat([buf, buf.flip(0)])
    for logn in range(8, 16):
        n = 1 << logn
        rows = total // n
        sc = float(n ** -0.5)

        def call():
            rc = lib.b200ht_fwht(buf.data_ptr(), buf.data_ptr(), rows, n, pkg._lib.BF16, sc, st)
            if rc:
                raise RuntimeError(pkg._lib.error_string(rc))

        for _ in range(2):
            call()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(2 * reps):     # an even count: the buffer ends as it started
            call()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / (2 * reps)
        gbs = total * 4 / (ms * 1e-3) / 1e9
        out[str(n)] = {"ms": ms, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"]}
    del buf
    return out


def time_gemv(pkg, torch, peaks, reps=20):
    """Small-batch fused GEMV, W 4096 x 4096 bf16, B in {1, 4, 16}.  W (33.5 MB)
    would sit in L2, so 16 copies are rotated (537 MB per rotation)."""
    M = N = 4096
    out = {}
    g = torch.Generator(device="cuda").manual_seed(3)
    Ws = [(torch.randn(M, N, generator=g, device="cuda") / 64).bfloat16() for _ in range(16)]
    lib = pkg._lib.load()
    st = torch.cuda.current_stream().cuda_stream
    for B in (1, 4, 16):
        X = torch.randn(N, B, generator=g, device="cuda").bfloat16()
        Y = torch.empty(M, B, dtype=torch.float32, device="cuda")

        def call(Wt):
            rc = lib.b200ht_fused_gemv(Wt.data_ptr(), X.data_ptr(), Y.data_ptr(), M, N, B, pkg._lib.BF16,
                                       pkg._lib.F32, float(N ** -0.5), st)
            if rc:
                raise RuntimeError(pkg._lib.error_string(rc))

        for Wt in Ws[:3]:
            call(Wt)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            for Wt in Ws:
                call(Wt)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / (reps * len(Ws))
        nbytes = M * N * 2 + N * B * 2 + M * B * 4
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[str(B)] = {"ms": ms, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"]}
    del Ws
    # the same call on a large weight (the C5 matrix, 28672 x 8192 = 470 MB, two rotating copies), B = 4: a long
    # stream instead of a 9 us call
    M, N, B = 28672, 8192, 4
    Ws = [(torch.randn(M, N, generator=g, device="cuda") / 90).bfloat16() for _ in range(2)]
    X = torch.randn(N, B, generator=g, device="cuda").bfloat16()
    Y = torch.empty(M, B, dtype=torch.float32, device="cuda")
    for Wt in Ws * 2:
        rc = lib.b200ht_fused_gemv(Wt.data_ptr(), X.data_ptr(), Y.data_ptr(), M, N, B, pkg._lib.BF16, pkg._lib.F32,
                                   float(N ** -0.5), st)
        if rc:
            raise RuntimeError(pkg._lib.error_string(rc))
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        for Wt in Ws:
            lib.b200ht_fused_gemv(Wt.data_ptr(), X.data_ptr(), Y.data_ptr(), M, N, B, pkg._lib.BF16, pkg._lib.F32,
                                  float(N ** -0.5), st)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / (reps * len(Ws))
    gbs = (M * N * 2 + N * B * 2 + M * B * 4) / (ms * 1e-3) / 1e9
    out["28672x8192_b4"] = {"ms": ms, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"]}
    return out


def time_gemv_rows(pkg, torch, dist, rank, world, reps=20):
    """Row-sharded small-batch GEMV (world > 1): every rank keeps M/world rows of W, computes its rows of Y and sends
    them, tagged with the number of the call, into a slot array on every other rank through peer-mapped pointers; the
    same kernel collects the other ranks' rows (RowShardedGemv: no collective, no fence, no flag).  Timed per call,
    launched from the host and replayed from a CUDA graph, 8 rotating copies of the W shard, B = 4; W 4096 x 4096 (the
    C4 shape) and 28672 x 8192 (the C5 weight).  `parity`: rank 0 compares the assembled Y of one call with the
    single-GPU call on the full W (same seeded data on every rank).  `nccl_ms` is the same split with an NCCL
    all-gather of Y after a plain GEMV, for comparison."""
    out = {}
    for M, N in ((4096, 4096), (28672, 8192)):
        g = torch.Generator(device="cuda").manual_seed(6)       # same W and X on every rank
        W_full = (torch.randn(M, N, generator=g, device="cuda") / math.sqrt(N)).bfloat16()
        X = torch.randn(N, 4, generator=g, device="cuda").bfloat16()
        a, b = pkg.row_range(M, rank, world)
        Ws = [W_full[a:b].clone() if i == 0 else (torch.randn(b - a, N, generator=g, device="cuda") / math.sqrt(N)).bfloat16()
              for i in range(8)]
        ops = [pkg.RowShardedGemv(Wt, M, 4) for Wt in Ws]
        got = ops[0](X).clone()
        torch.cuda.synchronize()
        ref = pkg.fused_ht_gemv(W_full, X)
        err = float((got - ref).norm() / ref.norm())
        parity = torch.tensor([1 if err < 1e-5 else 0], device="cuda")
        dist.all_reduce(parity, op=dist.ReduceOp.MIN)
        del W_full

        def timed(call):
            for i in range(3):
                call(i)
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            h0 = time.perf_counter()
            e0.record()
            for _ in range(reps):
                for i in range(len(Ws)):
                    call(i)
            e1.record()
            h1 = time.perf_counter()       # the host has enqueued everything; the device may still be running
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / (reps * len(Ws)), (h1 - h0) * 1e3 / (reps * len(Ws))], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t[0].item()), float(t[1].item())

        ms, host_ms = timed(lambda i: ops[i](X))
        nccl_ms, _ = timed(lambda i: pkg.gather_rows(pkg.fused_ht_gemv(Ws[i], X), M))
        # The same calls replayed from a CUDA graph (two rotations of the 8 shards per graph: an even number of calls
        # per op, as its two result buffers require): the hosts' launch pace and jitter drop out of the loop.
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(2):
                    for op in ops:
                        op(X)
            graph.replay()
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            for _ in range(reps):
                graph.replay()
            e1.record(side)
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / (reps * 2 * len(ops))], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            graph_ms = float(t.item())
        got2 = ops[0](X).clone()                       # an ordinary call behind the replays still gives the same rows
        torch.cuda.synchronize()
        err2 = float((got2 - ref).norm() / ref.norm())
        parity2 = torch.tensor([1 if err2 < 1e-5 else 0], device="cuda")
        dist.all_reduce(parity2, op=dist.ReduceOp.MIN)
        parity = torch.minimum(parity, parity2)
        del graph
        status = pkg.device_status()
        out[f"{M}x{N}"] = {"ms": ms, "gbs_all_gpus": M * N * 2 / (ms * 1e-3) / 1e9, "rows_per_gpu": b - a,
                           "parity": bool(parity.item()) and status == 0, "rel_err_vs_one_gpu": err,
                           "graph_replay_ms": graph_ms, "gbs_all_gpus_graph": M * N * 2 / (graph_ms * 1e-3) / 1e9,
                           "nccl_all_gather_ms": nccl_ms, "host_enqueue_ms": host_ms,
                           "exchange": "peer stores of (value, call number) slots, collected by the kernel"}
        for op in ops:
            op.close()
        del Ws, ops
    return out


def time_c3(pkg, torch, peaks, reps=10):
    """Fused W.H(X) at K=1024, 4096 tokens, M=4096: fp32 (exact FFMA path), fp32 through the tensor cores
    (three bf16 terms per operand) and bf16 (tcgen05 path)."""
    K, N, M = 1024, 4096, 4096
    g = torch.Generator(device="cuda").manual_seed(2)
    out = {}
    for name, dt in (("fp32", torch.float32), ("fp32_tc", torch.float32), ("bf16", torch.bfloat16)):
        # 4 rotating input sets (X, W): 2 x 16/8 MB each, C 64 MB fp32 -> every call misses L2 for C at least
        sets = [(torch.randn(N, K, generator=g, device="cuda").to(dt), torch.randn(M, K, generator=g, device="cuda").to(dt))
                for _ in range(4)]
        C = torch.empty(M, N, dtype=torch.float32, device="cuda")
        # fp32: the minimal workspace keeps the exact FFMA kernel, the larger one selects the split-bf16 tensor-core path
        ws = torch.empty(pkg.fused_gemm_workspace_bytes(M, N, K, dt, exact=(name == "fp32")), dtype=torch.uint8,
                         device="cuda")
        lib = pkg._lib.load()
        st = torch.cuda.current_stream().cuda_stream
        code = pkg._lib.F32 if dt == torch.float32 else pkg._lib.BF16

        def call(X, W):   # straight through the C ABI: at 25-800 us per call the Python wrapper would show
            rc = lib.b200ht_fused_gemm(X.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K, code, pkg._lib.F32,
                                       pkg._lib.OUT_MN, float(K ** -0.5), ws.data_ptr(), ws.numel(), st)
            if rc:
                raise RuntimeError(pkg._lib.error_string(rc))

        for X, W in sets[:3]:
            call(X, W)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            for X, W in sets:
                call(X, W)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / (reps * len(sets))
        tf = 2.0 * M * N * K / (ms * 1e-3) / 1e12
        peak = {"fp32": 74.0, "fp32_tc": peaks["bf16_tflops"] / 6.0, "bf16": peaks["bf16_tflops"]}[name]
        src = {"fp32": "nominal fp32 FFMA 148*128*2*1.965e9",
               "fp32_tc": "measured cuBLAS bf16 burst / 6 (six bf16 products per fp32 product)",
               "bf16": "measured cuBLAS bf16 burst"}[name]
        out[name] = {"ms": ms, "tflops": tf, "peak_tflops": peak, "frac": tf / peak, "peak_source": src}
    return out


def time_k4096(pkg, torch, peaks, reps=5):
    """Fused W.H(X) at Hadamard size 4096 (bf16 in, fp32 accumulate, bf16 token-major out): M=16384, 16384 tokens.
    W (134 MB) plus the tokens (134 MB) and the output (537 MB) exceed L2."""
    K, N, M = 4096, 16384, 16384
    g = torch.Generator(device="cuda").manual_seed(5)
    X = torch.randn(N, K, generator=g, device="cuda").bfloat16()
    W = (torch.randn(M, K, generator=g, device="cuda") / math.sqrt(K)).bfloat16()
    C = torch.empty(N, M, dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(pkg.fused_gemm_workspace_bytes(M, N, K, torch.bfloat16), dtype=torch.uint8, device="cuda")
    lib = pkg._lib.load()
    st = torch.cuda.current_stream().cuda_stream

    def call():
        rc = lib.b200ht_fused_gemm(X.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K, pkg._lib.BF16, pkg._lib.BF16,
                                   pkg._lib.OUT_NM, float(K ** -0.5), ws.data_ptr(), ws.numel(), st)
        if rc:
            raise RuntimeError(pkg._lib.error_string(rc))

    for _ in range(3):
        call()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        call()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    tf = 2.0 * M * N * K / (ms * 1e-3) / 1e12
    return {"shape": {"K": K, "M": M, "tokens": N}, "ms": ms, "tflops": tf,
            "frac_of_sustained": tf / peaks["bf16_tflops_sustained"], "frac_of_burst": tf / peaks["bf16_tflops"],
            "frac_of_nominal_2250": tf / 2250.0}


def time_sustained(torch, dist, step, flops_rank, rank, local_rank, world, seconds=2.0):
    """The fused call back to back for at least `seconds` on every rank at once, with this rank's SM clock sampled
    meanwhile: TFLOP/s, median SM MHz and TFLOP/s per MHz.  A burst of a few milliseconds runs at the boost clock,
    a long loop at whatever the 1 kW power cap allows, so scaling across N is read here at equal clock state."""
    for _ in range(2):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    step()
    e1.record()
    torch.cuda.synchronize()
    calls = max(4, int(seconds * 1e3 / max(e0.elapsed_time(e1), 1e-3)) + 1)
    if world > 1:
        c = torch.tensor([calls], device="cuda")
        dist.all_reduce(c, op=dist.ReduceOp.MAX)
        calls = int(c.item())
        dist.barrier()
    sampler = ClockSampler(local_rank, period_ms=50)
    sampler.start()
    e0.record()
    for _ in range(calls):
        step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    mine = torch.tensor([ms, flops_rank * calls / (ms * 1e-3) / 1e12, float(clocks["sm_mhz"] or 0.0)], device="cuda")
    if world > 1:
        allr = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
    else:
        allr = [mine]
    per_rank = [[float(v) for v in t.tolist()] for t in allr]
    t_max = max(r[0] for r in per_rank)
    tf = flops_rank * calls * world / (t_max * 1e-3) / 1e12
    mhz = [r[2] for r in per_rank]
    med = statistics.median(mhz) if mhz else 0.0
    return {"seconds": t_max * 1e-3, "calls": calls, "tflops": tf, "tflops_per_gpu": [r[1] for r in per_rank],
            "sm_mhz_per_gpu": mhz, "sm_mhz_median": med, "tflops_per_gpu_per_mhz": (tf / world / med) if med else None,
            "reasons": clocks["reasons"]}


def time_copy_floor(torch, dist, pipe, Xh, Ch, world, steps=3):
    """The host<->device copies of one end-to-end step alone: the same chunks on the same streams as HostPipeline,
    one cudaMemcpyAsync per chunk and direction, no kernels, on all ranks at once.  An end-to-end step cannot be
    faster than this; max over ranks, in ms."""
    n = int(Xh.shape[0])

    def copies():
        cur = torch.cuda.current_stream()
        for st in pipe.streams:
            st.wait_stream(cur)
        for i, t0 in enumerate(range(0, n, pipe.chunk)):
            t1 = min(t0 + pipe.chunk, n)
            k = i % len(pipe.streams)
            with torch.cuda.stream(pipe.streams[k]):
                pipe.x[k][: t1 - t0].copy_(Xh[t0:t1], non_blocking=True)
                Ch[t0:t1].copy_(pipe.c[k][: t1 - t0], non_blocking=True)
        for st in pipe.streams:
            cur.wait_stream(st)

    copies()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        copies()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_host_call_cost(pkg, torch, calls=200):
    """Host time of one C-ABI call (CPU clock around a burst of calls that are only enqueued, no synchronisation in
    between; the burst is shorter than the launch queue).  The trivial transform (one row of two elements) is the
    floor of a launch through the library; the GEMV adds a tensor map and a shared-memory attribute, which come from
    per-thread / per-device caches after the first call."""
    lib = pkg._lib.load()
    st = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(8)
    tiny = torch.zeros(8, dtype=torch.bfloat16, device="cuda")
    x = torch.randn(64, 1024, generator=g, device="cuda").bfloat16()
    W = (torch.randn(256, 4096, generator=g, device="cuda") / 64).bfloat16()
    X = torch.randn(4096, 4, generator=g, device="cuda").bfloat16()
    Y = torch.empty(256, 4, dtype=torch.float32, device="cuda")
    X3 = torch.randn(256, 1024, generator=g, device="cuda").bfloat16()
    W3 = torch.randn(256, 1024, generator=g, device="cuda").bfloat16()
    C3 = torch.empty(256, 256, dtype=torch.float32, device="cuda")
    ws = torch.empty(pkg.fused_gemm_workspace_bytes(256, 256, 1024, torch.bfloat16), dtype=torch.uint8, device="cuda")
    BF16, F32 = pkg._lib.BF16, pkg._lib.F32
    cases = {
        "ctypes_call_of_a_no_op": lambda: lib.b200ht_launch_count(),   # what the Python binding itself costs
        "fwht_trivial": lambda: lib.b200ht_fwht(tiny.data_ptr(), tiny.data_ptr(), 1, 2, BF16, 1.0, st),
        "fwht_64x1024": lambda: lib.b200ht_fwht(x.data_ptr(), x.data_ptr(), 64, 1024, BF16, 1.0 / 32, st),
        "gemv_256x4096_b4": lambda: lib.b200ht_fused_gemv(W.data_ptr(), X.data_ptr(), Y.data_ptr(), 256, 4096, 4, BF16,
                                                          F32, 1.0 / 64, st),
        "gemm_256x256x1024": lambda: lib.b200ht_fused_gemm(X3.data_ptr(), W3.data_ptr(), C3.data_ptr(), 256, 256, 1024,
                                                           BF16, F32, pkg._lib.OUT_MN, 1.0 / 32, ws.data_ptr(),
                                                           ws.numel(), st),
    }
    out = {}
    for name, fn in cases.items():
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        best = 1e30
        for _ in range(3):
            t0 = time.perf_counter()
            for _ in range(calls):
                fn()
            best = min(best, time.perf_counter() - t0)
            torch.cuda.synchronize()
        out[name] = {"host_us_per_call": best / calls * 1e6}
    return out


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    pkg = importlib.import_module("6s894_project_2025_b200")
    peaks = load_peaks()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    a, b = pkg.token_range(N_TOKENS, rank, world)
    n_local = b - a
    g = torch.Generator(device="cuda").manual_seed(4)
    d = (2 * torch.randint(0, 2, (K_DIM,), generator=g, device="cuda") - 1).float()
    W = (torch.randn(M_DIM, K_DIM, generator=g, device="cuda") / math.sqrt(K_DIM)).bfloat16()
    g.manual_seed(1000 + rank)
    X = (torch.randn(n_local, K_DIM, generator=g, device="cuda") * d).bfloat16()
    C = torch.empty(n_local, M_DIM, dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(pkg.fused_gemm_workspace_bytes(M_DIM, n_local, K_DIM, torch.bfloat16), dtype=torch.uint8,
                     device="cuda")

    def step():
        pkg.fused_ht_gemm(X, W, out=C, out_layout="nm", out_dtype=torch.bfloat16, workspace=ws)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    launches0 = int(pkg._lib.load().b200ht_launch_count())
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    gpu_launches = int(pkg._lib.load().b200ht_launch_count()) - launches0   # kernels of this rank in the timed region
    clocks = sampler.stop() if rank == 0 else None
    ms_local = e0.elapsed_time(e1) / args.steps
    status = pkg.device_status()
    if status != 0:
        raise RuntimeError(f"device status word = {status} after the timed region")
    t = torch.tensor([ms_local], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    flops_total = 2.0 * M_DIM * N_TOKENS * K_DIM
    value = flops_total / (ms * 1e-3) / 1e12

    # end to end: pinned host tokens in, result back to pinned host memory
    Xh = torch.empty(X.shape, dtype=X.dtype, pin_memory=True).copy_(X)
    Ch = torch.empty(C.shape, dtype=C.dtype, pin_memory=True)

    # chunks of 2048 tokens, but at least eight chunks per rank so that copy-in, compute and copy-out overlap
    pipe = pkg.HostPipeline(W, n_local, chunk_tokens=max(256, min(2048, n_local // 8)), n_streams=3,
                            out_dtype=torch.bfloat16)

    def e2e_step():
        pipe(Xh, Ch)   # per chunk: copy in, transform + GEMM, copy out, on three streams

    e2e_steps = max(2, min(args.steps, 5))
    e2e_step()
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1) / e2e_steps], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    e2e_val = flops_total / (e2e_ms * 1e-3) / 1e12
    copy_floor_ms = time_copy_floor(torch, dist, pipe, Xh, Ch, world)
    del pipe, Xh, Ch

    sustained = time_sustained(torch, dist, step, 2.0 * M_DIM * n_local * K_DIM, rank, local_rank, world)
    fwht = time_fwht_sweep(pkg, torch, peaks)
    fwht_ref_shape = time_fwht_reference_shape(pkg, torch, peaks)
    host_cost = time_host_call_cost(pkg, torch) if rank == 0 else None
    gemv = time_gemv(pkg, torch, peaks)
    c3 = time_c3(pkg, torch, peaks)
    k4096 = time_k4096(pkg, torch, peaks)
    if world > 1:
        agg = torch.tensor([fwht[k]["gbs"] for k in sorted(fwht, key=int)], device="cuda")
        dist.all_reduce(agg, op=dist.ReduceOp.SUM)
        for k, v in zip(sorted(fwht, key=int), agg.tolist()):
            fwht[k]["gbs_all_gpus"] = v

    def emit(gemv_rows):
        if rank != 0:
            return
        cpu = None
        if world == 1:
            import torch as _t
            tokens = CPU_SAMPLE_TOKENS
            Xc, Wc, Hc = cpu_setup(tokens)
            cpu_reference_step(Xc, Wc, Hc)
            best = 1e30
            for _ in range(3):
                t0 = time.perf_counter()
                cpu_reference_step(Xc, Wc, Hc)
                best = min(best, time.perf_counter() - t0)
            cpu = {"value": 2.0 * M_DIM * tokens * K_DIM / best / 1e12, "unit": "TFLOP/s",
                   "cores": _t.get_num_threads(), "kind": "port",
                   "sample": f"{tokens} of {N_TOKENS} tokens, min of 3; explicit {K_DIM}x{K_DIM} Hadamard matmul "
                             "then W matmul, fp32 torch on host cores"}
        achieved = 2.0 * M_DIM * n_local * K_DIM / (ms_local * 1e-3) / 1e12
        peak = peaks["bf16_tflops_sustained"]
        # the transform's roofline line is its WORST size from n = 512 up (n = 256 moves 8 MB per launch and is
        # bound by launch latency, which the per-n table shows)
        worst_n, worst_fwht = min(((k, v) for k, v in fwht.items() if int(k) >= 512), key=lambda kv: kv[1]["gbs"])
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "c5 fused W.H(X): K=8192, M=28672, 16384 tokens split by token columns",
                       "tokens_per_gpu": n_local, "parallelism": f"token-shard x{world}, W replicated",
                       "l2": "inputs (W 470 MB + tokens) exceed the 126 MB L2; fwht sweep runs in place on >= 512 MB of rotating buffers",
                       "out": "bf16 token-major"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak,
                         # DRAM read + write bytes of the contraction kernels of one full-size fused call on one GPU
                         # (8 token chunks: 8 launches with 256-row tiles + 8 tail launches), from a one-pass ncu capture
                         # of `bench.py --profile-case gemm-full` with the caches left alone between launches
                         # (profiles/gemm_tc_kernel_fused_k8192.md); scaled by the token share of a rank
                         "traffic": 5.509e9 * n_local / N_TOKENS, "traffic_unit": "B/fused call",
                         "algorithmic_bytes": (M_DIM * K_DIM * 2 + n_local * K_DIM * 2 + n_local * M_DIM * 2),
                         "peak_source": f"{peaks['source']} sustained cuBLAS bf16 (burst {peaks['bf16_tflops']})",
                         "frac_of_burst": achieved / peaks["bf16_tflops"]},
            "roofline_fwht": {"bound": "hbm", "achieved": worst_fwht["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                              "frac": worst_fwht["gbs"] / peaks["hbm_gbs"], "traffic": worst_fwht["traffic"],
                              "n": int(worst_n), "rule": "minimum over n >= 512 of the 16384-row sweep",
                              "peak_source": f"{peaks['source']} copy bandwidth"},
            "fwht": fwht,
            "fwht_2p30_elements": fwht_ref_shape,
            "sustained": sustained,
            "host_call_cost": host_cost,
            "gemv": gemv,
            "c3": c3,
            "k4096": k4096,
            "gemv_rows": gemv_rows,
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_val, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": X.numel() * 2 * world, "d2h_bytes_per_step": C.numel() * 2 * world,
                    # the same copies without any kernel (max over ranks): the PCIe / host-memory floor of a step
                    "copy_floor_ms": copy_floor_ms, "frac_of_copy_floor": copy_floor_ms / e2e_ms},
            "gpu_launches": gpu_launches,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)

    # The row-sharded GEMV block runs last and under a time limit: it is the only part of the run in which ranks wait
    # for one another outside a collective of the headline path, and a secondary block must not take the line down
    # with it.  If it fails, or does not return in time, the line is printed without its figures.
    gemv_rows = None
    if world > 1:
        def give_up():
            emit({"error": f"no result within {GEMV_ROWS_LIMIT_S} s"})
            os._exit(0)

        timer = threading.Timer(GEMV_ROWS_LIMIT_S, give_up)
        timer.daemon = True
        timer.start()
        try:
            gemv_rows = time_gemv_rows(pkg, torch, dist, rank, world)
        except Exception as e:   # noqa: BLE001
            gemv_rows = {"error": f"{type(e).__name__}: {e}"[:300]}
        timer.cancel()
    emit(gemv_rows)
    if world > 1:
        dist.destroy_process_group()


def run_profile_case(case: str):
    """A handful of launches on a reduced shape (inputs larger than the 126 MB L2, a
    few hundred MB on the device) so that an ncu capture of the kernel ends quickly."""
    import torch

    pkg = importlib.import_module("6s894_project_2025_b200")
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(0)
    if case in ("gemm", "gemm-full"):
        # reduced: K=8192, M=8192, 4096 tokens (W 134 MB, X 67 MB, C 67 MB); full: the bench shape (1.95 GB on the
        # device), meant for a one-pass capture of DRAM bytes only
        K, M, N = (8192, 8192, 4096) if case == "gemm" else (K_DIM, M_DIM, N_TOKENS)
        W = (torch.randn(M, K, generator=g, device="cuda") / math.sqrt(K)).bfloat16()
        X = torch.randn(N, K, generator=g, device="cuda").bfloat16()
        for _ in range(3):
            C = pkg.fused_ht_gemm(X, W, out_layout="nm", out_dtype=torch.bfloat16)
        # the fourth call is bracketed for the profiler: `ncu --profile-from-start off` then captures the kernels of
        # exactly one fused call (transform and contraction launches alike), however many launches a call makes
        torch.cuda.synchronize()
        torch.cuda.cudart().cudaProfilerStart()
        C = pkg.fused_ht_gemm(X, W, out_layout="nm", out_dtype=torch.bfloat16)
        torch.cuda.synchronize()
        torch.cuda.cudart().cudaProfilerStop()
        print("gemm case done", float(C.float().abs().mean()))
    elif case == "c3":      # fused W.H(X) at K=1024, 4096 tokens, M=4096, bf16 in, fp32 M x N out; rotating inputs
        K, M, N = 1024, 4096, 4096
        sets = [(torch.randn(N, K, generator=g, device="cuda").bfloat16(), torch.randn(M, K, generator=g, device="cuda").bfloat16())
                for _ in range(4)]
        for X, W in sets:
            C = pkg.fused_ht_gemm(X, W)
        print("c3 case done", float(C.abs().mean()))
    elif case == "fwht":    # standalone transform, n = 1024, 4096, 8192 and 32768 (bf16), 134-268 MB, distinct buffers
        for n, rows in ((1024, 65536), (4096, 16384), (8192, 16384), (32768, 4096)):
            bufs = [torch.randn(rows, n, generator=g, device="cuda").bfloat16() for _ in range(3)]
            for b in bufs:
                y = pkg.hadamard_transform(b)
            print("fwht case", n, float(y.float().abs().mean()))
    elif case == "fwht-sweep":
        # the bench's transform loop (16384 rows, n = 2^8..2^15, in place on >= 512 MB of rotating buffers), two
        # rotations per n: a one-pass capture of the DRAM counters with `--cache-control none` sees the steady state
        # of the second rotation, in which every launch's reads miss L2 and as many dirty lines are written back as
        # the launch produces
        lib = pkg._lib.load()
        st = torch.cuda.current_stream().cuda_stream
        rows = 16384
        for logn in range(8, 16):
            n = 1 << logn
            nbuf = max(2, math.ceil((512 << 20) / (rows * n * 2)))
            bufs = [torch.randn(rows, n, generator=g, device="cuda").bfloat16() for _ in range(nbuf)]
            for _ in range(2):
                for b in bufs:
                    rc = lib.b200ht_fwht(b.data_ptr(), b.data_ptr(), rows, n, pkg._lib.BF16, float(n ** -0.5), st)
                    assert rc == 0
            torch.cuda.synchronize()
            print("fwht-sweep case", n, nbuf, float(bufs[0].float().abs().mean()))
            del bufs
    elif case == "gemv-large":   # fused GEMV on the C5 weight, 28672 x 8192 bf16 (470 MB), B = 4, two rotating copies
        Ws = [(torch.randn(28672, 8192, generator=g, device="cuda") / 90).bfloat16() for _ in range(2)]
        X = torch.randn(8192, 4, generator=g, device="cuda").bfloat16()
        for _ in range(3):
            for W in Ws:
                Y = pkg.fused_ht_gemv(W, X)
        print("gemv-large case", float(Y.abs().mean()))
    else:                   # fused GEMV, W 4096 x 4096 bf16, B = 16 and 1, distinct W buffers
        Ws = [(torch.randn(4096, 4096, generator=g, device="cuda") / 64).bfloat16() for _ in range(6)]
        for B in (16, 1):
            X = torch.randn(4096, B, generator=g, device="cuda").bfloat16()
            for W in Ws:
                Y = pkg.fused_ht_gemv(W, X)
            print("gemv case", B, float(Y.abs().mean()))
    torch.cuda.synchronize()


_ORDERS_CHILD = r"""
import importlib, json, math, sys, torch
sys.path.insert(0, %r)
pkg = importlib.import_module("6s894_project_2025_b200")
lib = pkg._lib.load()
st = torch.cuda.current_stream().cuda_stream
g = torch.Generator(device="cuda").manual_seed(4)
def run(K, M, N, reps, layout, odt, ocode):
    W = (torch.randn(M, K, generator=g, device="cuda") / math.sqrt(K)).bfloat16()
    X = torch.randn(N, K, generator=g, device="cuda").bfloat16()
    C = torch.empty((N, M) if layout == 1 else (M, N), dtype=odt, device="cuda")
    ws = torch.empty(pkg.fused_gemm_workspace_bytes(M, N, K, torch.bfloat16), dtype=torch.uint8, device="cuda")
    def call():
        rc = lib.b200ht_fused_gemm(X.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K, 1, ocode, layout, float(K ** -0.5),
                                   ws.data_ptr(), ws.numel(), st)
        assert rc == 0
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    tot = 0.0
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); call(); e1.record(); torch.cuda.synchronize()
        tot += e0.elapsed_time(e1)
    return tot / reps
print(json.dumps({"c5_ms": run(8192, 28672, 16384, 8, 1, torch.bfloat16, 1),
                  "c5_shard_2048_tokens_ms": run(8192, 28672, 2048, 10, 1, torch.bfloat16, 1),
                  "k4096_ms": run(4096, 16384, 16384, 8, 1, torch.bfloat16, 1),
                  "c3_ms": run(1024, 4096, 4096, 20, 0, torch.float32, 2)}))
"""


def run_compare_orders():
    """``--compare orders``: the fused GEMM's tile order and chunking knobs (read once per process, hence one child
    process per setting, two rounds), mean ms of single calls on four shapes.  One JSON line."""
    settings = {
        "default (token groups of 8, 32 MB chunks)": {},
        "row groups of 16, one chunk": {"B200HT_GEMM_ORDER": "0", "B200HT_GEMM_GROUP": "16", "B200HT_GEMM_CHUNK_MB": "0"},
        "row groups of 8, one chunk": {"B200HT_GEMM_ORDER": "0", "B200HT_GEMM_GROUP": "8", "B200HT_GEMM_CHUNK_MB": "0"},
        "token groups of 8, one chunk": {"B200HT_GEMM_CHUNK_MB": "0"},
        "token groups of 12, 48 MB chunks": {"B200HT_GEMM_GROUP": "12", "B200HT_GEMM_CHUNK_MB": "48"},
        "128-row tiles only": {"B200HT_GEMM_MT": "1"},
    }
    out = {k: [] for k in settings}
    for _ in range(2):
        for name, env in settings.items():
            r = subprocess.run([sys.executable, "-c", _ORDERS_CHILD % str(ROOT)], capture_output=True, text=True,
                               env=dict(os.environ, **env))
            try:
                out[name].append(json.loads(r.stdout.strip().splitlines()[-1]))
            except (IndexError, ValueError):
                out[name].append({"error": (r.stdout + r.stderr)[-300:]})
    print(json.dumps({"compare": "orders", "ms_per_call": out}))


def run_compare(which: str):
    """Same-box library comparators (``--compare cublas``), one JSON line.  Nothing here is on the product path: the
    library kernels are timed beside this repository's calls on the same buffers.
      c5    the bench shape in alternating 10-call blocks: b200ht_fused_gemm | torch.matmul (cuBLAS) on already
            transformed tokens | b200ht_fwht followed by that matmul
      gemv  W 4096 x 4096 bf16 on 16 rotating copies, B = 1, 4, 16: b200ht_fused_gemv | F.linear (cuBLAS, no
            transform) | torch.sum(W) | a copy of W
    """
    import torch
    import torch.nn.functional as F

    if which == "orders":
        return run_compare_orders()
    assert which == "cublas"
    pkg = importlib.import_module("6s894_project_2025_b200")
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(4)
    ev = lambda: torch.cuda.Event(enable_timing=True)   # noqa: E731

    def timed(fn, reps):
        e0, e1 = ev(), ev()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    W = (torch.randn(M_DIM, K_DIM, generator=g, device="cuda") / math.sqrt(K_DIM)).bfloat16()
    X = torch.randn(N_TOKENS, K_DIM, generator=g, device="cuda").bfloat16()
    Y = pkg.hadamard_transform(X)
    C = torch.empty(N_TOKENS, M_DIM, dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(pkg.fused_gemm_workspace_bytes(M_DIM, N_TOKENS, K_DIM, torch.bfloat16), dtype=torch.uint8,
                     device="cuda")
    legs = {
        "b200ht_fused_gemm": lambda: pkg.fused_ht_gemm(X, W, out=C, out_layout="nm", out_dtype=torch.bfloat16,
                                                       workspace=ws),
        "cublas_gemm_only": lambda: torch.matmul(Y, W.t(), out=C),
        "b200ht_fwht_then_cublas": lambda: torch.matmul(pkg.hadamard_transform(X), W.t(), out=C),
    }
    for fn in legs.values():
        for _ in range(3):
            fn()
    torch.cuda.synchronize()
    c5 = {k: [] for k in legs}
    for _ in range(4):
        for k, fn in legs.items():
            c5[k].append(timed(fn, 10))
    del W, X, Y, C, ws

    M = N = 4096
    Ws = [(torch.randn(M, N, generator=g, device="cuda") / 64).bfloat16() for _ in range(16)]
    dst = torch.empty_like(Ws[0])
    gemv = {}
    for B in (1, 4, 16):
        Xc = torch.randn(N, B, generator=g, device="cuda").bfloat16()
        Xr = Xc.t().contiguous()
        out = torch.empty(M, B, dtype=torch.float32, device="cuda")
        state = {"i": 0}

        def nxt():
            state["i"] = (state["i"] + 1) % len(Ws)
            return Ws[state["i"]]

        row = {
            "b200ht_fused_gemv": lambda: pkg.fused_ht_gemv(nxt(), Xc, out=out),
            "cublas_linear_no_transform": lambda: F.linear(Xr, nxt()),
            "torch_sum_W": lambda: torch.sum(nxt()),
            "copy_W": lambda: dst.copy_(nxt()),
        }
        res = {}
        for k, fn in row.items():
            for _ in range(5):
                fn()
            torch.cuda.synchronize()
            res[k] = timed(fn, 160) * 1e3
        gemv[str(B)] = res
    print(json.dumps({"compare": "cublas", "c5_ms_per_call_blocks_of_10": c5, "gemv_us_per_call": gemv,
                      "note": "device time by CUDA events; the GEMV rows include the Python call of each leg"}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--profile-case", default=None, choices=["gemm", "gemm-full", "fwht", "fwht-sweep", "gemv", "gemv-large", "c3"],
                    help="run a few launches of ONE kernel on a reduced shape and exit (for ncu captures)")
    ap.add_argument("--compare", default=None, choices=["cublas", "orders"],
                    help="time library comparators beside this repository's calls on one GPU and exit")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args.profile_case)
    elif args.compare:
        run_compare(args.compare)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
