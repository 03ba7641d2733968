#!/usr/bin/env python3
"""Benchmark of the quantized-weight hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Headline workload (config.workload = "c1_q4k_decode_gemv"): the decode-shape
Q4_K quantized_matmul of the reference's first benchmark cell - W [4096, 4096]
in q4_k wire bytes, activations fp16 [M, 4096] (M = 1 unless --m is given). One
STEP is one pass of that matmul over a stack of `layers` DISTINCT weight
matrices (64 x 9.4 MB = 604 MB, several times the 126 MB L2), so every launch
streams its weights cold from HBM - the way the reference measures
("working set streamed far past the SLC", src/kquant_matmul.cpp:1436-1437).
metric = weight wire bytes processed per second (GB/s), the reference's own
definition (benchmarks/bench_qmm_bm128_ab.py:18-19).

value   device-resident: inputs already in HBM, the step is one CUDA-graph
        replay of the `layers` launches; CUDA events on the launching stream.
e2e     the same step through the public op with HOST buffers: pinned-host x
        -> device copy, the launches, device -> pinned-host copy of the outputs,
        all inside the timed region.
N > 1   weak scaling: every rank holds its own [4096, 4096] column shard (rows
        r*4096 .. (r+1)*4096 of a [N*4096, 4096] matrix) per layer and the
        [layers, M, 4096] output shards are all-gathered over NCCL each step.
--impl reference   times the reference's own CPU implementation of the path
        (oracle/_ref/libkqref.so = its kquant_qmm_cpu compiled in place; the
        oracle's C port if that library is absent) on a bounded sample of the
        same workload with all host threads.

Weights are synthetic valid wire bytes (mlx_kquant_b200/synth.py); activations
are seeded N(0, 1).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

N_ROWS = 4096
K_COLS = 4096
CODEC = "q4_k"
ROW_BYTES = K_COLS // 256 * 144
MATRIX_BYTES = N_ROWS * ROW_BYTES  # 9 437 184
# the kernel that runs this workload, and its DRAM bytes per launch from the ncu capture summarised in
# profiles/gemv_q4k_imma_decode.md (dram__bytes_read.sum + dram__bytes_write.sum)
ROOFLINE_KERNEL = "gemv_q4k_imma_kernel<__half, 1>"
ROOFLINE_TRAFFIC = 9470208


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=64, help="distinct weight matrices per step")
    ap.add_argument("--m", type=int, default=1, help="activation rows (decode batch), <= 16")
    ap.add_argument("--cpu-sample", type=int, default=16, help="matrices in the CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary cells (prefill, dequantize, MoE)")
    return ap.parse_args()


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                smax.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def host_wire(layers: int, seed: int = 0):
    """Synthetic valid q4_k wire bytes on the host (numpy), same recipe as synth.random_wire."""
    import numpy as np

    rng = np.random.default_rng(seed)
    w = rng.integers(0, 256, (layers, N_ROWS, K_COLS // 256, 144), dtype=np.uint8)
    d = rng.uniform(0.001, 0.02, (layers, N_ROWS, K_COLS // 256)).astype(np.float16).view(np.uint16)
    for off in (0, 2):
        w[..., off] = (d & 0xFF).astype(np.uint8)
        w[..., off + 1] = (d >> 8).astype(np.uint8)
    return w.reshape(layers, N_ROWS, ROW_BYTES)


def cpu_arm(m: int, sample: int, repeats: int):
    """The reference's CPU path on `sample` matrices; returns (GB/s, kind, cores, seconds per pass)."""
    import numpy as np

    from oracle import kq_oracle

    wire = host_wire(sample, seed=1)
    x = np.random.default_rng(2001).normal(0, 1, (m, K_COLS)).astype(np.float16)
    if kq_oracle.Ref.available():
        impl, kind = kq_oracle.Ref(), "reference"
    else:
        impl, kind = kq_oracle.Oracle(), "port"
    cores = impl.threads()
    impl.qmm(x, wire[0], CODEC, "f16")  # warm the pool
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        for i in range(sample):
            impl.qmm(x, wire[i], CODEC, "f16")
        best = min(best, time.perf_counter() - t0)
    return sample * MATRIX_BYTES / best / 1e9, kind, cores, best


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = args.cpu_sample
    # each "step" is one pass over the bounded sample
    t_all = []
    gbs, kind, cores, _ = cpu_arm(args.m, sample, max(1, args.warmup))
    import numpy as np

    from oracle import kq_oracle

    impl = kq_oracle.Ref() if kq_oracle.Ref.available() else kq_oracle.Oracle()
    wire = host_wire(sample, seed=1)
    x = np.random.default_rng(2001).normal(0, 1, (args.m, K_COLS)).astype(np.float16)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for i in range(sample):
            impl.qmm(x, wire[i], CODEC, "f16")
    total = time.perf_counter() - t0
    value = args.steps * sample * MATRIX_BYTES / total / 1e9
    line = {
        "impl": "reference", "metric": "q4k_gemv_weight_GBps", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "c1_q4k_decode_gemv", "codec": CODEC, "N": N_ROWS, "K": K_COLS, "M": args.m,
                   "layers": args.layers, "x_dtype": "f16", "accumulate": "f32",
                   "cold_cache": f"a step is a bounded sample: {sample} of the {args.layers} distinct matrices",
                   "parallelism": "host threads"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": kind,
                         "sample": f"{sample} of the step's matrices per step, x86_64 scalar/threaded eval_cpu path"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def measured_tflops():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops"]), "measured"
        except Exception:
            pass
    return 1590.0, "fallback"


def extra_cells(dev):
    """Secondary cells of the metric, single GPU, CUDA events, 5 timed repeats after 2 warm-ups:
    prefill TFLOP/s (config 3), dequantize GB/s (config 2, q4_k), MoE tokens/s (config 4)."""
    import torch

    import mlx_kquant_b200 as kq
    from mlx_kquant_b200.moe import fuse_gate_up, moe_glu, route_topk
    from mlx_kquant_b200.synth import random_wire

    def timed(fn, reps=5):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e-3

    out = {}
    peak_tf, kind = measured_tflops()
    hbm, _ = measured_peak()
    N, K = 14336, 4096
    for codec in ("q4_k", "q6_k"):
        W = random_wire(codec, N, K, seed=3, device=dev)
        for M in (512, 8192):
            x = torch.randn(M, K, device=dev).to(torch.bfloat16)
            t = timed(lambda: kq.quantized_matmul(x, W, None, codec))
            tf = 2.0 * M * N * K / t / 1e12
            out[f"prefill_{codec}_m{M}_bf16"] = {"tflops": tf, "ms": t * 1e3, "frac_of_bf16_peak": tf / peak_tf,
                                                  "peak_kind": kind}
    W = random_wire("q4_k", N, K, seed=4, device=dev, lead=(4,))       # 4 x 150 MB of traffic > L2
    def dq():
        for i in range(4):
            kq.dequantize(W[i], None, "q4_k", torch.float16)
    t = timed(dq) / 4
    gbs = (W[0].numel() + N * K * 2) / t / 1e9
    out["dequant_q4k_f16"] = {"GBps": gbs, "frac_of_hbm_peak": gbs / hbm}
    # MoE: 128 experts, hidden 2048, expert FFN 768, top-8
    E, H, F, k = 128, 2048, 768, 8
    wg = random_wire("q4_k", F, H, seed=5, device=dev, lead=(E,))
    wu = random_wire("q4_k", F, H, seed=6, device=dev, lead=(E,))
    wd = random_wire("q4_k", H, F, seed=7, device=dev, lead=(E,))
    wgu = fuse_gate_up(wg, wu)  # gate | up of every expert as one [E, 2F, bytes] stack: a load-time layout choice
    g = torch.Generator(device="cpu").manual_seed(3000)
    for T in (1, 64, 4096):
        x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev)
        ids, probs = route_topk(torch.randn(T, E, generator=g).to(dev), k)
        t = timed(lambda: moe_glu(x, None, None, wd, "q4_k", ids, probs, w_gate_up=wgu), reps=3)
        out[f"moe_glu_q4k_T{T}"] = {"tokens_per_s": T / t, "ms": t * 1e3}
        # the same block replayed from a CUDA graph (no host sync inside it): what a serving loop pays
        try:
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for _ in range(2):
                    moe_glu(x, None, None, wd, "q4_k", ids, probs, w_gate_up=wgu)
                side.synchronize()
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=side):
                    y_cap = moe_glu(x, None, None, wd, "q4_k", ids, probs, w_gate_up=wgu)
            torch.cuda.current_stream(dev).wait_stream(side)
            tg = timed(gr.replay, reps=5)
            out[f"moe_glu_q4k_T{T}"]["graph_tokens_per_s"] = T / tg
            out[f"moe_glu_q4k_T{T}"]["graph_ms"] = tg * 1e3
            del gr, y_cap
        except Exception as e:  # capture is an optimisation of the caller, not part of the op
            out[f"moe_glu_q4k_T{T}"]["graph_error"] = str(e)[:120]
            torch.cuda.synchronize()
    return out


def moe_ep_cell(dev, rank, world):
    """MoE SwiGLU block, 128 experts partitioned over the ranks, all-to-all dispatch and combine over
    NCCL; weak scaling: T = 4096 tokens per rank. Device time, max over ranks."""
    import torch
    import torch.distributed as dist

    from mlx_kquant_b200.dist import shard_bounds
    from mlx_kquant_b200.moe import fuse_gate_up, moe_glu_expert_parallel, route_topk
    from mlx_kquant_b200.synth import random_wire

    E, H, F, k, T = 128, 2048, 768, 8, 4096
    lo, hi = shard_bounds(E, rank, world)
    wg = random_wire("q4_k", F, H, seed=50 + rank, device=dev, lead=(hi - lo,))
    wu = random_wire("q4_k", F, H, seed=60 + rank, device=dev, lead=(hi - lo,))
    wd = random_wire("q4_k", H, F, seed=70 + rank, device=dev, lead=(hi - lo,))
    g = torch.Generator(device="cpu").manual_seed(3000 + rank)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev)
    ids, probs = route_topk(torch.randn(T, E, generator=g).to(dev), k)
    wgu = fuse_gate_up(wg, wu)
    fn = lambda: moe_glu_expert_parallel(x, None, None, wd, "q4_k", ids, probs, E, w_gate_up=wgu)
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    reps = 3
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    out = {f"moe_glu_q4k_ep{world}_T4096_per_rank": {"tokens_per_s": world * T / (ms * 1e-3), "ms": ms,
                                                      "experts_per_rank": hi - lo}}
    # fixed-shape form (all-gather, local experts as a CUDA graph, reduce-scatter): no host read inside a step
    from mlx_kquant_b200.moe import GatheredExpertParallel

    for Tg in (64, 4096):
        ep = GatheredExpertParallel(Tg, H, k, E, wgu, wd, "q4_k")
        xg, idg, prg = x[:Tg].contiguous(), ids[:Tg].contiguous(), probs[:Tg].contiguous()
        ep.capture()
        for _ in range(3):
            ep(xg, idg, prg)
        torch.cuda.synchronize()
        dist.barrier()
        reps = 20 if Tg <= 64 else 5
        e0.record()
        for _ in range(reps):
            ep(xg, idg, prg)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        out[f"moe_glu_q4k_ep{world}_gathered_T{Tg}_per_rank"] = {"tokens_per_s": world * Tg / (ms * 1e-3), "ms": ms}
        del ep
    return out


def run_b200(args):
    import torch
    import torch.distributed as dist

    import mlx_kquant_b200 as kq
    from mlx_kquant_b200.synth import random_wire

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.pop("NCCL_DEBUG", None)  # NCCL's version banner would share stdout with the one JSON line
        dist.init_process_group("nccl", device_id=dev)

    layers, M = args.layers, args.m
    # this rank's column shard of every layer: rows [rank*4096, (rank+1)*4096) of a [world*4096, 4096] matrix
    W = random_wire(CODEC, N_ROWS, K_COLS, seed=1000 + rank, device=dev, lead=(layers,))
    g = torch.Generator(device="cpu").manual_seed(2000 + M)
    x_host = torch.randn(M, K_COLS, generator=g).to(torch.float16).pin_memory()
    x_dev = x_host.to(dev)
    # two output buffers: at N > 1 the all-gather of step i overlaps the matmuls of step i + 1
    y_devs = [torch.empty(layers, M, N_ROWS, dtype=torch.float16, device=dev) for _ in range(2)]
    y_alls = [torch.empty(world, layers, M, N_ROWS, dtype=torch.float16, device=dev) for _ in range(2)] if world > 1 else None
    y_dev = y_devs[0]
    y_host = torch.empty(layers, M, N_ROWS, dtype=torch.float16).pin_memory()

    from mlx_kquant_b200 import _lib
    L = _lib.lib()
    stream = torch.cuda.Stream(dev)

    def launch_all(s, yb):
        for i in range(layers):
            rc = L.kq_quantized_matmul(x_dev.data_ptr(), _lib.KQ_F16, M, K_COLS, K_COLS, W[i].data_ptr(), ROW_BYTES,
                                       N_ROWS, CODEC.encode(), 1, yb[i].data_ptr(), N_ROWS, None, 0, s.cuda_stream)
            _lib.check(rc)

    # ---- correctness guard: the captured path equals the public op
    with torch.cuda.stream(stream):
        launch_all(stream, y_dev)
        ref0 = kq.quantized_matmul(x_dev, W[0], None, CODEC)
    stream.synchronize()
    assert torch.equal(ref0, y_dev[0]), "C-ABI launch and public op disagree"

    # ---- device-resident arm: one CUDA graph of `layers` launches (one graph per output buffer)
    def capture(yb, with_copies):
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(gr, stream=stream):
                if with_copies:
                    x_dev.copy_(x_host, non_blocking=True)
                launch_all(stream, yb)
                if with_copies:
                    y_host.copy_(yb, non_blocking=True)
        return gr

    graphs = [capture(yb, False) for yb in y_devs]
    # ---- end-to-end arm: H2D of x, the launches, D2H of y, captured as one graph of the public path
    graphs_e2e = [capture(yb, True) for yb in y_devs]

    # At N > 1 every step ends with the all-gather of its output shards. It is issued asynchronously and
    # the buffer it reads is not written again before it has finished, so it overlaps the next step.
    state = {"i": 0, "works": [None, None]}

    def run_step(gs):
        b = state["i"] & 1
        state["i"] += 1
        if world > 1 and state["works"][b] is not None:
            state["works"][b].wait()      # stream-side wait: buffer b is free again
        gs[b].replay()
        if world > 1:
            state["works"][b] = dist.all_gather_into_tensor(y_alls[b], y_devs[b], async_op=True)

    def drain():
        for b in range(2):
            if state["works"][b] is not None:
                state["works"][b].wait()
                state["works"][b] = None

    def step_device():
        run_step(graphs)

    def step_e2e():
        run_step(graphs_e2e)

    def timed(fn, steps, warmup):
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                fn()
            drain()
            stream.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                fn()
            drain()                      # the timed region ends when the last all-gather has landed
            e1.record(stream)
            stream.synchronize()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_dev = timed(step_device, args.steps, max(3, args.warmup))
    ms_e2e = timed(step_e2e, args.steps, max(3, args.warmup))
    clocks = sampler.stop() if rank == 0 else None

    step_bytes = layers * MATRIX_BYTES * world
    value = step_bytes / (ms_dev / args.steps * 1e-3) / 1e9
    e2e = step_bytes / (ms_e2e / args.steps * 1e-3) / 1e9
    # dominant kernel: average launch duration over the timed region of the device arm (rank-local bytes)
    launch_s = ms_dev * 1e-3 / (args.steps * layers)
    peak, peak_kind = measured_peak()
    achieved = MATRIX_BYTES / launch_s / 1e9

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            gbs, kind, cores, secs = cpu_arm(M, args.cpu_sample, 5)
            cpu = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": kind,
                   "sample": f"{args.cpu_sample} of the {layers} matrices, best of 5 passes ({secs * 1e3:.1f} ms per pass)"}
        except Exception as e:  # the checker is optional for timing; say why it is missing
            cpu = {"value": None, "unit": "GB/s", "cores": 0, "kind": "port", "sample": f"unavailable: {e}"}

    # expert-parallel MoE (config 4) at N > 1: every rank brings T = 4096 tokens, experts are partitioned
    ep = None
    if world > 1 and not args.no_extra:
        try:
            ep = moe_ep_cell(dev, rank, world)
        except Exception as e:
            ep = {"error": str(e)[:200]}

    if rank == 0:
        line = {
            "metric": "q4k_gemv_weight_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_dev / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "c1_q4k_decode_gemv", "codec": CODEC, "N": N_ROWS, "K": K_COLS, "M": M,
                       "layers": layers, "x_dtype": "f16", "accumulate": "f32",
                       "cold_cache": f"{layers} distinct weight matrices per step = {layers * MATRIX_BYTES / 1e6:.0f} MB > 126 MB L2",
                       "parallelism": "single GPU" if world == 1 else f"column shard x{world} + NCCL all-gather of outputs, overlapped with the next step"},
            "e2e": {"value": e2e, "unit": "GB/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2},
            "gpu_launches": args.steps * layers,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "traffic": ROOFLINE_TRAFFIC, "kernel": ROOFLINE_KERNEL,
                         "algorithmic_bytes_per_launch": MATRIX_BYTES},
            "cpu_baseline": cpu,
            "clocks": clocks,
        }
        if world == 1 and not args.no_extra:
            try:
                line["extra"] = extra_cells(dev)
            except Exception as e:
                line["extra"] = {"error": str(e)[:200]}
        if world > 1 and ep is not None:
            line["extra"] = ep
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
