#!/usr/bin/env python3
"""Benchmark of the quantized-weight hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference]
    python bench.py --case matmul q4_k 4096 4096 1 40        (one op a few times: the driver of profiler captures)

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
        all inside the timed region. The read of step i's outputs runs on a second
        stream beside the launches of step i + 1 (two output buffers), the last
        step's read closes the region.
extra   (N = 1) the other cells of the metric, each with its roofline fraction
        and a bounded CPU sample of the reference's own code: the headline
        shape at M = 8 and as a dependent chain (every launch consumes the
        output of the one before), dequantize of all ten codecs [14336, 4096]
        to f16 and f32, prefill of q4_k / q6_k at M = 128 .. 8192, the
        [28672, 8192] iq4_xs / iq2_xxs decode at M = 1, 4, 16, and the
        128-expert MoE block at T = 1, 64, 4096.
N > 1   weak scaling of the headline: every rank holds its own [4096, 4096]
        column shard (rows r*4096 .. (r+1)*4096 of a [N*4096, 4096] matrix) per
        layer and the [layers, M, 4096] output shards are all-gathered over
        NCCL each step. Before timing, the shards' outputs are compared with
        single-GPU products (`parity_n`). `extra` then carries the sharded
        cells: [28672, 8192] iq4_xs decode and [14336, 4096] q4_k prefill
        column-sharded over the FIXED N (strong scaling, with and without the
        all-gather), and the expert-parallel MoE block.
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
# profiles/gemv_q4k_stream_decode.md (dram__bytes_read.sum + dram__bytes_write.sum)
ROOFLINE_KERNEL = "gemv_q4k_stream_kernel<__half>"
ROOFLINE_TRAFFIC = 9491000
TEN_CODECS = ("q2_k", "q3_k", "q4_k", "q5_k", "q6_k", "q4_0", "q8_0", "iq4_nl", "iq4_xs", "iq2_xxs")


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
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary cells")
    ap.add_argument("--case", nargs="+", default=None,
                    help="run one op a few times and exit: matmul <codec> N K M launches [f16|bf16] | "
                         "dequant <codec> rows K dtype launches | gather <codec> N K tokens top_k | "
                         "moe T (the 128-expert block)")
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


def _peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return json.loads(p.read_text())
        except Exception:
            pass
    return {}


def measured_peak():
    try:
        return float(_peaks()["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def measured_tflops():
    try:
        return float(_peaks()["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, "fallback"


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


def cpu_impl():
    """The reference's compiled CPU library when present, else the C restatement: (object, kind)."""
    from oracle import kq_oracle

    if kq_oracle.Ref.available():
        return kq_oracle.Ref(), "reference"
    return kq_oracle.Oracle(), "port"


def cpu_arm(m: int, sample: int, repeats: int):
    """The reference's CPU path on `sample` matrices; returns (GB/s, kind, cores, seconds per pass)."""
    import numpy as np

    wire = host_wire(sample, seed=1)
    x = np.random.default_rng(2001).normal(0, 1, (m, K_COLS)).astype(np.float16)
    impl, kind = cpu_impl()
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
    gbs, kind, cores, _ = cpu_arm(args.m, sample, max(1, args.warmup))
    import numpy as np

    impl, _ = cpu_impl()
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


# ------------------------------------------------------------------------------------------ timing helpers
def _events(torch):
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def timed_eager(torch, fn, reps=5, warm=2):
    """Seconds per call of fn(), CUDA events on the current stream."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = _events(torch)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e-3


def timed_graph(torch, dev, fn, reps=10, warm=3):
    """Seconds per replay of a CUDA graph that holds one call of fn() (captured on a side stream)."""
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        for _ in range(2):
            fn()
        side.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=side):
            keep = fn()
    torch.cuda.current_stream(dev).wait_stream(side)
    t = timed_eager(torch, gr.replay, reps=reps, warm=warm)
    del gr, keep
    return t


def best_of(fn, repeats=3):
    fn()
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        fn()
        best = min(best, time.perf_counter() - t0)
    return best


# ------------------------------------------------------------------------------------------ secondary cells
def extra_cells(dev, with_cpu: bool):
    """Secondary cells of the metric on one GPU. GPU numbers: CUDA events, warm-ups first, inputs larger than L2
    or distinct per launch. `cpu`: the reference's CPU code on a bounded sample of the same cell (host threads)."""
    import numpy as np
    import torch

    import mlx_kquant_b200 as kq
    from mlx_kquant_b200 import _lib
    from mlx_kquant_b200.moe import fuse_gate_up, moe_glu, route_topk
    from mlx_kquant_b200.synth import random_wire

    out = {}
    peak_tf, tf_kind = measured_tflops()
    hbm, hbm_kind = measured_peak()
    impl = kind = None
    cores = 0
    if with_cpu:
        try:
            impl, kind = cpu_impl()
            cores = impl.threads()
        except Exception:
            impl = None
    L = _lib.lib()

    def cpu_cell(seconds, units, unit, sample):
        return {"value": units / seconds, "unit": unit, "cores": cores, "kind": kind, "sample": sample}

    # ---- config 1 at M = 8, and as a dependent chain (launch i reads what launch i - 1 wrote)
    layers = 64
    W = random_wire(CODEC, N_ROWS, K_COLS, seed=1000, device=dev, lead=(layers,))
    g = torch.Generator(device="cpu").manual_seed(2008)
    x8 = torch.randn(8, K_COLS, generator=g).to(torch.float16).to(dev)
    y8 = torch.empty(layers, 8, N_ROWS, dtype=torch.float16, device=dev)

    def launch(xp, M, wp, yp, s):
        _lib.check(L.kq_quantized_matmul(xp, _lib.KQ_F16, M, K_COLS, K_COLS, wp, ROW_BYTES, N_ROWS, CODEC.encode(), 1,
                                         yp, N_ROWS, None, 0, s))

    def c1_m8():
        s = torch.cuda.current_stream(dev).cuda_stream
        for i in range(layers):
            launch(x8.data_ptr(), 8, W[i].data_ptr(), y8[i].data_ptr(), s)

    t = timed_graph(torch, dev, c1_m8) / layers
    gbs = MATRIX_BYTES / t / 1e9
    out["c1_q4k_m8"] = {"GBps": gbs, "us_per_launch": t * 1e6, "frac_of_hbm_peak": gbs / hbm, "peak_kind": hbm_kind}
    if impl is not None:
        wh = W[:4].cpu().numpy()
        xh = x8.cpu().numpy()
        secs = best_of(lambda: [impl.qmm(xh, wh[i], CODEC, "f16") for i in range(4)])
        out["c1_q4k_m8"]["cpu"] = cpu_cell(secs, 4 * MATRIX_BYTES / 1e9, "GB/s", "4 of the 64 matrices, M = 8")
    # chain: super-scale d = 6.1e-5 and dmin = 7.5 d give zero-mean weights of gain ~1 per product, so that 64
    # products in a row stay inside fp16; the buffers between the launches are cleared at the start of every
    # replay, so a launch that reads ahead of its producer does not find last replay's values
    Wc = W.clone().view(layers, N_ROWS, K_COLS // 256, 144)
    for off, val in ((0, 6.1e-5), (2, 4.575e-4)):
        b = torch.tensor([val], dtype=torch.float16).view(torch.uint8).to(dev)
        Wc[..., off] = b[0]
        Wc[..., off + 1] = b[1]
    Wc = Wc.view(layers, N_ROWS, ROW_BYTES)
    ych = torch.empty(layers + 1, 1, N_ROWS, dtype=torch.float16, device=dev)
    ych[0] = torch.randn(1, K_COLS, generator=g).to(torch.float16).to(dev)

    def c1_chain():
        s = torch.cuda.current_stream(dev).cuda_stream
        ych[1:].zero_()
        for i in range(layers):
            launch(ych[i].data_ptr(), 1, Wc[i].data_ptr(), ych[i + 1].data_ptr(), s)

    t = timed_graph(torch, dev, c1_chain) / layers
    gbs = MATRIX_BYTES / t / 1e9
    out["c1_q4k_m1_dependent_chain"] = {
        "GBps": gbs, "us_per_launch": t * 1e6, "frac_of_hbm_peak": gbs / hbm, "peak_kind": hbm_kind,
        "note": "every launch consumes the preceding launch's output: its products cannot start before that "
                "launch has finished, only its weight stream overlaps",
        "finite": bool(torch.isfinite(ych[-1]).all().item()), "last_rms": float(ych[-1].float().pow(2).mean().sqrt())}
    del W, Wc, y8, ych

    # ---- config 2: dequantize [14336, 4096], all ten codecs, to f16 and f32 (wire + output > L2 per call)
    N, K = 14336, 4096
    for codec in TEN_CODECS:
        Wq = random_wire(codec, N, K, seed=4, device=dev, lead=(2,))
        wire_bytes = Wq[0].numel()
        cell = {}
        for dt, tdt, nbytes in (("f16", torch.float16, 2), ("f32", torch.float32, 4)):
            def dq():
                kq.dequantize(Wq[0], None, codec, tdt)
                kq.dequantize(Wq[1], None, codec, tdt)
            t = timed_eager(torch, dq) / 2
            gbs = (wire_bytes + N * K * nbytes) / t / 1e9
            cell[dt] = {"GBps": gbs, "frac_of_hbm_peak": gbs / hbm}
        if impl is not None:
            wh = Wq[0, :2048].cpu().numpy()
            secs = best_of(lambda: impl.dequantize(wh, codec, "f16"))
            cell["cpu"] = cpu_cell(secs, (wh.size + 2048 * K * 2) / 1e9, "GB/s", "2048 of the 14336 rows, to f16")
        cell["peak_kind"] = hbm_kind
        out[f"c2_dequant_{codec}"] = cell
        del Wq
    out["dequant_q4k_f16"] = {"GBps": out["c2_dequant_q4_k"]["f16"]["GBps"],
                              "frac_of_hbm_peak": out["c2_dequant_q4_k"]["f16"]["frac_of_hbm_peak"]}

    # ---- config 3: prefill [14336, 4096], bf16 rows
    for codec in ("q4_k", "q6_k"):
        Wq = random_wire(codec, N, K, seed=3, device=dev)
        for M in (128, 512, 2048, 8192):
            x = torch.randn(M, K, device=dev).to(torch.bfloat16)
            t = timed_eager(torch, lambda: kq.quantized_matmul(x, Wq, None, codec), reps=8 if M <= 512 else 5)
            tf = 2.0 * M * N * K / t / 1e12
            out[f"prefill_{codec}_m{M}_bf16"] = {"tflops": tf, "ms": t * 1e3, "frac_of_bf16_peak": tf / peak_tf,
                                                  "peak_kind": tf_kind}
        if impl is not None:
            wh = Wq[:1024].cpu().numpy()
            xh = torch.randn(128, K).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
            secs = best_of(lambda: impl.qmm(xh, wh, codec, "bf16"), repeats=2)
            out[f"prefill_{codec}_m128_bf16"]["cpu"] = cpu_cell(
                secs, 2.0 * 128 * 1024 * K / 1e12, "TFLOP/s", "1024 of the 14336 weight rows, M = 128")
        del Wq

    # ---- config 5: 70B-class decode [28672, 8192], fp16 rows; distinct matrices in turn (> L2 between reuses)
    N5, K5 = 28672, 8192
    for codec, copies in (("iq4_xs", 2), ("iq2_xxs", 3)):
        Wq = random_wire(codec, N5, K5, seed=5, device=dev, lead=(copies,))
        wire_bytes = Wq[0].numel()
        for M in (1, 4, 16):
            x = torch.randn(M, K5, device=dev).to(torch.float16)

            def c5():
                return [kq.quantized_matmul(x, Wq[i % copies], None, codec) for i in range(2 * copies)]
            t = timed_graph(torch, dev, c5) / (2 * copies)
            gbs = wire_bytes / t / 1e9
            out[f"c5_{codec}_m{M}"] = {"GBps": gbs, "us_per_launch": t * 1e6, "frac_of_hbm_peak": gbs / hbm,
                                       "peak_kind": hbm_kind}
        if impl is not None:
            wh = Wq[0, :4096].cpu().numpy()
            xh = torch.randn(1, K5).to(torch.float16).numpy()
            secs = best_of(lambda: impl.qmm(xh, wh, codec, "f16"))
            out[f"c5_{codec}_m1"]["cpu"] = cpu_cell(secs, wh.size / 1e9, "GB/s", "4096 of the 28672 rows, M = 1")
        del Wq

    # ---- config 4: MoE block, 128 experts, hidden 2048, expert FFN 768, top-8
    E, H, F, k = 128, 2048, 768, 8
    wg = random_wire("q4_k", F, H, seed=5, device=dev, lead=(E,))
    wu = random_wire("q4_k", F, H, seed=6, device=dev, lead=(E,))
    wd = random_wire("q4_k", H, F, seed=7, device=dev, lead=(E,))
    wgu = fuse_gate_up(wg, wu)  # gate | up of every expert as one [E, 2F, bytes] stack: a load-time layout choice
    del wg, wu
    g = torch.Generator(device="cpu").manual_seed(3000)
    for T in (1, 64, 512, 4096):
        x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev)
        ids, probs = route_topk(torch.randn(T, E, generator=g).to(dev), k)
        fn = lambda: moe_glu(x, None, None, wd, "q4_k", ids, probs, w_gate_up=wgu)
        t = timed_eager(torch, fn, reps=3)
        cell = {"tokens_per_s": T / t, "ms": t * 1e3}
        # the same block replayed from a CUDA graph (no host sync inside it): what a serving loop pays
        try:
            tg = timed_graph(torch, dev, fn, reps=5)
            cell["graph_tokens_per_s"] = T / tg
            cell["graph_ms"] = tg * 1e3
            experts = int(torch.unique(ids).numel())
            if T <= 64:   # weight-streaming regime
                cell["frac_of_hbm_peak"] = experts * 2654208 / tg / 1e9 / hbm
            else:
                cell["frac_of_bf16_peak"] = T * 75497472 / tg / 1e12 / peak_tf
        except Exception as e:  # capture is an optimisation of the caller, not part of the op
            cell["graph_error"] = str(e)[:120]
            torch.cuda.synchronize()
        out[f"moe_glu_q4k_T{T}"] = cell
    return out


# ------------------------------------------------------------------------------------------ N > 1
def parity_n(dev, rank, world, W0, x_dev, y0):
    """Correctness at N > 1, before anything is timed. Dense: every rank's output shard of layer 0 equals,
    bit for bit, the product of that shard computed alone on rank 0 (same kernel, K is not split), and agrees
    with the matching slice of the product with the whole [world * 4096, 4096] matrix. MoE: both
    expert-parallel forms against the single-GPU block on the same tokens."""
    import torch
    import torch.distributed as dist

    import mlx_kquant_b200 as kq
    from mlx_kquant_b200.dist import shard_bounds
    from mlx_kquant_b200.moe import GatheredExpertParallel, fuse_gate_up, moe_glu, moe_glu_expert_parallel, route_topk
    from mlx_kquant_b200.synth import random_wire

    problems = []
    shards = [torch.empty_like(W0) for _ in range(world)]
    dist.all_gather(shards, W0.contiguous())
    ys = [torch.empty_like(y0) for _ in range(world)]
    dist.all_gather(ys, y0.contiguous())
    if rank == 0:
        full = kq.quantized_matmul(x_dev, torch.cat(shards, dim=0), None, CODEC).float()
        for r in range(world):
            alone = kq.quantized_matmul(x_dev, shards[r], None, CODEC)
            if not torch.equal(alone, ys[r]):
                problems.append(f"dense shard {r}: not bit-identical to the single-GPU product of that shard")
            sl = full[:, r * N_ROWS:(r + 1) * N_ROWS]
            err = float((ys[r].float() - sl).norm() / sl.norm())
            if not err <= 2e-3:
                problems.append(f"dense shard {r}: rel error {err:.2e} against the full-matrix product")
    del shards

    # MoE: T = 64 tokens per rank
    E, H, F, k, T = 128, 2048, 768, 8, 64
    lo, hi = shard_bounds(E, rank, world)
    wg = random_wire("q4_k", F, H, seed=50 + rank, device=dev, lead=(hi - lo,))
    wu = random_wire("q4_k", F, H, seed=60 + rank, device=dev, lead=(hi - lo,))
    wd = random_wire("q4_k", H, F, seed=70 + rank, device=dev, lead=(hi - lo,))
    wgu = fuse_gate_up(wg, wu)
    g = torch.Generator(device="cpu").manual_seed(3100 + rank)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev)
    ids, probs = route_topk(torch.randn(T, E, generator=g).to(dev), k)
    y_a2a = moe_glu_expert_parallel(x, None, None, wd, "q4_k", ids, probs, E, w_gate_up=wgu)
    ep = GatheredExpertParallel(T, H, k, E, wgu, wd, "q4_k")
    y_gat = ep(x, ids, probs).clone()
    del ep
    from mlx_kquant_b200.moe import PeerExpertParallel, PipelinedExpertParallel
    ep = PipelinedExpertParallel(T, H, k, E, wgu, wd, "q4_k", chunks=2, reduce_dtype=torch.bfloat16)
    y_pip = ep(x, ids, probs).clone()
    del ep
    ep = PeerExpertParallel(T, H, k, E, wgu, wd, "q4_k")
    y_peer = ep(x, ids, probs).clone()
    ep.close()
    del ep
    y_pp = None
    from mlx_kquant_b200.moe import PeerPipelinedExpertParallel
    try:   # each of the two slices must reach the one-call block's sizes (the same answer on every rank)
        ep = PeerPipelinedExpertParallel(T, H, k, E, wgu, wd, "q4_k", chunks=2)
    except ValueError:
        ep = None
    if ep is not None:
        y_pp = ep(x, ids, probs).clone()
        ep.close()
        del ep

    def gather(t):
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous())
        return parts

    same = (hi - lo) * world == E   # equal shards: the stacks can be all-gathered as they are
    if same:
        all_wgu, all_wd = torch.cat(gather(wgu), 0), torch.cat(gather(wd), 0)
        all_x, all_ids, all_p = gather(x), gather(ids), gather(probs)
        all_a, all_g, all_pl = gather(y_a2a), gather(y_gat.to(y_a2a.dtype)), gather(y_pip.to(y_a2a.dtype))
        all_pe = gather(y_peer.to(y_a2a.dtype))
        all_pp = gather(y_pp.to(y_a2a.dtype)) if y_pp is not None else None
        if rank == 0:
            for r in range(world):
                ref = moe_glu(all_x[r], None, None, all_wd, "q4_k", all_ids[r], all_p[r], w_gate_up=all_wgu).float()
                for name, got, bar in (("all-to-all", all_a[r], 6e-3), ("gathered", all_g[r], 6e-3),
                                       ("pipelined, bfloat16 sums", all_pl[r], 8e-3),
                                       ("peer-memory, bfloat16 slots", all_pe[r], 8e-3),
                                       ("peer-memory, copy-engine gather over two slices",
                                        all_pp[r] if all_pp is not None else all_pe[r], 8e-3)):
                    err = float((got.float() - ref).norm() / ref.norm())
                    if not err <= bar:
                        problems.append(f"MoE {name} form, rank {r}: rel error {err:.2e} against the single-GPU block")
    flag = torch.tensor([len(problems)], device=dev)
    dist.broadcast(flag, 0)
    if rank == 0 and problems:
        raise AssertionError("; ".join(problems))
    if int(flag.item()):
        raise AssertionError("parity at N > 1 failed on rank 0")
    return "ok"


def sharded_cells(dev, rank, world):
    """Strong scaling of the sharded configurations: the FIXED matrix is column-sharded over the ranks.
    Device time, max over ranks; `gather` adds the NCCL all-gather of the output shards."""
    import torch
    import torch.distributed as dist

    import mlx_kquant_b200 as kq
    from mlx_kquant_b200.dist import shard_bounds
    from mlx_kquant_b200.synth import random_wire

    out = {}
    hbm, _ = measured_peak()
    peak_tf, _ = measured_tflops()

    def max_ms(ms):
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def run(fn, reps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = _events(torch)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return max_ms(e0.elapsed_time(e1) / reps)

    from mlx_kquant_b200 import _lib
    L = _lib.lib()

    def abi_matmul(x, Wm, codec, ybuf, ws):
        """The C-ABI call writing straight into the (wider) gather buffer: no copy between product and collective."""
        code = _lib.KQ_F16 if x.dtype == torch.float16 else _lib.KQ_BF16
        _lib.check(L.kq_quantized_matmul(x.data_ptr(), code, x.shape[0], x.shape[1], x.stride(0), Wm.data_ptr(),
                                         Wm.shape[1], Wm.shape[0], codec.encode(), 1, ybuf.data_ptr(), ybuf.stride(0),
                                         ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
                                         torch.cuda.current_stream(dev).cuda_stream))

    def graphs_of(fns):
        """One CUDA graph per callable (captured on a side stream)."""
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        out_g = []
        with torch.cuda.stream(side):
            for fn in fns:
                fn()
                side.synchronize()
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=side):
                    fn()
                out_g.append(gr)
        torch.cuda.current_stream(dev).wait_stream(side)
        return out_g

    # config 5: iq4_xs [28672, 8192], M = 1, fp16; four copies of the shard in turn (together larger than L2)
    N5, K5 = 28672, 8192
    lo, hi = shard_bounds(N5, rank, world)
    copies = 4
    Wq = random_wire("iq4_xs", hi - lo, K5, seed=500 + rank, device=dev, lead=(copies,))
    shard_bytes = Wq[0].numel()
    x = torch.randn(1, K5, device=dev, generator=torch.Generator(device=dev).manual_seed(5)).to(torch.float16)
    widest = (N5 + world - 1) // world
    ybuf = torch.zeros(1, widest, dtype=torch.float16, device=dev)
    yall = torch.empty(world, widest, dtype=torch.float16, device=dev)
    gs = graphs_of([(lambda i=i: abi_matmul(x, Wq[i], "iq4_xs", ybuf, None)) for i in range(copies)])
    state = {"i": 0}

    def c5(gather):
        i = state["i"] = (state["i"] + 1) % copies
        gs[i].replay()
        if gather:
            dist.all_gather_into_tensor(yall, ybuf)

    for gather in (False, True):
        ms = run(lambda: c5(gather), 40)
        gbs = shard_bytes / (ms * 1e-3) / 1e9
        out[f"c5_iq4_xs_m1_shard{world}" + ("_gather" if gather else "")] = {
            "per_gpu_GBps": gbs, "aggregate_GBps": gbs * world, "us": ms * 1e3, "frac_of_hbm_peak": gbs / hbm,
            "rows_per_rank": hi - lo}
    del gs, Wq

    # config 3: q4_k [14336, 4096], M = 512, bf16
    N3, K3, M = 14336, 4096, 512
    lo, hi = shard_bounds(N3, rank, world)
    Wq = random_wire("q4_k", hi - lo, K3, seed=300 + rank, device=dev)
    x = torch.randn(M, K3, device=dev, generator=torch.Generator(device=dev).manual_seed(3)).to(torch.bfloat16)
    widest = (N3 + world - 1) // world
    ybuf = torch.zeros(M, widest, dtype=torch.bfloat16, device=dev)
    yall = torch.empty(world * M, widest, dtype=torch.bfloat16, device=dev)
    ws = torch.empty(max(1, L.kq_quantized_matmul_workspace_bytes(_lib.KQ_BF16, M, K3)), dtype=torch.uint8, device=dev)
    g3 = graphs_of([lambda: abi_matmul(x, Wq, "q4_k", ybuf, ws)])[0]

    def c3(gather):
        g3.replay()
        if gather:
            dist.all_gather_into_tensor(yall, ybuf)

    for gather in (False, True):
        ms = run(lambda: c3(gather), 20)
        tf = 2.0 * M * (hi - lo) * K3 / (ms * 1e-3) / 1e12
        out[f"prefill_q4_k_m512_shard{world}" + ("_gather" if gather else "")] = {
            "per_gpu_tflops": tf, "aggregate_tflops": 2.0 * M * N3 * K3 / (ms * 1e-3) / 1e12, "us": ms * 1e3,
            "frac_of_bf16_peak": tf / peak_tf, "rows_per_rank": hi - lo}
    del g3
    return out


def moe_ep_cell(dev, rank, world):
    """MoE SwiGLU block, 128 experts partitioned over the ranks; weak scaling: T tokens per rank. Device time,
    max over ranks. Two forms: all-to-all dispatch and combine, and the fixed-shape gathered form."""
    import torch
    import torch.distributed as dist

    from mlx_kquant_b200.dist import shard_bounds
    from mlx_kquant_b200.moe import GatheredExpertParallel, fuse_gate_up, moe_glu_expert_parallel, route_topk
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
    del wg, wu
    fn = lambda: moe_glu_expert_parallel(x, None, None, wd, "q4_k", ids, probs, E, w_gate_up=wgu)
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = _events(torch)
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
    # fixed-shape form (all-gather, local experts as a CUDA graph, reduce-scatter): no host read inside a step;
    # "pipelined": two token slices, collectives of one overlapping the products of the other, bfloat16 partial sums
    from mlx_kquant_b200.moe import PipelinedExpertParallel

    def timed_ep(ep, xg, idg, prg, reps):
        ep.capture()
        for _ in range(3):
            ep(xg, idg, prg)
        torch.cuda.synchronize()
        dist.barrier()
        e0.record()
        for _ in range(reps):
            ep(xg, idg, prg)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed_part(fn, reps=5):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for Tg in (64, 4096):
        xg, idg, prg = x[:Tg].contiguous(), ids[:Tg].contiguous(), probs[:Tg].contiguous()
        for tag, rd in (("", torch.float32), ("_bf16sum", torch.bfloat16)):
            ep = GatheredExpertParallel(Tg, H, k, E, wgu, wd, "q4_k", reduce_dtype=rd)
            ms = timed_ep(ep, xg, idg, prg, 20 if Tg <= 64 else 5)
            cell = {"tokens_per_s": world * Tg / (ms * 1e-3), "ms": ms}
            if Tg == 4096:  # where the step goes: the two collectives and the local stage, each timed alone
                cell["all_gather_ms"] = timed_part(lambda: dist.all_gather_into_tensor(ep.recv, ep.send))
                cell["local_stage_ms"] = timed_part(lambda: ep._graph.replay())
                cell["reduce_scatter_ms"] = timed_part(lambda: dist.reduce_scatter_tensor(ep.y32, ep.partial))
            out[f"moe_glu_q4k_ep{world}_gathered{tag}_T{Tg}_per_rank"] = cell
            del ep
            torch.cuda.empty_cache()
    # the weighted sum written into the owners' memory through peer mappings instead of a reduce-scatter
    from mlx_kquant_b200.moe import PeerExpertParallel

    for Tg in (64, 4096):
        try:
            ep = PeerExpertParallel(Tg, H, k, E, wgu, wd, "q4_k")
        except ValueError:  # sizes the one-call block does not take (few routed rows per local expert)
            continue
        xg, idg, prg = x[:Tg].contiguous(), ids[:Tg].contiguous(), probs[:Tg].contiguous()
        ms = timed_ep(ep, xg, idg, prg, 20 if Tg <= 64 else 5)
        cell = {"tokens_per_s": world * Tg / (ms * 1e-3), "ms": ms}
        if Tg == 4096:
            cell["local_stage_with_peer_stores_ms"] = timed_part(lambda: ep._graph.replay())
        out[f"moe_glu_q4k_ep{world}_peer_T{Tg}_per_rank"] = cell
        ep.close()
        del ep
        torch.cuda.empty_cache()

    # ... and with the gather moved by the copy engines beside the products of the other token slice
    from mlx_kquant_b200.moe import PeerPipelinedExpertParallel

    for chunks in (2, 4):
        try:
            ep = PeerPipelinedExpertParallel(T, H, k, E, wgu, wd, "q4_k", chunks=chunks)
        except ValueError:
            continue
        ms = timed_ep(ep, x, ids, probs, 5)
        out[f"moe_glu_q4k_ep{world}_peer_pipelined{chunks}_T{T}_per_rank"] = {"tokens_per_s": world * T / (ms * 1e-3),
                                                                              "ms": ms}
        ep.close()
        del ep
        torch.cuda.empty_cache()

    # The collectives of the pipelined form run beside the tile kernel, which wants whole SMs: communicators limited
    # to a few CTAs leave it more of the machine (ncclConfig max_ctas through torch's process-group options).
    def narrow_group(ctas):
        try:
            opts = dist.ProcessGroupNCCL.Options()
            opts.config.max_ctas = ctas
            opts.config.min_ctas = 1
            return dist.new_group(pg_options=opts)
        except Exception:  # noqa: BLE001 - an older torch without these options: the cell is left out
            return None

    cells = [("pipelined2_bf16sum", dict(chunks=2, reduce_dtype=torch.bfloat16), None),
             ("pipelined4_bf16sum", dict(chunks=4, reduce_dtype=torch.bfloat16), None),
             ("pipelined2_f32sum", dict(chunks=2), None)]
    if world > 2:
        cells += [(f"pipelined2_bf16sum_{c}ctas", dict(chunks=2, reduce_dtype=torch.bfloat16), c) for c in (4, 8, 16)]
    for name, kw, ctas in cells:
        grp = narrow_group(ctas) if ctas else None
        if ctas and grp is None:
            continue
        ep = PipelinedExpertParallel(T, H, k, E, wgu, wd, "q4_k", group=grp, **kw)
        ms = timed_ep(ep, x, ids, probs, 5)
        out[f"moe_glu_q4k_ep{world}_{name}_T{T}_per_rank"] = {"tokens_per_s": world * T / (ms * 1e-3), "ms": ms}
        del ep
        torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------------ single cases
def run_case(argv):
    """One op a few times on synthetic inputs: what profiler captures are taken from."""
    import torch

    import mlx_kquant_b200 as kq
    from mlx_kquant_b200.synth import random_wire

    DT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}
    what = argv[0]
    if what == "matmul":
        codec = argv[1]
        N, K, M, launches = (int(v) for v in argv[2:6])
        dt = DT[argv[6]] if len(argv) > 6 else torch.float16
        W = random_wire(codec, N, K, seed=1, lead=(launches,))
        x = torch.randn(M, K, device="cuda").to(dt)
        for i in range(launches):
            y = kq.quantized_matmul(x, W[i], None, codec)
    elif what == "dequant":
        codec = argv[1]
        rows, K = int(argv[2]), int(argv[3])
        dt, launches = DT[argv[4]], int(argv[5])
        W = random_wire(codec, rows, K, seed=2, lead=(launches,))
        for i in range(launches):
            y = kq.dequantize(W[i], None, codec, dt)
    elif what == "gather":
        codec = argv[1]
        N, K, T, top_k = (int(v) for v in argv[2:6])
        W = random_wire(codec, N, K, seed=3, lead=(128,))
        x = torch.randn(T, 1, K, device="cuda").to(torch.bfloat16)
        idx = torch.randint(0, 128, (T, top_k), device="cuda")
        y = kq.gather_qmm(x, W, None, codec, lhs_indices=torch.arange(T, device="cuda")[:, None].expand(T, top_k),
                          rhs_indices=idx)
    elif what == "moe":
        from mlx_kquant_b200.moe import fuse_gate_up, moe_glu, route_topk

        T = int(argv[1])
        E, H, F, k = 128, 2048, 768, 8
        wgu = fuse_gate_up(random_wire("q4_k", F, H, seed=5, lead=(E,)), random_wire("q4_k", F, H, seed=6, lead=(E,)))
        wd = random_wire("q4_k", H, F, seed=7, lead=(E,))
        x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        ids, probs = route_topk(torch.randn(T, E, device="cuda"), k)
        for _ in range(3):
            y = moe_glu(x, None, None, wd, "q4_k", ids, probs, w_gate_up=wgu)
    elif what == "ep_local":
        # the local stage of one expert-parallel rank of eight, on one GPU (no communicator): all ranks' tokens and
        # routing in the gathered buffer, this rank's sixteen experts
        from mlx_kquant_b200.moe import GatheredExpertParallel, fuse_gate_up, route_topk

        T = int(argv[1]) if len(argv) > 1 else 4096
        rd = torch.float32 if (len(argv) > 2 and argv[2] == "f32") else torch.bfloat16
        E, H, F, k, world = 128, 2048, 768, 8, 8
        el = E // world
        wgu = fuse_gate_up(random_wire("q4_k", F, H, seed=5, lead=(el,)), random_wire("q4_k", F, H, seed=6, lead=(el,)))
        wd = random_wire("q4_k", H, F, seed=7, lead=(el,))
        ep = GatheredExpertParallel(T, H, k, E, wgu, wd, "q4_k", rank=3, world=world, reduce_dtype=rd)
        g = torch.Generator(device="cpu").manual_seed(1)
        rows = T + ep.pad_rows
        for r in range(world):
            xr = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
            ids, probs = route_topk(torch.randn(T, E, generator=g).cuda(), k)
            ep.pack(xr, ids, probs)
            ep.recv[r * rows:(r + 1) * rows].copy_(ep.send)
        ep.capture()
        e0, e1 = _events(torch)
        for _ in range(3):
            ep._graph.replay()
        e0.record()
        for _ in range(10):
            ep._graph.replay()
        e1.record()
        torch.cuda.synchronize()
        print(f"local stage of rank 3 of 8, T = {T} per rank: {e0.elapsed_time(e1) / 10:.4f} ms")
        y = ep.partial
    else:
        print(__doc__)
        return 2
    torch.cuda.synchronize()
    print("ok", tuple(y.shape), float(y.float().abs().mean()))
    return 0


# ------------------------------------------------------------------------------------------ headline
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
        # NCCL's own log (when NCCL_DEBUG asks for one) goes to stderr: stdout carries the one JSON line
        if os.environ.get("NCCL_DEBUG") and not os.environ.get("NCCL_DEBUG_FILE"):
            os.environ["NCCL_DEBUG_FILE"] = "/dev/stderr"
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
    y_hosts = [torch.empty(layers, M, N_ROWS, dtype=torch.float16).pin_memory() for _ in range(2)]
    y_host = y_hosts[0]

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
    parity = None
    if world > 1:
        parity = parity_n(dev, rank, world, W[0], x_dev, y_dev[0])

    # ---- device-resident arm: one CUDA graph of `layers` launches (one graph per output buffer)
    copy_stream = torch.cuda.Stream(dev)

    def capture(b, with_copies):
        """The step into output buffer b. End to end: the step's x comes from pinned host memory first; the
        device-to-host read of the PRECEDING step's outputs (the other buffer) runs on a second stream beside this
        step's launches, as a serving loop would overlap it - every step's result is still read inside the timed
        region (the last one by finish_e2e below)."""
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(gr, stream=stream):
                if with_copies:
                    copy_stream.wait_stream(stream)
                    with torch.cuda.stream(copy_stream):
                        y_hosts[1 - b].copy_(y_devs[1 - b], non_blocking=True)
                    x_dev.copy_(x_host, non_blocking=True)
                launch_all(stream, y_devs[b])
                if with_copies:
                    stream.wait_stream(copy_stream)
        return gr

    graphs = [capture(b, False) for b in range(2)]
    # ---- end-to-end arm: H2D of x, the launches, D2H of y, captured as one graph of the public path
    graphs_e2e = [capture(b, True) for b in range(2)]

    def finish_e2e():
        b = (state["i"] - 1) & 1     # the last step's buffer: its read has not been issued yet
        y_hosts[b].copy_(y_devs[b], non_blocking=True)

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

    def timed(fn, steps, warmup, finish=None):
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
            if finish is not None:
                finish()
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
    ms_e2e = timed(step_e2e, args.steps, max(3, args.warmup), finish_e2e)
    # the read of a step's outputs arrives intact: the last two steps' host copies equal the device buffers
    for b in range(2):
        assert torch.equal(y_hosts[b], y_devs[b].cpu()), "end-to-end arm: host copy differs from the device result"
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

    del graphs, graphs_e2e, W, y_devs, y_alls
    torch.cuda.empty_cache()
    extra = None
    if not args.no_extra:
        try:
            if world > 1:
                extra = sharded_cells(dev, rank, world)
                extra.update(moe_ep_cell(dev, rank, world))
            elif rank == 0:
                extra = extra_cells(dev, with_cpu=not args.no_cpu_baseline)
        except Exception as e:
            extra = {"error": f"{type(e).__name__}: {str(e)[:200]}"}

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
                    "overlap": "device-to-host read of step i beside the launches of step i + 1; all reads inside the timed region",
                    "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2},
            "gpu_launches": args.steps * layers,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "traffic": ROOFLINE_TRAFFIC, "kernel": ROOFLINE_KERNEL,
                         "algorithmic_bytes_per_launch": MATRIX_BYTES,
                         "note": "all launches of a step read the same activations, so each launch multiplies while "
                                 "the launch before it still runs; extra.c1_q4k_m1_dependent_chain is the same "
                                 "kernel when every launch has to wait for the output of the one before"},
            "cpu_baseline": cpu,
            "clocks": clocks,
        }
        if parity is not None:
            line["parity_n"] = parity
        if extra is not None:
            line["extra"] = extra
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    if args.case:
        sys.exit(run_case(args.case))
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
