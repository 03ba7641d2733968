"""The one-wave q4_k decode kernel (csrc/kq_gemv_stream.cu: one activation row, N <= 32 x SM count, K <= 4096)
against the CPU oracle, through the C-ABI.

The kernel multiplies BEFORE the preceding kernel of the stream has finished and checks its activations
afterwards, so besides the shapes the tests drive both outcomes of that check: activations that were final
when the kernel started, and activations that the preceding launch writes (a chain y1 = W1 x, y2 = W2 y1
replayed from a CUDA graph, the buffer between them filled with other values first)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import mlx_kquant_b200 as kq
from conftest import assert_close
from gpu_util import mint_wire, synthetic_wire, x_to_torch, y_to_f32
from oracle.kq_oracle import to_f32

pytestmark = pytest.mark.gpu
TOL = 2e-3


def fp64_ref(oracle, store, dt, wire):
    Wd = oracle.dequantize(wire, "q4_k", "f32").astype(np.float64)
    return to_f32(store, dt).astype(np.float64) @ Wd.T


@pytest.mark.parametrize("N,K", [(4096, 4096), (4100, 4096), (2048, 1024), (300, 256), (4736, 2048), (1000, 3840)])
@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_one_row_vs_oracle(oracle, N, K, dt):
    rng = np.random.default_rng(N + K)
    if N * K <= 4096 * 1024:
        wire = mint_wire("q4_k", rng.normal(0, 0.02, (N, K)).astype(np.float32))
    else:   # really-encoded rows for the first 512, valid random wire bytes for the rest (encoding is slow)
        wire = synthetic_wire("q4_k", N, K, seed=N)
        wire[:512] = mint_wire("q4_k", rng.normal(0, 0.02, (512, K)).astype(np.float32))
    xf = rng.normal(0, 1, (1, K)).astype(np.float32)
    xf[0, 5] = 37.0                      # an outlier in the first superblock
    xf[0, K - 40:K - 8] = 0.0            # a sub-block of zeros
    x, store = x_to_torch(xf, dt)
    y = kq.quantized_matmul(x, torch.from_numpy(wire).cuda(), None, "q4_k")
    assert tuple(y.shape) == (1, N)
    assert_close(y_to_f32(y), fp64_ref(oracle, store, dt, wire), dt, TOL)
    # and the reference-order CPU result itself (src/kquant_cpu_decode.cpp:1032-1065)
    cpu = to_f32(oracle.qmm(store, wire, "q4_k", dt), dt)
    assert np.linalg.norm(y_to_f32(y) - cpu) <= TOL * np.linalg.norm(cpu)


def test_back_to_back_launches_with_distinct_inputs(oracle):
    """Launches of a stream overlap (programmatic dependent launch): every result must belong to its own
    weights and activations."""
    N = K = 4096
    wires = [synthetic_wire("q4_k", N, K, seed=70 + i) for i in range(4)]
    wd = [torch.from_numpy(w).cuda() for w in wires]
    rng = np.random.default_rng(71)
    xs = [x_to_torch(rng.normal(0, 1, (1, K)).astype(np.float32), "f16") for _ in range(4)]
    ys = [kq.quantized_matmul(xs[i][0], wd[i], None, "q4_k") for i in range(4) for _ in range(3)]
    torch.cuda.synchronize()
    for j, y in enumerate(ys):
        i = j // 3
        assert_close(y_to_f32(y), fp64_ref(oracle, xs[i][1], "f16", wires[i]), "f16", TOL)


@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_activations_written_by_the_preceding_launch(oracle, dt):
    """y2 = W2 (W1 x): the second launch starts while the first still runs and reads a buffer that the first
    has not written yet. Its check after the wait must catch that and multiply again."""
    N = K = 4096
    tdt = torch.float16 if dt == "f16" else torch.bfloat16
    w1 = synthetic_wire("q4_k", N, K, seed=81)
    w2 = synthetic_wire("q4_k", N, K, seed=82)
    w1d, w2d = torch.from_numpy(w1).cuda(), torch.from_numpy(w2).cuda()
    x, _ = x_to_torch(np.random.default_rng(83).normal(0, 0.002, (1, K)).astype(np.float32), dt)  # keeps y2 inside fp16
    from mlx_kquant_b200 import _lib
    L = _lib.lib()
    code = _lib.KQ_F16 if dt == "f16" else _lib.KQ_BF16
    y1 = torch.empty(1, N, dtype=tdt, device="cuda")
    y2 = torch.empty(1, N, dtype=tdt, device="cuda")
    stream = torch.cuda.Stream()

    def chain(s):
        y1.fill_(1.0)      # what a too-early read of the second launch sees
        y2.zero_()
        for (xi, w, yo) in ((x, w1d, y1), (y1, w2d, y2)):
            _lib.check(L.kq_quantized_matmul(xi.data_ptr(), code, 1, K, K, w.data_ptr(), K // 256 * 144, N, b"q4_k", 1,
                                             yo.data_ptr(), N, None, 0, s.cuda_stream))

    with torch.cuda.stream(stream):
        chain(stream)                       # eager
        stream.synchronize()
        y1_e, y2_e = y1.clone(), y2.clone()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            chain(stream)
        for _ in range(5):
            g.replay()
        stream.synchronize()
    store1 = y1.cpu().view(torch.int16).numpy().view(np.uint16) if dt == "bf16" else y1.cpu().numpy()
    ref2 = fp64_ref(oracle, store1, dt, w2)
    assert_close(y_to_f32(y2), ref2, dt, TOL)
    assert torch.equal(y1, y1_e) and torch.equal(y2, y2_e)   # the same bits eagerly and from the graph


def test_non_finite_activations_propagate():
    wire = synthetic_wire("q4_k", 512, 1024, seed=90)
    wd = torch.from_numpy(wire).cuda()
    for bad in (float("inf"), float("nan")):
        for tdt in (torch.float16, torch.bfloat16):
            x = torch.ones(1, 1024, device="cuda", dtype=tdt)
            x[0, 700] = bad
            y = kq.quantized_matmul(x, wd, None, "q4_k")
            assert not torch.isfinite(y).any()
    y = kq.quantized_matmul(torch.zeros(1, 1024, device="cuda", dtype=torch.float16), wd, None, "q4_k")
    assert torch.count_nonzero(y) == 0
