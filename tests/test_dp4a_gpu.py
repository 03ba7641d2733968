"""The integer dot-product decode kernels (one to four activation rows; task lists of gather_qmm) against the
CPU oracle, on shapes chosen to reach their corners: every codec with every activation dtype, random wire
bytes (all scale / sign bit patterns), a ragged N, a K long enough for the weight ring to wrap, the large
iq2_xxs case that takes the lattice kernel, and expert task lists with more rows than one four-row slice.
Tolerance as in test_matmul_gpu.py: 2e-3 relative Frobenius and peak-normalised max error (after the one
rounding to the output dtype) against the fp64-accumulated fp32 math."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import mlx_kquant_b200 as kq
from conftest import assert_close
from gpu_util import mint_wire, synthetic_wire, x_to_torch, y_to_f32
from oracle.kq_oracle import CODECS, to_f32

pytestmark = pytest.mark.gpu
TOL = 2e-3


def ref64(oracle, x_store, dt, wire, codec):
    Wd = oracle.dequantize(wire, codec, "f32").astype(np.float64)
    if dt == "f32":  # the op rounds float32 activations to bfloat16 first (src/kquant_ops.cpp:159-168)
        xs = torch.from_numpy(x_store).to(torch.bfloat16).float().numpy().astype(np.float64)
    else:
        xs = to_f32(x_store, dt).astype(np.float64)
    return xs @ Wd.T


@pytest.mark.parametrize("codec", CODECS)
@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("M", [1, 4])
def test_random_wire_bytes_all_dtypes(oracle, codec, dt, M):
    N, K = 100, 2048  # N is not a multiple of the 32-row CTA
    wire = synthetic_wire(codec, N, K, seed=40 + M)
    x, store = x_to_torch(np.random.default_rng(41).normal(0, 1, (M, K)).astype(np.float32), dt)
    y = kq.quantized_matmul(x, torch.from_numpy(wire).cuda(), None, codec)
    out = "f16" if dt == "f16" else "bf16"
    assert tuple(y.shape) == (M, N)
    assert_close(y_to_f32(y), ref64(oracle, store, dt, wire, codec), out, TOL)


@pytest.mark.parametrize("codec", ["q4_k", "q6_k", "q3_k", "q8_0", "iq4_xs"])
@pytest.mark.parametrize("M", [1, 3])
def test_long_k_wraps_the_weight_ring(oracle, codec, M):
    N, K = 64, 8192  # four 256-weight chunks per warp: the two-slot ring is reused
    wire = synthetic_wire(codec, N, K, seed=50)
    x, store = x_to_torch(np.random.default_rng(51).normal(0, 1, (M, K)).astype(np.float32), "f16")
    y = kq.quantized_matmul(x, torch.from_numpy(wire).cuda(), None, codec)
    assert_close(y_to_f32(y), ref64(oracle, store, "f16", wire, codec), "f16", TOL)


def test_outlier_and_zero_groups(oracle):
    """One huge activation and an all-zero 32-group: the per-group 16-bit quantisation must keep both exact enough."""
    N, K = 96, 1024
    wire = mint_wire("q4_k", np.random.default_rng(60).normal(0, 0.02, (N, K)).astype(np.float32))
    xf = np.random.default_rng(61).normal(0, 1, (1, K)).astype(np.float32)
    xf[0, 37] = 3000.0
    xf[0, 64:96] = 0.0
    x, store = x_to_torch(xf, "f16")
    y = kq.quantized_matmul(x, torch.from_numpy(wire).cuda(), None, "q4_k")
    assert_close(y_to_f32(y), ref64(oracle, store, "f16", wire, "q4_k"), "f16", TOL)


def test_large_iq2_xxs_takes_the_lattice_kernel(oracle):
    N, K = 6144, 8192  # 50 M weights: above the size from which the integer kernel serves iq2_xxs
    wire = synthetic_wire("iq2_xxs", N, K, seed=70)
    x, store = x_to_torch(np.random.default_rng(71).normal(0, 1, (1, K)).astype(np.float32), "f16")
    y = kq.quantized_matmul(x, torch.from_numpy(wire).cuda(), None, "iq2_xxs")
    assert_close(y_to_f32(y), ref64(oracle, store, "f16", wire, "iq2_xxs"), "f16", TOL)


@pytest.mark.parametrize("codec", ["q4_k", "q6_k", "q5_k", "q8_0", "q2_k"])
def test_gather_task_lists_bf16(oracle, codec):
    """Decode-regime gather_qmm with bf16 rows: 6 experts, 40 routed rows, so some experts own more than one
    four-row slice."""
    E, N, K, B = 6, 96, 768, 40
    rng = np.random.default_rng(80)
    wire = np.stack([synthetic_wire(codec, N, K, seed=81 + e) for e in range(E)])
    xf = rng.normal(0, 1, (B, 1, K)).astype(np.float32)
    x, store = x_to_torch(xf, "bf16")
    rhs = rng.integers(0, E, B)
    y = kq.gather_qmm(x, torch.from_numpy(wire).cuda(), None, codec, rhs_indices=torch.from_numpy(rhs).cuda())
    assert tuple(y.shape) == (B, 1, N)
    got = y_to_f32(y).reshape(B, N)
    xs = to_f32(store.reshape(B, K), "bf16").astype(np.float64)
    want = np.empty((B, N))
    for e in range(E):
        sel = np.nonzero(rhs == e)[0]
        if len(sel):
            want[sel] = xs[sel] @ oracle.dequantize(wire[e], codec, "f32").astype(np.float64).T
    assert_close(got, want, "bf16", TOL)
