"""Prefill regime (M > 16): the tcgen05 tile kernel against the CPU oracle.

Reference for the tolerance is the fp32 math accumulated in float64 (on the GPU,
from the oracle's bit-exact dequantized weights); bar as in test_matmul_gpu.py.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest
import torch

import mlx_kquant_b200 as kq
from conftest import assert_close, rel_fro
from gpu_util import TORCH_DT, mint_wire, synthetic_wire, y_to_f32
from mlx_kquant_b200 import _lib
from oracle.kq_oracle import CODECS

pytestmark = pytest.mark.gpu
TOL = 2e-3


def no_device_errors():
    flags = C.c_int(-1)
    _lib.check(_lib.lib().kq_device_error_flags(C.byref(flags), 1))
    return flags.value == 0


def ref64(oracle, x: torch.Tensor, wire: np.ndarray, codec: str) -> np.ndarray:
    Wd = torch.from_numpy(oracle.dequantize(wire, codec, "f32")).cuda().double()
    xs = x.to(torch.bfloat16) if x.dtype == torch.float32 else x   # the op rounds f32 activations to bf16
    return (xs.double() @ Wd.T).cpu().numpy()


@pytest.mark.parametrize("M", [17, 40, 128, 129, 300])
@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
def test_q4k_tile_kernel_shapes(oracle, M, dt):
    rng = np.random.default_rng(M)
    N, K = 200, 1024                                   # N is not a multiple of the 128-column tile
    wire = mint_wire("q4_k", rng.normal(0, 0.02, (N, K)).astype(np.float32))
    g = torch.Generator(device="cuda").manual_seed(M)
    x = torch.randn(M, K, device="cuda", generator=g).to(TORCH_DT[dt])
    y = kq.quantized_matmul(x, torch.from_numpy(wire).cuda(), None, "q4_k")
    assert tuple(y.shape) == (M, N) and y.dtype == (torch.float16 if dt == "f16" else torch.bfloat16)
    assert_close(y_to_f32(y), ref64(oracle, x, wire, "q4_k"), "f16" if dt == "f16" else "bf16", TOL)
    assert no_device_errors()


@pytest.mark.parametrize("codec", CODECS)
def test_all_codecs_through_tile_kernel(oracle, codec):
    rng = np.random.default_rng(3)
    N, K, M = 136, 512, 70
    wire = mint_wire(codec, rng.normal(0, 0.02, (N, K)).astype(np.float32))
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    y = kq.quantized_matmul(x, torch.from_numpy(wire).cuda(), None, codec)
    assert_close(y_to_f32(y), ref64(oracle, x, wire, codec), "bf16", TOL)
    assert no_device_errors()


@pytest.mark.parametrize("codec", ["q4_0", "q8_0", "iq4_nl"])
def test_k_tail_in_tile_kernel(oracle, codec):
    rng = np.random.default_rng(5)
    N, K, M = 64, 288, 33                              # K = 4.5 tile steps of 64
    wire = mint_wire(codec, rng.normal(0, 0.02, (N, K)).astype(np.float32))
    g = torch.Generator(device="cuda").manual_seed(6)
    x = torch.randn(M, K, device="cuda", generator=g).half()
    y = kq.quantized_matmul(x, torch.from_numpy(wire).cuda(), None, codec)
    assert_close(y_to_f32(y), ref64(oracle, x, wire, codec), "f16", TOL)


def test_matches_reference_cpu_gemm_regime(oracle):
    """Against the reference's own dequantize-then-GEMM order (M > 16), not just the fp64 math."""
    rng = np.random.default_rng(8)
    N, K, M = 256, 1024, 64
    wire = mint_wire("q6_k", rng.normal(0, 0.02, (N, K)).astype(np.float32))
    x = torch.from_numpy(rng.normal(0, 1, (M, K)).astype(np.float32)).half()
    cpu = oracle.qmm(x.numpy(), wire, "q6_k", "f16").astype(np.float32)
    y = kq.quantized_matmul(x.cuda(), torch.from_numpy(wire).cuda(), None, "q6_k")
    assert rel_fro(y_to_f32(y), cpu) <= TOL


@pytest.mark.parametrize("codec", ["q4_k", "q6_k"])
def test_config3_shape_m512(oracle, codec):
    """Benchmark config 3 at M = 512: W [14336, 4096], x bf16. Weights are really encoded for
    the first 256 rows (checked against the oracle); the rest are synthetic and checked through a
    size-independent property: linearity in x."""
    rng = np.random.default_rng(3000)
    N, K, M = 14336, 4096, 512
    wire = synthetic_wire(codec, N, K, seed=9)
    wire[:256] = mint_wire(codec, rng.normal(0, 0.02, (256, K)).astype(np.float32))
    wd = torch.from_numpy(wire).cuda()
    g = torch.Generator(device="cuda").manual_seed(10)
    x1 = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    x2 = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    y1 = kq.quantized_matmul(x1, wd, None, codec)
    assert_close(y_to_f32(y1[:, :256]), ref64(oracle, x1, wire[:256], codec), "bf16", TOL)
    y2 = kq.quantized_matmul(x2, wd, None, codec).float()
    y12 = kq.quantized_matmul((x1.float() + x2.float()).to(torch.bfloat16), wd, None, codec).float()
    lin = (y12 - (y1.float() + y2)).norm() / (y1.float() + y2).norm()
    assert float(lin) < 6e-3, float(lin)               # three bf16 roundings of the outputs + one of x1+x2
    assert no_device_errors()
