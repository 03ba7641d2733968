"""The torch module layer (mlx_kquant_b200/nn.py) against the ops it wraps; mirrors what the reference's
tests/test_nn.py and tests/test_switch_gemm.py check of mlx_kquant/nn.py."""
from __future__ import annotations

import pytest
import torch

import mlx_kquant_b200 as kq
from mlx_kquant_b200.nn import KQuantEmbedding, KQuantLinear, KQuantSwitchLinear, bytes_per_row
from mlx_kquant_b200.synth import random_wire


def test_shapes_and_state_dict_keys():
    lin = KQuantLinear(512, 96, bias=True, codec="q4_k")
    assert tuple(lin.weight.shape) == (96, bytes_per_row("q4_k", 512)) and lin.weight.dtype == torch.uint8
    assert set(lin.state_dict()) == {"weight", "scales", "bias"} and lin.mode == "kquant" and lin.bits == 4
    sw = KQuantSwitchLinear(4, 64, 256, bias=False, codec="q6_k")
    assert tuple(sw.weight.shape) == (4, 64, 210) and set(sw.state_dict()) == {"weight", "scales"}
    emb = KQuantEmbedding(100, 256, "q8_0")
    assert tuple(emb.weight.shape) == (100, 8 * 34)
    with pytest.raises(ValueError):
        KQuantLinear(100, 8, bias=False, codec="q4_k")        # 100 is not a whole number of 256-weight blocks
    with pytest.raises(ValueError):
        KQuantLinear(256, 8, bias=False, codec="q9_k")


@pytest.mark.gpu
def test_linear_and_embedding():
    dev = torch.device("cuda")
    lin = KQuantLinear(512, 96, bias=True, codec="q4_k").to(dev)
    lin.weight.copy_(random_wire("q4_k", 96, 512, seed=1, device=dev))
    lin.bias.copy_(torch.linspace(-1, 1, 96))
    x = torch.randn(3, 5, 512, device=dev).to(torch.bfloat16)
    y = lin(x)
    want = kq.quantized_matmul(x, lin.weight, None, "q4_k") + lin.bias.to(torch.bfloat16)
    assert tuple(y.shape) == (3, 5, 96) and torch.equal(y, want)

    emb = KQuantEmbedding(50, 512, "q6_k").to(dev)
    emb.weight.copy_(random_wire("q6_k", 50, 512, seed=2, device=dev))
    tok = torch.tensor([[3, 49, 0], [7, 7, 12]], device=dev)
    table = kq.dequantize(emb.weight, None, "q6_k", torch.bfloat16)
    got = emb(tok)
    assert tuple(got.shape) == (2, 3, 512) and got.dtype == torch.bfloat16 and torch.equal(got, table[tok])
    h = torch.randn(2, 512, device=dev).to(torch.bfloat16)
    assert torch.equal(emb.as_linear(h), kq.quantized_matmul(h, emb.weight, None, "q6_k"))


@pytest.mark.gpu
def test_switch_linear_gather_and_sorted_segment_paths():
    dev = torch.device("cuda")
    E, N, K = 6, 128, 512
    sw = KQuantSwitchLinear(E, N, K, bias=True, codec="q4_k").to(dev)
    sw.weight.copy_(random_wire("q4_k", N, K, seed=3, device=dev, lead=(E,)))
    sw.bias.copy_(torch.randn(E, N))
    g = torch.Generator(device="cpu").manual_seed(4)
    # decode-shaped, unsorted
    x = torch.randn(7, 1, K, generator=g).to(torch.float16).to(dev)
    idx = torch.tensor([5, 0, 3, 3, 1, 5, 2], device=dev)
    y = sw(x, idx)
    want = kq.gather_qmm(x, sw.weight, None, "q4_k", rhs_indices=idx) + sw.bias[idx].unsqueeze(-2).half()
    assert tuple(y.shape) == (7, 1, N) and torch.equal(y, want)
    # prefill-shaped, sorted: the segment product with a device-built tile map (experts 2 absent)
    counts = torch.tensor([130, 70, 0, 257, 64, 100])
    B = int(counts.sum())
    idx = torch.repeat_interleave(torch.arange(E), counts).to(dev)
    xb = (torch.randn(B, 1, K, generator=g) * 0.5).to(torch.float16).to(dev)
    y = sw(xb, idx, sorted_indices=True)
    want = kq.gather_qmm(xb, sw.weight, None, "q4_k", rhs_indices=idx, sorted_indices=True).float() + \
        sw.bias[idx].unsqueeze(-2)
    assert tuple(y.shape) == (B, 1, N)
    assert float((y.float() - want).norm() / want.norm()) < 2e-3


@pytest.mark.gpu
@pytest.mark.parametrize("K", [1024, 288])      # integer-kernel shape; generic-kernel shape (K not a multiple of 256)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_qmv_bias_is_fused_with_one_rounding(K, dtype):
    dev = torch.device("cuda")
    N = 200
    w = random_wire("q8_0", N, K, seed=9, device=dev)
    x = torch.randn(1, 1, K, device=dev).to(dtype)
    out_dt = torch.bfloat16 if dtype == torch.float32 else dtype
    bias = (torch.randn(N, device=dev) * 3).to(out_dt)
    y = kq.quantized_matmul_qmv_bias(x, w, None, bias, "q8_0")
    assert tuple(y.shape) == (1, 1, N) and y.dtype == out_dt
    xr = x.to(torch.bfloat16) if dtype == torch.float32 else x
    exact = xr.double().reshape(1, K) @ kq.dequantize(w, None, "q8_0", torch.float32).double().T + bias.double()
    # one rounding of sum + bias: half an ulp of the output dtype plus the kernels' 2e-3 budget on the product
    ulp = 2.0 ** (-10 if out_dt == torch.float16 else -7)
    err = (y.double().reshape(1, N) - exact).abs()
    assert bool((err <= 0.5 * ulp * exact.abs() + 2e-3 * (exact - bias.double()).abs().max() + 1e-6).all())
    lin = KQuantLinear(K, N, bias=True, codec="q8_0").to(dev)
    lin.weight.copy_(w)
    lin.bias.copy_(bias.float())
    assert torch.equal(lin(x), y)
    with pytest.raises(ValueError):
        kq.quantized_matmul_qmv_bias(torch.cat([x, x]), w, None, bias, "q8_0")      # two rows
    with pytest.raises(ValueError):
        kq.quantized_matmul_qmv_bias(x, w, None, bias[:-1], "q8_0")
    with pytest.raises(ValueError):
        kq.quantized_matmul_qmv_bias(x, w, None, bias, "q4_k")


@pytest.mark.gpu
def test_multi_linear_both_orientations():
    from mlx_kquant_b200.nn import KQuantMultiLinear
    dev = torch.device("cuda")
    nh, out_dims, in_dims, B, L = 4, 64, 256, 2, 3
    ml = KQuantMultiLinear(in_dims, out_dims, nh, "q6_k").to(dev)
    ml.weight.copy_(random_wire("q6_k", out_dims, in_dims, seed=5, device=dev, lead=(nh,)))
    W = kq.dequantize(ml.weight.reshape(nh * out_dims, -1), None, "q6_k", torch.float32).reshape(nh, out_dims, in_dims).double()
    # transpose=True, per-head activations: [B, nh, L, in] @ W[h].T -> [B, nh, L, out]
    x = torch.randn(B, nh, L, in_dims, device=dev).to(torch.bfloat16)
    y = ml(x)
    want = torch.einsum("bhld,hod->bhlo", x.double(), W)
    assert tuple(y.shape) == (B, nh, L, out_dims)
    assert float((y.double() - want).norm() / want.norm()) < 4e-3
    # transpose=False, one activation shared by the heads: [B, 1, L, out] @ W[h] -> [B, nh, L, in]
    z = torch.randn(B, 1, L, out_dims, device=dev).to(torch.bfloat16)
    y2 = ml(z, transpose=False)
    want2 = torch.einsum("blo,hod->bhld", z[:, 0].double(), W)
    assert tuple(y2.shape) == (B, nh, L, in_dims)
    assert float((y2.double() - want2).norm() / want2.norm()) < 4e-3
    with pytest.raises(ValueError):
        ml(torch.zeros(B, 3, L, in_dims, device=dev, dtype=torch.bfloat16))
