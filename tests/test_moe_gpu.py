"""MoE SwiGLU composition (benchmark config 4, scaled down) against the oracle:
three reference-order gather_qmm calls with bf16 intermediates and float32
activation / mixing, plus an all-float reference for information."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import rel_fro
from gpu_util import mint_wire
from mlx_kquant_b200.moe import moe_glu, route_topk
from oracle.kq_oracle import bf16_bits_to_f32, f32_to_bf16_bits

pytestmark = pytest.mark.gpu


def oracle_moe(oracle, x_bits, wg, wu, wd, ids, probs, codec):
    T, k = ids.shape
    tok = np.repeat(np.arange(T), k).astype(np.uint32)
    e = ids.reshape(-1).astype(np.uint32)
    x3 = x_bits.reshape(T, 1, -1)
    g = bf16_bits_to_f32(oracle.gather_qmm(x3, wg, tok, e, codec, "bf16"))
    u = bf16_bits_to_f32(oracle.gather_qmm(x3, wu, tok, e, codec, "bf16"))
    h = f32_to_bf16_bits((g / (1.0 + np.exp(-g.astype(np.float64)))).astype(np.float32) * u)
    d = bf16_bits_to_f32(oracle.gather_qmm(h, wd, np.arange(T * k, dtype=np.uint32), e, codec, "bf16"))
    return (d.reshape(T, k, -1) * probs[:, :, None]).sum(axis=1)


@pytest.mark.parametrize("T", [1, 40, 256])   # 256 tokens x top-4 = 1024 routed rows: the grouped tile-kernel regime
def test_moe_glu_matches_oracle_composition(oracle, T):
    codec, E, H, F, k = "q4_k", 16, 512, 256, 4
    rng = np.random.default_rng(4000 + T)
    wg = np.stack([mint_wire(codec, rng.normal(0, 0.02, (F, H)).astype(np.float32)) for _ in range(E)])
    wu = np.stack([mint_wire(codec, rng.normal(0, 0.02, (F, H)).astype(np.float32)) for _ in range(E)])
    wd = np.stack([mint_wire(codec, rng.normal(0, 0.02, (H, F)).astype(np.float32)) for _ in range(E)])
    x = torch.from_numpy(rng.normal(0, 1, (T, H)).astype(np.float32)).to(torch.bfloat16)
    logits = torch.from_numpy(rng.normal(0, 1, (T, E)).astype(np.float32))
    ids, probs = route_topk(logits.cuda(), k)
    assert torch.allclose(probs.sum(-1), torch.ones(T, device="cuda"), atol=1e-6)
    y = moe_glu(x.cuda(), torch.from_numpy(wg).cuda(), torch.from_numpy(wu).cuda(), torch.from_numpy(wd).cuda(),
                codec, ids, probs)
    assert tuple(y.shape) == (T, H) and y.dtype == torch.bfloat16
    x_bits = x.view(torch.int16).numpy().view(np.uint16)
    want = oracle_moe(oracle, x_bits, wg, wu, wd, ids.cpu().numpy(), probs.cpu().numpy(), codec)
    err = rel_fro(y.float().cpu().numpy(), want)
    assert err < 6e-3, err      # three chained bf16 roundings (gate/up, h, down) + the bf16 output
    # gate | up as one stacked weight matrix: one gather_qmm instead of two, same numbers up to summation order
    from mlx_kquant_b200.moe import fuse_gate_up
    wgu = fuse_gate_up(torch.from_numpy(wg).cuda(), torch.from_numpy(wu).cuda())
    y2 = moe_glu(x.cuda(), None, None, torch.from_numpy(wd).cuda(), codec, ids, probs, w_gate_up=wgu)
    assert rel_fro(y2.float().cpu().numpy(), want) < 6e-3


def test_swiglu_and_combine_kernels_match_torch():
    from mlx_kquant_b200.moe import combine, swiglu
    g = torch.Generator(device="cpu").manual_seed(5)
    for dt in (torch.bfloat16, torch.float16):
        gu = (torch.randn(37, 2 * 264, generator=g) * 3).to(dt).cuda()
        got = swiglu(gu[:, :264], gu[:, 264:])
        want = (torch.nn.functional.silu(gu[:, :264].float()) * gu[:, 264:].float()).to(dt)
        assert torch.allclose(got.float(), want.float(), rtol=2 ** -7 if dt == torch.bfloat16 else 2 ** -10, atol=1e-6)
        d = torch.randn(5 * 4, 520, generator=g).to(dt).cuda()
        p = torch.rand(5, 4, generator=g).cuda()
        got = combine(d, p, 4)
        want = (d.reshape(5, 4, 520).float() * p.reshape(5, 4, 1)).sum(1).to(dt)
        assert torch.allclose(got.float(), want.float(), rtol=2 ** -7 if dt == torch.bfloat16 else 2 ** -10, atol=1e-5)


def test_topk_ties_go_to_the_lowest_index():
    logits = torch.zeros(2, 8)
    ids, probs = route_topk(logits, 3)
    assert ids.tolist() == [[0, 1, 2], [0, 1, 2]]
    assert torch.allclose(probs, torch.full((2, 3), 1 / 3))
