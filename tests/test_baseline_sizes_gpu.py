"""The benchmark configurations at their FULL sizes against the oracle.

config 2  the ten codecs, W [14336, 4096] really encoded, decoded to float16 and float32: bit-exact.
config 3  q4_k / q6_k W [14336, 4096] really encoded, bfloat16 x [M, 4096], M in {128, 2048, 8192}, against the
          float64 product of the oracle's bit-exact dequantized weights (computed on the GPU).
config 4  128 experts x {gate, up [768, 2048], down [2048, 768]} q4_k really encoded, top-8 of 128:
          T in {1, 64} against the oracle's three-gather composition, T = 4096 against a float64 composition of
          the oracle-dequantized weights with the same bfloat16 intermediates.
config 5  iq4_xs / iq2_xxs W [28672, 8192], float16 x, M in {1, 4, 16}: 256 really-encoded rows against the
          oracle's CPU product, every row against the float64 product of the dequantized weights.

Encoding uses the reference's own encoder (oracle/_ref) on all host threads; iq2_xxs with the all-ones
importance matrix (the reference rejects None for it, src/kquant_ops.cpp:594-599). Tolerances as in
test_matmul_gpu.py (2e-3) and test_moe_gpu.py (6e-3 for the three chained bfloat16 roundings)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import mlx_kquant_b200 as kq
from conftest import OUT_ULP
from gpu_util import mint_wire, synthetic_wire, t2np_bits, np_bits
from mlx_kquant_b200.moe import fuse_gate_up, moe_glu, route_topk
from oracle import kq_oracle
from oracle.kq_oracle import bf16_bits_to_f32, f32_to_bf16_bits

pytestmark = pytest.mark.gpu
TEN = ("q2_k", "q3_k", "q4_k", "q5_k", "q6_k", "q4_0", "q8_0", "iq4_nl", "iq4_xs", "iq2_xxs")


def cpu_dequantize(oracle, wire, codec, dt):
    """The reference's own decoder when its library is built (threaded), else the C restatement (bit-identical)."""
    if kq_oracle.Ref.available():
        return kq_oracle.Ref().dequantize(wire, codec, dt)
    return oracle.dequantize(wire, codec, dt)


def close_on_gpu(got: torch.Tensor, ref64: torch.Tensor, out_dtype: str, tol: float):
    """conftest.assert_close on device tensors: relative Frobenius error and peak-normalised max error beyond
    the output rounding, both <= tol."""
    got = got.double()
    rf = float((got - ref64).norm() / ref64.norm())
    if rf > tol:   # measure against the reference rounded the same way before calling it a failure
        rounded = ref64.float().to(torch.float16 if out_dtype == "f16" else torch.bfloat16).double()
        rf = min(rf, float((got - rounded).norm() / rounded.norm()))
    excess = ((got - ref64).abs() - OUT_ULP[out_dtype] * ref64.abs()).clamp_min(0).max()
    mx = float(excess / ref64.abs().max())
    assert rf <= tol, f"rel_fro {rf:.3e} > {tol}"
    assert mx <= tol, f"max/peak {mx:.3e} > {tol}"


@pytest.fixture(scope="module")
def w_ffn():
    """The seeded N(0, 0.02) weight [14336, 4096] of configs 2 and 3."""
    return np.random.default_rng(1002).normal(0, 0.02, (14336, 4096)).astype(np.float32)


@pytest.mark.parametrize("codec", TEN)
def test_config2_dequantize_full_size_bit_exact(oracle, w_ffn, codec):
    wire = mint_wire(codec, w_ffn)
    wd = torch.from_numpy(wire).cuda()
    for dt, tdt in (("f32", torch.float32), ("f16", torch.float16)):
        got = kq.dequantize(wd, None, codec, tdt)
        assert tuple(got.shape) == w_ffn.shape
        want = torch.from_numpy(np_bits(cpu_dequantize(oracle, wire, codec, dt)).astype(np.int64)).cuda()
        bits = got.view(torch.int32 if dt == "f32" else torch.int16).to(torch.int64) & (0xFFFFFFFF if dt == "f32" else 0xFFFF)
        assert torch.equal(bits, want), f"{codec} -> {dt}: {int((bits != want).sum())} weights differ"
        del got, want, bits


@pytest.mark.parametrize("codec", ["q4_k", "q6_k"])
def test_config3_prefill_full_size(oracle, w_ffn, codec):
    wire = mint_wire(codec, w_ffn)
    wd = torch.from_numpy(wire).cuda()
    Wd64 = torch.from_numpy(cpu_dequantize(oracle, wire, codec, "f32")).cuda().double()
    for M in (128, 2048, 8192):
        g = torch.Generator(device="cuda").manual_seed(6000 + M)
        x = torch.randn(M, 4096, device="cuda", generator=g).to(torch.bfloat16)
        y = kq.quantized_matmul(x, wd, None, codec)
        assert tuple(y.shape) == (M, 14336) and y.dtype == torch.bfloat16
        close_on_gpu(y, x.double() @ Wd64.T, "bf16", 2e-3)
        del y


# ------------------------------------------------------------------------------------------ config 4
E4, H4, F4, K4 = 128, 2048, 768, 8


@pytest.fixture(scope="module")
def experts():
    rng = np.random.default_rng(4004)

    def stack(n, k):
        W = rng.normal(0, 0.02, (E4 * n, k)).astype(np.float32)
        return mint_wire("q4_k", W).reshape(E4, n, -1)

    return stack(F4, H4), stack(F4, H4), stack(H4, F4)


def oracle_moe(oracle, x_bits, wg, wu, wd, ids, probs):
    T, k = ids.shape
    tok = np.repeat(np.arange(T), k).astype(np.uint32)
    e = ids.reshape(-1).astype(np.uint32)
    x3 = x_bits.reshape(T, 1, -1)
    g = bf16_bits_to_f32(oracle.gather_qmm(x3, wg, tok, e, "q4_k", "bf16"))
    u = bf16_bits_to_f32(oracle.gather_qmm(x3, wu, tok, e, "q4_k", "bf16"))
    h = f32_to_bf16_bits((g / (1.0 + np.exp(-g.astype(np.float64)))).astype(np.float32) * u)
    d = bf16_bits_to_f32(oracle.gather_qmm(h, wd, np.arange(T * k, dtype=np.uint32), e, "q4_k", "bf16"))
    return (d.reshape(T, k, -1) * probs[:, :, None]).sum(axis=1)


@pytest.mark.parametrize("T", [1, 64])
def test_config4_moe_decode_sizes(oracle, experts, T):
    wg, wu, wd = experts
    rng = np.random.default_rng(4100 + T)
    x = torch.from_numpy(rng.normal(0, 1, (T, H4)).astype(np.float32)).to(torch.bfloat16)
    ids, probs = route_topk(torch.from_numpy(rng.normal(0, 1, (T, E4)).astype(np.float32)).cuda(), K4)
    wgu = fuse_gate_up(torch.from_numpy(wg).cuda(), torch.from_numpy(wu).cuda())
    y = moe_glu(x.cuda(), None, None, torch.from_numpy(wd).cuda(), "q4_k", ids, probs, w_gate_up=wgu)
    assert tuple(y.shape) == (T, H4) and y.dtype == torch.bfloat16
    want = oracle_moe(oracle, x.view(torch.int16).numpy().view(np.uint16), wg, wu, wd, ids.cpu().numpy(),
                      probs.cpu().numpy())
    got = y.float().cpu().numpy().astype(np.float64)
    err = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert err < 6e-3, err


def test_config4_moe_prefill_size(oracle, experts):
    """T = 4096 (32 768 routed rows, the grouped tile kernel): float64 composition on the GPU from the oracle's
    dequantized weights, with the composition's own bfloat16 roundings of gate / up, h and down."""
    wg, wu, wd = experts
    T = 4096
    g = torch.Generator(device="cuda").manual_seed(4200)
    x = torch.randn(T, H4, device="cuda", generator=g).to(torch.bfloat16)
    ids, probs = route_topk(torch.randn(T, E4, device="cuda", generator=g), K4)
    wgu = fuse_gate_up(torch.from_numpy(wg).cuda(), torch.from_numpy(wu).cuda())
    y = moe_glu(x, None, None, torch.from_numpy(wd).cuda(), "q4_k", ids, probs, w_gate_up=wgu)
    ref = torch.zeros(T, H4, dtype=torch.float64, device="cuda")
    bf = lambda t: t.float().to(torch.bfloat16).double()
    for e in range(E4):
        tok, slot = torch.nonzero(ids == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        Wg = torch.from_numpy(cpu_dequantize(oracle, wg[e], "q4_k", "f32")).cuda().double()
        Wu = torch.from_numpy(cpu_dequantize(oracle, wu[e], "q4_k", "f32")).cuda().double()
        Wdn = torch.from_numpy(cpu_dequantize(oracle, wd[e], "q4_k", "f32")).cuda().double()
        xe = x[tok].double()
        gate, up = bf(xe @ Wg.T), bf(xe @ Wu.T)
        h = bf(torch.nn.functional.silu(gate.float()).double() * up)
        d = bf(h @ Wdn.T)
        ref.index_add_(0, tok, d * probs[tok, slot].double()[:, None])
    err = float((y.double() - ref).norm() / ref.norm())
    assert err < 6e-3, err


# ------------------------------------------------------------------------------------------ config 5
@pytest.mark.parametrize("codec", ["iq4_xs", "iq2_xxs"])
def test_config5_iq_decode_full_size(oracle, codec):
    N, K, ENC = 28672, 8192, 256
    rng = np.random.default_rng(5005)
    wire = synthetic_wire(codec, N, K, seed=55)
    wire[:ENC] = mint_wire(codec, rng.normal(0, 0.02, (ENC, K)).astype(np.float32))
    wd = torch.from_numpy(wire).cuda()
    Wd64 = kq.dequantize(wd, None, codec, torch.float32).double()       # bit-exact against the oracle elsewhere
    enc64 = torch.from_numpy(cpu_dequantize(oracle, wire[:ENC], codec, "f32")).cuda().double()
    assert torch.equal(Wd64[:ENC], enc64)
    for M in (1, 4, 16):
        xh = rng.normal(0, 1, (M, K)).astype(np.float32).astype(np.float16)
        x = torch.from_numpy(xh).cuda()
        y = kq.quantized_matmul(x, wd, None, codec)
        assert tuple(y.shape) == (M, N) and y.dtype == torch.float16
        close_on_gpu(y, x.double() @ Wd64.T, "f16", 2e-3)
        # the really-encoded rows against the reference-order CPU product (src/kquant_cpu_decode.cpp:1032-1065)
        cpu = oracle.qmm(xh, wire[:ENC], codec, "f16").astype(np.float64)
        got = y[:, :ENC].float().cpu().numpy().astype(np.float64)
        assert np.linalg.norm(got - cpu) <= 2e-3 * np.linalg.norm(cpu)
