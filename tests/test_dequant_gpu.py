"""dequantize on the GPU must be bit-exact with the reference's CPU decoders for
float32 and float16 (and bfloat16), for all ten codecs (the reference pins f32
bit-exactness in tests/test_cpu_decode.py:156 and tests/test_codecs.py:154-159)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import mlx_kquant_b200 as kq
from gpu_util import TORCH_DT, mint_wire, np_bits, synthetic_wire, t2np_bits
from oracle.kq_oracle import CODECS, GEOMETRY

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("codec", CODECS)
@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_golden_bit_exact(golden, codec, dt):
    wire = torch.from_numpy(golden[f"enc_{codec}_wire"]).cuda()
    got = kq.dequantize(wire, None, codec, TORCH_DT[dt])
    want = golden[f"enc_{codec}_{dt}"]
    assert got.shape == want.shape
    assert np.array_equal(t2np_bits(got), np_bits(want) if dt == "f32" else want)


@pytest.mark.parametrize("codec", ["q2_k", "q3_k", "q4_k", "q5_k", "q6_k"])
def test_reference_fixtures_bit_exact(golden, codec):
    wire = torch.from_numpy(golden[f"fxmoe_{codec}_wire"]).cuda()      # [2, 4, bytes]: leading dims kept
    got = kq.dequantize(wire, None, codec, torch.float32)
    assert tuple(got.shape) == golden[f"fxmoe_{codec}_f32"].shape
    assert np.array_equal(t2np_bits(got), np_bits(golden[f"fxmoe_{codec}_f32"]))


@pytest.mark.parametrize("codec", CODECS)
def test_default_dtype_is_float16(golden, codec):
    wire = torch.from_numpy(golden[f"enc_{codec}_wire"]).cuda()
    assert kq.dequantize(wire, None, codec).dtype == torch.float16


@pytest.mark.parametrize("codec", CODECS)
@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_seeded_matrix_vs_oracle(oracle, codec, dt):
    # N(0, 0.02) weights as in the benchmark configs; rows x K large enough to span many CTA tiles,
    # with a ragged last tile (rows * K is not a multiple of the 8192-weight tile).
    rng = np.random.default_rng(42)
    rows, K = 67, 2048
    W = rng.normal(0, 0.02, (rows, K)).astype(np.float32)
    wire = mint_wire(codec, W)
    want = oracle.dequantize(wire, codec, dt)
    got = kq.dequantize(torch.from_numpy(wire).cuda(), None, codec, TORCH_DT[dt])
    assert np.array_equal(t2np_bits(got), np_bits(want))


@pytest.mark.parametrize("codec", CODECS)
def test_random_wire_bytes_and_single_block(oracle, codec):
    wpb, bpb, _, _ = GEOMETRY[codec]
    wire = synthetic_wire(codec, 33, wpb * 9, seed=7)          # every bit pattern of quants and scales
    want = oracle.dequantize(wire, codec, "f32")
    got = kq.dequantize(torch.from_numpy(wire).cuda(), None, codec, torch.float32)
    assert np.array_equal(t2np_bits(got), np_bits(want))
    one = wire[0, :bpb]                                          # 1-D input, exactly one block
    got1 = kq.dequantize(torch.from_numpy(one.copy()).cuda(), None, codec, torch.float16)
    assert tuple(got1.shape) == (wpb,)
    assert np.array_equal(t2np_bits(got1), np_bits(oracle.dequantize(one, codec, "f16")))


@pytest.mark.parametrize("codec", ["q4_k", "q6_k", "q8_0", "iq2_xxs"])
def test_unaligned_base_pointer(oracle, codec):
    # a view that starts one byte into an allocation: no 16-byte (or even 2-byte) alignment
    wpb, bpb, _, _ = GEOMETRY[codec]
    wire = synthetic_wire(codec, 5, wpb * 4, seed=3)
    buf = torch.zeros(wire.size + 1, dtype=torch.uint8, device="cuda")
    buf[1:] = torch.from_numpy(wire.reshape(-1)).cuda()
    view = buf[1:].view(5, -1)
    assert view.data_ptr() % 2 == 1
    got = kq.dequantize(view, None, codec, torch.float32)
    assert np.array_equal(t2np_bits(got), np_bits(oracle.dequantize(wire, codec, "f32")))


def test_empty_input():
    out = kq.dequantize(torch.zeros((3, 0), dtype=torch.uint8, device="cuda"), None, "q4_k")
    assert tuple(out.shape) == (3, 0)


def test_roundtrip_property_full_size(oracle):
    """Full benchmark shape [14336, 4096] q4_k: size-independent checks - decoding
    twice is idempotent, and a checksum over 64 sampled rows equals the oracle's."""
    rows, K = 14336, 4096
    wire = synthetic_wire("q4_k", rows, K, seed=11)
    dev = torch.from_numpy(wire).cuda()
    a = kq.dequantize(dev, None, "q4_k", torch.float16)
    b = kq.dequantize(dev, None, "q4_k", torch.float16)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    pick = np.linspace(0, rows - 1, 64).astype(int)
    want = oracle.dequantize(wire[pick], "q4_k", "f16")
    assert np.array_equal(t2np_bits(a[torch.from_numpy(pick).cuda()]), np_bits(want))
