"""The CPU oracle (oracle/kq_oracle.c) pinned against the reference.

Three independent anchors:
  * the committed golden vectors (tests/golden/kq_golden.npz), produced by the
    reference's own compiled CPU library from the reference's test fixtures and
    from seeded weights (tests/golden/make_golden.py);
  * gguf-py's decoders - the oracle the reference's own tests use
    (tests/test_cpu_decode.py:29-30, 96-107, 156);
  * the reference library itself, live, where it has been built.
"""
from __future__ import annotations

import numpy as np
import pytest

from conftest import imatrix_for, rel_fro
from oracle import kq_oracle
from oracle.kq_oracle import CODECS, GEOMETRY, bf16_bits_to_f32, from_f32, to_f32

KQUANTS = ["q2_k", "q3_k", "q4_k", "q5_k", "q6_k"]
GGUF_NAME = {"q2_k": "Q2_K", "q3_k": "Q3_K", "q4_k": "Q4_K", "q5_k": "Q5_K", "q6_k": "Q6_K", "q4_0": "Q4_0",
             "q8_0": "Q8_0", "iq4_nl": "IQ4_NL", "iq4_xs": "IQ4_XS", "iq2_xxs": "IQ2_XXS", "q4_1": "Q4_1", "q5_0": "Q5_0",
             "q5_1": "Q5_1", "iq3_xxs": "IQ3_XXS", "iq3_s": "IQ3_S", "iq2_xs": "IQ2_XS", "iq2_s": "IQ2_S",
             "iq1_s": "IQ1_S", "iq1_m": "IQ1_M", "mxfp4": "MXFP4", "nvfp4": "NVFP4"}


def bits(a):
    return a.view(np.uint32) if a.dtype == np.float32 else a.view(np.uint16)


@pytest.mark.parametrize("codec", KQUANTS)
def test_reference_fixtures_decode_bit_exact(oracle, golden, codec):
    got = oracle.dequantize(golden[f"fx_{codec}_wire"], codec, "f32")
    assert np.array_equal(bits(got), bits(golden[f"fx_{codec}_f32"]))
    got = oracle.dequantize(golden[f"fxmoe_{codec}_wire"], codec, "f32")
    assert got.shape == golden[f"fxmoe_{codec}_f32"].shape
    assert np.array_equal(bits(got), bits(golden[f"fxmoe_{codec}_f32"]))


@pytest.mark.parametrize("codec", CODECS)
@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_encoded_golden_decode_bit_exact(oracle, golden, codec, dt):
    got = oracle.dequantize(golden[f"enc_{codec}_wire"], codec, dt)
    assert np.array_equal(bits(got), bits(golden[f"enc_{codec}_{dt}"]) if dt == "f32" else golden[f"enc_{codec}_{dt}"])


@pytest.mark.parametrize("codec", CODECS)
def test_decode_matches_gguf_py(oracle, golden, codec):
    gguf = pytest.importorskip("gguf")
    wire = golden[f"enc_{codec}_wire"]
    want = gguf.quants.dequantize(wire, getattr(gguf.GGMLQuantizationType, GGUF_NAME[codec])).astype(np.float32)
    got = oracle.dequantize(wire, codec, "f32")
    assert np.array_equal(bits(got), bits(want))
    # f16 = one IEEE round-to-nearest-even of the exact f32 value
    assert np.array_equal(oracle.dequantize(wire, codec, "f16").view(np.uint16), want.astype(np.float16).view(np.uint16))


@pytest.mark.parametrize("codec", CODECS)
@pytest.mark.parametrize("M,dt", [(1, "f16"), (8, "f16"), (24, "bf16")])
def test_qmm_matches_golden(oracle, golden, codec, M, dt):
    x = from_f32(golden[f"x_m{M}"], dt)
    got = oracle.qmm(x, golden[f"enc_{codec}_wire"], codec, dt)
    want = golden[f"qmm_{codec}_m{M}_{dt}"]
    # Same association order as the reference; compilers may contract a*b+c
    # differently in the two builds, so allow the last bit of the 16-bit output.
    g = to_f32(got.view(np.uint16) if dt == "bf16" else got, dt)
    w = bf16_bits_to_f32(want) if dt == "bf16" else want.view(np.float16).astype(np.float32)
    assert rel_fro(g, w) < 1e-3
    assert np.mean(got.view(np.uint16) == want) > 0.95


@pytest.mark.parametrize("codec", CODECS)
def test_live_reference_agrees(oracle, ref, codec):
    rng = np.random.default_rng(123)
    K = 1024
    W = rng.normal(0, 0.02, (24, K)).astype(np.float32)
    if codec in kq_oracle.DECODE_ONLY:
        wire = kq_oracle.synthetic_wire(codec, 24, K, seed=9)
    else:
        wire = ref.quantize(W, codec, imatrix_for(codec, K), threads=2)
    wpb, bpb, _, _ = GEOMETRY[codec]
    assert wire.shape == (24, K // wpb * bpb)
    for dt in ("f32", "f16", "bf16"):
        assert oracle.dequantize(wire, codec, dt).tobytes() == ref.dequantize(wire, codec, dt).tobytes()
    for M in (1, 5, 16, 17):
        x = rng.normal(0, 1, (M, K)).astype(np.float16)
        a, b = oracle.qmm(x, wire, codec, "f16"), ref.qmm(x, wire, codec, "f16")
        assert rel_fro(a, b) < 1e-3


def test_gather_restatement_is_per_entry_qmm(oracle, golden):
    """kqo_gather_qmm must equal running the plain matmul on each expert's packed rows."""
    codec = "q4_k"
    wire = np.stack([golden[f"enc_{codec}_wire"], golden[f"enc_{codec}_wire"][::-1].copy()])  # 2 experts
    rng = np.random.default_rng(5)
    x = rng.normal(0, 1, (6, 1, 512)).astype(np.float16)
    lhs = np.array([0, 1, 2, 3, 4, 5, 5, 0], np.uint32)
    rhs = np.array([1, 0, 1, 1, 0, 0, 1, 1], np.uint32)
    got = oracle.gather_qmm(x, wire, lhs, rhs, codec, "f16")
    assert got.shape == (8, 1, 16)
    for b in range(8):
        want = oracle.qmm(x[lhs[b]], wire[rhs[b]], codec, "f16")
        assert np.array_equal(got[b].view(np.uint16), want.view(np.uint16))


def test_gather_large_group_takes_gemm_regime(oracle, golden):
    codec = "q6_k"
    wire = golden[f"enc_{codec}_wire"][None]
    rng = np.random.default_rng(6)
    x = rng.normal(0, 1, (20, 1, 512)).astype(np.float16)
    lhs = np.arange(20, dtype=np.uint32)
    rhs = np.zeros(20, np.uint32)
    got = oracle.gather_qmm(x, wire, lhs, rhs, codec, "f16")
    want = oracle.qmm(x[:, 0, :], wire[0], codec, "f16")  # M = 20 > 16: dequantize-then-GEMM order
    assert np.array_equal(got[:, 0, :].view(np.uint16), want.view(np.uint16))
