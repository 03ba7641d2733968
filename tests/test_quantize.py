"""kq.quantize (host encoder of the product) against the reference's CPU encoder: the bytes must be
identical. Pins: the committed golden wire bytes (made by the reference itself, tests/golden/make_golden.py)
and, when the compiled reference is present, fresh seeded matrices with and without an imatrix and in all
three input dtypes."""
import numpy as np
import pytest
import torch

import mlx_kquant_b200 as kq
from oracle import kq_oracle

BUILT = ("q8_0", "q4_0", "q2_k", "q3_k", "q4_k", "q5_k", "q6_k", "iq4_nl", "iq4_xs", "iq2_xxs", "q4_1", "q5_0", "q5_1")


@pytest.fixture(scope="module")
def golden():
    import pathlib
    return np.load(pathlib.Path(__file__).parent / "golden" / "kq_golden.npz")


@pytest.mark.parametrize("codec", BUILT)
def test_golden_wire_bytes(golden, codec):
    W = torch.from_numpy(golden["W"])
    im = torch.ones(W.shape[-1]) if codec == "iq2_xxs" else None  # as the fixture script does
    wq, scales = kq.quantize(W, codec, im)
    assert wq.dtype == torch.uint8 and tuple(scales.shape) == (1,)
    assert np.array_equal(wq.numpy(), golden[f"enc_{codec}_wire"])


@pytest.mark.parametrize("codec", BUILT)
@pytest.mark.parametrize("with_imatrix", [False, True])
def test_matches_reference_encoder(codec, with_imatrix):
    if not kq_oracle.Ref.available():
        pytest.skip("oracle/_ref/libkqref.so not built (needs the reference checkout)")
    ref = kq_oracle.Ref()
    rng = np.random.default_rng(11)
    K = 1024
    W = rng.normal(0, 0.02, (48, K)).astype(np.float32)
    W[3] = 0.0                      # an all-zero row
    W[5, :256] = 1e-3               # a constant superblock
    W[7] *= 50.0                    # large magnitudes
    if codec == "iq2_xxs" and not with_imatrix:
        pytest.skip("iq2_xxs cannot be encoded without an imatrix")
    im = (rng.uniform(0.1, 4.0, K).astype(np.float32)) if with_imatrix else None
    want = ref.quantize(W, codec, im, threads=4)
    got, _ = kq.quantize(torch.from_numpy(W), codec, None if im is None else torch.from_numpy(im))
    assert np.array_equal(got.numpy(), want)


@pytest.mark.parametrize("codec", ("q4_k", "q6_k", "q8_0"))
@pytest.mark.parametrize("dt", (torch.float16, torch.bfloat16))
def test_half_inputs_encode_like_their_float_values(codec, dt):
    W = (torch.randn(8, 512, generator=torch.Generator().manual_seed(3)) * 0.02).to(dt)
    a, _ = kq.quantize(W, codec)
    b, _ = kq.quantize(W.float(), codec)
    assert torch.equal(a, b)


def test_leading_dims_and_threads_do_not_change_bytes():
    W = torch.randn(4, 6, 256, generator=torch.Generator().manual_seed(4)) * 0.02
    a, _ = kq.quantize(W, "q5_k")
    assert tuple(a.shape) == (4, 6, 176)
    rows = torch.stack([kq.quantize(r, "q5_k")[0] for r in W.reshape(24, 256)]).reshape(4, 6, 176)
    assert torch.equal(a, rows)


def test_argument_errors():
    W = torch.zeros(2, 256)
    with pytest.raises(ValueError, match="Unknown kquant_type"):
        kq.quantize(W, "q9_z")
    with pytest.raises(ValueError, match="multiple of weights_per_block"):
        kq.quantize(torch.zeros(2, 100), "q4_k")
    with pytest.raises(ValueError, match="imatrix must be float32"):
        kq.quantize(W, "q4_k", torch.zeros(256, dtype=torch.float64))
    with pytest.raises(ValueError, match="imatrix shape"):
        kq.quantize(W, "q4_k", torch.zeros(128))
    with pytest.raises(ValueError, match="real floating"):
        kq.quantize(torch.zeros(2, 256, dtype=torch.int32), "q4_k")
    with pytest.raises((ValueError, RuntimeError), match="requires an importance matrix"):
        kq.quantize(W, "iq2_xxs")
