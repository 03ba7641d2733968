#!/usr/bin/env python3
"""Regenerate tests/golden/kq_golden.npz from the reference itself.

Needs the reference checkout (for its test fixtures) and the reference's CPU
library compiled by oracle/Makefile into oracle/_ref/libkqref.so. The produced
file is what travels: the parity tests only ever read the .npz.

Contents (all little-endian numpy arrays):
  fx_<codec>_wire / fx_<codec>_f32     the first 8 rows of the reference's own
      fixtures tests/fixtures/<codec>.npz (q2_k..q6_k; N=256, K=512, minted by
      tests/gen_fixtures.py:62-87) and the reference decode of them to float32.
  fxmoe_<codec>_wire / _f32            expert 0..1, first 4 rows of *_moe.npz.
  enc_<codec>_wire                     wire bytes made by the reference encoder
      from W = default_rng(7).normal(0, 0.02, (16, 512)) (iq2_xxs: all-ones
      imatrix, which the reference requires for that codec).
  enc_<codec>_f32 / _f16 / _bf16       the reference decode of those bytes
      (f16/bf16 as uint16 bit patterns).
  qmm_<codec>_m{1,8}_f16, qmm_<codec>_m24_bf16
      reference quantized_matmul outputs for x = default_rng(11 + M).normal(0, 1,
      (M, 512)) rounded to the dtype: M = 1, 8 take the fused GEMV regime, M = 24
      the dequantize-then-GEMM regime (src/kquant_cpu_decode.cpp:1254-1352).
  W, x_m1, x_m8, x_m24                 the float32 inputs.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle.kq_oracle import CODECS, DECODE_ONLY, GEOMETRY, Ref, from_f32, synthetic_wire  # noqa: E402


def main(ref_dir: str) -> None:
    ref = Ref()
    fx = Path(ref_dir) / "tests" / "fixtures"
    out: dict[str, np.ndarray] = {}
    for c in ("q2_k", "q3_k", "q4_k", "q5_k", "q6_k"):
        wire = np.load(fx / f"{c}.npz")["wire"][:8]
        out[f"fx_{c}_wire"] = wire
        out[f"fx_{c}_f32"] = ref.dequantize(wire, c, "f32")
        moe = np.load(fx / f"{c}_moe.npz")["wire"][:2, :4]
        out[f"fxmoe_{c}_wire"] = moe
        out[f"fxmoe_{c}_f32"] = ref.dequantize(moe, c, "f32")
    W = np.random.default_rng(7).normal(0, 0.02, (16, 512)).astype(np.float32)
    out["W"] = W
    xs = {M: np.random.default_rng(11 + M).normal(0, 1, (M, 512)).astype(np.float32) for M in (1, 8, 24)}
    for M, x in xs.items():
        out[f"x_m{M}"] = x
    for c in CODECS:
        im = np.ones(512, np.float32) if GEOMETRY[c][3] else None
        if c in DECODE_ONLY:   # no encoder in the reference: seeded valid bytes
            wire = synthetic_wire(c, W.shape[0], W.shape[1], seed=77)
        else:
            wire = ref.quantize(W, c, im, threads=1)
        out[f"enc_{c}_wire"] = wire
        for dt in ("f32", "f16", "bf16"):
            d = ref.dequantize(wire, c, dt)
            out[f"enc_{c}_{dt}"] = d if dt == "f32" else d.view(np.uint16)
        for M, dt in ((1, "f16"), (8, "f16"), (24, "bf16")):
            y = ref.qmm(from_f32(xs[M], dt), wire, c, dt)
            out[f"qmm_{c}_m{M}_{dt}"] = y.view(np.uint16)
    np.savez_compressed(Path(__file__).with_name("kq_golden.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    import os

    where = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("KQ_REFERENCE_DIR")
    if not where:
        sys.exit("usage: make_golden.py <reference checkout>   (or set KQ_REFERENCE_DIR)")
    main(where)
