"""Shared test plumbing.

Markers: ``gpu`` = needs a CUDA device (the parity tests proper, which call the
CUDA kernels through the C-ABI). Everything else runs on CPU: the oracle against
the golden vectors, host-side logic, and the ABI's symbol table.

The CPU checkers under ``oracle/`` are test infrastructure; they are built on
first use with oracle/Makefile.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from oracle import kq_oracle  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    return kq_oracle.Oracle()


@pytest.fixture(scope="session")
def ref():
    """The reference's own compiled CPU library (encoder + decoder)."""
    if not kq_oracle.Ref.available():
        try:
            kq_oracle.build()
        except Exception:
            pass
    if not kq_oracle.Ref.available():
        pytest.skip("oracle/_ref/libkqref.so not built (needs the reference checkout)")
    return kq_oracle.Ref()


@pytest.fixture(scope="session")
def golden():
    return np.load(ROOT / "tests" / "golden" / "kq_golden.npz")


def imatrix_for(codec: str, K: int):
    """iq2_xxs cannot be encoded without an importance matrix (the reference
    rejects it, src/kquant_ops.cpp:594-599): use all-ones."""
    return np.ones(K, np.float32) if kq_oracle.GEOMETRY[codec][3] else None


def rel_fro(got: np.ndarray, want: np.ndarray) -> float:
    got = got.astype(np.float64)
    want = want.astype(np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


# Unit roundoff of the output type: the result is rounded ONCE from fp32 to it.
OUT_ULP = {"f16": 2.0 ** -11, "bf16": 2.0 ** -8, "f32": 2.0 ** -24}


def max_rel_to_peak(got: np.ndarray, want: np.ndarray, out_dtype: str = "f32") -> float:
    """max |got - want| / max |want| after discounting the unavoidable rounding of
    each element to the output dtype (half an ulp: up to 2^-8 relative for bf16,
    which alone exceeds 2e-3 of an element near the peak)."""
    got = got.astype(np.float64)
    want = want.astype(np.float64)
    excess = np.maximum(np.abs(got - want) - OUT_ULP[out_dtype] * np.abs(want), 0.0)
    return float(excess.max() / max(np.abs(want).max(), 1e-30))


def assert_close(got, ref, out_dtype: str, tol: float = 2e-3) -> None:
    """The matmul parity bar: relative Frobenius error <= tol and peak-normalised
    max error (beyond the output rounding) <= tol, against an fp64-accumulated
    reference of the fp32 math."""
    rf, mx = rel_fro(got, ref), max_rel_to_peak(got, ref, out_dtype)
    if rf > tol and out_dtype in ("f16", "bf16"):
        # On ~100 outputs the rounding of an exact result to bfloat16 alone can reach 2.1e-3 (2^-9 / sqrt(3) is
        # its expectation): measure against the reference rounded the same way before calling it a failure.
        r32 = np.asarray(ref, dtype=np.float64).astype(np.float32)
        if out_dtype == "f16":
            rounded = r32.astype(np.float16).astype(np.float64)
        else:
            rounded = kq_oracle.bf16_bits_to_f32(kq_oracle.f32_to_bf16_bits(r32)).astype(np.float64)
        rf = min(rf, rel_fro(got, rounded))
    assert rf <= tol, f"rel_fro {rf:.3e} > {tol}"
    assert mx <= tol, f"max/peak {mx:.3e} > {tol}"
