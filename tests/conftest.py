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


def max_rel_to_peak(got: np.ndarray, want: np.ndarray) -> float:
    got = got.astype(np.float64)
    want = want.astype(np.float64)
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))
