"""The C-ABI library without a GPU: it loads, exports every symbol that
include/kquant_b200.h declares, carries the reference's codec geometry, and
rejects bad arguments with the reference's messages before touching CUDA."""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

import pytest
import torch

import mlx_kquant_b200 as kq
from mlx_kquant_b200 import _lib
from oracle.kq_oracle import CODECS, GEOMETRY

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "kquant_b200.h").read_text()
    return re.findall(r"KQ_API\s+[\w\s\*]+?\b(kq_\w+)\s*\(", text)


def test_header_symbols_all_exported():
    names = declared_symbols()
    assert len(names) >= 9
    handle = C.CDLL(str(_lib.LIB_PATH))
    for n in names:
        assert hasattr(handle, n), f"{n} declared in the header but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signatures out of sync with the header"


def test_registry_matches_reference_geometry():
    # src/kquant_codec.cpp:12-37: the ten in-scope rows, then q4_1, q5_0, q5_1
    assert kq.codecs() == CODECS
    for c in CODECS:
        assert kq.codec_geometry(c) == GEOMETRY[c]
    with pytest.raises(ValueError, match="Unknown kquant_type"):
        kq.codec_geometry("q9_z")


def test_abi_validation_needs_no_gpu():
    L = _lib.lib()
    assert L.kq_dequantize(None, 144, b"nope", 1, None, None) == _lib.KQ_ERR_INVALID_ARGUMENT
    assert b"[mlx_kquant.dequantize] Unknown kquant_type: 'nope'." == L.kq_last_error()
    assert L.kq_dequantize(None, 145, b"q4_k", 1, None, None) == _lib.KQ_ERR_INVALID_ARGUMENT
    assert b"must be a multiple of bytes_per_block (144)" in L.kq_last_error()
    assert L.kq_dequantize(None, 144, b"q4_k", 7, None, None) == _lib.KQ_ERR_INVALID_ARGUMENT
    # K mismatch: 2 blocks of q4_k = 512 weights but K = 256
    rc = L.kq_quantized_matmul(None, 1, 1, 256, 256, None, 288, 4, b"q4_k", 1, None, 4, None, 0, None)
    assert rc == _lib.KQ_ERR_INVALID_ARGUMENT and b"does not match the expanded quantized matrix inner dim (512)" in L.kq_last_error()
    # transpose = 0: w is [K, bytes(N)], so the row's expanded width (512) must equal N
    rc = L.kq_quantized_matmul(None, 1, 1, 512, 512, None, 288, 4, b"q4_k", 0, None, 4, None, 0, None)
    assert rc == _lib.KQ_ERR_INVALID_ARGUMENT and b"transpose=false" in L.kq_last_error()
    assert L.kq_quantized_matmul(None, 1, 0, 300, 300, None, 288, 512, b"q4_k", 0, None, 512, None, 0, None) == 0
    # zero-sized problems succeed without touching memory
    assert L.kq_dequantize(None, 0, b"q4_k", 1, None, None) == 0
    assert L.kq_quantized_matmul(None, 1, 0, 512, 512, None, 288, 4, b"q4_k", 1, None, 4, None, 0, None) == 0
    assert L.kq_quantized_matmul_workspace_bytes(1, 4096, 4096) == 0        # fp16 needs none
    assert L.kq_quantized_matmul_workspace_bytes(2, 4096, 4096) >= 4096 * 4096 * 2
    assert L.kq_quantized_matmul_workspace_bytes(2, 16, 4096) >= 16 * 4096 * 2  # optional fp16 copy of 2-16 rows
    assert L.kq_quantized_matmul_workspace_bytes(2, 1, 4096) == 0           # a single row never needs one
    assert L.kq_gather_qmm_workspace_bytes(8, 1, 128, 2048) > 0


def test_python_ops_validate_like_the_reference():
    w = torch.zeros(4, 144, dtype=torch.uint8)
    with pytest.raises(ValueError, match="w must be uint8"):
        kq.dequantize(w.float(), None, "q4_k")
    with pytest.raises(ValueError, match="Unknown kquant_type"):
        kq.dequantize(w, None, "q4_z")
    with pytest.raises(ValueError, match="multiple of bytes_per_block"):
        kq.dequantize(w[:, :100], None, "q4_k")
    with pytest.raises(RuntimeError, match="no CPU path"):
        kq.dequantize(w, None, "q4_k")  # CPU weights: fail loudly, never fall back
    with pytest.raises(ValueError, match="batched"):
        kq.quantized_matmul(torch.zeros(2, 1, 256), torch.zeros(2, 4, 144, dtype=torch.uint8), None, "q4_k")
    with pytest.raises(ValueError, match="does not match the expanded"):
        kq.quantized_matmul(torch.zeros(1, 512, dtype=torch.float16), w, None, "q4_k")
    with pytest.raises(ValueError, match="at least two dimensions"):
        kq.gather_qmm(torch.zeros(256), w[None], None, "q4_k", rhs_indices=torch.zeros(1, dtype=torch.int64))
