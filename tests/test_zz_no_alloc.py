"""kq_gather_qmm_noalloc: the gather entry point for callers that cannot allocate.

Some users of this library may not call cudaMalloc at all - a plugin running
inside a host that owns the whole of HBM through its own arena, or a serving
loop that cannot afford the device-wide synchronisation an allocation implies.
For them the grouping scratch of gather_qmm sits in a fixed array inside the
library. This test calls that entry point straight through the C ABI, twice in
a row (the array keeps the first call's contents, so the second call proves the
counters are cleared), and requires the same bits as the ordinary entry point
with a caller-provided workspace. It also checks the size limit is enforced.

The file sorts last on purpose: a run that stops at the first failure has then
already executed every other test.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from mlx_kquant_b200 import _lib

pytestmark = pytest.mark.gpu

KQ_GATHER_STATIC_WS_BYTES = 1 << 20


def _wire(E, N, K, seed):
    # valid q4_k bytes: random quants and sub-scales, small finite fp16 d / dmin
    rng = np.random.default_rng(seed)
    nb = K // 256
    w = rng.integers(0, 256, (E, N, nb, 144), dtype=np.uint8)
    d = rng.uniform(0.001, 0.02, (E, N, nb)).astype(np.float16).view(np.uint16)
    for off in (0, 2):
        w[..., off] = (d & 0xFF).astype(np.uint8)
        w[..., off + 1] = (d >> 8).astype(np.uint8)
    return torch.from_numpy(w.reshape(E, N, nb * 144)).cuda()


def _call(L, fn, x, w, lhs, rhs, y, ws=None):
    E, N, rb = w.shape
    B, M, K = x.shape
    s = torch.cuda.current_stream().cuda_stream
    head = (x.data_ptr(), _lib.KQ_F16, B, M, K, w.data_ptr(), E, N * rb, rb, N, b"q4_k", lhs.data_ptr(),
            rhs.data_ptr(), lhs.numel(), 1, 0, y.data_ptr())
    if ws is None:
        return fn(*head, s)
    return fn(*head, ws.data_ptr(), ws.numel(), s)


def test_noalloc_matches_workspace_entry_point_twice():
    L = _lib.lib()
    E, N, K, M = 6, 80, 512, 1
    w = _wire(E, N, K, seed=77)
    g = torch.Generator(device="cuda").manual_seed(5)
    for n_entries, seed in ((40, 1), (23, 2)):          # second call: fewer entries, different routing
        x = torch.randn(n_entries, M, K, device="cuda", generator=g).half()
        rng = np.random.default_rng(seed)
        lhs = torch.from_numpy(rng.permutation(n_entries).astype(np.int32)).cuda()
        rhs = torch.from_numpy(rng.integers(0, E, n_entries).astype(np.int32)).cuda()
        want = torch.full((n_entries, M, N), float("nan"), dtype=torch.float16, device="cuda")
        got = torch.full_like(want, float("nan"))
        ws = torch.empty(L.kq_gather_qmm_workspace_bytes(n_entries, M, E, K), dtype=torch.uint8, device="cuda")
        _lib.check(_call(L, L.kq_gather_qmm, x, w, lhs, rhs, want, ws))
        _lib.check(_call(L, L.kq_gather_qmm_noalloc, x, w, lhs, rhs, got))
        torch.cuda.synchronize()
        assert not torch.isnan(got).any()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_noalloc_rejects_problems_beyond_the_fixed_array():
    L = _lib.lib()
    n_entries = 200_000
    assert L.kq_gather_qmm_workspace_bytes(n_entries, 1, 128, 0) > KQ_GATHER_STATIC_WS_BYTES
    # validation happens before any pointer is touched, so dummy non-null pointers are enough
    one = torch.zeros(16, dtype=torch.uint8, device="cuda")
    p = one.data_ptr()
    rc = L.kq_gather_qmm_noalloc(p, _lib.KQ_F16, 1, 1, 256, p, 128, 144, 144, 1, b"q4_k", p, p, n_entries, 1, 0, p, None)
    assert rc == _lib.KQ_ERR_INVALID_ARGUMENT
    assert b"too large for the built-in scratch" in L.kq_last_error()


def test_noalloc_checks_arguments_before_the_size_limit_and_only_where_scratch_is_used():
    """An unknown codec on an oversized call is reported as such, and the [K, N] orientation (transpose = 0),
    which uses no scratch, is not subject to the limit of the fixed array."""
    L = _lib.lib()
    one = torch.zeros(16, dtype=torch.uint8, device="cuda")
    p = one.data_ptr()
    rc = L.kq_gather_qmm_noalloc(p, _lib.KQ_F16, 1, 1, 256, p, 128, 144, 144, 1, b"q9_z", p, p, 200_000, 1, 0, p, None)
    assert rc == _lib.KQ_ERR_INVALID_ARGUMENT and b"Unknown kquant_type" in L.kq_last_error()
    # transpose = 0: w [E, K, bytes(N)], 100 000 entries (far beyond the limit of the other orientation)
    E, K, N, B = 2, 32, 256, 100_000
    w = _wire(E, K, N, seed=5)                       # [E, K rows, bytes of N weights]
    x = torch.randn(4, 1, K, device="cuda").half()
    rng = np.random.default_rng(6)
    lhs = torch.from_numpy(rng.integers(0, 4, B).astype(np.int32)).cuda()
    rhs = torch.from_numpy(rng.integers(0, E, B).astype(np.int32)).cuda()
    got = torch.empty(B, 1, N, dtype=torch.float16, device="cuda")
    want = torch.empty_like(got)
    s = torch.cuda.current_stream().cuda_stream
    args = (x.data_ptr(), _lib.KQ_F16, 4, 1, K, w.data_ptr(), E, w.stride(0), w.shape[2], N, b"q4_k", lhs.data_ptr(),
            rhs.data_ptr(), B, 0, 0)
    assert L.kq_gather_qmm_workspace_bytes(B, 1, E, 0) > KQ_GATHER_STATIC_WS_BYTES
    _lib.check(L.kq_gather_qmm_noalloc(*args, got.data_ptr(), s))
    ws = torch.empty(L.kq_gather_qmm_workspace_bytes(B, 1, E, K), dtype=torch.uint8, device="cuda")
    _lib.check(L.kq_gather_qmm(*args, want.data_ptr(), ws.data_ptr(), ws.numel(), s))
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
