"""expert_tile_map / gather_qmm_seg against the per-segment quantized_matmul loop, as the reference tests
them (tests/test_switch_gemm.py:145-310; the ops are Metal-only there, so the loop is the oracle)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import mlx_kquant_b200 as kq
from mlx_kquant_b200.moe import host_tile_maps
from mlx_kquant_b200.synth import random_wire

TOL = 2e-3


def _indices(counts):
    return torch.from_numpy(np.repeat(np.arange(len(counts), dtype=np.int32), counts)).cuda()


def _loop(x, w, codec, counts):
    outs, start = [], 0
    for e in np.flatnonzero(counts):
        c = int(counts[e])
        outs.append(kq.quantized_matmul(x[start:start + c], w[e], None, codec))
        start += c
    return torch.cat(outs)


def _rel(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-6))


@pytest.mark.gpu
@pytest.mark.parametrize("codec", ["iq2_xxs", "q2_k", "q8_0", "q4_k", "q6_k"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_gather_qmm_seg_matches_loop(codec, dtype):
    E, N, K = 8, 192, 512
    w = random_wire(codec, N, K, seed=7, device=torch.device("cuda"), lead=(E,))
    # ragged segments: absent experts and partial pieces at every boundary class
    counts = np.zeros(E, dtype=np.int64)
    counts[[0, 1, 2, 3, 4, 5, 7]] = [1, 17, 63, 96, 129, 200, 48]
    rows = int(counts.sum())
    g = torch.Generator(device="cpu").manual_seed(23)
    x = (torch.randn(rows, K, generator=g) * 0.1).to(dtype).cuda()
    ref = _loop(x, w, codec, counts)
    for label, maps in (("host", host_tile_maps(counts, device="cuda")),
                        ("gpu", kq.expert_tile_map(_indices(counts), E))):
        got = kq.gather_qmm_seg(x, w, None, codec, *maps)
        assert tuple(got.shape) == (rows, N) and got.dtype == ref.dtype
        assert _rel(got, ref) < TOL, (codec, dtype, label)


@pytest.mark.gpu
def test_gather_qmm_seg_unaligned_n_and_float32():
    E, N, K = 4, 72, 512          # N not a multiple of the tile width
    w = random_wire("iq2_xxs", N, K, seed=31, device=torch.device("cuda"), lead=(E,))
    counts = np.array([65, 0, 3, 64], dtype=np.int64)
    rows = int(counts.sum())
    g = torch.Generator(device="cpu").manual_seed(32)
    x = (torch.randn(rows, K, generator=g) * 0.1).cuda()
    for dt in (torch.float16, torch.float32):
        xd = x.to(dt)
        got = kq.gather_qmm_seg(xd, w, None, "iq2_xxs", *host_tile_maps(counts, device="cuda"))
        ref = _loop(xd, w, "iq2_xxs", counts)
        assert tuple(got.shape) == (rows, N) and got.dtype == ref.dtype
        assert _rel(got, ref) < TOL


@pytest.mark.gpu
def test_gather_qmm_seg_large_segments_and_irregular_map():
    # a 700-row segment is re-cut into 256-row tiles; a map whose pieces of one expert are two separate runs
    # (not what either builder makes) is taken piece by piece
    E, N, K = 3, 256, 1024
    w = random_wire("q4_k", N, K, seed=41, device=torch.device("cuda"), lead=(E,))
    counts = np.array([700, 5, 300], dtype=np.int64)
    rows = int(counts.sum())
    g = torch.Generator(device="cpu").manual_seed(42)
    x = (torch.randn(rows, K, generator=g) * 0.1).to(torch.bfloat16).cuda()
    ref = _loop(x, w, "q4_k", counts)
    got = kq.gather_qmm_seg(x, w, None, "q4_k", *kq.expert_tile_map(_indices(counts), E))
    assert _rel(got, ref) < TOL
    m = torch.tensor([[0, 0, 64], [2, 64, 300], [0, 364, 40], [1, 404, 5]], dtype=torch.int32, device="cuda")
    cnt = torch.tensor([4], dtype=torch.int32, device="cuda")
    xs = x[:409]
    want = torch.cat([kq.quantized_matmul(xs[0:64], w[0], None, "q4_k"), kq.quantized_matmul(xs[64:364], w[2], None, "q4_k"),
                      kq.quantized_matmul(xs[364:404], w[0], None, "q4_k"), kq.quantized_matmul(xs[404:409], w[1], None, "q4_k")])
    assert _rel(kq.gather_qmm_seg(xs, w, None, "q4_k", m, cnt), want) < TOL


@pytest.mark.gpu
@pytest.mark.parametrize("counts", [[1, 63, 64, 129, 200, 0, 0, 32], [512], [0, 0, 0, 5], [64] * 8, [65] * 8,
                                    [1, 7, 8, 9, 16, 17, 48, 96]],
                         ids=["ragged", "single", "tiny", "uniform64", "uniform65", "sub_frag"])
def test_expert_tile_map_matches_host(counts):
    counts = np.asarray(counts, dtype=np.int64)
    mh, cnth = host_tile_maps(counts)
    m, cnt = kq.expert_tile_map(_indices(counts), len(counts))
    rows = int(counts.sum())
    assert tuple(m.shape) == (max(rows // 64 + min(len(counts), rows), 1), 3)
    assert int(cnt.item()) == int(cnth.item())
    got = m.cpu().numpy()[: int(cnt.item())]
    want = mh.numpy()[: int(cnt.item())]
    order = lambda a: a[np.lexsort(a.T[::-1])]   # tile order is unspecified
    np.testing.assert_array_equal(order(got), order(want))


def test_gather_qmm_seg_rejects_bad_inputs():
    K, N = 4096, 64
    x = torch.zeros((64, 512), dtype=torch.float16)
    w = torch.zeros((2, N, 1056), dtype=torch.uint8)          # iq2_xxs bytes per row for K = 4096
    good = torch.zeros((1, 3), dtype=torch.int32)
    cnt = torch.zeros(1, dtype=torch.int32)
    with pytest.raises(ValueError):                            # K mismatch
        kq.gather_qmm_seg(x, w, None, "iq2_xxs", good, cnt)
    x_ok = torch.zeros((64, K), dtype=torch.float16)
    with pytest.raises(ValueError):                            # bad map shape
        kq.gather_qmm_seg(x_ok, w, None, "iq2_xxs", torch.zeros(3, dtype=torch.int32), cnt)
    with pytest.raises(ValueError):                            # bad counts shape
        kq.gather_qmm_seg(x_ok, w, None, "iq2_xxs", good, torch.zeros(2, dtype=torch.int32))
    with pytest.raises(ValueError):                            # 3-D x
        kq.gather_qmm_seg(x_ok[None], w, None, "iq2_xxs", good, cnt)
    with pytest.raises(ValueError):                            # float weights
        kq.gather_qmm_seg(x_ok, w.float(), None, "iq2_xxs", good, cnt)
    with pytest.raises(ValueError):                            # unknown codec
        kq.gather_qmm_seg(x_ok, w, None, "q9_k", good, cnt)
    with pytest.raises(ValueError):
        kq.expert_tile_map(torch.zeros((2, 2), dtype=torch.int32), 4)
    with pytest.raises(ValueError):
        kq.expert_tile_map(torch.zeros(0, dtype=torch.int32), 4)
