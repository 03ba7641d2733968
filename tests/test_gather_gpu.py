"""gather_qmm on the GPU against the CPU restatement of the reference's
KQuantGatherQMM::eval_cpu (src/kquant_gather.cpp:496-731)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import mlx_kquant_b200 as kq
from conftest import assert_close, rel_fro
from gpu_util import mint_wire, x_to_torch, y_to_f32
from oracle.kq_oracle import to_f32

pytestmark = pytest.mark.gpu
TOL = 2e-3


def make_experts(codec, E, N, K, seed):
    rng = np.random.default_rng(seed)
    return np.stack([mint_wire(codec, rng.normal(0, 0.02, (N, K)).astype(np.float32)) for _ in range(E)])


def fp64_ref(oracle, store, dt, wire, codec, lhs, rhs):
    xs = to_f32(store, dt).astype(np.float64)
    Wd = oracle.dequantize(wire, codec, "f32").astype(np.float64)
    return np.stack([xs[l] @ Wd[r].T for l, r in zip(lhs.ravel(), rhs.ravel())])


@pytest.mark.parametrize("codec", ["q4_k", "q6_k", "q8_0", "iq4_xs", "iq2_xxs", "q2_k", "q3_k", "q5_k", "q4_0", "iq4_nl"])
@pytest.mark.parametrize("M", [1, 3])
def test_gather_sweep(oracle, codec, M):
    # B = 8 entries, lhs = arange and reversed-with-repeat (tests/test_cpu_decode.py:186-224)
    E, N, K, B = 4, 64, 512, 8
    wire = make_experts(codec, E, N, K, seed=21)
    x, store = x_to_torch(np.random.default_rng(22).normal(0, 1, (B, M, K)).astype(np.float32), "f16")
    wd = torch.from_numpy(wire).cuda()
    rhs = np.array([0, 3, 1, 1, 2, 0, 3, 3], np.uint32)
    for lhs in (np.arange(B, dtype=np.uint32), np.array([7, 6, 5, 4, 3, 3, 1, 0], np.uint32)):
        y = kq.gather_qmm(x, wd, None, codec, lhs_indices=torch.from_numpy(lhs.astype(np.int64)),
                          rhs_indices=torch.from_numpy(rhs.astype(np.int64)))
        assert tuple(y.shape) == (B, M, N) and y.dtype == torch.float16
        ref = fp64_ref(oracle, store, "f16", wire, codec, lhs, rhs)
        assert_close(y_to_f32(y), ref, "f16", TOL)
        cpu = oracle.gather_qmm(store, wire, lhs, rhs, codec, "f16").astype(np.float32)
        assert rel_fro(y_to_f32(y), cpu) <= TOL


def test_gather_defaults_and_index_shapes(oracle):
    # rhs only (the MoE call): lhs defaults to arange over x's batch dims; 2-D index tensors keep their shape
    codec, E, N, K = "q4_k", 8, 96, 512
    wire = make_experts(codec, E, N, K, seed=31)
    wd = torch.from_numpy(wire).cuda()
    x, store = x_to_torch(np.random.default_rng(32).normal(0, 1, (6, 1, K)).astype(np.float32), "bf16")
    rhs = np.array([5, 5, 0, 7, 2, 5], np.uint32)
    y = kq.gather_qmm(x, wd, None, codec, rhs_indices=torch.from_numpy(rhs.astype(np.int64)).cuda())
    assert tuple(y.shape) == (6, 1, N) and y.dtype == torch.bfloat16
    ref = fp64_ref(oracle, store, "bf16", wire, codec, np.arange(6), rhs)
    assert rel_fro(y_to_f32(y), ref) <= TOL
    # broadcast: one token against top-k experts, indices shaped [1, 4]
    rhs2 = torch.tensor([[1, 3, 4, 6]])
    lhs2 = torch.zeros((1, 1), dtype=torch.int64)
    y2 = kq.gather_qmm(x, wd, None, codec, lhs_indices=lhs2, rhs_indices=rhs2)
    assert tuple(y2.shape) == (1, 4, 1, N)
    ref2 = fp64_ref(oracle, store, "bf16", wire, codec, np.zeros(4, int), np.array([1, 3, 4, 6]))
    assert rel_fro(y_to_f32(y2).reshape(4, 1, N), ref2) <= TOL
    # no indices at all is a plain matmul (src/kquant_ops.cpp:303-312)
    y3 = kq.gather_qmm(x[:, 0], wd[0], None, codec)
    assert torch.equal(y3, kq.quantized_matmul(x[:, 0], wd[0], None, codec))


def test_duplicates_match_singletons_bitwise(oracle):
    # repeated (lhs, rhs) pairs give bit-identical rows (tests/test_gather.py:253-321)
    codec, E, N, K = "q4_k", 3, 64, 512
    wire = make_experts(codec, E, N, K, seed=41)
    wd = torch.from_numpy(wire).cuda()
    x, _ = x_to_torch(np.random.default_rng(42).normal(0, 1, (4, 1, K)).astype(np.float32), "f16")
    lhs = torch.tensor([2, 2, 2, 0, 2])
    rhs = torch.tensor([1, 1, 1, 1, 1])
    y = kq.gather_qmm(x, wd, None, codec, lhs_indices=lhs, rhs_indices=rhs)
    single = kq.gather_qmm(x, wd, None, codec, lhs_indices=torch.tensor([2]), rhs_indices=torch.tensor([1]))
    for i in (0, 1, 2, 4):
        assert torch.equal(y[i], single[0])


def test_sorted_large_group_and_strided_experts(oracle):
    # 700 rows sorted by expert (prefill shape, groups far above 16 rows) through a strided expert view:
    # the gate half of a fused [E, 2N, bytes] gate_up tensor (src/kquant_ops.cpp:24-49)
    codec, E, N, K, B = "q4_k", 4, 48, 512, 700
    fused = make_experts(codec, E, 2 * N, K, seed=51)
    fd = torch.from_numpy(fused).cuda()
    gate = fd[:, :N, :]
    assert not gate.is_contiguous()
    x, store = x_to_torch(np.random.default_rng(52).normal(0, 1, (B, 1, K)).astype(np.float32), "bf16")
    rhs = np.sort(np.random.default_rng(53).integers(0, E, B)).astype(np.uint32)
    y = kq.gather_qmm(x, gate, None, codec, rhs_indices=torch.from_numpy(rhs.astype(np.int64)), sorted_indices=True)
    ref = fp64_ref(oracle, store, "bf16", fused[:, :N, :], codec, np.arange(B), rhs)
    assert_close(y_to_f32(y), ref, "bf16", TOL)
    # sorted and shuffled orders agree row for row
    perm = np.random.default_rng(54).permutation(B)
    y_sh = kq.gather_qmm(x, gate, None, codec, lhs_indices=torch.from_numpy(perm), rhs_indices=torch.from_numpy(rhs[perm].astype(np.int64)))
    assert torch.equal(y_sh, y[torch.from_numpy(perm).cuda()])


def test_many_rows_regression():
    # more than 32767 routed rows in one call (tests/test_gather.py:197-250), K = 256
    codec, E, N, K, B = "q8_0", 2, 16, 256, 33000
    wire = make_experts(codec, E, N, K, seed=61)
    wd = torch.from_numpy(wire).cuda()
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(B, 1, K, device="cuda", generator=g).half()
    rhs = (torch.arange(B, device="cuda") * 2 // B).to(torch.int64)
    y = kq.gather_qmm(x, wd, None, codec, rhs_indices=rhs, sorted_indices=True)
    half = B // 2
    want0 = kq.quantized_matmul(x[:half, 0], wd[0], None, codec).float()   # dense tile kernel: fp16-rounded weights
    want1 = kq.quantized_matmul(x[half:, 0], wd[1], None, codec).float()
    e0 = (y[:half, 0].float() - want0).norm() / want0.norm()
    e1 = (y[half:, 0].float() - want1).norm() / want1.norm()
    assert float(e0) < TOL and float(e1) < TOL


@pytest.mark.parametrize("B", [12, 640])
def test_out_of_range_expert_ids_are_skipped(oracle, B):
    # Entries whose expert index is >= the expert count belong to no group: the other entries' rows are
    # computed as usual (both regimes: task lists at B = 12, the grouped tile kernel at B = 640).
    codec, E, N, K = "q4_k", 4, 64, 512
    wire = make_experts(codec, E, N, K, seed=71)
    wd = torch.from_numpy(wire).cuda()
    x, store = x_to_torch(np.random.default_rng(72).normal(0, 1, (B, 1, K)).astype(np.float32), "bf16")
    rhs = np.random.default_rng(73).integers(0, E, B).astype(np.int64)
    bad = np.arange(B) % 5 == 2
    rhs_bad = rhs.copy()
    rhs_bad[bad] = E + 3
    y = kq.gather_qmm(x, wd, None, codec, rhs_indices=torch.from_numpy(rhs_bad))
    good = kq.gather_qmm(x, wd, None, codec, rhs_indices=torch.from_numpy(rhs))
    torch.cuda.synchronize()
    keep = torch.from_numpy(~bad).cuda()
    ref = fp64_ref(oracle, store, "bf16", wire, codec, np.arange(B), rhs)
    assert rel_fro(y_to_f32(good), ref) <= TOL
    assert rel_fro(y_to_f32(y[keep]), ref[~bad]) <= TOL


@pytest.mark.parametrize("codec", ["q4_k", "q8_0", "iq4_xs", "q5_1"])
@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_gather_transpose_false(oracle, codec, dt):
    # [K, N] expert matrices: entry e is x[lhs[e]] @ dequant(w[rhs[e]]); an out-of-range expert index is skipped
    E, K, N, B, M = 3, 40, 512, 5, 2
    wire = make_experts(codec, E, K, N, seed=81)        # E matrices of K rows, N weights per row
    wd = torch.from_numpy(wire).cuda()
    x, store = x_to_torch(np.random.default_rng(82).normal(0, 1, (B, M, K)).astype(np.float32), dt)
    lhs = np.array([4, 0, 0, 2, 3, 1], np.int64)
    rhs = np.array([2, 0, 1, 1, 2, 0], np.int64)
    y = kq.gather_qmm(x, wd, None, codec, lhs_indices=torch.from_numpy(lhs), rhs_indices=torch.from_numpy(rhs),
                      transpose=False)
    assert tuple(y.shape) == (6, M, N)
    xs = to_f32(store, dt).astype(np.float64)
    Wd = oracle.dequantize(wire, codec, "f32").astype(np.float64)
    ref = np.stack([xs[l] @ Wd[r] for l, r in zip(lhs, rhs)])
    assert_close(y_to_f32(y), ref, dt, TOL)
    rhs_bad = rhs.copy()
    rhs_bad[1] = E + 1
    y2 = kq.gather_qmm(x, wd, None, codec, lhs_indices=torch.from_numpy(lhs), rhs_indices=torch.from_numpy(rhs_bad),
                       transpose=False)
    keep = [0, 2, 3, 4, 5]
    assert torch.equal(y2[keep], y[keep])


@pytest.mark.parametrize("scale", [1e-6, 1e-9])
def test_gather_small_magnitude_rows(oracle, scale):
    """Rows of bfloat16 activations far below fp16's normal range keep their accuracy through the fp16 copy
    that the q4_k task kernel and the grouped tile kernel read (both regimes: 8 and 600 entries)."""
    codec, E, N, K = "q4_k", 4, 64, 512
    wire = make_experts(codec, E, N, K, seed=61)
    wd = torch.from_numpy(wire).cuda()
    for B in (8, 600):
        rng = np.random.default_rng(62 + B)
        x, store = x_to_torch((rng.normal(0, 1, (B, 1, K)) * scale).astype(np.float32), "bf16")
        rhs = rng.integers(0, E, B).astype(np.uint32)
        y = kq.gather_qmm(x, wd, None, codec, rhs_indices=torch.from_numpy(rhs.astype(np.int64)).cuda())
        ref = fp64_ref(oracle, store.reshape(B, K), "bf16", wire, codec, np.arange(B), rhs)
        assert_close(y_to_f32(y).reshape(B, N), ref, "bf16", TOL)


@pytest.mark.parametrize("B", [12, 640])
def test_out_of_range_activation_indices_are_skipped(oracle, B):
    """Entries whose lhs index is >= the number of activation slots read nothing and leave their output rows
    unwritten, like entries with an out-of-range expert (both regimes). Called through the C-ABI: the Python
    op would reject such indices earlier."""
    from mlx_kquant_b200 import _lib
    L = _lib.lib()
    codec, E, N, K, XB = "q4_k", 4, 64, 512, 9
    wire = make_experts(codec, E, N, K, seed=91)
    wd = torch.from_numpy(wire).cuda()
    x, store = x_to_torch(np.random.default_rng(92).normal(0, 1, (XB, 1, K)).astype(np.float32), "bf16")
    rng = np.random.default_rng(93)
    rhs = rng.integers(0, E, B).astype(np.int32)
    lhs = rng.integers(0, XB, B).astype(np.int32)
    bad = np.arange(B) % 7 == 3
    lhs_bad = lhs.copy()
    lhs_bad[bad] = XB + 100
    y = torch.full((B, 1, N), 7.0, dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(L.kq_gather_qmm_workspace_bytes(B, 1, E, K), dtype=torch.uint8, device="cuda")
    lt, rt = torch.from_numpy(lhs_bad).cuda(), torch.from_numpy(rhs).cuda()
    _lib.check(L.kq_gather_qmm(x.data_ptr(), _lib.KQ_BF16, XB, 1, K, wd.data_ptr(), E, wd.stride(0), wd.shape[2], N,
                               codec.encode(), lt.data_ptr(), rt.data_ptr(), B, 1, 0, y.data_ptr(), ws.data_ptr(),
                               ws.numel(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    ref = fp64_ref(oracle, store.reshape(XB, K), "bf16", wire, codec, lhs, rhs)
    got = y_to_f32(y).reshape(B, N)
    assert rel_fro(got[~bad], ref[~bad]) <= TOL
    assert (got[bad] == 7.0).all()
