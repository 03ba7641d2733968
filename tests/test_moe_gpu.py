"""MoE SwiGLU composition (benchmark config 4, scaled down) against the oracle:
three reference-order gather_qmm calls with bf16 intermediates and float32
activation / mixing, plus an all-float reference for information."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import rel_fro
from gpu_util import mint_wire
from mlx_kquant_b200.moe import moe_glu, route_topk
from oracle.kq_oracle import bf16_bits_to_f32, f32_to_bf16_bits

pytestmark = pytest.mark.gpu


def oracle_moe(oracle, x_bits, wg, wu, wd, ids, probs, codec):
    T, k = ids.shape
    tok = np.repeat(np.arange(T), k).astype(np.uint32)
    e = ids.reshape(-1).astype(np.uint32)
    x3 = x_bits.reshape(T, 1, -1)
    g = bf16_bits_to_f32(oracle.gather_qmm(x3, wg, tok, e, codec, "bf16"))
    u = bf16_bits_to_f32(oracle.gather_qmm(x3, wu, tok, e, codec, "bf16"))
    h = f32_to_bf16_bits((g / (1.0 + np.exp(-g.astype(np.float64)))).astype(np.float32) * u)
    d = bf16_bits_to_f32(oracle.gather_qmm(h, wd, np.arange(T * k, dtype=np.uint32), e, codec, "bf16"))
    return (d.reshape(T, k, -1) * probs[:, :, None]).sum(axis=1)


@pytest.mark.parametrize("T", [1, 40, 256])   # 256 tokens x top-4 = 1024 routed rows: the grouped tile-kernel regime
def test_moe_glu_matches_oracle_composition(oracle, T):
    codec, E, H, F, k = "q4_k", 16, 512, 256, 4
    rng = np.random.default_rng(4000 + T)
    wg = np.stack([mint_wire(codec, rng.normal(0, 0.02, (F, H)).astype(np.float32)) for _ in range(E)])
    wu = np.stack([mint_wire(codec, rng.normal(0, 0.02, (F, H)).astype(np.float32)) for _ in range(E)])
    wd = np.stack([mint_wire(codec, rng.normal(0, 0.02, (H, F)).astype(np.float32)) for _ in range(E)])
    x = torch.from_numpy(rng.normal(0, 1, (T, H)).astype(np.float32)).to(torch.bfloat16)
    logits = torch.from_numpy(rng.normal(0, 1, (T, E)).astype(np.float32))
    ids, probs = route_topk(logits.cuda(), k)
    assert torch.allclose(probs.sum(-1), torch.ones(T, device="cuda"), atol=1e-6)
    y = moe_glu(x.cuda(), torch.from_numpy(wg).cuda(), torch.from_numpy(wu).cuda(), torch.from_numpy(wd).cuda(),
                codec, ids, probs)
    assert tuple(y.shape) == (T, H) and y.dtype == torch.bfloat16
    x_bits = x.view(torch.int16).numpy().view(np.uint16)
    want = oracle_moe(oracle, x_bits, wg, wu, wd, ids.cpu().numpy(), probs.cpu().numpy(), codec)
    err = rel_fro(y.float().cpu().numpy(), want)
    assert err < 6e-3, err      # three chained bf16 roundings (gate/up, h, down) + the bf16 output
    # gate | up as one stacked weight matrix: one gather_qmm instead of two, same numbers up to summation order
    from mlx_kquant_b200.moe import fuse_gate_up
    wgu = fuse_gate_up(torch.from_numpy(wg).cuda(), torch.from_numpy(wu).cuda())
    y2 = moe_glu(x.cuda(), None, None, torch.from_numpy(wd).cuda(), codec, ids, probs, w_gate_up=wgu)
    assert rel_fro(y2.float().cpu().numpy(), want) < 6e-3


def test_swiglu_and_combine_kernels_match_torch():
    from mlx_kquant_b200.moe import combine, swiglu
    g = torch.Generator(device="cpu").manual_seed(5)
    for dt in (torch.bfloat16, torch.float16):
        gu = (torch.randn(37, 2 * 264, generator=g) * 3).to(dt).cuda()
        got = swiglu(gu[:, :264], gu[:, 264:])
        want = (torch.nn.functional.silu(gu[:, :264].float()) * gu[:, 264:].float()).to(dt)
        assert torch.allclose(got.float(), want.float(), rtol=2 ** -7 if dt == torch.bfloat16 else 2 ** -10, atol=1e-6)
        d = torch.randn(5 * 4, 520, generator=g).to(dt).cuda()
        p = torch.rand(5, 4, generator=g).cuda()
        got = combine(d, p, 4)
        want = (d.reshape(5, 4, 520).float() * p.reshape(5, 4, 1)).sum(1).to(dt)
        assert torch.allclose(got.float(), want.float(), rtol=2 ** -7 if dt == torch.bfloat16 else 2 ** -10, atol=1e-5)


def test_topk_ties_go_to_the_lowest_index():
    logits = torch.zeros(2, 8)
    ids, probs = route_topk(logits, 3)
    assert ids.tolist() == [[0, 1, 2], [0, 1, 2]]
    assert torch.allclose(probs, torch.full((2, 3), 1 / 3))


def test_routed_swiglu_and_partial_combine_skip_foreign_rows():
    # rows of experts another rank owns hold NaN here: the routed forms must neither read nor write them
    from mlx_kquant_b200.moe import combine_partial, swiglu
    g = torch.Generator(device="cpu").manual_seed(6)
    rows, F, H, k = 48, 128, 256, 4
    gu = torch.randn(rows, 2 * F, generator=g).to(torch.bfloat16).cuda()
    ids = torch.randint(-3, 9, (rows,), generator=g).to(torch.int32).cuda()     # 6 local experts: 0..5
    mine = (ids >= 0) & (ids < 6)
    gu[~mine] = float("nan")
    out = swiglu(gu[:, :F], gu[:, F:], row_expert=ids, n_experts=6)
    want = (torch.nn.functional.silu(gu[:, :F].float()) * gu[:, F:].float()).to(torch.bfloat16)
    assert torch.equal(out[mine], want[mine])
    d = torch.randn(rows, H, generator=g).to(torch.bfloat16).cuda()
    d[~mine] = float("nan")
    p = torch.rand(rows // k, k, generator=g).cuda()
    p = torch.where(mine.reshape(-1, k), p, torch.zeros_like(p))
    y = combine_partial(d, p, k)
    ref = (torch.nan_to_num(d.float()).reshape(-1, k, H) * p[:, :, None]).sum(1)
    assert y.dtype == torch.float32 and torch.isfinite(y).all()
    assert torch.allclose(y, ref, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("T,E", [(24, 16), (320, 8)])   # task lists; grouped tile kernel (2560 routed rows, 4 local experts)
def test_gathered_expert_parallel_two_virtual_ranks(T, E):
    # Two ranks emulated on one GPU without a communicator: the all-gather is a concatenation of the two
    # packed send buffers and the reduce-scatter a sum of the two partial buffers.
    from mlx_kquant_b200.dist import shard_bounds
    from mlx_kquant_b200.moe import GatheredExpertParallel, fuse_gate_up
    from mlx_kquant_b200.synth import random_wire
    dev = torch.device("cuda")
    H, F, k, W = 512, 256, 4, 2
    wg = random_wire("q4_k", F, H, seed=1, device=dev, lead=(E,))
    wu = random_wire("q4_k", F, H, seed=2, device=dev, lead=(E,))
    wd = random_wire("q4_k", H, F, seed=3, device=dev, lead=(E,))
    ranks, xs, routes = [], [], []
    for r in range(W):
        g = torch.Generator(device="cpu").manual_seed(200 + r)
        xs.append(torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev))
        routes.append(route_topk(torch.randn(T, E, generator=g).to(dev), k))
        lo, hi = shard_bounds(E, r, W)
        ranks.append(GatheredExpertParallel(T, H, k, E, fuse_gate_up(wg[lo:hi], wu[lo:hi]), wd[lo:hi].contiguous(),
                                            "q4_k", rank=r, world=W))
    gathered = torch.cat([ranks[r].pack(xs[r], *routes[r]) for r in range(W)])
    total = torch.zeros((W * T, H), dtype=torch.float32, device=dev)
    for r in range(W):
        ranks[r].recv.copy_(gathered)
        ranks[r].local_stage()
        assert torch.isfinite(ranks[r].partial).all()
        total += ranks[r].partial
    for r in range(W):
        want = moe_glu(xs[r], wg, wu, wd, "q4_k", *routes[r], fused=False).float()   # the same composition
        got = total[r * T:(r + 1) * T].to(torch.bfloat16).float()
        assert float((got - want).norm() / want.norm()) < 2e-3


def test_peer_scatter_combine_two_virtual_ranks():
    """kq_moe_swiglu_block_scatter + kq_moe_sum_slots with both "ranks" on one GPU (the slot buffers are ordinary
    local tensors here; on two GPUs they are peer mappings, tests/test_moe_ep_gpu.py): every token's output is the
    single-GPU block's, and slots nobody owns a share of are never read (they hold NaNs)."""
    from mlx_kquant_b200.dist import shard_bounds
    from mlx_kquant_b200.moe import GatheredExpertParallel, fuse_gate_up, moe_sum_slots, moe_swiglu_block
    from mlx_kquant_b200.synth import random_wire
    dev = torch.device("cuda")
    T, E, H, F, k, W = 160, 16, 512, 256, 2, 2
    wg = random_wire("q4_k", F, H, seed=1, device=dev, lead=(E,))
    wu = random_wire("q4_k", F, H, seed=2, device=dev, lead=(E,))
    wd = random_wire("q4_k", H, F, seed=3, device=dev, lead=(E,))
    xs, routes, ranks = [], [], []
    for r in range(W):
        g = torch.Generator(device="cpu").manual_seed(300 + r)
        xs.append(torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev))
        routes.append(route_topk(torch.randn(T, E, generator=g).to(dev), k))
        lo, hi = shard_bounds(E, r, W)
        ranks.append(GatheredExpertParallel(T, H, k, E, fuse_gate_up(wg[lo:hi], wu[lo:hi]), wd[lo:hi].contiguous(),
                                            "q4_k", rank=r, world=W, reduce_dtype=torch.bfloat16))
        assert ranks[r].block_ok
    gathered = torch.cat([ranks[r].pack(xs[r], *routes[r]) for r in range(W)])
    slots = [torch.full((W, T, H), float("nan"), dtype=torch.bfloat16, device=dev) for _ in range(W)]
    ptrs = torch.tensor([t.data_ptr() for t in slots], dtype=torch.int64, device=dev)
    rank_lo = torch.tensor([shard_bounds(E, r, W)[0] for r in range(W)] + [E], dtype=torch.int32, device=dev)
    for r in range(W):
        ep = ranks[r]
        ep.recv.copy_(gathered)
        R = T + ep.pad_rows
        meta = ep._meta(ep.recv, R)
        ids = meta[:, :T * k].reshape(W * T * k) - ep.lo
        probs = meta[:, T * k:2 * T * k].reshape(W * T * k).view(torch.float32)
        assert moe_swiglu_block(ep.recv, ep.w_gate_up, ep.w_down, "q4_k", ids.view(W * T, k), probs.view(W * T, k),
                                token_rows=ep.tok_rows, tokens=W * T, scatter=(ptrs, torch.bfloat16, r, T)) is True
    some_nan = False
    for r in range(W):
        some_nan |= bool(torch.isnan(slots[r]).any())
        y = moe_sum_slots(slots[r], routes[r][0], rank_lo, torch.bfloat16)
        assert torch.isfinite(y.float()).all()
        want = moe_glu(xs[r], wg, wu, wd, "q4_k", *routes[r], fused=False).float()
        assert float((y.float() - want).norm() / want.norm()) < 4e-3   # two bf16 partial sums instead of one float32 sum
    assert some_nan   # with top-2 of 16 experts some tokens have no expert on one of the ranks
