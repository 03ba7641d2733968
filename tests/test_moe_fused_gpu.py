"""The fused mixture-of-experts decode ops (csrc/kq_moe_decode.cu) against the oracle.

The reference has no CPU evaluation of moe_glu_gather_kq / gather_qmv_mix_ns_kq / moe_router_topk
(src/kquant_moe_glu.cpp:1-8), so the expected values are the float64 statement of each op on the oracle's
bit-exact dequantized weights, and, for the router, the numpy statement the reference tests its op with
(tests/test_moe_glu.py:453-549) as restated in test_router.py for host tensors."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import assert_close
from gpu_util import mint_wire, x_to_torch, y_to_f32
from mlx_kquant_b200 import _lib
from mlx_kquant_b200.moe import (codec_has_moe_glu, gather_qmv_kq, gather_qmv_mix_ns_kq, moe_glu, moe_glu_gather_kq,
                                 moe_router_topk, route_topk)
from oracle.kq_oracle import to_f32

pytestmark = pytest.mark.gpu


def experts(E, N, K, seed):
    rng = np.random.default_rng(seed)
    return np.stack([mint_wire("q4_k", rng.normal(0, 0.02, (N, K)).astype(np.float32)) for _ in range(E)])


def act_ref(g, u, act, limit):
    if act == "gelu":
        return 0.5 * g * (1.0 + np.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3))) * u
    if act == "silu_limit":
        g = np.minimum(g, limit)
        u = np.clip(u, -limit, limit)
    return g / (1.0 + np.exp(-g)) * u


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("act,limit", [("silu", 0.0), ("gelu", 0.0), ("silu_limit", 0.5)])
def test_moe_glu_gather_kq(oracle, dt, act, limit):
    E, N, K, T, R = 6, 100, 512, 3, 4            # N = 100: the last 16-row tile holds 4 rows
    wg, wu = experts(E, N, K, 11), experts(E, N, K, 12)
    rng = np.random.default_rng(13)
    x, store = x_to_torch(rng.normal(0, 1, (T, K)).astype(np.float32), dt)
    ids = rng.integers(0, E, (T, R))
    y = moe_glu_gather_kq(x, torch.from_numpy(wg).cuda(), torch.from_numpy(wu).cuda(), "q4_k",
                          torch.from_numpy(ids).cuda(), act=act, limit=limit)
    assert tuple(y.shape) == (T, R, N) and y.dtype == x.dtype
    xs = to_f32(store, dt).astype(np.float64)
    Wg = oracle.dequantize(wg, "q4_k", "f32").astype(np.float64)
    Wu = oracle.dequantize(wu, "q4_k", "f32").astype(np.float64)
    ref = np.stack([np.stack([act_ref(xs[t] @ Wg[e].T, xs[t] @ Wu[e].T, act, limit) for e in ids[t]]) for t in range(T)])
    assert_close(y_to_f32(y).reshape(T * R, N), ref.reshape(T * R, N), dt, 2e-3)


def test_moe_glu_gather_kq_stacked_views_and_skipped_entries(oracle):
    """gate | up as the two halves of one stacked tensor (strided expert dimension), and an out-of-range expert
    index whose output row stays untouched."""
    E, F, K, T, R = 4, 48, 256, 2, 3
    wg, wu = experts(E, F, K, 21), experts(E, F, K, 22)
    wgu = torch.from_numpy(np.concatenate([wg, wu], axis=1)).cuda()
    x, store = x_to_torch(np.random.default_rng(23).normal(0, 1, (T, K)).astype(np.float32), "bf16")
    ids = torch.tensor([[0, 3, 9], [2, 2, 1]]).cuda()      # 9 >= E
    L = _lib.lib()
    y = torch.full((T, R, F), 5.0, dtype=torch.bfloat16, device="cuda")
    idx = ids.to(torch.int32).contiguous()
    g_v, u_v = wgu[:, :F], wgu[:, F:]
    _lib.check(L.kq_moe_glu_gather(x.data_ptr(), _lib.KQ_BF16, T, K, g_v.data_ptr(), g_v.stride(0), u_v.data_ptr(),
                                   u_v.stride(0), g_v.shape[2], F, E, b"q4_k", idx.data_ptr(), R, b"silu", 0.0,
                                   y.data_ptr(), None, 0, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    xs = to_f32(store, "bf16").astype(np.float64)
    Wg = oracle.dequantize(wg, "q4_k", "f32").astype(np.float64)
    Wu = oracle.dequantize(wu, "q4_k", "f32").astype(np.float64)
    got = y_to_f32(y)
    assert (got[0, 2] == 5.0).all()
    for t in range(T):
        for r in range(R):
            e = int(ids[t, r])
            if e < E:
                assert_close(got[t, r][None], act_ref(xs[t] @ Wg[e].T, xs[t] @ Wu[e].T, "silu", 0)[None], "bf16", 2e-3)


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("S", [3, 8, 11])
def test_gather_qmv_mix_ns_kq(oracle, dt, S):
    E, N, K, T = 5, 84, 768, 3                  # K = 768: three superblocks per row, rows of 432 bytes
    w = experts(E, N, K, 31)
    rng = np.random.default_rng(32 + S)
    x, store = x_to_torch(rng.normal(0, 1, (T, S, K)).astype(np.float32), dt)
    ids = rng.integers(0, E, (T, S))
    sc = rng.uniform(0.05, 0.4, (T, S)).astype(np.float32)
    wd = torch.from_numpy(w).cuda()
    y = gather_qmv_mix_ns_kq(x, wd, "q4_k", torch.from_numpy(ids).cuda(), torch.from_numpy(sc).cuda())
    assert tuple(y.shape) == (T, N) and y.dtype == x.dtype
    xs = to_f32(store, dt).astype(np.float64)
    W = oracle.dequantize(w, "q4_k", "f32").astype(np.float64)
    ref = np.stack([sum(sc[t, s] * (xs[t, s] @ W[ids[t, s]].T) for s in range(S)) for t in range(T)])
    assert_close(y_to_f32(y), ref, dt, 2e-3)
    # the unfused form of the same op: per-slot products (rounded), then the weighted sum
    d = gather_qmv_kq(x, wd, "q4_k", torch.from_numpy(ids).cuda()).float()
    unfused = (d * torch.from_numpy(sc).cuda()[:, :, None]).sum(1)
    assert float((y.float() - unfused).norm() / unfused.norm()) < 6e-3


def test_fused_block_equals_composition(oracle):
    """moe_glu takes the two fused launches for a few tokens; sort_rows=True forces the three-gather composition."""
    E, H, F, k, T = 16, 512, 256, 4, 5
    wg, wu, wd = experts(E, F, H, 41), experts(E, F, H, 42), experts(E, H, F, 43)
    rng = np.random.default_rng(44)
    x = torch.from_numpy(rng.normal(0, 1, (T, H)).astype(np.float32)).to(torch.bfloat16).cuda()
    ids, probs = route_topk(torch.from_numpy(rng.normal(0, 1, (T, E)).astype(np.float32)).cuda(), k)
    args = (x, torch.from_numpy(wg).cuda(), torch.from_numpy(wu).cuda(), torch.from_numpy(wd).cuda(), "q4_k", ids, probs)
    assert codec_has_moe_glu("q4_k") and not codec_has_moe_glu("q6_k")
    y = moe_glu(*args)
    # float64 statement of the block
    xs = x.float().cpu().numpy().astype(np.float64)
    Wg, Wu, Wd = (oracle.dequantize(w, "q4_k", "f32").astype(np.float64) for w in (wg, wu, wd))
    idn, pn = ids.cpu().numpy(), probs.cpu().numpy().astype(np.float64)
    ref = np.zeros((T, H))
    for t in range(T):
        for j in range(k):
            e = idn[t, j]
            g, u = xs[t] @ Wg[e].T, xs[t] @ Wu[e].T
            ref[t] += pn[t, j] * ((g / (1 + np.exp(-g)) * u) @ Wd[e].T)
    err = np.linalg.norm(y_to_f32(y) - ref) / np.linalg.norm(ref)
    assert err < 4e-3, err                       # the rounding of h to bfloat16, then of y


def test_indices_written_by_the_preceding_launch(oracle):
    """router -> fused gate/up -> fused down replayed from a CUDA graph whose first node overwrites the index
    buffer: the product kernels start their weight copies from the stale indices and must copy again."""
    E, H, F, k, T = 16, 512, 256, 4, 2
    wg, wu, wd = (torch.from_numpy(experts(E, n, kk, s)).cuda() for n, kk, s in ((F, H, 51), (F, H, 52), (H, F, 53)))
    rng = np.random.default_rng(54)
    x = torch.from_numpy(rng.normal(0, 1, (T, H)).astype(np.float32)).to(torch.float16).cuda()
    logits = torch.from_numpy(rng.normal(0, 1, (T, E)).astype(np.float32)).cuda()
    L = _lib.lib()
    idx = torch.zeros(T, k, dtype=torch.int32, device="cuda")
    sc = torch.zeros(T, k, dtype=torch.float32, device="cuda")
    h = torch.empty(T, k, F, dtype=torch.float16, device="cuda")
    y = torch.empty(T, H, dtype=torch.float16, device="cuda")
    stream = torch.cuda.Stream()

    def block(s):
        idx.fill_(E - 1)          # stale: every slot points at the last expert
        _lib.check(L.kq_moe_router_topk(logits.data_ptr(), _lib.KQ_F32, T, E, k, 1, 0, None, None, b"softmax", 1.0,
                                        idx.data_ptr(), sc.data_ptr(), s.cuda_stream))
        _lib.check(L.kq_moe_glu_gather(x.data_ptr(), _lib.KQ_F16, T, H, wg.data_ptr(), wg.stride(0), wu.data_ptr(),
                                       wu.stride(0), wg.shape[2], F, E, b"q4_k", idx.data_ptr(), k, b"silu", 0.0,
                                       h.data_ptr(), None, 0, s.cuda_stream))
        _lib.check(L.kq_gather_qmv_mix(h.data_ptr(), _lib.KQ_F16, T, k, F, wd.data_ptr(), wd.stride(0), wd.shape[2], H, E,
                                       b"q4_k", idx.data_ptr(), sc.data_ptr(), y.data_ptr(), None, 0, 0, s.cuda_stream))

    with torch.cuda.stream(stream):
        block(stream)
        stream.synchronize()
        y_eager = y.clone()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            block(stream)
        for _ in range(5):
            g.replay()
        stream.synchronize()
    ids, probs = route_topk(logits, k)
    assert torch.equal(idx.long(), ids.long())
    want = moe_glu(x, wg, wu, wd, "q4_k", ids, probs)
    assert torch.equal(y, y_eager)
    assert torch.equal(y, want)


@pytest.mark.parametrize("case", ["softmax_shared", "pes", "sqrtsoftplus_bias", "wide"])
def test_router_kernel_matches_host_statement(case):
    rng = np.random.default_rng(61)
    if case == "softmax_shared":
        cfgs = [dict(E=256, k=8, norm=True, shared=True), dict(E=256, k=8, norm=False, shared=True),
                dict(E=16, k=2, norm=True, shared=True)]
    elif case == "pes":
        cfgs = [dict(E=128, k=8, norm=True, shared=False, pes=True), dict(E=100, k=5, norm=True, shared=False, pes=True)]
    elif case == "sqrtsoftplus_bias":
        cfgs = [dict(E=256, k=6, norm=True, shared=False, bias=True, scoring="sqrtsoftplus", scale=1.5)]
    else:
        cfgs = [dict(E=1024, k=16, norm=True, shared=False), dict(E=33, k=16, norm=False, shared=False)]
    for c in cfgs:
        E, k = c["E"], c["k"]
        T = 37
        logits = rng.standard_normal((T, E + (1 if c["shared"] else 0))).astype(np.float32)
        logits[3, 4:9] = logits[3, 4]              # exact ties: the lowest index wins
        pes = torch.from_numpy(rng.uniform(0.5, 1.5, E).astype(np.float32)) if c.get("pes") else None
        bias = torch.from_numpy(rng.standard_normal(E).astype(np.float32)) if c.get("bias") else None
        for dt in (torch.float32, torch.bfloat16, torch.float16):
            lt = torch.from_numpy(logits).to(dt)
            kw = dict(shared_gate=c["shared"], per_expert_scale=pes, bias=bias, scoring=c.get("scoring", "softmax"),
                      scale=c.get("scale", 1.0))
            i_h, s_h = moe_router_topk(lt, k, c["norm"], **kw)                  # host tensors: torch statement
            i_d, s_d = moe_router_topk(lt.cuda(), k, c["norm"], **kw)           # the kernel
            assert i_d.dtype == torch.int32 and tuple(s_d.shape) == tuple(s_h.shape)
            same = (i_d.cpu() == i_h).all(dim=1)
            # rows that differ may only differ by float32 rounding noise between equal-within-an-ulp scores
            for t in torch.nonzero(~same).flatten().tolist():
                assert set(i_d[t].tolist()) == set(i_h[t].tolist()) or c.get("scoring") == "sqrtsoftplus"
            ok = same
            np.testing.assert_allclose(s_d.cpu().numpy()[ok.numpy()], s_h.numpy()[ok.numpy()], rtol=2e-5, atol=1e-6)
            assert int(ok.sum()) >= T - 2


@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_grouped_forms_beyond_the_direct_limit(oracle, dt):
    """More than KQ_MOE_DIRECT_MAX_ENTRIES entries: entries grouped by expert, four per pass over the weights.
    One expert index is out of range (its rows stay unwritten / count as zero in the mix)."""
    E, F, K, T, R = 7, 104, 512, 60, 4          # 240 entries; F = 104: last tile of 8 rows, last 128-row block ragged
    wg, wu, wdn = experts(E, F, K, 71), experts(E, F, K, 72), experts(E, 200, 768, 73)
    rng = np.random.default_rng(74)
    x, store = x_to_torch(rng.normal(0, 1, (T, K)).astype(np.float32), dt)
    ids = rng.integers(0, E, (T, R))
    ids[5, 2] = E + 2
    idt = torch.from_numpy(ids).cuda()
    y = torch.full((T, R, F), 3.0, dtype=x.dtype, device="cuda")
    L = _lib.lib()
    code = _lib.KQ_F16 if dt == "f16" else _lib.KQ_BF16
    wgd, wud = torch.from_numpy(wg).cuda(), torch.from_numpy(wu).cuda()
    idx = idt.to(torch.int32).contiguous()
    ws = torch.empty(L.kq_moe_decode_workspace_bytes(T * R, E, 0), dtype=torch.uint8, device="cuda")
    assert ws.numel() > 0
    _lib.check(L.kq_moe_glu_gather(x.data_ptr(), code, T, K, wgd.data_ptr(), wgd.stride(0), wud.data_ptr(), wud.stride(0),
                                   wgd.shape[2], F, E, b"q4_k", idx.data_ptr(), R, b"silu", 0.0, y.data_ptr(),
                                   ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    xs = to_f32(store, dt).astype(np.float64)
    Wg = oracle.dequantize(wg, "q4_k", "f32").astype(np.float64)
    Wu = oracle.dequantize(wu, "q4_k", "f32").astype(np.float64)
    got = y_to_f32(y)
    assert (got[5, 2] == 3.0).all()
    ok = ids < E
    ref = np.zeros((T, R, F))
    for t in range(T):
        for r in range(R):
            if ok[t, r]:
                ref[t, r] = act_ref(xs[t] @ Wg[ids[t, r]].T, xs[t] @ Wu[ids[t, r]].T, "silu", 0)
    assert_close(got[ok], ref[ok], dt, 2e-3)
    # the same call without a workspace takes the per-entry kernel: same values up to summation order
    y2 = moe_glu_gather_kq(x[:8], wgd, wud, "q4_k", idt[:8])
    assert float((y2.float() - y[:8].float())[torch.from_numpy(ok[:8]).cuda()].abs().max()) <= 2e-2 * float(y.float().abs().max())

    # down stage with the weighted sum: x [T, S, 768], N = 200
    S = R
    xm, storem = x_to_torch(rng.normal(0, 1, (T, S, 768)).astype(np.float32), dt)
    sc = rng.uniform(0.05, 0.4, (T, S)).astype(np.float32)
    ym = gather_qmv_mix_ns_kq(xm, torch.from_numpy(wdn).cuda(), "q4_k", idt, torch.from_numpy(sc).cuda())
    xms = to_f32(storem, dt).astype(np.float64)
    Wd = oracle.dequantize(wdn, "q4_k", "f32").astype(np.float64)
    refm = np.stack([sum(sc[t, s] * (xms[t, s] @ Wd[ids[t, s]].T) for s in range(S) if ok[t, s]) for t in range(T)])
    err = np.linalg.norm(y_to_f32(ym) - refm) / np.linalg.norm(refm)
    assert err < 4e-3, err          # every slot's product is rounded once before the weighted sum


# ------------------------------------------------------------------------------------------ the one-call block
def _block_case(codec, E, H, F, seed):
    rng = np.random.default_rng(seed)
    mk = lambda n, k: torch.from_numpy(np.stack([mint_wire(codec, rng.normal(0, 0.02, (n, k)).astype(np.float32))
                                                 for _ in range(E)])).cuda()
    return mk(2 * F, H), mk(H, F)


@pytest.mark.parametrize("codec,dt", [("q4_k", torch.bfloat16), ("q4_k", torch.float16), ("q6_k", torch.bfloat16)])
def test_block_same_bits_as_the_composition(codec, dt):
    """kq_moe_swiglu_block against the three-gather composition (gather_qmm x2, the activation kernel, the weighted
    sum): the same roundings in the same places, so bit-identical outputs - including tokens routed to an expert
    outside [0, E), which contribute nothing in either form."""
    from mlx_kquant_b200.moe import moe_swiglu_block

    E, H, F, k, T = 8, 512, 256, 2, 640
    wgu, wd = _block_case(codec, E, H, F, 71)
    g = torch.Generator(device="cuda").manual_seed(72)
    x = torch.randn(T, H, device="cuda", generator=g).to(dt)
    x[5] *= 1e-6                                  # a row that only survives the fp16 pre-pass through its row factor
    ids, probs = route_topk(torch.randn(T, E, device="cuda", generator=g), k)
    y = moe_swiglu_block(x, wgu, wd, codec, ids, probs)
    assert y is not None and tuple(y.shape) == (T, H) and y.dtype == dt
    ref = moe_glu(x, None, None, wd, codec, ids, probs, w_gate_up=wgu, fused=False)
    assert torch.equal(y.view(torch.int16), ref.view(torch.int16))
    # moe_glu takes the block by itself at this size
    assert torch.equal(moe_glu(x, None, None, wd, codec, ids, probs, w_gate_up=wgu).view(torch.int16), y.view(torch.int16))
    if dt == torch.bfloat16:                      # float16 rows take no row factor (nor do they in the composition)
        assert float(y[5].float().abs().max()) > 0

    # experts of another rank: index E + something, weight irrelevant
    ids2 = ids.clone()
    ids2[::3, 0] = E + 3
    y2 = moe_swiglu_block(x, wgu, wd, codec, ids2, probs)
    p2 = probs.clone()
    p2[::3, 0] = 0
    ids_safe = ids2.clone()
    ids_safe[::3, 0] = 0
    ref2 = moe_glu(x, None, None, wd, codec, ids_safe, p2, w_gate_up=wgu, fused=False)
    assert torch.equal(y2.view(torch.int16), ref2.view(torch.int16))


def test_block_token_rows_and_float32_partial_sums():
    from mlx_kquant_b200.moe import moe_swiglu_block

    E, H, F, k, T = 4, 256, 256, 4, 256
    wgu, wd = _block_case("q4_k", E, H, F, 81)
    g = torch.Generator(device="cuda").manual_seed(82)
    big = torch.randn(2 * T + 7, H, device="cuda", generator=g).to(torch.bfloat16)
    rows = torch.randperm(2 * T + 7, device="cuda", generator=g)[:T].to(torch.int32)
    ids, probs = route_topk(torch.randn(T, E, device="cuda", generator=g), k)
    out = torch.empty(T, H, dtype=torch.float32, device="cuda")
    y = moe_swiglu_block(big, wgu, wd, "q4_k", ids, probs, token_rows=rows, tokens=T, out=out)
    assert y is out
    ref = moe_swiglu_block(big[rows.long()].contiguous(), wgu, wd, "q4_k", ids, probs)
    # the float32 form is the same sum before its one rounding
    assert torch.equal(out.to(torch.bfloat16).view(torch.int16), ref.view(torch.int16))


def test_block_refuses_small_calls():
    lib = _lib.lib()
    assert lib.kq_moe_block_workspace_bytes(8, 2, 8, 512, 256) == 0          # 16 routed rows
    assert lib.kq_moe_block_workspace_bytes(640, 2, 8, 512, 250) == 0        # F not a multiple of 8
    assert lib.kq_moe_block_workspace_bytes(640, 2, 8, 512, 256) > 0
    x = torch.zeros(8, 512, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(8, 512, 288, dtype=torch.uint8, device="cuda")
    wd = torch.zeros(8, 512, 144, dtype=torch.uint8, device="cuda")
    idx = torch.zeros(8, 2, dtype=torch.int32, device="cuda")
    sc = torch.zeros(8, 2, dtype=torch.float32, device="cuda")
    rc = lib.kq_moe_swiglu_block(x.data_ptr(), 2, 8, 512, 512, None, w.data_ptr(), w.stride(0), 288, 256, wd.data_ptr(),
                                 wd.stride(0), 144, 8, b"q4_k", idx.data_ptr(), sc.data_ptr(), 2, x.data_ptr(), 2, None, 0,
                                 None)
    assert rc == _lib.KQ_ERR_UNSUPPORTED


def test_block_with_more_tiles_than_the_grid_cap():
    """The grouped tile kernel launches at most 256 tile rows and loops over longer lists: 300 experts with rows
    make 300 tiles or more. Against the composition per expert on the plain matmul."""
    import mlx_kquant_b200 as kq
    from mlx_kquant_b200.moe import moe_swiglu_block, swiglu

    E, H, F, k, T = 300, 256, 256, 1, 300 * 40
    rng = np.random.default_rng(91)
    wgu = torch.from_numpy(mint_wire("q4_k", rng.normal(0, 0.02, (E * 2 * F, H)).astype(np.float32))).cuda().reshape(E, 2 * F, -1)
    wd = torch.from_numpy(mint_wire("q4_k", rng.normal(0, 0.02, (E * H, F)).astype(np.float32))).cuda().reshape(E, H, -1)
    g = torch.Generator(device="cuda").manual_seed(92)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    ids = (torch.arange(T, device="cuda") % E).to(torch.int32).reshape(T, 1)
    probs = torch.rand(T, 1, device="cuda", generator=g) + 0.5
    y = moe_swiglu_block(x, wgu, wd, "q4_k", ids, probs)
    assert y is not None
    for e in (0, 1, 149, 255, 256, 299):                       # experts on both sides of the cap
        rows = torch.nonzero(ids[:, 0] == e)[:, 0]
        gu = kq.quantized_matmul(x[rows], wgu[e], None, "q4_k")
        h = swiglu(gu[:, :F], gu[:, F:])
        d = kq.quantized_matmul(h, wd[e], None, "q4_k")
        ref = (d.float() * probs[rows]).to(torch.bfloat16)
        err = float((y[rows].float() - ref.float()).norm() / ref.float().norm())
        assert err < 4e-3, (e, err)


def test_block_q6k_rows_on_8_byte_boundaries():
    """The grouped tile kernel with the q6_k producer that needs 8-byte aligned rows (H and F multiples of 1024)."""
    from mlx_kquant_b200.moe import moe_swiglu_block

    E, H, F, k, T = 4, 1024, 1024, 2, 320
    wgu, wd = _block_case("q6_k", E, H, F, 93)
    g = torch.Generator(device="cuda").manual_seed(94)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    ids, probs = route_topk(torch.randn(T, E, device="cuda", generator=g), k)
    y = moe_swiglu_block(x, wgu, wd, "q6_k", ids, probs)
    assert y is not None
    ref = torch.zeros(T, H, dtype=torch.float64, device="cuda")
    bf = lambda t: t.float().to(torch.bfloat16).double()
    import mlx_kquant_b200 as kq
    for e in range(E):
        tok, slot = torch.nonzero(ids == e, as_tuple=True)
        Wgu = kq.dequantize(wgu[e], None, "q6_k", torch.float32).double()      # bit-exact against the oracle elsewhere
        Wd = kq.dequantize(wd[e], None, "q6_k", torch.float32).double()
        gu = bf(x[tok].double() @ Wgu.T)
        h = bf(torch.nn.functional.silu(gu[:, :F].float()).double() * gu[:, F:])
        ref.index_add_(0, tok, bf(h @ Wd.T) * probs[tok, slot].double()[:, None])
    assert float((y.double() - ref).norm() / ref.norm()) < 6e-3
