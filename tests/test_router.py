"""moe_router_topk against the numpy statement the reference checks its op with (tests/test_moe_glu.py:453-549)."""
import numpy as np
import pytest
import torch

from mlx_kquant_b200.moe import moe_router_topk


def test_softmax_with_shared_gate():
    rng = np.random.default_rng(5)
    for e, r, norm in ((256, 8, True), (256, 8, False), (128, 4, True), (16, 2, True)):
        logits = rng.standard_normal((5, e + 1)).astype(np.float32)
        inds, sc = moe_router_topk(torch.from_numpy(logits), r, norm)
        assert inds.dtype == torch.int32 and tuple(sc.shape) == (5, r + 1)
        p = np.exp(logits[:, :e] - logits[:, :e].max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        top = np.argsort(-p, axis=-1, kind="stable")[:, :r]
        assert np.array_equal(inds.numpy(), top)
        for t in range(5):
            pk = p[t, top[t]]
            np.testing.assert_allclose(sc.numpy()[t, :r], pk / (pk.sum() if norm else 1.0), rtol=1e-5, atol=1e-6)
            assert abs(float(sc[t, r]) - 1.0 / (1.0 + np.exp(-logits[t, e]))) < 1e-5


def test_per_expert_scale_without_shared_gate():
    rng = np.random.default_rng(6)
    for e, r in ((128, 8), (16, 4)):
        logits = rng.standard_normal((5, e)).astype(np.float32)
        pes = rng.uniform(0.5, 1.5, e).astype(np.float32)
        inds, sc = moe_router_topk(torch.from_numpy(logits), r, True, shared_gate=False,
                                   per_expert_scale=torch.from_numpy(pes))
        assert tuple(sc.shape) == (5, r)
        p = np.exp(logits - logits.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        top = np.argsort(-p, axis=-1, kind="stable")[:, :r]
        assert np.array_equal(inds.numpy(), top)
        for t in range(5):
            pk = p[t, top[t]]
            np.testing.assert_allclose(sc.numpy()[t], pk / pk.sum() * pes[top[t]], rtol=1e-5, atol=1e-6)


def test_sqrtsoftplus_bias_scale_and_ties():
    rng = np.random.default_rng(7)
    for e, r, spread in ((256, 6, 1.0), (256, 6, 30.0), (64, 4, 1.0)):
        logits = (rng.standard_normal((7, e)) * spread).astype(np.float32)
        logits[5, 10:20] = logits[5, 10]                      # exact ties at the boundary: lowest index wins
        bias = rng.standard_normal(e).astype(np.float32)
        for dt in (torch.float32, torch.bfloat16):
            lt = torch.from_numpy(logits).to(dt)
            inds, sc = moe_router_topk(lt, r, True, shared_gate=False, bias=torch.from_numpy(bias),
                                       scoring="sqrtsoftplus", scale=1.5)
            lf = lt.float().numpy()
            p = np.sqrt(np.logaddexp(lf, 0.0))
            top = np.argsort(-(p + bias), axis=-1, kind="stable")[:, :r]
            got = inds.numpy()
            for t in range(7):
                if set(got[t]) != set(top[t]):   # float32 softplus ulp noise at the boundary
                    np.testing.assert_allclose(np.sort((p + bias)[t, got[t]]), np.sort((p + bias)[t, top[t]]), rtol=0, atol=3e-6)
                pk = p[t, got[t]]
                np.testing.assert_allclose(sc.numpy()[t], pk / (pk.sum() + 1e-20) * 1.5, rtol=1e-5, atol=1e-6)
        neg = torch.from_numpy((-np.abs(logits) - 50.0).astype(np.float32))
        _, sc = moe_router_topk(neg, r, True, shared_gate=False, bias=torch.from_numpy(bias), scoring="sqrtsoftplus",
                                scale=1.5)
        assert torch.isfinite(sc).all()


def test_rejects_bad_arguments():
    x = torch.zeros(2, 9)
    with pytest.raises(ValueError):
        moe_router_topk(x, 2, True, scoring="tanh")
    with pytest.raises(ValueError):
        moe_router_topk(x, 20, True)
    with pytest.raises(ValueError):
        moe_router_topk(x, 2, False, shared_gate=False, scoring="sqrtsoftplus")
    with pytest.raises(ValueError):
        moe_router_topk(torch.zeros(9), 2, True)
