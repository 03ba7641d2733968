"""Mixture-of-experts SwiGLU block composed from gather_qmm, the way the
reference's callers compose it (three gather calls per FFN, mlx_kquant/nn.py:185-220):

    h = silu(x . Wg[e]^T) * (x . Wu[e]^T);  y = sum_k p_k * (h_k . Wd[e_k]^T)

Routing: softmax over the router logits, top-k with ties to the lowest index,
probabilities renormalised over the k winners. Each gather output is rounded to
the activation dtype (as every reference op does, src/kquant_ops.cpp:354); the
activation and the weighted sum run in float32.
"""
from __future__ import annotations

import torch

from .ops import gather_qmm


def route_topk(router_logits: torch.Tensor, top_k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """(expert ids [T, k] int64, renormalised probabilities [T, k] float32)."""
    probs = torch.softmax(router_logits.float(), dim=-1)
    # a stable descending sort puts the lowest index first among equal probabilities
    order = torch.sort(probs, dim=-1, descending=True, stable=True)
    p, idx = order.values[:, :top_k], order.indices[:, :top_k]
    return idx, p / p.sum(dim=-1, keepdim=True)


def moe_glu(x, w_gate, w_up, w_down, kquant_type, expert_ids, expert_probs, *, sort_rows: bool = True):
    """x [T, H] (f16 / bf16), expert stacks [E, F, bytes(H)] x2 and [E, H, bytes(F)],
    expert_ids / expert_probs [T, k]. Returns y [T, H] in x's dtype."""
    T, H = x.shape
    k = expert_ids.shape[1]
    rows = T * k
    flat_e = expert_ids.reshape(rows)
    tok = torch.arange(T, device=x.device).repeat_interleave(k)
    if sort_rows and rows >= 64:
        # expert-sorted rows, as the reference's callers do from 64 routed rows up (src/kquant_gather.cpp:8-16)
        order = torch.argsort(flat_e, stable=True)
        flat_e, tok = flat_e[order], tok[order]
    else:
        order = None
    x3 = x.reshape(T, 1, H)
    g = gather_qmm(x3, w_gate, None, kquant_type, lhs_indices=tok, rhs_indices=flat_e)
    u = gather_qmm(x3, w_up, None, kquant_type, lhs_indices=tok, rhs_indices=flat_e)
    h = (torch.nn.functional.silu(g.float()) * u.float()).to(x.dtype)          # [rows, 1, F]
    d = gather_qmm(h, w_down, None, kquant_type, rhs_indices=flat_e, sorted_indices=order is not None)
    d = d.reshape(rows, H).float()
    if order is not None:
        unsort = torch.empty_like(order)
        unsort[order] = torch.arange(rows, device=x.device)
        d = d[unsort]
    y = (d.reshape(T, k, H) * expert_probs.reshape(T, k, 1).float()).sum(dim=1)
    return y.to(x.dtype)
