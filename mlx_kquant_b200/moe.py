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


def moe_glu_expert_parallel(x, w_gate, w_up, w_down, kquant_type, expert_ids, expert_probs, n_experts, group=None):
    """The same block with the experts partitioned over the ranks of `group`.

    Every rank holds its own tokens x [T, H] and routing, and only the expert
    matrices of its contiguous share (`dist.shard_bounds(n_experts, rank, world)`;
    w_* are the LOCAL stacks). Routed rows travel to the rank that owns their
    expert with one all-to-all (activations + expert id), are multiplied there, and
    come back with a second all-to-all; the weighted sum over the k experts happens
    where the token lives. The reference has no counterpart (it is single-device).
    """
    import torch.distributed as dist

    from .dist import expert_owner, shard_bounds, split_by_owner

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    T, H = x.shape
    k = expert_ids.shape[1]
    rows = T * k
    flat_e = expert_ids.reshape(rows)
    tok = torch.arange(T, device=x.device).repeat_interleave(k)
    owner = expert_owner(flat_e, n_experts, world)
    order, send_counts = split_by_owner(owner, world)
    recv_counts_t = torch.empty(world, dtype=torch.int64, device=x.device)
    dist.all_to_all_single(recv_counts_t, torch.tensor(send_counts, dtype=torch.int64, device=x.device), group=group)
    recv_counts = recv_counts_t.tolist()
    n_recv = sum(recv_counts)
    # dispatch: activations and expert ids of the routed rows, grouped by destination
    send_x = x[tok[order]].contiguous()
    send_e = flat_e[order].to(torch.int32).contiguous()
    recv_x = torch.empty((n_recv, H), dtype=x.dtype, device=x.device)
    recv_e = torch.empty(n_recv, dtype=torch.int32, device=x.device)
    dist.all_to_all_single(recv_x, send_x, output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
    dist.all_to_all_single(recv_e, send_e, output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
    # local experts
    lo, _ = shard_bounds(n_experts, rank, world)
    local_e = (recv_e.to(torch.int64) - lo)
    if n_recv > 0:
        sort = torch.argsort(local_e, stable=True)
        xs = recv_x[sort].reshape(n_recv, 1, H)
        es = local_e[sort]
        g = gather_qmm(xs, w_gate, None, kquant_type, rhs_indices=es, sorted_indices=True)
        u = gather_qmm(xs, w_up, None, kquant_type, rhs_indices=es, sorted_indices=True)
        h = (torch.nn.functional.silu(g.float()) * u.float()).to(x.dtype)
        d = gather_qmm(h, w_down, None, kquant_type, rhs_indices=es, sorted_indices=True).reshape(n_recv, H)
        out_rows = torch.empty_like(d)
        out_rows[sort] = d
    else:
        out_rows = torch.empty((0, H), dtype=x.dtype, device=x.device)
    # combine: results return to the rank of their token
    back = torch.empty((rows, H), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(back, out_rows.contiguous(), output_split_sizes=send_counts, input_split_sizes=recv_counts,
                           group=group)
    d_all = torch.empty((rows, H), dtype=torch.float32, device=x.device)
    d_all[order] = back.float()
    y = (d_all.reshape(T, k, H) * expert_probs.reshape(T, k, 1).float()).sum(dim=1)
    return y.to(x.dtype)
