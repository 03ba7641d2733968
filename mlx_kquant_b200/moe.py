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

from . import _lib
from .ops import gather_qmm


def route_topk(router_logits: torch.Tensor, top_k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """(expert ids [T, k] int32 - the index type every kernel here takes, so no conversion sits between the router
    and the block - and renormalised probabilities [T, k] float32)."""
    if router_logits.is_cuda and router_logits.shape[1] <= 1024 and top_k <= 16:
        return moe_router_topk(router_logits, top_k, True, shared_gate=False)
    probs = torch.softmax(router_logits.float(), dim=-1)
    # a stable descending sort puts the lowest index first among equal probabilities
    order = torch.sort(probs, dim=-1, descending=True, stable=True)
    p, idx = order.values[:, :top_k], order.indices[:, :top_k]
    return idx.to(torch.int32), p / p.sum(dim=-1, keepdim=True)


def swiglu(gate: torch.Tensor, up: torch.Tensor, row_expert: torch.Tensor | None = None,
           n_experts: int = 0) -> torch.Tensor:
    """silu(gate) * up in float32, rounded once to the inputs' dtype. gate / up: [rows, F] views that may be
    the two halves of one [rows, 2F] product (same row stride). With `row_expert` (int32 [rows]), rows whose
    expert index is outside [0, n_experts) are skipped and their output rows stay unwritten."""
    rows, F = gate.shape
    if row_expert is not None:
        if not (gate.is_cuda and gate.dtype in (torch.float16, torch.bfloat16) and F % 8 == 0):
            raise ValueError("[mlx_kquant.swiglu] the routed form needs float16 / bfloat16 CUDA rows with F % 8 == 0.")
        re32 = row_expert.reshape(rows).to(torch.int32).contiguous()
        out = torch.empty((rows, F), dtype=gate.dtype, device=gate.device)
        with torch.cuda.device(gate.device):
            _lib.check(_lib.lib().kq_swiglu_routed(gate.data_ptr(), up.data_ptr(), gate.stride(0), rows, F,
                                                   _lib.KQ_F16 if gate.dtype == torch.float16 else _lib.KQ_BF16,
                                                   out.data_ptr(), re32.data_ptr(), n_experts,
                                                   torch.cuda.current_stream(gate.device).cuda_stream))
        return out
    if (gate.is_cuda and gate.dtype in (torch.float16, torch.bfloat16) and F % 8 == 0 and gate.stride(1) == 1
            and up.stride(1) == 1 and gate.stride(0) == up.stride(0) and gate.stride(0) % 8 == 0
            and gate.data_ptr() % 16 == 0 and up.data_ptr() % 16 == 0):
        out = torch.empty((rows, F), dtype=gate.dtype, device=gate.device)
        with torch.cuda.device(gate.device):
            _lib.check(_lib.lib().kq_swiglu(gate.data_ptr(), up.data_ptr(), gate.stride(0), rows, F,
                                            _lib.KQ_F16 if gate.dtype == torch.float16 else _lib.KQ_BF16,
                                            out.data_ptr(), torch.cuda.current_stream(gate.device).cuda_stream))
        return out
    return (torch.nn.functional.silu(gate.float()) * up.float()).to(gate.dtype)


def combine_partial(d: torch.Tensor, probs: torch.Tensor, k: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """y[t] = sum_j probs[t, j] * d[t k + j]; rows of d whose weight is exactly 0 are not read. The partial sum
    of a rank that computed only the rows of its own experts: float32 by default, or rounded once to d's dtype
    when `out` has that dtype (half the bytes for the reduce-scatter that follows)."""
    rows, H = d.shape
    T = rows // k
    if not (d.is_cuda and d.dtype in (torch.float16, torch.bfloat16) and H % 8 == 0 and d.is_contiguous()):
        raise ValueError("[mlx_kquant.moe_combine] needs contiguous float16 / bfloat16 CUDA rows with H % 8 == 0.")
    p = probs.reshape(T * k).float().contiguous()
    y = torch.empty((T, H), dtype=torch.float32, device=d.device) if out is None else out
    if y.dtype not in (torch.float32, d.dtype):
        raise ValueError("[mlx_kquant.moe_combine] out must be float32 or of d's dtype.")
    fn = _lib.lib().kq_moe_combine_f32 if y.dtype == torch.float32 else _lib.lib().kq_moe_combine
    with torch.cuda.device(d.device):
        _lib.check(fn(d.data_ptr(), p.data_ptr(), T, k, H, _lib.KQ_F16 if d.dtype == torch.float16 else _lib.KQ_BF16,
                      y.data_ptr(), torch.cuda.current_stream(d.device).cuda_stream))
    return y


def combine(d: torch.Tensor, probs: torch.Tensor, k: int) -> torch.Tensor:
    """y[t] = sum_j probs[t, j] * d[t k + j] in float32, rounded once. d [T k, H], probs [T, k] float32."""
    rows, H = d.shape
    T = rows // k
    if d.is_cuda and d.dtype in (torch.float16, torch.bfloat16) and H % 8 == 0 and d.is_contiguous():
        p = probs.reshape(T * k).float().contiguous()
        y = torch.empty((T, H), dtype=d.dtype, device=d.device)
        with torch.cuda.device(d.device):
            _lib.check(_lib.lib().kq_moe_combine(d.data_ptr(), p.data_ptr(), T, k, H,
                                                 _lib.KQ_F16 if d.dtype == torch.float16 else _lib.KQ_BF16,
                                                 y.data_ptr(), torch.cuda.current_stream(d.device).cuda_stream))
        return y
    return (d.reshape(T, k, H).float() * probs.reshape(T, k, 1).float()).sum(dim=1).to(d.dtype)


def fuse_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """[E, F, bytes] x2 -> [E, 2F, bytes]: rows are independent codec streams, so stacking the two matrices of
    every expert along N is a valid weight matrix whose product is gate | up side by side. Done once, at load."""
    return torch.cat([w_gate, w_up], dim=1).contiguous()


_DT = {torch.float32: _lib.KQ_F32, torch.float16: _lib.KQ_F16, torch.bfloat16: _lib.KQ_BF16}
FUSED_MAX_ENTRIES = 512   # beyond (measured on the 128-expert block): the three-gather composition is faster


def _fused_regime(rows: int, n_experts: int) -> bool:
    """The fused decode kernels serve calls below the prefill regime of gather_qmm (512 or more routed entries
    with 16 or more per expert on average go to the tensor-core tile kernel)."""
    return not (rows >= 512 and rows >= 16 * n_experts) and rows <= FUSED_MAX_ENTRIES


def _decode_ws(n_entries: int, n_experts: int, n_mix: int, device):
    need = _lib.lib().kq_moe_decode_workspace_bytes(n_entries, n_experts, n_mix)
    if need == 0:
        return None
    return torch.empty(need, dtype=torch.uint8, device=device)


def codec_has_moe_glu(kquant_type: str) -> bool:
    """True when the codec has the fused MoE decode kernels (the reference's codec_has_moe_glu, src/kquant.h:359)."""
    return bool(_lib.lib().kq_codec_has_moe_glu(kquant_type.encode()))


def _u32(idx: torch.Tensor, device) -> torch.Tensor:
    return idx.to(device=device, dtype=torch.int32).contiguous()


def moe_glu_gather_kq(x, gate_w, up_w, kquant_type, indices, act="silu", limit=0.0, *, workspace=None):
    """The reference's moe_glu_gather_kq (src/kquant.h:335-357): x [T, K], gate_w / up_w [E, N, bytes] (views of
    one stacked tensor are fine: only the last two dims must be dense), indices [T, R] ->
    [T, R, N] = act(x . Wg[e]^T) * (x . Wu[e]^T) in x's dtype, one rounding. Raises NotImplementedError when the
    call has no fused kernel (see kq_moe_glu_gather in include/kquant_b200.h)."""
    if x.dim() != 2 or indices.dim() != 2 or indices.shape[0] != x.shape[0]:
        raise ValueError("[mlx_kquant.moe_glu_gather_kq] x must be [T, K] and indices [T, R].")
    if gate_w.dim() != 3 or up_w.shape != gate_w.shape or gate_w.dtype != torch.uint8 or up_w.dtype != torch.uint8:
        raise ValueError("[mlx_kquant.moe_glu_gather_kq] gate_w / up_w must be uint8 [E, N, bytes] of one shape.")
    for w in (gate_w, up_w):
        if w.stride(2) != 1 or w.stride(1) != w.shape[2]:
            raise ValueError("[mlx_kquant.moe_glu_gather_kq] the expert matrices must be dense in their last two dims.")
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise NotImplementedError("[mlx_kquant.moe_glu_gather_kq] float16 / bfloat16 activations only.")
    T, K = x.shape
    E, N, rb = gate_w.shape
    R = indices.shape[1]
    xc = x.contiguous()
    idx = _u32(indices, x.device)
    y = torch.empty((T, R, N), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        ws = workspace if workspace is not None else _decode_ws(T * R, E, 0, x.device)
        _lib.check(_lib.lib().kq_moe_glu_gather(xc.data_ptr(), _DT[x.dtype], T, K, gate_w.data_ptr(), gate_w.stride(0),
                                                up_w.data_ptr(), up_w.stride(0), rb, N, E, kquant_type.encode(),
                                                idx.data_ptr(), R, act.encode(), float(limit), y.data_ptr(),
                                                ws.data_ptr() if ws is not None else None,
                                                ws.numel() if ws is not None else 0,
                                                torch.cuda.current_stream(x.device).cuda_stream))
    return y


def gather_qmv_kq(x, w, kquant_type, indices):
    """The reference's gather_qmv_kq without bias (src/kquant.h:505-515): x [T, R, K] (one row per expert slot),
    indices [T, R] -> [T, R, N]. This is gather_qmm over the flattened slots."""
    T, R, K = x.shape
    y = gather_qmm(x.reshape(T * R, 1, K), w, None, kquant_type, rhs_indices=indices.reshape(T * R))
    return y.reshape(T, R, -1)


def gather_qmv_mix_ns_kq(x, w, kquant_type, indices, scores, *, workspace=None, reuse_grouping=False):
    """The reference's gather_qmv_mix_ns_kq (src/kquant.h:549-558): x [T, S, K], w [E, N, bytes], indices [T, S],
    scores [T, S] -> [T, N] = sum_s scores[t, s] * (x[t, s] . W[e_s]^T), accumulated in float32, one rounding."""
    if x.dim() != 3 or indices.shape != x.shape[:2] or scores.shape != x.shape[:2]:
        raise ValueError("[mlx_kquant.gather_qmv_mix_ns_kq] x must be [T, S, K], indices and scores [T, S].")
    if w.dim() != 3 or w.dtype != torch.uint8 or w.stride(2) != 1 or w.stride(1) != w.shape[2]:
        raise ValueError("[mlx_kquant.gather_qmv_mix_ns_kq] w must be uint8 [E, N, bytes], dense in its last two dims.")
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise NotImplementedError("[mlx_kquant.gather_qmv_mix_ns_kq] float16 / bfloat16 activations only.")
    T, S, K = x.shape
    E, N, rb = w.shape
    xc = x.contiguous()
    idx = _u32(indices, x.device)
    sc = scores.to(device=x.device, dtype=torch.float32).contiguous()
    y = torch.empty((T, N), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        ws = workspace if workspace is not None else _decode_ws(T * S, E, N, x.device)
        _lib.check(_lib.lib().kq_gather_qmv_mix(xc.data_ptr(), _DT[x.dtype], T, S, K, w.data_ptr(), w.stride(0), rb, N, E,
                                                kquant_type.encode(), idx.data_ptr(), sc.data_ptr(), y.data_ptr(),
                                                ws.data_ptr() if ws is not None else None,
                                                ws.numel() if ws is not None else 0,
                                                1 if (reuse_grouping and ws is not None) else 0,
                                                torch.cuda.current_stream(x.device).cuda_stream))
    return y


def moe_swiglu_block(x, w_gate_up, w_down, kquant_type, expert_ids, expert_probs, *, token_rows=None, tokens=None,
                     out=None, workspace=None, scatter=None):
    """A whole SwiGLU block on the tile kernel (kq_moe_swiglu_block in include/kquant_b200.h): x [T, H] float16 /
    bfloat16, w_gate_up [E, 2F, bytes(H)] (`fuse_gate_up`), w_down [E, H, bytes(F)], expert_ids / expert_probs [T, k]
    -> y [T, H]. Same bits as the three-gather composition with its activation and weighted-sum kernels.
    token_rows [T] (with tokens = T): token t's activation is row token_rows[t] of x. out: a [T, H] tensor of x's
    dtype or float32 to write into. Returns None when the sizes are outside the block's regime.
    scatter = (slot_ptrs int64 [world] on the device, slot dtype, my_rank, tokens_per_rank): the expert-parallel
    form over peer memory (kq_moe_swiglu_block_scatter); nothing is returned but True."""
    T = int(tokens) if tokens is not None else x.shape[0]
    H = x.shape[1]
    k = expert_ids.shape[1]
    E, F2, rb_h = w_gate_up.shape
    F = F2 // 2
    if not (x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and x.stride(1) == 1):
        return None
    if w_down.shape[0] != E or w_down.shape[1] != H:
        raise ValueError("[mlx_kquant.moe_swiglu_block] w_down must be [E, H, bytes] for w_gate_up [E, 2F, bytes].")
    for w in (w_gate_up, w_down):
        if w.dtype != torch.uint8 or w.stride(2) != 1 or w.stride(1) != w.shape[2]:
            raise ValueError("[mlx_kquant.moe_swiglu_block] expert stacks must be uint8, dense in their last two dims.")
    need = _lib.lib().kq_moe_block_workspace_bytes(T, k, E, H, F)
    if need == 0 or x.data_ptr() % 16 or (x.stride(0) * 2) % 16:
        return None
    idx = _u32(expert_ids, x.device)
    sc = expert_probs.to(device=x.device, dtype=torch.float32).contiguous()
    tr = _u32(token_rows, x.device) if token_rows is not None else None
    if scatter is not None:
        ptrs, slot_dtype, my_rank, per_rank = scatter
        with torch.cuda.device(x.device):
            ws = workspace if workspace is not None else torch.empty(need, dtype=torch.uint8, device=x.device)
            _lib.check(_lib.lib().kq_moe_swiglu_block_scatter(
                x.data_ptr(), _DT[x.dtype], T, H, x.stride(0), tr.data_ptr() if tr is not None else None,
                w_gate_up.data_ptr(), w_gate_up.stride(0), rb_h, F, w_down.data_ptr(), w_down.stride(0), w_down.shape[2],
                E, kquant_type.encode(), idx.data_ptr(), sc.data_ptr(), k, ptrs.data_ptr(), _DT[slot_dtype], int(my_rank),
                int(per_rank), ws.data_ptr(), ws.numel(), torch.cuda.current_stream(x.device).cuda_stream))
        return True
    y = out if out is not None else torch.empty((T, H), dtype=x.dtype, device=x.device)
    if y.dtype not in (x.dtype, torch.float32) or not y.is_contiguous() or tuple(y.shape) != (T, H):
        raise ValueError("[mlx_kquant.moe_swiglu_block] out must be a contiguous [T, H] tensor of x's dtype or float32.")
    with torch.cuda.device(x.device):
        ws = workspace if workspace is not None else torch.empty(need, dtype=torch.uint8, device=x.device)
        _lib.check(_lib.lib().kq_moe_swiglu_block(
            x.data_ptr(), _DT[x.dtype], T, H, x.stride(0), tr.data_ptr() if tr is not None else None,
            w_gate_up.data_ptr(), w_gate_up.stride(0), rb_h, F, w_down.data_ptr(), w_down.stride(0), w_down.shape[2], E,
            kquant_type.encode(), idx.data_ptr(), sc.data_ptr(), k, y.data_ptr(), _DT[y.dtype], ws.data_ptr(), ws.numel(),
            torch.cuda.current_stream(x.device).cuda_stream))
    return y


def _fused_decode_ok(x, kquant_type, rows, *stacks) -> bool:
    if not (x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and _fused_regime(rows, stacks[0].shape[0])):
        return False
    if not codec_has_moe_glu(kquant_type):
        return False
    for w in stacks:
        if w.stride(2) != 1 or w.stride(1) != w.shape[2] or w.data_ptr() % 16 or (w.stride(0) % 16):
            return False
        if (w.shape[2] // 144 * 256) % 256 or w.shape[2] % 144:
            return False
    return True


def moe_glu(x, w_gate, w_up, w_down, kquant_type, expert_ids, expert_probs, *, sort_rows: bool = False,
            w_gate_up=None, fused: bool | None = None):
    """x [T, H] (f16 / bf16), expert stacks [E, F, bytes(H)] x2 and [E, H, bytes(F)],
    expert_ids / expert_probs [T, k]. Returns y [T, H] in x's dtype. With w_gate_up = fuse_gate_up(w_gate,
    w_up) the gate and up products are one gather_qmm call (w_gate / w_up may then be None).
    fused: None = the two fused decode launches when the call is small enough and has them, False = always the
    three-gather composition (the reference callers' form, with its bf16 intermediates)."""
    T, H = x.shape
    k = expert_ids.shape[1]
    rows = T * k
    # A few tokens: two launches - gate | up with the activation fused, then down with the weighted sum fused.
    # One rounding (h) where the composition below has three (gate / up, h, down): not bit-identical to it.
    if not sort_rows and fused is not False:
        if w_gate_up is not None:
            F = w_gate_up.shape[1] // 2
            wg_v, wu_v = w_gate_up[:, :F], w_gate_up[:, F:]
        else:
            wg_v, wu_v = w_gate, w_up
        if _fused_decode_ok(x, kquant_type, rows, wg_v, wu_v, w_down):
            # one scratch buffer for both launches: the second reuses the grouping the first made
            ws = _decode_ws(rows, w_down.shape[0], w_down.shape[1], x.device)
            h = moe_glu_gather_kq(x, wg_v, wu_v, kquant_type, expert_ids, workspace=ws)
            return gather_qmv_mix_ns_kq(h, w_down, kquant_type, expert_ids, expert_probs, workspace=ws,
                                        reuse_grouping=True)
        # Prefill sizes with a stacked gate | up: the whole block in one call (one grouping, the first product
        # kept in expert order, the activation inside the pre-pass of the down product); same bits as below.
        if w_gate_up is not None:
            y = moe_swiglu_block(x, w_gate_up, w_down, kquant_type, expert_ids, expert_probs)
            if y is not None:
                return y
    flat_e = expert_ids.reshape(rows)
    tok = torch.arange(T, device=x.device).repeat_interleave(k)
    # Rows go in routing order: gather_qmm groups them by expert on the device itself, so the explicit
    # argsort / unsort that the reference's callers do from 64 routed rows up (src/kquant_gather.cpp:8-16)
    # would only add passes over the activations. sort_rows=True keeps that composition for comparison.
    if sort_rows and rows >= 64:
        order = torch.argsort(flat_e, stable=True)
        flat_e, tok = flat_e[order], tok[order]
    else:
        order = None
    x3 = x.reshape(T, 1, H)
    if w_gate_up is not None:
        F = w_gate_up.shape[1] // 2
        gu = gather_qmm(x3, w_gate_up, None, kquant_type, lhs_indices=tok, rhs_indices=flat_e).reshape(rows, 2 * F)
        h = swiglu(gu[:, :F], gu[:, F:])
    else:
        g = gather_qmm(x3, w_gate, None, kquant_type, lhs_indices=tok, rhs_indices=flat_e)
        u = gather_qmm(x3, w_up, None, kquant_type, lhs_indices=tok, rhs_indices=flat_e)
        F = g.shape[-1]
        h = swiglu(g.reshape(rows, F), u.reshape(rows, F))
    d = gather_qmm(h.reshape(rows, 1, F), w_down, None, kquant_type, rhs_indices=flat_e,
                   sorted_indices=order is not None)
    d = d.reshape(rows, H)
    probs = expert_probs.reshape(rows)
    if order is not None:
        unsort = torch.empty_like(order)
        unsort[order] = torch.arange(rows, device=x.device)
        d = d[unsort]
    return combine(d, probs.reshape(T, k), k)


def moe_glu_expert_parallel(x, w_gate, w_up, w_down, kquant_type, expert_ids, expert_probs, n_experts, group=None,
                            *, w_gate_up=None):
    """The same block with the experts partitioned over the ranks of `group`.

    Every rank holds its own tokens x [T, H] and routing, and only the expert
    matrices of its contiguous share (`dist.shard_bounds(n_experts, rank, world)`;
    w_* are the LOCAL stacks). Routed rows travel to the rank that owns their
    expert with one all-to-all (activations + expert id), are multiplied there, and
    come back with a second all-to-all; the weighted sum over the k experts happens
    where the token lives. The reference has no counterpart (it is single-device).
    """
    import torch.distributed as dist

    from .dist import expert_owner, shard_bounds

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    T, H = x.shape
    k = expert_ids.shape[1]
    rows = T * k
    flat_e = expert_ids.reshape(rows)
    tok = torch.arange(T, device=x.device).repeat_interleave(k)
    owner = expert_owner(flat_e, n_experts, world)
    # rows grouped by destination rank; every rank's per-destination counts are gathered so that one
    # host read gives both the send and the receive splits of the all-to-alls
    order = torch.argsort(owner, stable=True)
    counts = torch.bincount(owner, minlength=world)
    all_counts = torch.empty(world * world, dtype=counts.dtype, device=x.device)
    dist.all_gather_into_tensor(all_counts, counts, group=group)
    table = all_counts.view(world, world).tolist()
    send_counts = table[rank]
    recv_counts = [table[r][rank] for r in range(world)]
    n_recv = sum(recv_counts)
    # dispatch: activations and expert ids of the routed rows, grouped by destination
    send_x = x[tok[order]].contiguous()
    send_e = flat_e[order].to(torch.int32).contiguous()
    recv_x = torch.empty((n_recv, H), dtype=x.dtype, device=x.device)
    recv_e = torch.empty(n_recv, dtype=torch.int32, device=x.device)
    dist.all_to_all_single(recv_x, send_x, output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
    dist.all_to_all_single(recv_e, send_e, output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
    # local experts: rows stay in arrival order, gather_qmm groups them by expert on the device
    lo, _ = shard_bounds(n_experts, rank, world)
    if n_recv > 0:
        es = recv_e.to(torch.int64) - lo
        xs = recv_x.reshape(n_recv, 1, H)
        if w_gate_up is not None:  # the local experts' gate | up stacked along N (fuse_gate_up)
            Fh = w_gate_up.shape[1] // 2
            gu = gather_qmm(xs, w_gate_up, None, kquant_type, rhs_indices=es).reshape(n_recv, 2 * Fh)
            h = swiglu(gu[:, :Fh], gu[:, Fh:]).reshape(n_recv, 1, Fh)
        else:
            g = gather_qmm(xs, w_gate, None, kquant_type, rhs_indices=es)
            u = gather_qmm(xs, w_up, None, kquant_type, rhs_indices=es)
            Fh = g.shape[-1]
            h = swiglu(g.reshape(n_recv, Fh), u.reshape(n_recv, Fh)).reshape(n_recv, 1, Fh)
        out_rows = gather_qmm(h, w_down, None, kquant_type, rhs_indices=es).reshape(n_recv, H)
    else:
        out_rows = torch.empty((0, H), dtype=x.dtype, device=x.device)
    # combine: results return to the rank of their token and are summed there with the routing weights
    back = torch.empty((rows, H), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(back, out_rows.contiguous(), output_split_sizes=send_counts, input_split_sizes=recv_counts,
                           group=group)
    w_sorted = expert_probs.reshape(rows)[order].float()
    y = torch.zeros((T, H), dtype=torch.float32, device=x.device)
    y.index_add_(0, tok[order], back.float() * w_sorted[:, None])
    return y.to(x.dtype)


class GatheredExpertParallel:
    """Expert-parallel MoE SwiGLU block with fixed shapes and no host read inside a step.

    Where `moe_glu_expert_parallel` sends each routed row to the rank of its expert (two all-to-alls whose
    split sizes the host must read first), this form moves the same bytes when top-k equals the rank count
    but needs no sizes: one all-gather gives every rank all tokens with their routing; each rank multiplies
    the rows routed to ITS experts (the other rows carry an out-of-range expert index, which `gather_qmm`,
    the routed `swiglu` and the zero-weight rule of `combine_partial` all skip), forms the float32 partial
    sum per token, and one reduce-scatter adds the partial sums and leaves every rank its own tokens. The
    local stage touches no communicator, so `capture()` can record it into a CUDA graph.

    x [T, H] float16 / bfloat16 with the same T on every rank; w_gate_up [E_local, 2F, bytes] and
    w_down [E_local, H, bytes] are the local experts' stacks (`fuse_gate_up`, `dist.shard_bounds`).
    """

    def __init__(self, T, H, k, n_experts, w_gate_up, w_down, kquant_type, dtype=torch.bfloat16, group=None,
                 *, rank=None, world=None, reduce_dtype=torch.float32):
        from .dist import shard_bounds

        if world is None:  # rank / world given explicitly: no communicator (pack() and local_stage() only)
            import torch.distributed as dist

            world, rank = dist.get_world_size(group), dist.get_rank(group)
        self.group, self.world, self.rank = group, world, rank
        self.T, self.H, self.k, self.kquant_type = T, H, k, kquant_type
        self.w_gate_up, self.w_down = w_gate_up, w_down
        self.lo, hi = shard_bounds(n_experts, self.rank, self.world)
        self.e_local = hi - self.lo
        dev = w_down.device
        row_bytes = H * torch.empty((), dtype=dtype).element_size()
        # routing (ids int32 + weights float32 per routed row) rides in extra rows behind the T activation rows,
        # so that one all-gather moves everything and all ranks' activations form one [W * rows, H] matrix
        self.pad_rows = -(-(T * k * 8) // row_bytes)
        R = T + self.pad_rows
        self.send = torch.zeros((R, H), dtype=dtype, device=dev)
        self.recv = torch.empty((self.world * R, H), dtype=dtype, device=dev)
        # reduce_dtype: float32 partial sums (default), or the activation dtype - half the bytes through the
        # reduce-scatter, at one extra rounding per rank's partial sum and the collective's own sums in that type
        self.partial = torch.empty((self.world * T, H), dtype=reduce_dtype, device=dev)
        self.y32 = torch.empty((T, H), dtype=reduce_dtype, device=dev)
        tok = torch.arange(T, device=dev).repeat_interleave(k)
        self.lhs = (torch.arange(self.world, device=dev)[:, None] * R + tok[None, :]).reshape(-1)
        # row of `recv` that holds token t of rank w, for the one-call block (taken when the sizes allow it)
        self.tok_rows = (torch.arange(self.world, device=dev)[:, None] * R +
                         torch.arange(T, device=dev)[None, :]).reshape(-1).to(torch.int32)
        self.block_ok = bool(dev.type == "cuda" and dtype in (torch.float16, torch.bfloat16) and
                             reduce_dtype in (dtype, torch.float32) and
                             _lib.lib().kq_moe_block_workspace_bytes(self.world * T, k, self.e_local, H,
                                                                     w_gate_up.shape[1] // 2) > 0)
        self._graph = None

    def _meta(self, buf, R):
        return buf.view(-1, R, self.H)[:, self.T:, :].reshape(buf.shape[0] // R, -1).view(torch.int32)

    def local_stage(self):
        """recv (all ranks' tokens and routing) -> partial (this rank's float32 partial sums for all tokens)."""
        T, k, W = self.T, self.k, self.world
        R = T + self.pad_rows
        meta = self._meta(self.recv, R)
        ids = meta[:, :T * k].reshape(W * T * k) - self.lo
        probs = meta[:, T * k:2 * T * k].reshape(W * T * k).view(torch.float32)
        rows = W * T * k
        if self.block_ok:
            # the block skips every entry whose index is outside [0, e_local) by itself (a negative difference
            # reads as a huge unsigned index)
            moe_swiglu_block(self.recv, self.w_gate_up, self.w_down, self.kquant_type, ids.view(W * T, k),
                             probs.view(W * T, k), token_rows=self.tok_rows, tokens=W * T, out=self.partial)
            return
        mine = (ids >= 0) & (ids < self.e_local)
        probs = torch.where(mine, probs, torch.zeros_like(probs))
        Fh = self.w_gate_up.shape[1] // 2
        gu = gather_qmm(self.recv.view(W * R, 1, self.H), self.w_gate_up, None, self.kquant_type,
                        lhs_indices=self.lhs, rhs_indices=ids).reshape(rows, 2 * Fh)
        h = swiglu(gu[:, :Fh], gu[:, Fh:], row_expert=ids, n_experts=self.e_local)
        d = gather_qmm(h.reshape(rows, 1, Fh), self.w_down, None, self.kquant_type, rhs_indices=ids)
        combine_partial(d.reshape(rows, self.H), probs, k, out=self.partial)

    def capture(self):
        """Record the local stage into a CUDA graph (three warm-up runs on a side stream first)."""
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(3):
                self.local_stage()
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.local_stage()
        self._graph = g

    def pack(self, x, expert_ids, expert_probs):
        """Fill `send`: this rank's T activation rows, then ids and weights of its routed rows."""
        T, k = self.T, self.k
        self.send[:T].copy_(x)
        tail = self.send[T:].view(torch.int32).reshape(-1)
        tail[:T * k].copy_(expert_ids.reshape(T * k))
        tail[T * k:2 * T * k].copy_(expert_probs.reshape(T * k).float().view(torch.int32))
        return self.send

    def __call__(self, x, expert_ids, expert_probs):
        import torch.distributed as dist

        self.pack(x, expert_ids, expert_probs)
        dist.all_gather_into_tensor(self.recv, self.send, group=self.group)
        if self._graph is not None:
            self._graph.replay()
        else:
            self.local_stage()
        dist.reduce_scatter_tensor(self.y32, self.partial, group=self.group)
        return self.y32.to(x.dtype)


def moe_sum_slots(slots, expert_ids, rank_lo, out_dtype, *, shape=None, dtype=None):
    """kq_moe_sum_slots: slots [world, T, H] (a tensor, or a raw device pointer with shape= and dtype=), expert_ids
    [T, k] (global indices), rank_lo int32 [world + 1] on the device -> y [T, H] = the sum of the slots of the ranks
    that own one of the token's experts."""
    if isinstance(slots, torch.Tensor):
        ptr, (W, T, H), dtype, dev = slots.data_ptr(), slots.shape, slots.dtype, slots.device
    else:
        ptr, (W, T, H), dev = int(slots), shape, rank_lo.device
    ids = _u32(expert_ids, dev)
    y = torch.empty((T, H), dtype=out_dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().kq_moe_sum_slots(ptr, _DT[dtype], ids.data_ptr(), rank_lo.data_ptr(), W, T, ids.shape[1], H,
                                               y.data_ptr(), _DT[out_dtype], torch.cuda.current_stream(dev).cuda_stream))
    return y


class PeerBuffers:
    """One device buffer per rank, each mapped into every other rank's process (one process per GPU, one node):
    the kq_peer_buffer_* entry points (cudaMalloc + CUDA IPC, opened on the opener's own device with lazy peer
    access); the 64-byte handles travel through the process group's object all-gather. `ptrs[r]` is rank r's
    buffer as seen from this process. close() is collective."""

    def __init__(self, nbytes: int, device, group=None):
        import ctypes as C

        import torch.distributed as dist

        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        L = _lib.lib()
        with torch.cuda.device(device):
            own, handle = C.c_void_p(), (C.c_ubyte * 64)()
            _lib.check(L.kq_peer_buffer_create(nbytes, C.byref(own), handle))
            self.own = own.value
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
            self.ptrs = []
            try:
                for r, h in enumerate(handles):
                    if r == self.rank:
                        self.ptrs.append(self.own)
                        continue
                    p = C.c_void_p()
                    _lib.check(L.kq_peer_buffer_open((C.c_ubyte * 64).from_buffer_copy(h), C.byref(p)))
                    self.ptrs.append(p.value)
            except Exception:
                # give back what this rank holds; the other ranks will time out in the barrier below
                for r, p in enumerate(self.ptrs):
                    if r != self.rank:
                        L.kq_peer_buffer_close(p)
                L.kq_peer_buffer_destroy(self.own)
                self.ptrs = None
                raise
        dist.barrier(group=group)   # every rank has opened every buffer before anyone stores

    def own_tensor(self, shape, dtype):
        """This rank's buffer as a torch tensor (no copy; the buffer stays owned by this object)."""
        n = 1
        for d in shape:
            n *= int(d)
        n *= torch.empty((), dtype=dtype).element_size()

        class _Raw:   # the CUDA array interface over the raw pointer
            __cuda_array_interface__ = {"shape": (n,), "typestr": "|u1", "data": (self.own, False), "version": 2}

        return torch.as_tensor(_Raw(), device=self.device).view(dtype).view(*shape)

    def close(self):
        import torch.distributed as dist

        if self.ptrs is None:
            return
        L = _lib.lib()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for r, p in enumerate(self.ptrs):
                if r != self.rank:
                    _lib.check(L.kq_peer_buffer_close(p))
            dist.barrier(group=self.group)   # nobody still maps this rank's buffer
            _lib.check(L.kq_peer_buffer_destroy(self.own))
        self.ptrs = None


class PeerExpertParallel(GatheredExpertParallel):
    """GatheredExpertParallel whose weighted sum goes straight into the owners' memory: the local stage ends with
    the combine kernel writing each token's partial row into slot [my_rank] of the token's home rank through a
    peer mapping (only tokens with an expert here write), one small collective tells every rank that all writes
    have landed, and a local kernel adds the slots of the ranks that contribute to each token. Against the
    reduce-scatter form: the partial rows cross NVLink once and only the non-empty ones (two thirds at 8 ranks
    and top-8), and no [world * T, H] buffer is written and read again. Needs the one-call block
    (`moe_swiglu_block`) sizes; slots of `reduce_dtype` (default: the activation dtype). close() is collective."""

    def __init__(self, T, H, k, n_experts, w_gate_up, w_down, kquant_type, dtype=torch.bfloat16, group=None, *,
                 reduce_dtype=None, copy_engine_gather=False):
        from .dist import shard_bounds

        reduce_dtype = reduce_dtype or dtype
        super().__init__(T, H, k, n_experts, w_gate_up, w_down, kquant_type, dtype, group, reduce_dtype=reduce_dtype)
        if not self.block_ok:
            raise ValueError("[mlx_kquant.moe] PeerExpertParallel needs sizes the one-call block takes "
                             "(512 or more routed rows over all ranks, 16 per local expert).")
        dev = w_down.device
        self.partial = None   # no local [world * T, H] buffer in this form
        self.slot_dtype = reduce_dtype
        item = torch.empty((), dtype=reduce_dtype).element_size()
        self.buffers = PeerBuffers(self.world * T * H * item, dev, group)
        self.slot_ptrs = torch.tensor(self.buffers.ptrs, dtype=torch.int64, device=dev)
        self.rank_lo = torch.tensor([shard_bounds(n_experts, r, self.world)[0] for r in range(self.world)] + [n_experts],
                                    dtype=torch.int32, device=dev)
        self.flag = torch.zeros(1, dtype=torch.int32, device=dev)
        self.out_dtype = dtype
        # copy_engine_gather: the gathered buffer is peer memory too, and every rank pushes its packed rows into
        # all ranks' buffers with asynchronous copies (copy engines over NVLink: no SM) instead of an all-gather
        self.recv_buffers = None
        if copy_engine_gather:
            rows = T + self.pad_rows
            self.recv_buffers = PeerBuffers(self.world * rows * H * self.send.element_size(), dev, group)
            self.recv = self.recv_buffers.own_tensor((self.world * rows, H), dtype)
            self.recv.zero_()
            self.flag_in = torch.zeros(1, dtype=torch.int32, device=dev)

    def close(self):
        self._graph = None
        self.buffers.close()
        if self.recv_buffers is not None:
            self.recv = None
            self.recv_buffers.close()

    def push(self):
        """Copy-engine form of the all-gather: this rank's packed rows into every rank's gathered buffer, then a
        one-element collective - once it completes here, every rank's rows have landed here."""
        import torch.distributed as dist

        nbytes = self.send.numel() * self.send.element_size()
        st = torch.cuda.current_stream(self.send.device).cuda_stream
        L = _lib.lib()
        for r in range(self.world):
            _lib.check(L.kq_peer_copy_async(self.recv_buffers.ptrs[r] + self.rank * nbytes, self.send.data_ptr(), nbytes, st))
        dist.all_reduce(self.flag_in, group=self.group)

    def finish(self, expert_ids):
        return moe_sum_slots(self.buffers.own, expert_ids, self.rank_lo, self.out_dtype,
                             shape=(self.world, self.T, self.H), dtype=self.slot_dtype)

    def local_stage(self):
        T, k, W = self.T, self.k, self.world
        R = T + self.pad_rows
        meta = self._meta(self.recv, R)
        ids = meta[:, :T * k].reshape(W * T * k) - self.lo
        probs = meta[:, T * k:2 * T * k].reshape(W * T * k).view(torch.float32)
        moe_swiglu_block(self.recv, self.w_gate_up, self.w_down, self.kquant_type, ids.view(W * T, k),
                         probs.view(W * T, k), token_rows=self.tok_rows, tokens=W * T,
                         scatter=(self.slot_ptrs, self.slot_dtype, self.rank, T))

    def __call__(self, x, expert_ids, expert_probs):
        import torch.distributed as dist

        self.pack(x, expert_ids, expert_probs)
        dist.all_gather_into_tensor(self.recv, self.send, group=self.group)
        if self._graph is not None:
            self._graph.replay()
        else:
            self.local_stage()
        # every rank's stores into this rank's slots are complete once every rank has joined this collective
        # (it is queued behind the local stage on each rank's stream)
        dist.all_reduce(self.flag, group=self.group)
        return self.finish(expert_ids)


class PeerPipelinedExpertParallel:
    """PeerExpertParallel over `chunks` token slices with the gather moved by the copy engines: while the expert
    products of slice c run, the rows of slice c + 1 travel over NVLink without taking an SM from the tile
    kernel (NCCL's all-gather beside it costs more than it hides). Per step: pack all slices; on a side
    stream push slice after slice (peer copies + a one-element collective that says "everybody's rows are
    here"); on the main stream, per slice, wait for its rows and replay its local stage (whose weighted sum
    stores into the owners' slots); one collective after the last slice says "all stores have landed"; the
    slot sums. close() is collective."""

    def __init__(self, T, H, k, n_experts, w_gate_up, w_down, kquant_type, dtype=torch.bfloat16, group=None, *,
                 chunks=2, reduce_dtype=None):
        if T % chunks:
            raise ValueError("[mlx_kquant.moe] T must be a multiple of the number of chunks.")
        self.T, self.chunks, self.group = T, chunks, group
        self.parts = [PeerExpertParallel(T // chunks, H, k, n_experts, w_gate_up, w_down, kquant_type, dtype, group,
                                         reduce_dtype=reduce_dtype, copy_engine_gather=True) for _ in range(chunks)]
        dev = w_down.device
        self.side = torch.cuda.Stream(device=dev)
        self.events = [torch.cuda.Event() for _ in range(chunks)]
        self.flag = torch.zeros(1, dtype=torch.int32, device=dev)

    def capture(self):
        for p in self.parts:
            p.capture()

    def close(self):
        for p in self.parts:
            p.close()

    def __call__(self, x, expert_ids, expert_probs):
        import torch.distributed as dist

        n = self.T // self.chunks
        main = torch.cuda.current_stream(x.device)
        for c, p in enumerate(self.parts):
            sl = slice(c * n, (c + 1) * n)
            p.pack(x[sl], expert_ids[sl], expert_probs[sl])
        self.side.wait_stream(main)
        with torch.cuda.stream(self.side):
            for c, p in enumerate(self.parts):
                p.push()
                self.events[c].record(self.side)
        for c, p in enumerate(self.parts):
            main.wait_event(self.events[c])
            if p._graph is not None:
                p._graph.replay()
            else:
                p.local_stage()
        dist.all_reduce(self.flag, group=self.group)   # every rank's stores into the slots have landed
        return torch.cat([p.finish(expert_ids[c * n:(c + 1) * n]) for c, p in enumerate(self.parts)])


class PipelinedExpertParallel:
    """GatheredExpertParallel over `chunks` slices of the tokens, so that the collectives of one slice overlap the
    expert products of another: all slices' all-gathers are issued first (asynchronously, on the communicator's
    stream), then slice by slice "wait for its gather, replay its local stage, issue its reduce-scatter". Same
    results as the unsliced form (every token's sum is formed the same way). T must be a multiple of `chunks`."""

    def __init__(self, T, H, k, n_experts, w_gate_up, w_down, kquant_type, dtype=torch.bfloat16, group=None, *,
                 chunks=2, reduce_dtype=torch.float32):
        if T % chunks:
            raise ValueError("[mlx_kquant.moe] T must be a multiple of the number of chunks.")
        self.T, self.chunks, self.group = T, chunks, group
        self.parts = [GatheredExpertParallel(T // chunks, H, k, n_experts, w_gate_up, w_down, kquant_type, dtype,
                                             group, reduce_dtype=reduce_dtype) for _ in range(chunks)]

    def capture(self):
        for p in self.parts:
            p.capture()

    def __call__(self, x, expert_ids, expert_probs):
        import torch.distributed as dist

        n = self.T // self.chunks
        gathers, sums = [], []
        for c, p in enumerate(self.parts):
            sl = slice(c * n, (c + 1) * n)
            p.pack(x[sl], expert_ids[sl], expert_probs[sl])
            gathers.append(dist.all_gather_into_tensor(p.recv, p.send, group=self.group, async_op=True))
        for c, p in enumerate(self.parts):
            gathers[c].wait()
            if p._graph is not None:
                p._graph.replay()
            else:
                p.local_stage()
            sums.append(dist.reduce_scatter_tensor(p.y32, p.partial, group=self.group, async_op=True))
        for w in sums:
            w.wait()
        return torch.cat([p.y32 for p in self.parts]).to(x.dtype)


def host_tile_maps(counts, device=None):
    """Host-built equivalent of `expert_tile_map` from per-expert row counts (mlx_kquant/nn.py:33-47): segments
    cut into 64-row pieces, only the last piece of a segment partial. Returns (map int32 [n, 3], count int32 [1])."""
    tiles, row = [], 0
    for e, c in enumerate(int(v) for v in counts):
        for off in range(0, c, 64):
            tiles.append((e, row + off, min(64, c - off)))
        row += c
    m = torch.tensor(tiles or [(0, 0, 0)], dtype=torch.int32, device=device)
    return m, torch.tensor([len(tiles)], dtype=torch.int32, device=device)


def moe_router_topk(logits, top_k, norm_topk_prob, shared_gate=True, per_expert_scale=None, bias=None,
                    scoring="softmax", scale=1.0):
    """Router top-k with the reference op's semantics (src/kquant.h:560-585): score the E expert columns in
    float32 ("softmax", or "sqrtsoftplus" = sqrt(softplus(x))), pick the `top_k` largest of score (+ `bias` [E],
    which ranks the selection only), lowest index first among equals, optionally renormalise the picked scores
    (the sqrtsoftplus renormalisation carries a 1e-20 guard), multiply by `per_expert_scale` [E] of the picked
    experts and by the uniform `scale`. With `shared_gate`, logits are [T, E + 1] and the sigmoid of column E
    lands in an extra last scores slot. Returns (indices [T, top_k] int32, scores float32 [T, top_k (+ 1)]).
    One kernel launch for CUDA logits (kq_moe_router_topk); torch ops for host tensors. E <= 1024 and
    top_k <= 16 as in the reference."""
    if scoring not in ("softmax", "sqrtsoftplus"):
        raise ValueError(f"[mlx_kquant.moe_router_topk] unknown scoring '{scoring}'.")
    if logits.dim() != 2:
        raise ValueError(f"[mlx_kquant.moe_router_topk] logits must be [T, E] but got shape {tuple(logits.shape)}.")
    E = logits.shape[1] - (1 if shared_gate else 0)
    if E < 1 or E > 1024 or top_k < 1 or top_k > 16 or top_k > E:
        raise ValueError("[mlx_kquant.moe_router_topk] needs 1 <= top_k <= min(E, 16) and E <= 1024.")
    if scoring == "sqrtsoftplus" and not norm_topk_prob:
        raise ValueError("[mlx_kquant.moe_router_topk] sqrtsoftplus has no global normaliser: norm_topk_prob is required.")
    if logits.is_cuda and logits.dtype in _DT:
        T = logits.shape[0]
        lc = logits.contiguous()
        idx = torch.empty((T, top_k), dtype=torch.int32, device=logits.device)
        sc = torch.empty((T, top_k + (1 if shared_gate else 0)), dtype=torch.float32, device=logits.device)
        pes = per_expert_scale.to(device=logits.device, dtype=torch.float32).contiguous() if per_expert_scale is not None else None
        bs = bias.to(device=logits.device, dtype=torch.float32).contiguous() if bias is not None else None
        with torch.cuda.device(logits.device):
            _lib.check(_lib.lib().kq_moe_router_topk(lc.data_ptr(), _DT[logits.dtype], T, E, top_k,
                                                     1 if norm_topk_prob else 0, 1 if shared_gate else 0,
                                                     pes.data_ptr() if pes is not None else None,
                                                     bs.data_ptr() if bs is not None else None, scoring.encode(),
                                                     float(scale), idx.data_ptr(), sc.data_ptr(),
                                                     torch.cuda.current_stream(logits.device).cuda_stream))
        return idx, sc
    # host tensors: the same computation in torch ops
    lf = logits.float()
    x = lf[:, :E]
    if scoring == "softmax":
        p = torch.softmax(x, dim=-1)
    else:
        p = torch.sqrt(torch.nn.functional.softplus(x, threshold=88.0))
    rank = p if bias is None else p + bias.to(p.device).float()
    # a stable descending sort puts the lowest index first among equal scores
    idx = torch.sort(rank, dim=-1, descending=True, stable=True).indices[:, :top_k]
    picked = torch.gather(p, 1, idx)
    if norm_topk_prob:
        s = picked.sum(dim=-1, keepdim=True)
        picked = picked / (s + 1e-20 if scoring == "sqrtsoftplus" else s)
    if per_expert_scale is not None:
        picked = picked * per_expert_scale.to(p.device).float()[idx]
    if scale != 1.0:
        picked = picked * float(scale)
    if shared_gate:
        picked = torch.cat([picked, torch.sigmoid(lf[:, E:E + 1])], dim=1)
    return idx.to(torch.int32), picked
