"""Sharding of the quantized-weight path across the GPUs of one box.

The reference has no multi-device code; the two shardings below are the ones
its wire format allows without touching a byte of it:

* column shard (dense FFN weights): rows of the wire matrix are independent
  codec streams, so rank r simply keeps rows [r*N/g, (r+1)*N/g). Activations are
  replicated, every rank computes y_r [M, N/g] with the ordinary kernels (K is
  not split, so each output element is bit-identical to the single-GPU result)
  and one all-gather assembles [M, N].
* expert partition (MoE): rank r keeps experts [r*E/g, (r+1)*E/g); routed rows
  are exchanged with all-to-all (`expert_owner`, `split_by_owner`).

Collectives go through torch.distributed (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_bounds(n: int, rank: int, world: int) -> tuple[int, int]:
    """Rows [lo, hi) of an n-row matrix kept by `rank`; the first n % world ranks get one extra row."""
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def column_shard(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """This rank's rows of a wire matrix [N, bytes] (a view, no copy)."""
    lo, hi = shard_bounds(w.shape[-2], rank, world)
    return w[..., lo:hi, :]


def gather_columns(y_shard: torch.Tensor, n_total: int, group=None) -> torch.Tensor:
    """All-gather per-rank outputs [M, N_r] into [M, N]. Shards may differ in width by one row
    (ragged N); they are padded to the widest for the collective and trimmed afterwards."""
    world = dist.get_world_size(group)
    M = y_shard.shape[0]
    widest = (n_total + world - 1) // world
    send = y_shard
    if y_shard.shape[1] != widest:
        send = torch.zeros((M, widest), dtype=y_shard.dtype, device=y_shard.device)
        send[:, : y_shard.shape[1]] = y_shard
    flat = torch.empty((world * M, widest), dtype=y_shard.dtype, device=y_shard.device)
    dist.all_gather_into_tensor(flat, send.contiguous(), group=group)  # rank-major concatenation along dim 0
    out = flat.view(world, M, widest)
    parts = []
    for r in range(world):
        lo, hi = shard_bounds(n_total, r, world)
        parts.append(out[r, :, : hi - lo])
    return torch.cat(parts, dim=1)


def expert_owner(expert_ids: torch.Tensor, n_experts: int, world: int) -> torch.Tensor:
    """Rank that holds each expert under the contiguous partition of shard_bounds()."""
    base, extra = divmod(n_experts, world)
    cut = extra * (base + 1)
    return torch.where(expert_ids < cut, expert_ids // (base + 1), extra + (expert_ids - cut) // max(base, 1))


def split_by_owner(owner: torch.Tensor, world: int) -> tuple[torch.Tensor, list[int]]:
    """Stable permutation that groups routed rows by destination rank, and the per-rank counts
    (the send splits of the dispatch all-to-all)."""
    order = torch.argsort(owner, stable=True)
    counts = torch.bincount(owner, minlength=world).tolist()
    return order, counts
