"""Host-side sharding logic with two gloo ranks on CPU: a column-sharded matmul
all-gathered over the ranks equals the unsharded result bit for bit (K is never
split, so each output element is computed identically), and the expert-partition
helpers route every row to the rank that owns its expert."""
from __future__ import annotations

import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mlx_kquant_b200.dist import column_shard, expert_owner, gather_columns, shard_bounds, split_by_owner


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle.kq_oracle import Oracle

        golden = np.load(os.path.join(os.path.dirname(__file__), "golden", "kq_golden.npz"))
        oracle = Oracle()
        wire = golden["enc_q4_k_wire"][:15]                     # N = 15: ragged over two ranks (8 + 7)
        x = golden["x_m8"].astype(np.float16)
        full = oracle.qmm(x, wire, "q4_k", "f16")
        mine = column_shard(torch.from_numpy(wire), rank, world).numpy()
        y_r = torch.from_numpy(oracle.qmm(x, np.ascontiguousarray(mine), "q4_k", "f16"))
        y = gather_columns(y_r, wire.shape[0])
        ok = bool(np.array_equal(y.numpy().view(np.uint16), full.view(np.uint16)))
        # expert partition: 5 experts over 2 ranks -> ranks own {0,1,2} and {3,4}
        ids = torch.tensor([4, 0, 3, 2, 1, 4, 0])
        owner = expert_owner(ids, 5, world)
        order, counts = split_by_owner(owner, world)
        ok = ok and owner.tolist() == [1, 0, 1, 0, 0, 1, 0] and counts == [4, 3]
        ok = ok and ids[order].tolist() == [0, 2, 1, 0, 4, 3, 4]
        # dispatch: every rank sends its routed rows to the owners and gets back what it owns
        recv_counts = torch.zeros(world, dtype=torch.int64)
        dist.all_to_all_single(recv_counts, torch.tensor(counts))
        send = ids[order].to(torch.int64)
        recv = torch.empty(int(recv_counts.sum()), dtype=torch.int64)
        dist.all_to_all_single(recv, send, output_split_sizes=recv_counts.tolist(), input_split_sizes=counts)
        lo, hi = shard_bounds(5, rank, world)
        ok = ok and bool(((recv >= lo) & (recv < hi)).all())
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_shard_bounds_cover_everything():
    for n in (1, 7, 16, 4096, 14336):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))


def test_two_rank_column_shard_and_expert_dispatch():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]
