"""Host-side multi-GPU logic on CPU ranks (gloo, world size 2): the M-shard partition covers every
row exactly once, and the N-split form (column shards of W, one all-gather, re-layout) reproduces
the unsharded result bit for bit."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from aitemplate_b200 import sharding


def test_shard_range_partitions_exactly():
    for total in (0, 1, 7, 64, 65536, 1000003):
        for world in (1, 2, 3, 4, 8):
            spans = [sharding.shard_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(8, 2, 2)
    with pytest.raises(ValueError):
        sharding.split_weight_columns(torch.zeros(7, 4), None, 2, 0)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(7)
        x = torch.randn((37, 24), generator=g).half().float()
        w = torch.randn((16, 24), generator=g).half().float()
        b = torch.randn((16,), generator=g).half().float()
        full = torch.relu(torch.nn.functional.linear(x, w, b)).half()
        # M-sharded: each rank computes its rows, nothing is exchanged on the data path
        rows = sharding.shard_rows(x, world, rank)
        mine = torch.relu(torch.nn.functional.linear(rows, w, b)).half()
        start, stop = sharding.shard_range(x.shape[0], world, rank)
        ok_m = torch.equal(mine, full[start:stop])
        # N-split: column shard of the weight, one all-gather, re-layout
        w_r, b_r = sharding.split_weight_columns(w, b, world, rank)
        y_r = torch.relu(torch.nn.functional.linear(x, w_r, b_r)).half()
        y = sharding.gather_columns(y_r, world, relayout=lambda t: t.permute(1, 0, 2).contiguous())
        ok_n = torch.equal(y, full)
        # max-over-ranks timing reduction used by the benchmark
        t = torch.tensor([float(rank + 1)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        results[rank] = (ok_m, ok_n, float(t.item()))
    finally:
        dist.destroy_process_group()


def test_m_shard_and_n_split_on_two_gloo_ranks():
    world = 2
    port = _free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert len(results) == world
        for rank in range(world):
            ok_m, ok_n, tmax = results[rank]
            assert ok_m and ok_n and tmax == float(world)
