"""Host-side sharding logic, including the multi-process path on CPU (gloo, world size 2)."""
import os
import random

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from bladedisc_b200 import sharding


def test_row_and_column_ranges_partition_exactly():
    for total in (0, 1, 7, 64, 333, 16384):
        for world in (1, 2, 3, 4, 8):
            spans = [sharding.row_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for a, b in zip(spans, spans[1:]):
                assert a[1] == b[0]
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    cols = [sharding.column_range(11008, 8, r) for r in range(8)]
    assert cols[0][0] == 0 and cols[-1][1] == 11008
    assert all(b % 128 == 0 for b, _ in cols)
    with pytest.raises(ValueError):
        sharding.row_range(10, 2, 2)


def test_balance_sequences_properties():
    rng = random.Random(0)
    for trial in range(20):
        n = rng.randint(1, 70)
        lens = [rng.randint(16, 512) for _ in range(n)]
        for world in (1, 2, 4, 8):
            a = sharding.balance_sequences(lens, world)
            assert len(a) == world
            assert sorted(sum(a, [])) == list(range(n))          # every sequence exactly once
            cost = sharding.padded_cost(lens, a)
            if n >= world:
                assert all(len(x) >= 1 for x in a)
            # never worse than the trivial contiguous split of the sorted order
            order = sorted(range(n), key=lambda i: -lens[i])
            naive = [order[sharding.row_range(n, world, r)[0]:sharding.row_range(n, world, r)[1]] for r in range(world)]
            assert max(cost) <= max(sharding.padded_cost(lens, naive))
    assert sharding.balance_sequences([], 4) == [[], [], [], []]
    assert sharding.balance_sequences([5, 5, 5], 8)[:3] == [[0], [1], [2]]


def _worker(rank, world, port, lens, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = sharding.balance_sequences(lens, world)[rank]
        # what bench.py does around a timed region: barrier, per-rank time, MAX over ranks, SUM of work
        dist.barrier()
        t = torch.tensor([10.0 + rank, 3.0], dtype=torch.float64)
        work = torch.tensor([float(len(mine)), float(sum(lens[i] for i in mine))], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(work, op=dist.ReduceOp.SUM)
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        b, e = sharding.row_range(1000, world, rank)
        rows = torch.tensor([float(e - b)])
        dist.all_reduce(rows)
        q.put((rank, t.tolist(), work.tolist(), gathered, rows.item()))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_sharding():
    rng = random.Random(1)
    lens = [rng.randint(16, 512) for _ in range(32)]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_worker, args=(r, 2, port, lens, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, t, work, gathered, rows in results:
        assert t == [11.0, 3.0]                        # max over ranks
        assert work == [32.0, float(sum(lens))]        # every sequence counted once
        assert sorted(sum(gathered, [])) == list(range(32))
        assert rows == 1000.0
