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


# ------------------------------------------------ column-parallel (N-split) host logic
def test_column_share_and_gathered_layout():
    from bladedisc_b200 import tp
    for world in (1, 2, 4, 8):
        spans = [tp.column_share(11008, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == 11008
        assert len({e - b for b, e in spans}) == 1 and all((e - b) % 16 == 0 for b, e in spans)
    with pytest.raises(ValueError):
        tp.column_share(11008, 3, 0)      # not an even split
    with pytest.raises(ValueError):
        tp.column_share(4096, 8, 8)
    x = torch.arange(6 * 8).reshape(6, 8)
    g = tp.rowmajor_to_gathered(x, 4)
    assert g.shape == (4, 6, 2) and torch.equal(g[1, :, 0], x[:, 2])
    assert torch.equal(tp.gathered_to_rowmajor(g), x)


def _tp_worker(rank, world, port, q):
    """Each rank computes its shard of a quantized linear with the CPU oracle; the
    shards meet through a real all-gather (gloo) in the rank-major layout the GPU
    path produces, and the next linear reads that layout slab by slab."""
    import numpy as np
    from oracle import c
    from bladedisc_b200 import tp
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)  # same data on every rank
        M, K, N, N2 = 9, 64, 32 * world, 16
        a = rng.integers(-127, 128, (M, K), dtype=np.int8)
        w = rng.integers(-127, 128, (N, K), dtype=np.int8)
        w2 = rng.integers(-127, 128, (N2, N), dtype=np.int8)
        sw = (rng.random(N) * 9e-3 + 1e-3).astype(np.float32)
        b, e = tp.column_share(N, world, rank)
        _, mine = c.qgemm_epilogue(c.qgemm_acc(a, w[b:e]), x_scale=np.float32(0.02), w_scale=sw[b:e],
                                   out_scale=np.float32(0.05), div_out=True)
        slots = [torch.empty((M, e - b), dtype=torch.int8) for _ in range(world)]
        dist.all_gather(slots, torch.from_numpy(mine))
        gathered = torch.stack(slots)                      # [g, M, N / g]
        _, full = c.qgemm_epilogue(c.qgemm_acc(a, w), x_scale=np.float32(0.02), w_scale=sw,
                                   out_scale=np.float32(0.05), div_out=True)
        ok_layout = bool((tp.gathered_to_rowmajor(gathered).numpy() == full).all())
        # K of the next linear walked slab by slab equals the row-major product
        acc = np.zeros((M, N2), dtype=np.int32)
        share = e - b
        for s in range(world):
            acc += c.qgemm_acc(np.ascontiguousarray(gathered[s].numpy()), np.ascontiguousarray(w2[:, s * share:(s + 1) * share]))
        ok_chain = bool((acc == c.qgemm_acc(full, w2)).all())
        # per-row scale of a row spread over the ranks = max of the local scales
        local = torch.tensor(np.abs(mine).max(axis=1) / 127.0)
        dist.all_reduce(local, op=dist.ReduceOp.MAX)
        ok_scale = bool(np.allclose(local.numpy(), np.abs(full).max(axis=1) / 127.0))
        q.put((rank, ok_layout, ok_chain, ok_scale))
    finally:
        dist.destroy_process_group()


def test_two_rank_column_parallel_on_cpu(golden):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + random.randint(0, 200)
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == [(0, True, True, True), (1, True, True, True)]


def test_balance_packed_properties():
    """Every sequence exactly once, the same answer on every call, no rank idle while sequences remain, and the
    heaviest rank within one longest sequence of the mean."""
    import random
    rnd = random.Random(7)
    for world in (1, 2, 4, 8):
        for n in (0, 1, 3, 8, 32, 64):
            lens = [rnd.randint(16, 512) for _ in range(n)]
            a = sharding.balance_packed(lens, world)
            assert a == sharding.balance_packed(lens, world)
            assert sorted(i for part in a for i in part) == list(range(n))
            assert sum(1 for part in a if part) == min(world, n)
            if n:
                loads = [sum(sharding.packed_cost(lens[i]) for i in part) for part in a]
                mean = sum(loads) / world
                assert max(loads) <= mean + sharding.packed_cost(max(lens)) + 1e-9
