"""The multi-GPU host logic (sequence sharding, slowest-rank timing) on two CPU ranks over gloo."""
import os
import sys

import pytest
import torch.multiprocessing as mp

from tenzo_b200.sharding import shard_sequences


def test_shards_partition_the_batch():
    for batch in (0, 1, 7, 256, 257):
        for world in (1, 2, 3, 8):
            spans = [shard_sequences(batch, world, r) for r in range(world)]
            assert sum(c for _, c in spans) == batch
            nxt = 0
            for first, count in spans:
                assert first == nxt
                nxt += count
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    with pytest.raises(ValueError):
        shard_sequences(4, 2, 2)


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from tenzo_b200.sharding import max_over_ranks, shard_sequences
    first, count = shard_sequences(257, world, rank)
    ids = torch.full((130,), -1, dtype=torch.int64)
    ids[:count] = torch.arange(first, first + count)
    gathered = [torch.empty_like(ids) for _ in range(world)]
    dist.all_gather(gathered, ids)
    seen = sorted(int(v) for g in gathered for v in g if v >= 0)
    slow = max_over_ranks(1.0 + rank, device="cpu")
    dist.barrier()
    dist.destroy_process_group()
    q.put((rank, seen == list(range(257)), slow))


def test_two_ranks_cover_every_sequence_once_and_report_the_slowest():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29000 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in res)
    assert all(slow == 2.0 for _, _, slow in res)
