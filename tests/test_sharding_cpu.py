"""CPU tests of the multi-GPU host logic: partitioning rules, and a world-size-2 gloo run of the
rank protocol bench.py uses (deterministic shards, barrier, max-over-ranks of the timed interval)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from composable_kernel_b200.sharding import batch_shard, grouped_gemm_shard, lpt_partition

MS = [256 * (1 + g % 16) for g in range(64)]  # the 64-group configuration


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_grouped_shards_are_balanced_and_cover_every_group_once(world):
    parts = lpt_partition(MS, world)
    assert sorted(i for p in parts for i in p) == list(range(64))
    loads = [sum(MS[i] for i in p) for p in parts]
    assert sum(loads) == sum(MS) == 139264
    # weights 1..16 (x4 each): 544 units split exactly (68 per GPU at 8 GPUs)
    assert max(loads) - min(loads) <= 256
    if world == 8:
        assert loads == [68 * 256] * 8


@pytest.mark.parametrize("n,world", [(128, 1), (128, 2), (128, 8), (10, 4), (3, 8)])
def test_batch_shards_partition_the_batch(n, world):
    spans = [batch_shard(n, r, world) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == n
    for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
        assert a1 == b0 and a1 >= a0 and b1 >= b0
    sizes = [b - a for a, b in spans]
    assert max(sizes) - min(sizes) <= 1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_main(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = grouped_gemm_shard(MS, rank, world)
        b0, b1 = batch_shard(128, rank, world)
        # every rank contributes what it owns; together they must cover the job exactly once
        owned = torch.zeros(64, dtype=torch.int64)
        owned[mine] = 1
        dist.all_reduce(owned)
        images = torch.tensor([b1 - b0], dtype=torch.int64)
        dist.all_reduce(images)
        # timing protocol: barrier, local interval, MAX over ranks
        dist.barrier()
        t = torch.tensor([1.0 + rank], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        flop = sum(2 * MS[i] * 4096 * 4096 for i in mine)
        total = torch.tensor([float(flop)], dtype=torch.float64)
        dist.all_reduce(total)
        q.put((rank, owned.tolist(), int(images.item()), float(t.item()), float(total.item())))
    finally:
        dist.destroy_process_group()


def test_two_rank_protocol_over_gloo():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, owned, images, tmax, total in results:
        assert owned == [1] * 64          # each group on exactly one rank
        assert images == 128              # batch shards add up
        assert tmax == float(world)       # max over ranks
        assert total == float(sum(2 * m * 4096 * 4096 for m in MS))
