"""World-size-2 (gloo, CPU) checks of the multi-GPU host logic: voice sharding, the global-batch loss
mean, max-over-ranks timing aggregation and the gradient all-reduce wrapper.  The per-shard losses are
computed with the CPU oracle, so the identity tested is the one the GPU ranks rely on:
mean over the global batch == sum_r(mean_r * B_r) / B."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dgen_b200 import sharding
from oracle import oracle as orc


def test_shard_ranges_partition_the_batch():
    for total, world in ((256, 8), (16, 2), (10, 4), (3, 8), (1, 1)):
        spans = [sharding.shard_range(total, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
        sizes = [e - b for b, e in spans]
        assert max(sizes) - min(sizes) <= 1


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(7)
    B, T = 5, 2048                                    # uneven shards: 3 + 2
    x = rng.standard_normal((B, T)).astype(np.float32)
    y = rng.standard_normal((B, T)).astype(np.float32)
    b0, b1 = sharding.shard_range(B, rank, world)
    local = orc.mss_loss(x[b0:b1], y[b0:b1], sizes=(256, 64))
    glob = sharding.global_mean_loss(local, b1 - b0)
    tmax = sharding.max_over_ranks([1.0 + rank, 5.0 - rank])
    g = torch.full((4,), float(rank + 1))
    sharding.allreduce_sum_(g)
    if rank == 0:
        q.put((glob, orc.mss_loss(x, y, sizes=(256, 64)), tmax, g.tolist()))
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_single_rank_loss():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    glob, single, tmax, g = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert abs(glob - single) < 1e-6 * abs(single)
    assert tmax == [2.0, 5.0]
    assert g == [3.0] * 4
