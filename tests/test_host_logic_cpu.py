"""Host-side logic that needs no GPU: row sharding and the world-size-2
all-gather of pooled rows over gloo."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from svod_b200.encoders import gather_pooled, shard_rows


def test_shard_rows_deals_longest_first_round_robin():
    lens = [5, 100, 7, 64, 33, 90, 1, 2]
    shards = shard_rows(lens, 2)
    assert sorted(shards[0] + shards[1]) == list(range(8))
    assert shards[0][0] == 1 and shards[1][0] == 5          # longest two lead the two ranks
    tot = [sum(lens[i] for i in s) for s in shards]
    assert abs(tot[0] - tot[1]) <= max(lens)
    assert shard_rows(lens, 1) == [sorted(range(8), key=lambda i: -lens[i])]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, rows, d, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    gathered = torch.zeros(world * rows, d)
    local = gathered[rank * rows:(rank + 1) * rows]          # this rank's slot of the gather buffer
    local.copy_(torch.arange(rows * d, dtype=torch.float32).view(rows, d) + 1000 * rank)
    gather_pooled(local, gathered)
    ret[rank] = gathered.clone().numpy()
    dist.barrier()
    dist.destroy_process_group()


def test_all_gather_of_pooled_rows_world_size_2():
    world, rows, d = 2, 3, 8
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), rows, d, ret), nprocs=world, join=True)
    want = np.concatenate([np.arange(rows * d, dtype=np.float32).reshape(rows, d) + 1000 * r for r in range(world)])
    for r in range(world):
        assert np.array_equal(ret[r], want)
