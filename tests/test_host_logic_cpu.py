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


# ---- plan-shape bucketing and packing (model/src/encoder_head.rs:366-533; qwen3/embed.rs:26-62) ----
from svod_b200 import encoder_head as EH


def test_plan_shape_buckets_rows_and_length():
    assert EH.plan_shape(1, 1, 64) == (1, 128)
    assert EH.plan_shape(3, 128, 64) == (4, 128)
    assert EH.plan_shape(5, 129, 64) == (8, 256)
    assert EH.plan_shape(70, 500, 64) == (64, 512)
    assert EH.plan_shape(2, 0, 8) == (2, 128)


def test_pack_ids_and_mask_pad_rows_and_tails():
    batch = [[5, 6, 7], [9]]
    ids = EH.pack_ids(batch, 4, 128, pad_id=1)
    assert ids.shape == (4, 128) and list(ids[0, :4]) == [5, 6, 7, 1] and ids[1, 0] == 9 and np.all(ids[2:] == 1)
    m = EH.pack_mask(batch, 4, 128)
    assert m[0, :3].all() and not m[0, 3:].any() and m[1, 0] and not m[1, 1:].any()
    # an unused row attends to its first (pad) token alone
    assert m[2, 0] and m[3, 0] and not m[2:, 1:].any()


def test_first_fit_packing_longest_first():
    lens = [300, 20, 100, 100, 128, 7, 1]
    batches = EH.pack(lens, max_batch=2)
    placed = sorted(i for b in batches for row in b.rows for i in row)
    assert placed == list(range(len(lens)))
    first = batches[0]
    assert first.bucket == 384                       # 300 rounded up to the 128-token tile
    for b in batches:
        for row in b.rows:
            assert sum(lens[i] for i in row) <= b.bucket and len(row) <= b.bucket // EH.SLOT_TOKENS
    assert first.rows[0][0] == 0                      # the longest row opens the first plan row
    # slots bound: sixteen tokens of capacity per pooled slot
    many = EH.pack([1] * 40, max_batch=1)
    assert many[0].bucket == 128 and len(many[0].rows[0]) == 8 and len(many) == 5


def test_packed_inputs_positions_segments_and_pool_slots():
    rows = [[11, 12, 13], [21, 22], []]
    lens = [3, 2, 1]
    batch = EH.PackedBatch(128, [[0, 1, 2], []])
    ids, pos, seg, pool = EH.packed_inputs(batch, rows, lens, 2, pad_id=0)
    assert list(ids[0, :6]) == [11, 12, 13, 21, 22, 0]
    assert list(pos[0, :6]) == [0, 1, 2, 0, 1, 0]
    assert list(seg[0, :7]) == [0, 0, 0, 3, 3, 5, 6]   # padding: each token its own segment
    assert list(pool[0, :3]) == [2, 4, 5]
    assert list(seg[1, :3]) == [0, 1, 2] and np.all(ids[1] == 0)
