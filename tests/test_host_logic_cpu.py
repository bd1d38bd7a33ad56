"""Host-side logic that needs no GPU: row sharding and the world-size-2
all-gather of pooled rows over gloo."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from svod_b200.encoders import gather_pooled, shard_rows, unshard_rows


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


def _embed_stub(ids):
    """Stands in for the stack: a row's output depends on that row alone."""
    return torch.stack([ids.float().sum(1), ids.float().max(1).values, ids[:, 0].float()], 1)


def _strong_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(5)                       # the same batch on every rank
    ids = torch.randint(0, 1000, (8, 16), generator=g)
    lens = [int(x) for x in torch.randint(1, 17, (8,), generator=g)]
    shards = shard_rows(lens, world)
    per = len(shards[rank])
    gathered = torch.zeros(world * per, 3)
    local = gathered[rank * per:(rank + 1) * per]
    local.copy_(_embed_stub(ids[torch.tensor(shards[rank])]))
    gather_pooled(local, gathered)
    ret[rank] = (unshard_rows(gathered, shards).numpy(), _embed_stub(ids).numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_one_batch_dealt_over_two_ranks_comes_back_in_input_order():
    """The strong-scaling path: one batch's rows dealt by length over the ranks,
    each rank's rows gathered, the deal undone: every rank holds what one process
    computes on the whole batch."""
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_strong_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    for r in range(2):
        got, want = ret[r]
        assert np.array_equal(got, want)


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


# ---- config store (the small stand-in for tk/src/tune.rs) ----------------------------------------
def test_tune_store_round_trips_and_tolerates_bad_files(tmp_path, monkeypatch):
    from svod_b200 import tune
    from svod_b200 import _lib as L
    lib = L.load()
    lib.svodb_config_clear()
    st = tune.TuneStore("NVIDIA B200", "0.1", tmp_path)
    assert st.load() == 0  # no file: a miss, not an error
    st.put("gemm|bf16|1024|4096|1024|plain", 128, 1234.5)
    st.put("attention|bfloat16|2|1|4096|16|128|cache", 8, 99.0)
    assert lib.svodb_config_get(b"gemm|bf16|1024|4096|1024|plain") == 128
    assert lib.svodb_config_get(b"attention|bfloat16|2|1|4096|16|128|cache") == 0  # host-side entry
    lib.svodb_config_clear()
    st2 = tune.TuneStore("NVIDIA B200", "0.1", tmp_path)
    assert st2.load() == 2 and st2.get("gemm|bf16|1024|4096|1024|plain") == 128
    assert lib.svodb_config_get(b"gemm|bf16|1024|4096|1024|plain") == 128  # pushed into the library on load
    # a line that does not parse is dropped at the next write
    with open(st2.path, "a") as f:
        f.write("garbage line\nkey notanumber 1\n")
    st3 = tune.TuneStore("NVIDIA B200", "0.1", tmp_path)
    assert st3.load() == 2 and st3.dropped == 2
    st3.save()
    assert "garbage" not in st3.path.read_text()
    # another format orphans the file
    st3.path.write_text("format 0\nx 1 1\n")
    assert tune.TuneStore("NVIDIA B200", "0.1", tmp_path).load() == 0
    # one file per device and version; the directory comes from the environment
    monkeypatch.setenv("SVODB_TUNE_DIR", str(tmp_path / "elsewhere"))
    other = tune.TuneStore("NVIDIA H100", "0.1")
    assert other.path.parent == tmp_path / "elsewhere" and other.path.name != st3.path.name
    # an unwritable store is a miss
    ro = tune.TuneStore("x", "0.1", "/proc/definitely/not/writable")
    ro.put("gemm|bf16|1|8|16|plain", 64, 1.0)
    assert ro.get("gemm|bf16|1|8|16|plain") == 64 and not ro.save()
    lib.svodb_config_set(b"gemm|bf16|1|8|16|plain", 0)
    assert lib.svodb_config_get(b"gemm|bf16|1|8|16|plain") == 0
    lib.svodb_config_clear()


# ---- text pipeline front end (arch/src/pipelines/text.rs:575-667, 883-1134) ----------------------
class _WordTokenizer:
    """[CLS] word ids [SEP]; offsets = byte position of each word."""
    def encode(self, text):
        from svod_b200.pipeline import Encoding
        ids, offs, at = [0], [0], 0
        for w in text.split(" "):
            ids.append(100 + len(w)), offs.append(at)
            at += len(w) + 1
        return Encoding(ids + [2], [1] + [0] * (len(ids) - 1) + [1], offs + [at])


class _FakeHead:
    def __init__(self, max_batch, max_seq):
        self.cap, self.batches = (max_batch, max_seq), []
    def capacity(self):
        return self.cap
    def run_batch(self, encodings):
        self.batches.append([len(e) for e in encodings])
        return [np.array([len(e), sum(e)], dtype=np.float32) for e in encodings]


def test_sliding_window_chunker_geometry():
    from svod_b200.pipeline import ChunkerError, Encoding, SlidingWindowChunker
    enc = Encoding([0] + list(range(10, 20)) + [2], [1] + [0] * 10 + [1])
    ch = SlidingWindowChunker(6, 3).chunk(enc)  # 4 content tokens per window, step 3
    assert [c.first_token for c in ch] == [0, 3, 6]
    assert [c.encoding.ids for c in ch] == [[0, 10, 11, 12, 13, 2], [0, 13, 14, 15, 16, 2], [0, 16, 17, 18, 19, 2]]
    ch = SlidingWindowChunker(6, 4).chunk(enc)
    assert [c.encoding.ids for c in ch][-1] == [0, 18, 19, 2]  # a short last window
    ch = SlidingWindowChunker(6, 4, full_last_window=True).chunk(enc)
    assert [c.encoding.ids for c in ch][-1] == [0, 16, 17, 18, 19, 2]  # backed up to a whole one
    assert SlidingWindowChunker(6, 3).chunk(Encoding([])) == []
    only_specials = SlidingWindowChunker(2, 1).chunk(Encoding([0, 2], [1, 1]))
    assert len(only_specials) == 1 and only_specials[0].encoding.ids == [0, 2]
    with pytest.raises(ChunkerError):
        SlidingWindowChunker(2, 1).chunk(enc)  # no room past the two specials
    with pytest.raises(ChunkerError):
        SlidingWindowChunker(4, 5)


def test_encoder_pipeline_batches_longest_first_and_restores_order():
    from svod_b200.pipeline import EncoderPipeline, PipelineBuildError, SlidingWindowChunker
    head = _FakeHead(max_batch=3, max_seq=8)
    with pytest.raises(PipelineBuildError):
        EncoderPipeline(_WordTokenizer(), SlidingWindowChunker(9, 4), head)
    pipe = EncoderPipeline(_WordTokenizer(), SlidingWindowChunker(6, 4), head)
    texts = ["a bb ccc dddd eeeee ffffff", "x", "one two three four five six seven eight nine"]
    out = pipe.embed_texts(texts)
    assert [len(o) for o in out] == [2, 1, 3]
    # sub-batches of at most 3, each sorted longest first
    assert all(len(b) <= 3 and b == sorted(b, reverse=True) for b in head.batches)
    assert max(head.batches[0]) >= max(head.batches[-1])
    for chunks in out:
        for chunk, value in chunks:  # each output belongs to its own chunk
            assert value[0] == len(chunk.encoding) and value[1] == sum(chunk.encoding.ids)
    assert out[0][1][0].byte_offset == len("a bb ccc dddd ")  # second window starts at its 5th word
    assert pipe.embed("x")[0][1][0] == 3
    built = EncoderPipeline.assemble(_WordTokenizer(), SlidingWindowChunker(5, 2), lambda n: _FakeHead(2, n))
    assert built.head.capacity() == (2, 5)
    built.warm_up([(2, 5)])
    assert built.head.batches == [[5, 5]]
