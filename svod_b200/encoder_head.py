"""Host-side batching around the encoder stacks: plan-shape bucketing with a
plan cache (the reference's `HeadPlans`, model/src/encoder_head.rs:366-533) and
Qwen3's first-fit sequence packing with segment starts
(model/src/qwen3/embed.rs:26-163).

Everything here is host logic over `svod_b200.encoders.Plan` (one captured CUDA
graph per plan shape); the device work is the same op sequence as the stacks.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

from . import ops
from .encoders import Plan, Qwen3Embedder

# One plan per 128 tokens of length (model/src/encoder_head.rs:364-366).
LEN_MULTIPLE = 128
# Qwen3 pads packed rows to whole attention tiles (model/src/qwen3/model.rs:56).
SEQUENCE_TILE = 128
# Tokens of row capacity per pooled slot (model/src/qwen3/embed.rs:24-26).
SLOT_TOKENS = 16


def next_pow2(n: int) -> int:
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


def plan_shape(b: int, longest: int, max_batch: int) -> Tuple[int, int]:
    """`plan_shape` (model/src/encoder_head.rs:370-372): rows = next power of two
    of the batch capped at `max_batch`, length rounded up to 128 tokens."""
    rows = min(next_pow2(b), max_batch)
    length = -(-max(longest, 1) // LEN_MULTIPLE) * LEN_MULTIPLE
    return rows, length


def pack_ids(batch: Sequence[Sequence[int]], rows: int, length: int, pad_id: int) -> np.ndarray:
    """`pack_ids` (model/src/encoder_head.rs:510-512): each chunk's ids padded
    into `[rows, length]`, unused positions and rows filled with `pad_id`."""
    out = np.full((rows, length), pad_id, dtype=np.int32)
    for r, ids in enumerate(batch):
        take = min(len(ids), length)
        out[r, :take] = np.asarray(ids[:take], dtype=np.int32)
    return out


def pack_mask(batch: Sequence[Sequence[int]], rows: int, length: int) -> np.ndarray:
    """`pack_mask` (model/src/encoder_head.rs:514-523): 1 = real token; an
    unused row attends to its first (pad) token alone, so no softmax runs over
    nothing."""
    out = np.zeros((rows, length), dtype=bool)
    for r, ids in enumerate(batch):
        out[r, :min(len(ids), length)] = True
    out[len(batch):, 0] = True
    return out


class HeadPlans:
    """Per-shape plan cache of an encoder head (model/src/encoder_head.rs:384-500):
    a batch runs on the plan of its `(rows, len)` bucket, captured on first use
    and replayed afterwards; only the live rows of the output are returned."""

    def __init__(self, model, max_batch: int = 64, max_seq: int = 8192, pad_id: int = 1, device="cuda"):
        self.model, self.max_batch, self.max_seq, self.pad_id, self.device = model, max_batch, max_seq, pad_id, device
        self.plans: Dict[Tuple[int, int], Plan] = {}
        self._host: Dict[Tuple[int, int], Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}

    def run(self, batch: Sequence[Sequence[int]]) -> np.ndarray:
        assert 0 < len(batch) <= self.max_batch
        longest = min(max(len(x) for x in batch), self.max_seq)
        shape = plan_shape(len(batch), longest, self.max_batch)
        rows, length = shape
        if shape not in self.plans:
            self.plans[shape] = Plan(self.model, rows, length, "mask", device=self.device).capture()
            D = self.model.cfg.hidden_size
            self._host[shape] = (torch.empty(rows, length, dtype=torch.int32).pin_memory(),
                                 torch.empty(rows, length, dtype=torch.bool).pin_memory(),
                                 torch.empty(rows, D, dtype=torch.float32).pin_memory())
        plan = self.plans[shape]
        ids_h, mask_h, out_h = self._host[shape]
        ids_h.copy_(torch.from_numpy(pack_ids(batch, rows, length, self.pad_id)))
        mask_h.copy_(torch.from_numpy(pack_mask(batch, rows, length)))
        plan.run(ids_h, mask_h, out_h)
        plan.stream.synchronize()
        return out_h[:len(batch)].numpy().copy()


# the head interface the text pipeline drives (`EncoderHead::capacity` / `run_batch`,
# model/src/encoder_head.rs:46-70)
HeadPlans.capacity = lambda self: (self.max_batch, self.max_seq)
HeadPlans.run_batch = lambda self, encodings: self.run(encodings)


def embed_chunks(plans: HeadPlans, chunks: Sequence[Sequence[int]]) -> np.ndarray:
    """`run_chunks_flat` (arch/src/pipelines/text.rs:968-985): chunks sorted
    longest first, cut into sub-batches of `max_batch`, results restored to
    input order."""
    order = sorted(range(len(chunks)), key=lambda i: -len(chunks[i]))
    out = [None] * len(chunks)
    for at in range(0, len(order), plans.max_batch):
        idx = order[at:at + plans.max_batch]
        res = plans.run([chunks[i] for i in idx])
        for i, row in zip(idx, res):
            out[i] = row
    return np.stack(out) if out else np.zeros((0, plans.model.cfg.hidden_size), dtype=np.float32)


# --------------------------------------------------------------------------- Qwen3 packing
@dataclass
class PackedBatch:
    bucket: int
    rows: List[List[int]]  # per plan row, the input rows packed into it in order


def pack(lens: Sequence[int], max_batch: int) -> List[PackedBatch]:
    """`pack` (model/src/qwen3/embed.rs:40-62): longest first; each batch's
    bucket is its longest row rounded up to the tile; the rest first-fit by
    tokens and by pooled slots."""
    pending = sorted(range(len(lens)), key=lambda i: -lens[i])
    batches = []
    while pending:
        bucket = -(-lens[pending[0]] // SEQUENCE_TILE) * SEQUENCE_TILE
        slots = bucket // SLOT_TOKENS
        fill = [0] * max_batch
        rows: List[List[int]] = [[] for _ in range(max_batch)]
        rest = []
        for i in pending:
            for r in range(max_batch):
                if fill[r] + lens[i] <= bucket and len(rows[r]) < slots:
                    fill[r] += lens[i]
                    rows[r].append(i)
                    break
            else:
                rest.append(i)
        pending = rest
        batches.append(PackedBatch(bucket, rows))
    return batches


def packed_inputs(batch: PackedBatch, rows_ids: Sequence[Sequence[int]], lens: Sequence[int], max_batch: int,
                  pad_id: int):
    """The four `[max_batch, bucket | slots]` i32 inputs of one packed plan
    (model/src/qwen3/embed.rs:119-136): padding is pad tokens at position 0,
    each its own segment, pooled nowhere."""
    bucket, slots = batch.bucket, batch.bucket // SLOT_TOKENS
    ids = np.full((max_batch, bucket), pad_id, dtype=np.int32)
    positions = np.zeros((max_batch, bucket), dtype=np.int32)
    seg_start = np.tile(np.arange(bucket, dtype=np.int32), (max_batch, 1))
    pool_idx = np.zeros((max_batch, slots), dtype=np.int32)
    for r, packed in enumerate(batch.rows):
        cursor = 0
        for slot, i in enumerate(packed):
            n = lens[i]
            src = list(rows_ids[i])
            ids[r, cursor:cursor + len(src)] = src
            positions[r, cursor:cursor + len(src)] = np.arange(len(src))
            seg_start[r, cursor:cursor + n] = cursor
            cursor += n
            pool_idx[r, slot] = cursor - 1
    return ids, positions, seg_start, pool_idx


class Qwen3PackedEmbedder:
    """`Qwen3Embedder::embed` (model/src/qwen3/embed.rs:86-163): rows packed end
    to end into `[max_batch, bucket]` plan rows with per-token positions and
    segment starts, one unit-norm embedding per input row in input order."""

    def __init__(self, model: Qwen3Embedder, max_batch: int, max_len: int, pad_id: int = 0, device="cuda"):
        self.model, self.max_batch, self.pad_id, self.device = model, max(max_batch, 1), pad_id, device
        self.max_len = -(-max(max_len, 1) // SEQUENCE_TILE) * SEQUENCE_TILE

    def _forward(self, ids, positions, seg_start, pool_idx):
        c = self.model.cfg
        B, L = ids.shape
        hd = c.head_dim
        cos, sin = ops.rope_table(c.rope_theta, positions.reshape(-1), hd, c.dtype, self.device)
        rope = (cos.view(B, L, 1, hd // 2), sin.view(B, L, 1, hd // 2))
        h = self.model.hidden(ids, seg_start=seg_start, rope=rope)
        return ops.pool(h, pool_idx, ops.POOL_GATHER, True)

    def embed(self, rows: Sequence[Sequence[int]]) -> List[np.ndarray]:
        rows = [list(r[:self.max_len]) for r in rows]
        lens = [max(len(r), 1) for r in rows]  # an empty row embeds as one pad token
        out: List[np.ndarray] = [None] * len(rows)
        for batch in pack(lens, self.max_batch):
            slots = batch.bucket // SLOT_TOKENS
            arrays = packed_inputs(batch, rows, lens, self.max_batch, self.pad_id)
            ids, positions, seg_start, pool_idx = (torch.from_numpy(a).to(self.device) for a in arrays)
            flat = self._forward(ids, positions, seg_start, pool_idx).float().cpu().numpy()
            for r, packed in enumerate(batch.rows):
                for slot, i in enumerate(packed):
                    out[i] = flat[r * slots + slot].copy()
        return out
