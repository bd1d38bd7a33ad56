"""Text-pipeline front end over an encoder head: tokenize -> chunk -> encode,
the host logic of the reference's `EncoderPipeline`
(arch/src/pipelines/text.rs:883-1134) and its `SlidingWindowChunker`
(:575-667), so a caller of that pipeline finds the same verbs here. Tokenizers
are an interface only (no vocabulary files travel with this package): anything
with `encode(text) -> Encoding` serves.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Protocol, Sequence, Tuple

import numpy as np


@dataclass
class Encoding:
    """Token ids with the mask of special tokens (1 = special) and each token's
    byte offset in the source text."""
    ids: List[int]
    special: List[int] = field(default_factory=list)
    offsets: List[int] = field(default_factory=list)

    def __post_init__(self):
        if not self.special:
            self.special = [0] * len(self.ids)
        if not self.offsets:
            self.offsets = list(range(len(self.ids)))

    def __len__(self):
        return len(self.ids)


@dataclass
class TextChunk:
    encoding: Encoding
    byte_offset: int   # where the chunk's first content token begins in the text
    first_token: int   # index of that token among the content tokens


class Tokenizer(Protocol):
    def encode(self, text: str) -> Encoding: ...


class ChunkerError(ValueError):
    pass


class SlidingWindowChunker:
    """Windows of `window` tokens in total (boundary specials repeated in every
    chunk), starting every `stride` content tokens; the last window is short
    unless `full_last_window` backs it up to a whole one
    (arch/src/pipelines/text.rs:597-667)."""

    def __init__(self, window: int, stride: int, full_last_window: bool = False):
        if window < 1:
            raise ChunkerError("window must be >= 1")
        if not 1 <= stride <= window:
            raise ChunkerError("stride must be in 1..=window")
        self.window, self.stride, self.full_last_window = window, stride, full_last_window

    def max_seq(self) -> int:
        return self.window

    def chunk(self, enc: Encoding) -> List[TextChunk]:
        if len(enc) == 0:
            return []
        n = len(enc)
        lead = next((i for i, m in enumerate(enc.special) if m != 1), n)
        trail = min(next((i for i, m in enumerate(reversed(enc.special)) if m != 1), n), n - lead)
        content = range(lead, n - trail)
        fixed = lead + trail
        if len(content) == 0:
            if fixed > self.window:
                raise ChunkerError(f"window ({self.window}) leaves no room for content past {fixed} fixed tokens")
            return [TextChunk(enc, 0, 0)]
        room = self.window - fixed
        if room < 1:
            raise ChunkerError(f"window ({self.window}) leaves no room for content past {fixed} fixed tokens")
        step = min(self.stride, room)
        pick = lambda idx: Encoding([enc.ids[i] for i in idx], [enc.special[i] for i in idx],
                                    [enc.offsets[i] for i in idx])
        chunks, start = [], 0
        while True:
            if self.full_last_window and start + room > len(content):
                start = max(len(content) - room, 0)
            end = min(start + room, len(content))
            idx = list(range(lead)) + [content.start + i for i in range(start, end)] + list(range(n - trail, n))
            chunks.append(TextChunk(pick(idx), enc.offsets[content.start + start], start))
            if end >= len(content):
                return chunks
            start += step


class PipelineBuildError(ValueError):
    pass


class EncoderPipeline:
    """`EncoderPipeline` (arch/src/pipelines/text.rs:883-1134) for the embedding
    verb: `head` is anything with `capacity() -> (max_batch, max_seq)` and
    `run_batch(list of id lists) -> [n, D] array` (`encoder_head.HeadPlans`
    does)."""

    def __init__(self, tokenizer: Tokenizer, chunker, head):
        chunker_max, head_max = chunker.max_seq(), head.capacity()[1]
        if chunker_max > head_max:
            raise PipelineBuildError(
                f"the chunker cuts chunks of up to {chunker_max} tokens, but the head takes up to {head_max}")
        self.tokenizer, self.chunker, self.head = tokenizer, chunker, head

    @classmethod
    def assemble(cls, tokenizer, chunker, build):
        """Builds the head sized to the chunker's longest chunk, then composes."""
        return cls(tokenizer, chunker, build(chunker.max_seq()))

    def run_chunks_flat(self, chunks: Sequence[TextChunk]) -> List[np.ndarray]:
        """Sub-batches of at most the head's `max_batch`, longest chunk first;
        outputs in input order (text.rs:968-985)."""
        max_batch = max(self.head.capacity()[0], 1)
        order = sorted(range(len(chunks)), key=lambda i: -len(chunks[i].encoding))
        out: List[np.ndarray] = [None] * len(chunks)
        for at in range(0, len(order), max_batch):
            batch = order[at:at + max_batch]
            values = self.head.run_batch([chunks[i].encoding.ids for i in batch])
            for i, value in zip(batch, values):
                out[i] = np.asarray(value)
        return out

    def embed_texts(self, texts: Sequence[str]) -> List[List[Tuple[TextChunk, np.ndarray]]]:
        """Every text's chunks flattened into one stream through the head, then
        handed back per text with their source positions."""
        per_text = [self.chunker.chunk(self.tokenizer.encode(t)) for t in texts]
        flat = [c for chunks in per_text for c in chunks]
        values = self.run_chunks_flat(flat)
        out, at = [], 0
        for chunks in per_text:
            out.append(list(zip(chunks, values[at:at + len(chunks)])))
            at += len(chunks)
        return out

    def embed(self, text: str) -> List[Tuple[TextChunk, np.ndarray]]:
        return self.embed_texts([text])[0]

    def warm_up(self, shapes: Sequence[Tuple[int, int]]):
        """Runs one batch per `(rows, length)` so the head prepares those plans
        ahead of the first real call (text.rs:1131-1134)."""
        for rows, length in shapes:
            self.head.run_batch([[0] * max(length, 1)] * max(rows, 1))
