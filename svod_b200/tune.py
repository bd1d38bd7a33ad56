"""Shape-keyed config store: a small stand-in for the reference's tune store
(tk/src/tune.rs): the config an op uses for a shape is measured once, kept in
the process and in a file, and replayed afterwards.

What is stored: the tile width of the tensor-core GEMM per `linear` shape (the
library keeps the process map and reports each call's key,
`svodb_last_config_key` / `svodb_config_set`) and the key-split count of a
decode-shaped attention (`Attn.splits = None` asks the store, as the
reference's `splits: None` does, tk/src/ops/attention.rs:74-80).

File: `$SVODB_TUNE_DIR`, else `$XDG_CACHE_HOME/svod_b200/tune`, else
`~/.cache/svod_b200/tune`; one file per device name and library version; a
`format N` line, then one `key value ns` line per entry. An unreadable or
unwritable store is a miss, never an error; lines that do not parse are dropped
at the next write and a file of another format is dropped whole. `SVODB_TUNE=0`
turns timing off: ops keep the library's own choice.
"""
from __future__ import annotations

import os
import re
from pathlib import Path
from typing import Callable, Dict, Iterable, Optional, Tuple

from . import _lib as L

FORMAT = 1
GEMM_WIDTHS = (64, 128, 256, 512)  # 512 = the CTA-pair kernel (256 x 256 tiles on two SMs)


def enabled() -> bool:
    return os.environ.get("SVODB_TUNE", "1") != "0"


def store_dir() -> Path:
    if os.environ.get("SVODB_TUNE_DIR"):
        return Path(os.environ["SVODB_TUNE_DIR"])
    base = os.environ.get("XDG_CACHE_HOME") or os.path.join(os.path.expanduser("~"), ".cache")
    return Path(base) / "svod_b200" / "tune"


def _slug(text: str) -> str:
    return re.sub(r"[^A-Za-z0-9._-]+", "_", text).strip("_") or "device"


class TuneStore:
    """`entries[key] = (value, ns)`; GEMM entries are mirrored into the library."""

    def __init__(self, device_name: str = "cpu", version: Optional[str] = None, directory: Optional[Path] = None):
        version = version or L.load().svodb_version().decode()
        self.path = Path(directory or store_dir()) / f"{_slug(device_name)}-{_slug(version)}.tune"
        self.entries: Dict[str, Tuple[int, float]] = {}
        self.dropped = 0

    # ------------------------------------------------------------------ file
    def load(self) -> int:
        """Reads the file and pushes GEMM entries into the library; returns the
        number of entries kept."""
        self.entries, self.dropped = {}, 0
        try:
            lines = self.path.read_text().splitlines()
        except OSError:
            return 0
        if not lines or lines[0].strip() != f"format {FORMAT}":
            return 0  # another format: the next save rewrites the file
        for line in lines[1:]:
            parts = line.split()
            try:
                key, value, ns = parts[0], int(parts[1]), float(parts[2])
            except (IndexError, ValueError):
                self.dropped += 1
                continue
            self.entries[key] = (value, ns)
        self._push()
        return len(self.entries)

    def save(self) -> bool:
        try:
            self.path.parent.mkdir(parents=True, exist_ok=True)
            tmp = self.path.with_suffix(".tmp")
            body = [f"format {FORMAT}"] + [f"{k} {v} {ns:.1f}" for k, (v, ns) in sorted(self.entries.items())]
            tmp.write_text("\n".join(body) + "\n")
            os.replace(tmp, self.path)
            return True
        except OSError:
            return False

    def _push(self):
        lib = L.load()
        for key, (value, _) in self.entries.items():
            if key.startswith("gemm|"):
                lib.svodb_config_set(key.encode(), value)

    # --------------------------------------------------------------- entries
    def get(self, key: str) -> Optional[int]:
        hit = self.entries.get(key)
        return hit[0] if hit else None

    def put(self, key: str, value: int, ns: float = 0.0, persist: bool = True):
        self.entries[key] = (int(value), float(ns))
        if key.startswith("gemm|"):
            L.load().svodb_config_set(key.encode(), int(value))
        if persist:
            self.save()

    # ---------------------------------------------------------------- timing
    @staticmethod
    def _time(fn: Callable[[], None], rounds: int = 3, reps: int = 5) -> float:
        """Minimum over `rounds` of the mean of `reps` back-to-back launches, ns."""
        import torch
        fn()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(rounds):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                fn()
            b.record()
            b.synchronize()
            best = min(best, a.elapsed_time(b) * 1e6 / reps)
        return best

    def pick(self, key: str, candidates: Iterable[int], run: Callable[[int], None]) -> int:
        """The stored value of `key`, or the fastest candidate, timed now and kept."""
        hit = self.get(key)
        if hit is not None:
            return hit
        timed = [(self._time(lambda c=c: run(c)), c) for c in candidates]
        ns, best = min(timed)
        self.put(key, best, ns)
        return best

    def tune_linear(self, x, w, opts=None) -> Optional[int]:
        """Measures the tile widths for this `linear` shape on a store miss and
        keeps the winner; returns the width in use (None when the shape runs
        the generic kernel, which has nothing to choose)."""
        from . import ops
        lib = L.load()
        ops.linear(x, w, opts)
        key = lib.svodb_last_config_key().decode()
        if not key:
            return None
        if self.get(key) is not None or not enabled():
            return self.get(key)

        def run(bn: int):
            lib.svodb_config_set(key.encode(), bn)
            ops.linear(x, w, opts)

        def takes(bn: int) -> bool:
            # a choice the shape or the epilogue cannot take is ignored by the library
            run(bn)
            chosen = ops.chosen()
            return ("cta_pair:1" in chosen) if bn == 512 else (f"bn:{bn}," in chosen and "cta_pair" not in chosen)

        best = self.pick(key, [bn for bn in GEMM_WIDTHS if takes(bn)], run)
        lib.svodb_config_set(key.encode(), best)
        return best

    @staticmethod
    def attention_key(q, k, opts) -> str:
        cached = opts is not None and opts.cache is not None
        app = opts.cache.appended[0].shape[1] if cached and opts.cache.appended is not None else 0
        return (f"attention|{str(q.dtype).split('.')[-1]}|{q.shape[0]}|{q.shape[1]}|{k.shape[1] + app}|"
                f"{q.shape[2]}|{q.shape[3]}|{'cache' if cached else 'plain'}")

    def tune_attention_splits(self, q, k, v, opts, sms: int = 148) -> int:
        """The split count of a decode-shaped attention: one, two, the counts
        around two key blocks per SM and the block count
        (tk/src/ops/attention.rs:74-80), timed on a miss."""
        from dataclasses import replace
        from . import ops
        key = self.attention_key(q, k, opts)
        hit = self.get(key)
        if hit is not None or not enabled():
            return hit or 1
        keys = k.shape[1] + (opts.cache.appended[0].shape[1] if opts.cache and opts.cache.appended else 0)
        blocks = max(1, -(-keys // 32))
        tiles = max(1, q.shape[0] * q.shape[2] * -(-q.shape[1] // 32))
        around = max(1, (2 * sms) // tiles)
        cands = sorted({c for c in (1, 2, around // 2, around, 2 * around, blocks) if 1 <= c <= blocks})
        return self.pick(key, cands, lambda s: ops.attention(q, k, v, replace(opts, splits=s if s > 1 else None)))


_active: Optional[TuneStore] = None


def activate(store: Optional[TuneStore]):
    """Makes `store` the one `ops.attention` consults when `Attn.splits` is None."""
    global _active
    _active = store


def active() -> Optional[TuneStore]:
    return _active
