"""ctypes face of the library's native Qwen3 runner (`svodb_qwen3_*`,
`svodb_plan_*`): the model borrows the device weights of a
`encoders.Qwen3Embedder`, a plan is one captured CUDA graph per `(rows, len)`
shape, a run takes host ids / lengths and returns host pooled rows — no Python
between the copies and the graph launch."""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from . import _lib as L
from . import ops
from .encoders import Qwen3Embedder


class NativeQwen3:
    def __init__(self, model: Qwen3Embedder, reference_ops: bool = False):
        lib = L.load()
        c, p = model.cfg, model.p
        self._keep = model  # the weights stay alive with the runner
        self.hidden = c.hidden_size
        cfg = L.Qwen3Config(c.vocab_size, c.hidden_size, c.num_hidden_layers, c.num_attention_heads,
                            c.num_key_value_heads, c.head_dim, c.intermediate_size, ops._DTYPES[c.dtype],
                            float(c.rms_norm_eps), float(c.rope_theta))
        names = ("in_w", "qkv_w", "qn_w", "kn_w", "o_w", "post_w", "gu_w", "down_w")
        self._layers = (L.Qwen3Layer * len(p["layers"]))(
            *[L.Qwen3Layer(*[lp[n].data_ptr() for n in names]) for lp in p["layers"]])
        w = L.Qwen3Weights(p["embed"].data_ptr(), self._layers, p["norm_w"].data_ptr())
        self._model = C.c_void_p()
        ops._check(lib.svodb_qwen3_create(C.byref(cfg), C.byref(w), C.byref(self._model)))
        self.reference_ops = int(reference_ops)
        self._plans: Dict[Tuple[int, int], C.c_void_p] = {}

    def plan(self, rows: int, length: int) -> C.c_void_p:
        key = (rows, length)
        if key not in self._plans:
            h = C.c_void_p()
            ops._check(L.load().svodb_qwen3_plan(self._model, rows, length, self.reference_ops, C.byref(h)))
            self._plans[key] = h
        return self._plans[key]

    def run(self, ids: np.ndarray, lengths: np.ndarray, out: Optional[np.ndarray] = None) -> np.ndarray:
        """ids `[rows, len]` i32, lengths `[rows]` i32 (host arrays; pinned memory
        makes the copies asynchronous) -> pooled unit-norm rows `[rows, hidden]` f32."""
        rows, length = ids.shape
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        lengths = np.ascontiguousarray(lengths, dtype=np.int32)
        if out is None:
            out = np.empty((rows, self.hidden), dtype=np.float32)
        ops._check(L.load().svodb_plan_run(self.plan(rows, length), ids.ctypes.data, lengths.ctypes.data,
                                           out.ctypes.data))
        return out

    def replay(self, rows: int, length: int):
        """Graph launch alone on the plan's stream (inputs as last written)."""
        ops._check(L.load().svodb_plan_run(self.plan(rows, length), None, None, None))

    def stream(self, rows: int, length: int) -> torch.cuda.ExternalStream:
        return torch.cuda.ExternalStream(L.load().svodb_plan_stream(self.plan(rows, length)))

    def close(self):
        lib = L.load()
        for h in self._plans.values():
            lib.svodb_plan_free(h)
        self._plans.clear()
        if self._model:
            lib.svodb_qwen3_free(self._model)
            self._model = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
