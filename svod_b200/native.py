"""ctypes face of the library's native runners (`svodb_{qwen3,xlmr,modernbert}_create`,
`svodb_model_plan`, `svodb_plan_*`): a model borrows the device weights of one
of the `encoders` stacks, a plan is one captured CUDA graph per `(rows, len)`
shape, a run takes host ids and lengths (Qwen3) or the padding mask (XLM-R,
ModernBERT) and returns host pooled rows — no Python between the copies and the
graph launch."""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from . import _lib as L
from . import ops
from .encoders import ModernBertEncoder, Qwen3Embedder, XlmRobertaEncoder


class _Native:
    """What the three runners share: plans by shape, run, replay, close."""

    aux_dtype = np.uint8

    def __init__(self, model, hidden: int, reference_ops: bool = False):
        self._keep = model  # the weights stay alive with the runner
        self.hidden = hidden
        self.reference_ops = int(reference_ops)
        self._model = C.c_void_p()
        self._plans: Dict[Tuple[int, int], C.c_void_p] = {}

    def plan(self, rows: int, length: int) -> C.c_void_p:
        key = (rows, length)
        if key not in self._plans:
            h = C.c_void_p()
            ops._check(L.load().svodb_model_plan(self._model, rows, length, self.reference_ops, C.byref(h)))
            self._plans[key] = h
        return self._plans[key]

    def run(self, ids: np.ndarray, aux: np.ndarray, out: Optional[np.ndarray] = None) -> np.ndarray:
        """ids `[rows, len]` i32 and `aux` = lengths `[rows]` i32 (Qwen3) or the
        padding mask `[rows, len]` (the others), host arrays (pinned memory makes
        the copies asynchronous) -> pooled unit-norm rows `[rows, hidden]` f32."""
        rows, length = ids.shape
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        aux = np.ascontiguousarray(aux, dtype=self.aux_dtype)
        if out is None:
            out = np.empty((rows, self.hidden), dtype=np.float32)
        ops._check(L.load().svodb_plan_run(self.plan(rows, length), ids.ctypes.data, aux.ctypes.data, out.ctypes.data))
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
            lib.svodb_model_free(self._model)
            self._model = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _ptr(t):
    return None if t is None else t.data_ptr()


class NativeQwen3(_Native):
    aux_dtype = np.int32

    def __init__(self, model: Qwen3Embedder, reference_ops: bool = False):
        c, p = model.cfg, model.p
        super().__init__(model, c.hidden_size, reference_ops)
        cfg = L.Qwen3Config(c.vocab_size, c.hidden_size, c.num_hidden_layers, c.num_attention_heads,
                            c.num_key_value_heads, c.head_dim, c.intermediate_size, ops._DTYPES[c.dtype],
                            float(c.rms_norm_eps), float(c.rope_theta))
        names = ("in_w", "qkv_w", "qn_w", "kn_w", "o_w", "post_w", "gu_w", "down_w")
        self._layers = (L.Qwen3Layer * len(p["layers"]))(
            *[L.Qwen3Layer(*[lp[n].data_ptr() for n in names]) for lp in p["layers"]])
        w = L.Qwen3Weights(p["embed"].data_ptr(), self._layers, p["norm_w"].data_ptr())
        ops._check(L.load().svodb_qwen3_create(C.byref(cfg), C.byref(w), C.byref(self._model)))


class NativeXlmRoberta(_Native):
    def __init__(self, model: XlmRobertaEncoder):
        c, p = model.cfg, model.p
        super().__init__(model, c.hidden_size)
        cfg = L.XlmrConfig(c.vocab_size, c.hidden_size, c.num_hidden_layers, c.num_attention_heads,
                           c.intermediate_size, p["pos"].shape[0], c.pad_token_id, ops._DTYPES[c.dtype],
                           0 if c.pooling == "cls" else 1, float(c.layer_norm_eps))
        names = ("qkv_w", "qkv_b", "o_w", "o_b", "ln1_w", "ln1_b", "fi_w", "fi_b", "fo_w", "fo_b", "ln2_w", "ln2_b")
        self._layers = (L.XlmrLayer * len(p["layers"]))(
            *[L.XlmrLayer(*[lp[n].data_ptr() for n in names]) for lp in p["layers"]])
        w = L.XlmrWeights(p["word"].data_ptr(), p["pos"].data_ptr(), p["type"].data_ptr(), p["emb_ln_w"].data_ptr(),
                          p["emb_ln_b"].data_ptr(), self._layers)
        ops._check(L.load().svodb_xlmr_create(C.byref(cfg), C.byref(w), C.byref(self._model)))


class NativeModernBert(_Native):
    def __init__(self, model: ModernBertEncoder):
        c, p = model.cfg, model.p
        super().__init__(model, c.hidden_size)
        cfg = L.ModernBertConfig(c.vocab_size, c.hidden_size, c.num_hidden_layers, c.num_attention_heads,
                                 c.intermediate_size, c.global_attn_every_n_layers, c.local_attention,
                                 ops._DTYPES[c.dtype], 0 if c.pooling == "cls" else 1, float(c.norm_eps),
                                 float(c.global_rope_theta), float(c.local_rope_theta))
        names = ("attn_ln_w", "qkv_w", "o_w", "mlp_ln_w", "wi_w", "wo_w")
        self._layers = (L.ModernBertLayer * len(p["layers"]))(
            *[L.ModernBertLayer(*[_ptr(lp[n]) for n in names]) for lp in p["layers"]])
        w = L.ModernBertWeights(p["embed"].data_ptr(), p["emb_ln_w"].data_ptr(), self._layers,
                                p["final_ln_w"].data_ptr())
        ops._check(L.load().svodb_modernbert_create(C.byref(cfg), C.byref(w), C.byref(self._model)))
