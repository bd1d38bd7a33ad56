"""ctypes binding of `libsvodb.so` (the C ABI declared in include/svodb.h).

The library is the product path. There is no CPU or PyTorch fallback: if the
shared library is missing, loading raises with the build command.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

# SVODB_LIB_PATH selects another build of the library (e.g. one with debug probes).
LIB_PATH = Path(os.environ.get("SVODB_LIB_PATH") or Path(__file__).resolve().parent / "lib" / "libsvodb.so")

MAX_RANK = 5

# status codes of include/svodb.h
OK, ERR_SHAPE, ERR_DTYPE, ERR_HEADS, ERR_GRAPH, ERR_LAUNCH, ERR_UNREALIZED, ERR_ALIAS, ERR_TIMEOUT, \
    ERR_POISONED, ERR_WORKSPACE, ERR_UNSUPPORTED = range(12)

F32, F16, BF16, I32, I64, U8 = range(6)

NOALLOC_SCRATCH_BYTES = 8 << 20  # SVODB_NOALLOC_SCRATCH_BYTES


class Tensor(C.Structure):
    _fields_ = [
        ("data", C.c_void_p),
        ("dtype", C.c_int32),
        ("rank", C.c_int32),
        ("shape", C.c_int64 * MAX_RANK),
        ("stride", C.c_int64 * MAX_RANK),
    ]


TensorP = C.POINTER(Tensor)


class LinearOpts(C.Structure):
    _fields_ = [
        ("bias", TensorP),
        ("act", C.c_int32),
        ("gated", C.c_int32),
        ("residual", TensorP),
        ("has_scale", C.c_int32),
        ("scale", C.c_float),
        ("rope_cos", TensorP),
        ("rope_sin", TensorP),
        ("rope_heads", C.c_int32),
        ("rope_head_dim", C.c_int32),
        ("into_at", C.c_int64),
        ("qkv", C.c_void_p),  # const svodb_qkv_opts* (QkvOpts is declared below)
        ("k_splits", C.c_int32),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
    ]


class PeerGather(C.Structure):
    _fields_ = [
        ("world", C.c_int32),
        ("rank", C.c_int32),
        ("stage", C.c_void_p * 8),
        ("flags", C.c_void_p * 8),
        ("local", C.c_void_p),
        ("wait_polls", C.c_uint32),
        ("phases", C.c_int32),
    ]


class AttnOpts(C.Structure):
    _fields_ = [
        ("causal", C.c_int32),
        ("key_lens", TensorP),
        ("key_mask", TensorP),
        ("has_window", C.c_int32),
        ("window_left", C.c_int64),
        ("window_right", C.c_int64),
        ("has_chunk", C.c_int32),
        ("chunk_size", C.c_int64),
        ("chunk_left", C.c_int64),
        ("chunk_right", C.c_int64),
        ("seg_start", TensorP),
        ("splits", C.c_int32),
        ("has_scale", C.c_int32),
        ("scale", C.c_float),
        ("bias", TensorP),
        ("lse", TensorP),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
        ("has_cache", C.c_int32),
        ("cache_head_start", C.c_int32),
        ("cache_kv_heads", C.c_int32),
        ("cache_row_map", TensorP),
        ("cache_app_k", TensorP),
        ("cache_app_v", TensorP),
        ("cache_app_lens", TensorP),
    ]


class QkvOpts(C.Structure):
    _fields_ = [
        ("heads", C.c_int32),
        ("kv_heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("q_norm", TensorP),
        ("k_norm", TensorP),
        ("eps", C.c_double),
        ("rope_cos", TensorP),
        ("rope_sin", TensorP),
    ]


class Qwen3Config(C.Structure):
    _fields_ = [("vocab", C.c_int32), ("hidden", C.c_int32), ("layers", C.c_int32), ("heads", C.c_int32),
                ("kv_heads", C.c_int32), ("head_dim", C.c_int32), ("ffn", C.c_int32), ("dtype", C.c_int32),
                ("eps", C.c_double), ("rope_theta", C.c_double)]


class Qwen3Layer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("in_w", "qkv_w", "qn_w", "kn_w", "o_w", "post_w", "gu_w", "down_w")]


class Qwen3Weights(C.Structure):
    _fields_ = [("embed", C.c_void_p), ("layers", C.POINTER(Qwen3Layer)), ("norm_w", C.c_void_p)]


class XlmrConfig(C.Structure):
    _fields_ = [("vocab", C.c_int32), ("hidden", C.c_int32), ("layers", C.c_int32), ("heads", C.c_int32),
                ("ffn", C.c_int32), ("max_positions", C.c_int32), ("pad_id", C.c_int32), ("dtype", C.c_int32),
                ("pooling", C.c_int32), ("eps", C.c_double)]


class XlmrLayer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("qkv_w", "qkv_b", "o_w", "o_b", "ln1_w", "ln1_b", "fi_w", "fi_b", "fo_w",
                                          "fo_b", "ln2_w", "ln2_b")]


class XlmrWeights(C.Structure):
    _fields_ = [("word", C.c_void_p), ("pos", C.c_void_p), ("type", C.c_void_p), ("emb_ln_w", C.c_void_p),
                ("emb_ln_b", C.c_void_p), ("layers", C.POINTER(XlmrLayer))]


class ModernBertConfig(C.Structure):
    _fields_ = [("vocab", C.c_int32), ("hidden", C.c_int32), ("layers", C.c_int32), ("heads", C.c_int32),
                ("ffn", C.c_int32), ("global_every", C.c_int32), ("local_window", C.c_int32), ("dtype", C.c_int32),
                ("pooling", C.c_int32), ("eps", C.c_double), ("global_theta", C.c_double), ("local_theta", C.c_double)]


class ModernBertLayer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("attn_ln_w", "qkv_w", "o_w", "mlp_ln_w", "wi_w", "wo_w")]


class ModernBertWeights(C.Structure):
    _fields_ = [("embed", C.c_void_p), ("emb_ln_w", C.c_void_p), ("layers", C.POINTER(ModernBertLayer)),
                ("final_ln_w", C.c_void_p)]


class AbiParam(C.Structure):
    _fields_ = [("slot", C.c_int32), ("kind", C.c_int32)]


# Every symbol include/svodb.h declares: (name, restype, argtypes).
SYMBOLS = [
    ("svodb_version", C.c_char_p, []),
    ("svodb_last_error", C.c_char_p, []),
    ("svodb_supported", C.c_int, [C.c_int]),
    ("svodb_last_chosen", C.c_char_p, []),
    ("svodb_last_config_key", C.c_char_p, []),
    ("svodb_config_set", C.c_int, [C.c_char_p, C.c_int32]),
    ("svodb_config_get", C.c_int32, [C.c_char_p]),
    ("svodb_config_clear", None, []),
    ("svodb_device_status", C.c_int, [C.c_void_p]),
    ("svodb_selftest_wait_timeout", C.c_int, [C.c_uint32, C.c_void_p]),
    ("svodb_selftest_latch_error", C.c_int, [C.c_int32]),
    ("svodb_selftest_clear_latch", None, []),
    ("svodb_qwen3_create", C.c_int, [C.POINTER(Qwen3Config), C.POINTER(Qwen3Weights), C.POINTER(C.c_void_p)]),
    ("svodb_xlmr_create", C.c_int, [C.POINTER(XlmrConfig), C.POINTER(XlmrWeights), C.POINTER(C.c_void_p)]),
    ("svodb_modernbert_create", C.c_int,
     [C.POINTER(ModernBertConfig), C.POINTER(ModernBertWeights), C.POINTER(C.c_void_p)]),
    ("svodb_model_free", None, [C.c_void_p]),
    ("svodb_model_plan", C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.POINTER(C.c_void_p)]),
    ("svodb_plan_run", C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    ("svodb_plan_stream", C.c_void_p, [C.c_void_p]),
    ("svodb_plan_output", C.c_void_p, [C.c_void_p]),
    ("svodb_plan_free", None, [C.c_void_p]),
    ("svodb_linear", C.c_int, [TensorP, TensorP, C.POINTER(LinearOpts), TensorP, C.c_void_p]),
    ("svodb_attention_workspace_bytes", C.c_size_t, [C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int32]),
    ("svodb_linear_workspace_bytes", C.c_size_t, [C.c_int64, C.c_int64, C.c_int32]),
    ("svodb_attention", C.c_int, [TensorP, TensorP, TensorP, C.POINTER(AttnOpts), TensorP, C.c_void_p]),
    ("svodb_attention_splits_noalloc", C.c_int, [TensorP, TensorP, TensorP, C.POINTER(AttnOpts), TensorP, C.c_void_p]),
    ("svodb_attention_packed", C.c_int, [TensorP, C.c_int32, C.c_int32, C.POINTER(AttnOpts), TensorP, C.c_void_p]),
    ("svodb_combine_splits", C.c_int, [TensorP, TensorP, TensorP, TensorP, C.c_void_p]),
    ("svodb_heads", C.c_int, [TensorP, C.POINTER(QkvOpts), TensorP, TensorP, TensorP, C.c_void_p]),
    ("svodb_layer_norm", C.c_int, [TensorP, TensorP, TensorP, C.c_double, TensorP, C.c_void_p]),
    ("svodb_add_layer_norm", C.c_int, [TensorP, TensorP, TensorP, TensorP, C.c_double, TensorP, TensorP, C.c_void_p]),
    ("svodb_rms_norm", C.c_int, [TensorP, TensorP, C.c_double, TensorP, C.c_void_p]),
    ("svodb_add_rms_norm", C.c_int, [TensorP, TensorP, TensorP, C.c_double, TensorP, TensorP, C.c_void_p]),
    ("svodb_embed", C.c_int, [TensorP, TensorP, TensorP, TensorP, C.c_int64, TensorP, C.c_void_p]),
    ("svodb_embed_norm", C.c_int, [TensorP, TensorP, TensorP, TensorP, C.c_int64, TensorP, TensorP, C.c_double, C.c_int32,
                                   TensorP, C.c_void_p]),
    ("svodb_pool", C.c_int, [TensorP, TensorP, C.c_int32, C.c_int32, TensorP, C.c_void_p]),
    ("svodb_norm_pool", C.c_int, [TensorP, TensorP, TensorP, C.c_double, C.c_int32, TensorP, TensorP, C.c_int32,
                                  C.c_int32, TensorP, C.c_void_p]),
    ("svodb_rope_table", C.c_int, [C.c_double, TensorP, C.c_int32, TensorP, TensorP, C.c_void_p]),
    ("svodb_module_load", C.c_int,
     [C.c_void_p, C.c_size_t, C.c_char_p, C.POINTER(AbiParam), C.c_int32, C.POINTER(C.c_void_p)]),
    ("svodb_program_launch", C.c_int,
     [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.c_int32, C.POINTER(C.c_int32), C.c_int32,
      C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), C.c_uint32]),
    ("svodb_program_free", C.c_int, [C.c_void_p]),
    ("svodb_graph_begin", C.c_int, [C.c_void_p]),
    ("svodb_graph_end", C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    ("svodb_graph_replay", C.c_int, [C.c_void_p, C.c_void_p]),
    ("svodb_graph_free", C.c_int, [C.c_void_p]),
    ("svodb_alloc", C.c_int, [C.c_size_t, C.c_int32, C.POINTER(C.c_void_p)]),
    ("svodb_free", C.c_int, [C.c_void_p, C.c_int32]),
    ("svodb_copy_h2d", C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    ("svodb_copy_d2h", C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    ("svodb_stream_sync", C.c_int, [C.c_void_p]),
    ("svodb_memset", C.c_int, [C.c_void_p, C.c_int32, C.c_size_t, C.c_void_p]),
    ("svodb_peer_stage_bytes", C.c_size_t, [C.c_int32, C.c_int64, C.c_int64]),
    ("svodb_ipc_export", C.c_int, [C.c_void_p, C.c_void_p]),
    ("svodb_ipc_open", C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    ("svodb_ipc_close", C.c_int, [C.c_void_p]),
    ("svodb_peer_all_gather", C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    ("svodb_norm_pool_gather", C.c_int, [TensorP, TensorP, TensorP, C.c_double, C.c_int32, TensorP, TensorP, C.c_int32,
                                        C.c_int32, C.c_void_p, TensorP, C.c_void_p]),
]

_lib = None


def load() -> C.CDLL:
    """Loads the library once and types every entry point."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m svod_b200.build` "
                "(there is no CPU or PyTorch fallback for these ops)")
        lib = C.CDLL(str(LIB_PATH))
        for name, res, args in SYMBOLS:
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
