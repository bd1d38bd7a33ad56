"""ctypes binding and build recipe of the C restatement (`svod_oracle.c`).

TEST INFRASTRUCTURE ONLY, like the rest of this folder: the tests, the smoke
check and the benchmark's CPU legs may use it; the product never does.

`build()` compiles `svod_oracle.c` with gcc + OpenMP into `oracle/lib/`, twice:
`libsvod_oracle_avx2.so` (`-mavx2 -mfma`) and `libsvod_oracle_generic.so` (no
ISA flags), so that a library built on one machine still runs on another;
`load()` picks the first the running CPU supports. The numpy float64
restatement is the pinned checker; `tests/test_oracle_pins.py` holds this C
code to it.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_DIR = HERE / "lib"
SRC = HERE / "svod_oracle.c"
VARIANTS = (("avx2", ["-mavx2", "-mfma"]), ("generic", []))

BF16, F16, F32 = 0, 1, 2
ACT_NONE, ACT_GELU, ACT_SILU, ACT_GELU_TANH = 0, 1, 2, 3
DTYPES = {"bf16": BF16, "f16": F16, "f32": F32}


def build(force: bool = False) -> list:
    LIB_DIR.mkdir(exist_ok=True)
    out = []
    for name, flags in VARIANTS:
        so = LIB_DIR / f"libsvod_oracle_{name}.so"
        if force or not so.exists() or so.stat().st_mtime < SRC.stat().st_mtime:
            cmd = ["gcc", "-O3", "-std=c11", "-fopenmp", "-fPIC", "-shared", "-fno-math-errno", "-Wno-psabi", *flags, str(SRC), "-o", str(so), "-lm"]
            subprocess.run(cmd, check=True)
        out.append(so)
    return out


def _cpu_flags() -> set:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


_LIB = None


def load():
    global _LIB
    if _LIB is not None:
        return _LIB
    flags = _cpu_flags()
    order = ["avx2", "generic"] if {"avx2", "fma"} <= flags else ["generic"]
    for name in order:
        so = LIB_DIR / f"libsvod_oracle_{name}.so"
        if so.exists():
            lib = ctypes.CDLL(str(so))
            break
    else:
        raise OSError(f"no C oracle library under {LIB_DIR}: run oracle.c_oracle.build()")
    fp, ip = ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_int32)
    i64, i32, f32 = ctypes.c_int64, ctypes.c_int, ctypes.c_float
    lib.so_threads.restype = i32
    lib.so_round.argtypes = [fp, i64, i32]
    lib.so_linear.argtypes = [fp, fp, fp, fp, fp, i64, i64, i64, i32, i32, i32, f32, i32]
    lib.so_norm_rows.argtypes = [i32, fp, fp, fp, fp, fp, fp, i64, i64, f32, i32]
    lib.so_rope_table.argtypes = [f32, ip, i64, i32, fp, fp, i32]
    lib.so_heads.argtypes = [fp, fp, fp, fp, fp, fp, fp, fp, i64, i64, i32, i32, i32, f32, i32]
    bp = ctypes.POINTER(ctypes.c_uint8)
    lib.so_set_threads.argtypes = [i32]
    lib.so_attention.argtypes = [fp, fp, fp, fp, i64, i64, i64, i32, i32, i32, i32, ip, bp, i32, i32, i32, f32, i32]
    lib.so_linear_rope.argtypes = [fp, fp, fp, fp, i64, i64, i64, i64, fp, fp, i32, i32, i32]
    lib.so_qwen3_layers.argtypes = [fp, ctypes.POINTER(fp), i32, i64, i64, i32, i32, i32, i32, i32, f32, f32, i32]
    lib.so_qwen3_layers.restype = i32
    lib.so_xlmr_layers.argtypes = [fp, ctypes.POINTER(fp), i32, i64, i64, i32, i32, i32, bp, f32, i32]
    lib.so_xlmr_layers.restype = i32
    lib.so_modernbert_layers.argtypes = [fp, ctypes.POINTER(fp), i32, i32, i64, i64, i32, i32, i32, bp, i32, f32, f32,
                                         i32, i32, f32, i32]
    lib.so_modernbert_layers.restype = i32
    for fn in (lib.so_round, lib.so_linear, lib.so_norm_rows, lib.so_rope_table, lib.so_heads, lib.so_attention,
               lib.so_linear_rope, lib.so_set_threads):
        fn.restype = None
    _LIB = lib
    return lib


def threads() -> int:
    return int(load().so_threads())


def use_all_cores() -> int:
    """Sizes the OpenMP team to every core this process may run on, whatever
    `OMP_NUM_THREADS` said (launchers such as torchrun export 1); returns the count."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    load().so_set_threads(n)
    return threads()


def _f(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _ip(a):
    return None if a is None else a.ctypes.data_as(ctypes.POINTER(ctypes.c_int32))


def linear(x, w, bias=None, act=ACT_NONE, gated=False, residual=None, scale=None, dtype=BF16):
    x, w, bias, residual = _f(x), _f(w), _f(bias), _f(residual)
    k = x.shape[-1]
    m = x.size // k
    n = w.shape[0] // (2 if gated else 1)
    out = np.empty(x.shape[:-1] + (n,), dtype=np.float32)
    load().so_linear(_p(x), _p(w), _p(bias), _p(residual), _p(out), m, n, k, act, int(gated), int(scale is not None),
                     float(scale if scale is not None else 1.0), dtype)
    return out


def norm_rows(kind, x, w, b=None, residual=None, eps=1e-5, dtype=BF16):
    x, w, b, residual = _f(x), _f(w), _f(b), _f(residual)
    d = x.shape[-1]
    out = np.empty_like(x)
    total = np.empty_like(x) if residual is not None else None
    load().so_norm_rows(0 if kind == "layer" else 1, _p(x), _p(w), _p(b), _p(residual), _p(out), _p(total), x.size // d, d,
                        float(eps), dtype)
    return out, total


def rope_table(theta, positions, head_dim, dtype=BF16):
    pos = np.ascontiguousarray(positions, dtype=np.int32)
    cos = np.empty((pos.size, head_dim // 2), dtype=np.float32)
    sin = np.empty_like(cos)
    load().so_rope_table(float(theta), _ip(pos), pos.size, head_dim, _p(cos), _p(sin), dtype)
    return cos, sin


def heads(qkv, heads_n, kv_heads, d, q_w=None, k_w=None, eps=1e-6, cos=None, sin=None, dtype=BF16):
    qkv, q_w, k_w, cos, sin = _f(qkv), _f(q_w), _f(k_w), _f(cos), _f(sin)
    b, t = qkv.shape[:2]
    q = np.empty((b, t, heads_n, d), dtype=np.float32)
    k = np.empty((b, t, kv_heads, d), dtype=np.float32)
    v = np.empty((b, t, kv_heads, d), dtype=np.float32)
    load().so_heads(_p(qkv), _p(q_w), _p(k_w), _p(cos), _p(sin), _p(q), _p(k), _p(v), b, t, heads_n, kv_heads, d,
                    float(eps), dtype)
    return q, k, v


def _bp(a):
    return None if a is None else a.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8))


def _mask(m):
    return None if m is None else np.ascontiguousarray(np.asarray(m) != 0, dtype=np.uint8)


def attention(q, k, v, *, causal=False, key_lens=None, key_mask=None, window=None, scale=None, dtype=BF16):
    q, k, v = _f(q), _f(k), _f(v)
    b, t, h, d = q.shape
    tk, hkv = k.shape[1], k.shape[2]
    lens = None if key_lens is None else np.ascontiguousarray(key_lens, dtype=np.int32)
    km = _mask(key_mask)
    o = np.empty_like(q)
    sc = float(np.float32(1.0 / np.sqrt(d))) if scale is None else float(scale)
    wl, wr = window if window is not None else (0, 0)
    load().so_attention(_p(q), _p(k), _p(v), _p(o), b, t, tk, h, hkv, d, int(causal), _ip(lens), _bp(km),
                        int(window is not None), int(wl), int(wr), sc, dtype)
    return o


def linear_rope(x, w, cos, sin, heads_n, head_dim, bias=None, dtype=BF16):
    """`x [B,T,K] . w^T (+ bias)` with the first `heads_n*head_dim` output columns
    turned in the store; tables `[T, head_dim/2]`."""
    x, w, bias, cos, sin = _f(x), _f(w), _f(bias), _f(cos), _f(sin)
    k = x.shape[-1]
    t = x.shape[-2]
    n = w.shape[0]
    out = np.empty(x.shape[:-1] + (n,), dtype=np.float32)
    load().so_linear_rope(_p(x), _p(w), _p(bias), _p(out), x.size // k, n, k, t, _p(cos), _p(sin), heads_n, head_dim,
                          dtype)
    return out


QWEN3_LAYER_KEYS = ("in_w", "qkv_w", "qn_w", "kn_w", "o_w", "post_w", "gu_w", "down_w")


def qwen3_layers(hidden, layers, *, heads_n, kv_heads, head_dim, theta=1e6, eps=1e-6, dtype=BF16):
    """Runs the Qwen3 layers over `hidden [B,T,D]` (a copy) and returns the result;
    `layers` is the list of per-layer weight dicts the numpy restatement takes."""
    hid = np.array(hidden, dtype=np.float32, order="C")
    b, t, dm = hid.shape
    keep = [[_f(lp[k]) for k in QWEN3_LAYER_KEYS] for lp in layers]
    fp = ctypes.POINTER(ctypes.c_float)
    flat = (fp * (8 * len(layers)))(*[_p(a) for lw in keep for a in lw])
    f = keep[0][7].shape[1]
    rc = load().so_qwen3_layers(_p(hid), flat, len(layers), b, t, dm, heads_n, kv_heads, head_dim, f, float(theta),
                                float(eps), dtype)
    if rc != 0:
        raise MemoryError("the C oracle could not allocate its scratch")
    return hid


XLMR_LAYER_KEYS = ("q_w", "q_b", "k_w", "k_b", "v_w", "v_b", "o_w", "o_b", "ln1_w", "ln1_b", "fi_w", "fi_b", "fo_w",
                   "fo_b", "ln2_w", "ln2_b")


def _flat(layers, keys):
    keep = [[_f(lp.get(k)) for k in keys] for lp in layers]
    fp = ctypes.POINTER(ctypes.c_float)
    return keep, (fp * (len(keys) * len(layers)))(*[_p(a) for lw in keep for a in lw])


def xlmr_layers(hidden, layers, mask, *, heads_n, eps=1e-5, dtype=F16):
    """Runs XLM-R encoder layers over `hidden [B,T,D]` (a copy); `mask [B,T]` nonzero = real token."""
    hid = np.array(hidden, dtype=np.float32, order="C")
    b, t, dm = hid.shape
    keep, flat = _flat(layers, XLMR_LAYER_KEYS)
    km = _mask(mask)
    rc = load().so_xlmr_layers(_p(hid), flat, len(layers), b, t, dm, heads_n, keep[0][10].shape[0], _bp(km), float(eps),
                               dtype)
    if rc != 0:
        raise MemoryError("the C oracle could not allocate its scratch")
    return hid


MODERNBERT_LAYER_KEYS = ("attn_ln_w", "qkv_w", "o_w", "mlp_ln_w", "wi_w", "wo_w")


def modernbert_layers(hidden, layers, mask, *, heads_n, first_layer=0, global_every=3, global_theta=160000.0,
                      local_theta=10000.0, local_window=(64, 64), eps=1e-5, dtype=BF16):
    """Runs ModernBERT layers `first_layer ...` over `hidden [B,T,D]` (a copy)."""
    hid = np.array(hidden, dtype=np.float32, order="C")
    b, t, dm = hid.shape
    keep, flat = _flat(layers, MODERNBERT_LAYER_KEYS)
    km = _mask(mask)
    rc = load().so_modernbert_layers(_p(hid), flat, len(layers), first_layer, b, t, dm, heads_n, keep[0][5].shape[1],
                                     _bp(km), global_every, float(global_theta), float(local_theta),
                                     int(local_window[0]), int(local_window[1]), float(eps), dtype)
    if rc != 0:
        raise MemoryError("the C oracle could not allocate its scratch")
    return hid
