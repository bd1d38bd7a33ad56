"""Writes `tests/golden/ops_golden.npz`: seeded inputs and the oracle's outputs
for a few small cases of each op on the path, stored as float32 (every value is
already rounded to bf16, so the upper 16 bits of its float32 form hold it
exactly: arrays are stored as those uint16 bit patterns; `load()` widens them).

The reference keeps no stored vectors for this path (its tests are generators
plus closed forms) and cannot be built here, so these fixtures pin the oracle
against itself across changes and give the GPU suite a reference that does not
depend on running the oracle. Regenerate with:

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", ".."))
from oracle import svod_oracle as O  # noqa: E402


def build():
    g = {}
    dt = O.BF16
    rng = np.random.default_rng(20240)
    n = lambda shape, s=1.0: O.round_to(dt, rng.standard_normal(shape) * s)
    # attention: causal + key lengths + GQA
    q, k, v = n((1, 96, 2, 64)), n((1, 96, 1, 64)), n((1, 96, 1, 64))
    lens = np.array([77])
    g["attn_q"], g["attn_k"], g["attn_v"], g["attn_lens"] = q, k, v, lens
    g["attn_o"] = O.attention(q, k, v, causal=True, key_lens=lens, dtype=dt)
    # attention: window + segments, d 128
    q, k, v = n((1, 64, 1, 128)), n((1, 64, 1, 128)), n((1, 64, 1, 128))
    seg = np.array([[i - i % 40 for i in range(64)]])
    g["attn2_q"], g["attn2_k"], g["attn2_v"], g["attn2_seg"] = q, k, v, seg
    g["attn2_o"] = O.attention(q, k, v, causal=True, window=(30, 0), seg_start=seg, dtype=dt)
    # cached attention: row map, appended rows, counted
    q, kc, vc = n((2, 3, 4, 64)), n((3, 32, 6, 64)), n((3, 32, 6, 64))
    ka, va = n((2, 4, 2, 64)), n((2, 4, 2, 64))
    g["cache_q"], g["cache_k"], g["cache_v"], g["cache_ka"], g["cache_va"] = q, kc, vc, ka, va
    g["cache_o"] = O.attention(q, kc, vc, key_lens=np.array([32, 11]), dtype=dt,
                               cache=dict(head_start=2, kv_heads=2, row_map=[2, 0], k_app=ka, v_app=va, app_lens=[4, 2]))
    # linear: bias + erf GELU; gated SiLU + residual + scale
    x, w, b = n((48, 64)), n((32, 64), 64 ** -0.5), n((32,))
    g["lin_x"], g["lin_w"], g["lin_b"] = x, w, b
    g["lin_gelu"] = O.linear(x, w, b, act=O.ACT_GELU, dtype=dt)
    wg, bg, r = n((64, 64), 64 ** -0.5), n((64,)), n((48, 32))
    g["lin_wg"], g["lin_bg"], g["lin_r"] = wg, bg, r
    g["lin_swiglu"] = O.linear(x, wg, bg, act=O.ACT_SILU, gated=True, residual=r, scale=0.5, dtype=dt)
    # heads: q/k norm + rotation
    qkv, qw, kw = n((2, 24, (2 + 2) * 64)), O.round_to(dt, 1 + 0.1 * rng.standard_normal(64)), \
        O.round_to(dt, 1 + 0.1 * rng.standard_normal(64))
    cos, sin = O.rope_table(1e6, np.arange(24), 64, dt)
    g["heads_qkv"], g["heads_qw"], g["heads_kw"], g["heads_cos"], g["heads_sin"] = qkv, qw, kw, cos, sin
    hq, hk, hv = O.heads(qkv, 2, 1, 64, qw, kw, 1e-6, cos, sin, dt)
    g["heads_q"], g["heads_k"], g["heads_v"] = hq, hk, hv
    # norms: fused add + RMSNorm, LayerNorm with bias
    x, r, w, b = n((10, 256), 2.0), n((10, 256)), O.round_to(dt, 1 + 0.5 * rng.standard_normal(256)), n((256,), 0.5)
    g["norm_x"], g["norm_r"], g["norm_w"], g["norm_b"] = x, r, w, b
    y, s = O.norm_rows("rms", x, w, residual=r, eps=1e-6, dtype=dt)
    g["norm_rms"], g["norm_sum"] = y, s
    g["norm_layer"], _ = O.norm_rows("layer", x, w, b, eps=1e-5, dtype=dt)
    out = {}
    for key, val in g.items():
        val = np.asarray(val)
        if val.dtype.kind == "f":
            bits = np.ascontiguousarray(val, dtype=np.float32).view(np.uint32)
            assert not np.any(bits & 0xFFFF), key  # bf16 values only
            out[key] = (bits >> 16).astype(np.uint16)
        else:
            out["i_" + key] = val.astype(np.int64)
    return out


def load(path=None):
    """The fixtures as float64 arrays (integers as int64), keyed as in `build`."""
    path = path or os.path.join(os.path.dirname(__file__), "ops_golden.npz")
    out = {}
    with np.load(path) as z:
        for key in z.files:
            if key.startswith("i_"):
                out[key[2:]] = z[key]
            else:
                out[key] = (z[key].astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    return out


if __name__ == "__main__":
    out = os.path.join(os.path.dirname(__file__), "ops_golden.npz")
    np.savez_compressed(out, **build())
    print(out, os.path.getsize(out), "bytes")
