"""CPU restatement (numpy, float64) of svod's `tk` transformer-encoder hot path.

THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE. Only the tests, the smoke check
and the benchmark's CPU-baseline leg import it; the product path is the CUDA
library and fails loudly when that library is missing.

The reference (npatsakula/svod, Rust) cannot be compiled in this build
environment (no rustc/cargo/libLLVM), so every function below restates the
arithmetic of the reference file:line it cites. The arithmetic is all in the
reference's own repository (no third-party crate computes any of it). Parity is
pinned two ways (see tests/test_oracle_pins.py):
  * the known-answer tests of tensor/src/test/unit/transformer.rs (rms_norm,
    SDPA causal/bool-mask/window, rotary split/rotation) are replayed here, and
  * the reference's seeded test recipes (64-bit LCG, tk/src/test/unit/mod.rs:441-450)
    with their closed-form f64 references are regenerated bit for bit.

Conventions follow the reference: activations are sequence-major `[B, T, H, D]`,
weights are `[N, K]` (PyTorch `nn.Linear`), every op computes in wide precision
from inputs already rounded to the storage dtype and rounds once at the store.
"""
from __future__ import annotations

import math

import numpy as np

# --------------------------------------------------------------------------
# dtype rounding — tk/src/interp.rs:37-71 (`round_to`, `f16_round`)
# --------------------------------------------------------------------------

F32, F16, BF16 = "f32", "f16", "bf16"


def round_bf16(x):
    """Round-to-nearest-even to bfloat16 precision, returned as float64.

    tk/src/interp.rs:41-45: `bits + 0x7fff + ((bits >> 16) & 1)` masked to the
    top 16 bits; NaN kept quiet.
    """
    x32 = np.asarray(x, dtype=np.float64).astype(np.float32)
    bits = x32.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    out = rounded.view(np.float32).astype(np.float64)
    return np.where(np.isnan(x32), np.nan, out)


def round_f16(x):
    """Round-to-nearest-even to IEEE half precision (tk/src/interp.rs:52-71).

    The reference saturates exponents above 15 to infinity and keeps fewer
    mantissa bits for subnormals; numpy's float16 cast does the same.
    """
    with np.errstate(over="ignore"):
        return np.asarray(x, dtype=np.float64).astype(np.float32).astype(np.float16).astype(np.float64)


def round_to(dtype, x):
    """tk/src/interp.rs:37-50."""
    if dtype == BF16:
        return round_bf16(x)
    if dtype == F16:
        return round_f16(x)
    if dtype == F32:
        return np.asarray(x, dtype=np.float64).astype(np.float32).astype(np.float64)
    raise ValueError(f"rounding to {dtype}")


def bf16_bits(x):
    """The 16-bit patterns of values already rounded by `round_bf16`."""
    return (np.asarray(x, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


def from_bf16_bits(bits):
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)


# --------------------------------------------------------------------------
# the reference's seeded generator — tk/src/test/unit/mod.rs:441-450
# --------------------------------------------------------------------------

_MASK64 = (1 << 64) - 1


class Lcg:
    """`s <- s*6364136223846793005 + 1442695040888963407 (mod 2^64)`;
    `x = (s >> 33) / 2^31 * 2 - 1`, uniform in [-1, 1)."""

    def __init__(self, seed: int):
        self.s = seed & _MASK64

    def draw(self, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.float64)
        s = self.s
        for i in range(n):
            s = (s * 6364136223846793005 + 1442695040888963407) & _MASK64
            out[i] = (s >> 33) / float(1 << 31) * 2.0 - 1.0
        self.s = s
        return out

    def rounded(self, dtype, n: int, f=lambda x: x) -> np.ndarray:
        """`rounded` of tk/src/test/unit/mod.rs:447-450."""
        return round_to(dtype, f(self.draw(n)))


def ops_rand(shape, seed: int, scale: float) -> np.ndarray:
    """`rand(shape, seed, scale)` of tk/src/test/unit/ops.rs:20-27: the LCG
    started at `seed*0x9e3779b97f4a7c15 | 1`, draws scaled (not yet rounded)."""
    g = Lcg(((seed * 0x9E3779B97F4A7C15) & _MASK64) | 1)
    return (g.draw(int(np.prod(shape))) * scale).reshape(shape)


# --------------------------------------------------------------------------
# activations — tk/src/kernels/mod.rs:272-335, tensor/src/activation.rs:198-243
# --------------------------------------------------------------------------

ACT_NONE, ACT_GELU, ACT_SILU, ACT_GELU_TANH = 0, 1, 2, 3

_erf = np.vectorize(math.erf, otypes=[np.float64])


def gelu_erf(x):
    """`0.5*x*(1+erf(x/sqrt2))`: `gelu_exact` (tensor/src/activation.rs:233-243)
    and the closed form the reference's GEMM test uses (tk/src/test/unit/rows.rs:67)."""
    x = np.asarray(x, dtype=np.float64)
    return 0.5 * x * (1.0 + _erf(x * math.sqrt(0.5)))


def gelu_as(x):
    """The in-kernel form: `0.5*(x+|x|*erf(|x|/sqrt2))` with erf by
    Abramowitz-Stegun 7.1.26 (tk/src/kernels/mod.rs:313-335), |error| <= 1.5e-7."""
    x = np.asarray(x, dtype=np.float64)
    p = 0.3275911
    a = [0.254829592, -0.284496736, 1.421413741, -1.453152027, 1.061405429]
    ax = np.abs(x)
    z = ax * math.sqrt(0.5)
    t = 1.0 / (z * p + 1.0)
    poly = np.full_like(t, a[4])
    for c in reversed(a[:4]):
        poly = poly * t + c
    poly = poly * t
    erf = 1.0 - poly * np.exp2(-(z * z) * math.log2(math.e))
    return 0.5 * (x + ax * erf)


def gelu_tanh(x):
    """`Tensor::gelu` (tensor/src/activation.rs:198-230), not reachable from
    `tk::ops`; kept for the benchmark sweep that names it."""
    x = np.asarray(x, dtype=np.float64)
    return 0.5 * x * (1.0 + np.tanh(0.7978845608 * (x + 0.044715 * x * x * x)))


def silu(x):
    """`x/(1+2^(-x*log2 e))` (tk/src/kernels/mod.rs:304-311) = `x*sigmoid(x)`."""
    x = np.asarray(x, dtype=np.float64)
    return x / (1.0 + np.exp(-x))


def activate(x, act):
    if act == ACT_NONE:
        return x
    if act == ACT_GELU:
        return gelu_erf(x)
    if act == ACT_SILU:
        return silu(x)
    if act == ACT_GELU_TANH:
        return gelu_tanh(x)
    raise ValueError(act)


# --------------------------------------------------------------------------
# RoPE — tensor/src/transformer.rs:72-164
# --------------------------------------------------------------------------


def rope_inv_freq(theta: float, head_dim: int) -> np.ndarray:
    """`theta^(-2i/head_dim)` evaluated in float32 (transformer.rs:153-164)."""
    expo = (np.arange(head_dim // 2, dtype=np.float32) * np.float32(-2.0 / head_dim)).astype(np.float32)
    return np.power(np.float32(theta), expo).astype(np.float32)


def rope_table(theta: float, positions, head_dim: int, dtype):
    """`(cos, sin)` of `[len(positions), head_dim/2]`: angles in float32, cos/sin
    in float32, cast to `dtype` last (transformer.rs:130-150)."""
    pos = np.asarray(positions, dtype=np.float32).reshape(-1, 1)
    ang = (pos * rope_inv_freq(theta, head_dim).reshape(1, -1)).astype(np.float32)
    return round_to(dtype, np.cos(ang).astype(np.float32)), round_to(dtype, np.sin(ang).astype(np.float32))


def apply_rotary_split(x, cos, sin):
    """Half-split (GPT-NeoX) rotation over the last dim (transformer.rs:72-117):
    `y1 = x1*cos - x2*sin`, `y2 = x1*sin + x2*cos`."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    return np.concatenate([x1 * cos - x2 * sin, x1 * sin + x2 * cos], axis=-1)


# --------------------------------------------------------------------------
# norms — tk/src/kernels/rows.rs:41-115, tk/src/test/unit/rows.rs:169-197
# --------------------------------------------------------------------------


def norm_rows(kind: str, x, w, b=None, residual=None, eps=1e-5, dtype=BF16):
    """LayerNorm / RMSNorm over the last dim with the optional fused residual.

    Returns `(out, sum)`; `sum` is `round(x + residual)` (None when not fused)
    and is what gets normalised (rows.rs:77-85). Biased variance,
    `1/sqrt(var+eps)`, one rounding at the store.
    """
    x = np.asarray(x, dtype=np.float64)
    summed = None
    if residual is not None:
        summed = round_to(dtype, x + np.asarray(residual, dtype=np.float64))
        x = summed
    mean = x.mean(axis=-1, keepdims=True) if kind == "layer" else 0.0
    c = x - mean
    var = (c * c).mean(axis=-1, keepdims=True)
    y = c / np.sqrt(var + eps) * np.asarray(w, dtype=np.float64)
    if b is not None:
        y = y + np.asarray(b, dtype=np.float64)
    return round_to(dtype, y), summed


# --------------------------------------------------------------------------
# heads — tk/src/kernels/heads.rs:36-125, tk/src/test/unit/heads.rs:59-105
# --------------------------------------------------------------------------


def heads(qkv, heads_n, kv_heads, d, q_w=None, k_w=None, eps=1e-6, cos=None, sin=None, dtype=BF16):
    """`qkv [B,T,(H+2Hkv)*D]` -> `q [B,T,H,D]`, `k,v [B,T,Hkv,D]`.

    q and k: optional RMSNorm over D (`x/sqrt(mean x^2+eps)*w`) then the
    half-split rotation with `cos,sin` of `[1|B, T, D/2]`; v copied. One
    rounding at the store.
    """
    qkv = np.asarray(qkv, dtype=np.float64)
    B, T, _ = qkv.shape
    x = qkv.reshape(B, T, heads_n + 2 * kv_heads, d)
    parts = [x[:, :, :heads_n], x[:, :, heads_n:heads_n + kv_heads], x[:, :, heads_n + kv_heads:]]
    out = []
    for which, (part, w) in enumerate(zip(parts, [q_w, k_w, None])):
        y = part
        if w is not None:
            inv = 1.0 / np.sqrt((y * y).mean(axis=-1, keepdims=True) + eps)
            y = y * inv * np.asarray(w, dtype=np.float64)
        if cos is not None and which < 2:
            c = np.asarray(cos, dtype=np.float64).reshape(-1, T, 1, d // 2)
            s = np.asarray(sin, dtype=np.float64).reshape(-1, T, 1, d // 2)
            y = apply_rotary_split(y, c, s)
        out.append(round_to(dtype, y))
    return tuple(out)


# --------------------------------------------------------------------------
# linear — tk/src/kernels/gemm.rs:605-651 (order of the epilogue),
# tk/src/ops/linear.rs:306-355 (graph), tk/src/test/unit/rows.rs:51-75
# --------------------------------------------------------------------------


def linear(x, w, bias=None, act=ACT_NONE, gated=False, residual=None, scale=None, rope=None, dtype=BF16):
    """`scale*act(x.w^T + bias) + residual`; gated: `w = [2N,K]`, gate rows
    first, `act(gate)*up`.

    Epilogue order on the wide accumulator: +bias -> act -> *up -> *scale ->
    RoPE turn -> +residual -> one rounding. `rope = (cos, sin, heads, head_dim)`
    with tables `[T, head_dim/2]` rotates the first `heads*head_dim` output
    columns of `x [B,T,K]`, row `t` at position `t` (gemm.rs:670-718); it is
    only ever combined with a bias (linear.rs:132-139).
    """
    x = np.asarray(x, dtype=np.float64)
    w = np.asarray(w, dtype=np.float64)
    y = x @ w.T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float64)
    if gated:
        n = w.shape[0] // 2
        y = activate(y[..., :n], act) * y[..., n:]
    else:
        y = activate(y, act)
    if scale is not None:
        y = y * float(np.float32(scale))
    if rope is not None:
        cos, sin, nh, hd = rope
        B, T, N = y.shape
        width = nh * hd
        turned = y[..., :width].reshape(B, T, nh, hd)
        c = np.asarray(cos, dtype=np.float64).reshape(1, T, 1, hd // 2)
        s = np.asarray(sin, dtype=np.float64).reshape(1, T, 1, hd // 2)
        turned = apply_rotary_split(turned, c, s).reshape(B, T, width)
        y = np.concatenate([turned, y[..., width:]], axis=-1)
    if residual is not None:
        y = y + np.asarray(residual, dtype=np.float64)
    return round_to(dtype, y)


# --------------------------------------------------------------------------
# attention — tk/src/test/unit/attention.rs:102-178 (f64 mirror of the kernel's
# masks), tensor/src/transformer.rs:358-531 (graph), kernels/attention.rs:971-980
# --------------------------------------------------------------------------


def attention(q, k, v, *, causal=False, key_lens=None, key_mask=None, window=None, chunk=None,
              seg_start=None, scale=None, bias=None, dtype=BF16, return_lse=False, cache=None):
    """`softmax(q.k^T*scale + bias) . v` over `q [B,T,H,D]`, `k,v [B,Tk,Hkv,D]`.

    Masks apply together: causal `j<=i`; `j < key_lens[b]`; window
    `i-left <= j <= i+right`; chunk `(size,left|None,right)`; key mask nonzero
    = visible; segment `j >= seg_start[b,i]`. A query with no visible key yields
    zeros. GQA: query head `h` reads KV head `h // (H/Hkv)`. `bias` is
    `[B|1,H,T,Tk]`, added after scaling and before the masks.

    `lse[b,h,i] = max + ln(sum exp(s - max))` of the masked scaled scores
    (`-inf` for an empty row): the natural-log form of the `(m, l)` statistics
    the reference keeps in log2 units (kernels/attention.rs:910-920).

    `cache = dict(head_start, kv_heads, row_map=None, k_app=None, v_app=None,
    app_lens=None)` (`ops::Cache`, tk/src/ops/attention.rs:39-55; graph at
    :496-535): `k, v` are `[rows, Tk, H_all, D]`; this attention reads heads
    `head_start .. head_start+kv_heads` of cache row `row_map[b]` (row `b`
    without a map), then the appended `[B, n, kv_heads, D]` keys. The masks
    above apply to the cached keys only; an appended key is hidden only past
    `app_lens[b]` (tk/src/test/unit/attention.rs:112-135). `bias` spans
    `Tk + n` columns, the appended ones last.
    """
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    n_app = 0
    cached_keys = k.shape[1]
    if cache is not None:
        hs, kvh = cache["head_start"], cache["kv_heads"]
        k, v = k[:, :, hs:hs + kvh], v[:, :, hs:hs + kvh]
        if cache.get("row_map") is not None:
            rm = np.asarray(cache["row_map"]).astype(np.int64)
            k, v = k[rm], v[rm]
        else:
            k, v = k[:q.shape[0]], v[:q.shape[0]]  # lane b reads row b
        if cache.get("k_app") is not None:
            ka = np.asarray(cache["k_app"], dtype=np.float64)
            va = np.asarray(cache["v_app"], dtype=np.float64)
            n_app = ka.shape[1]
            k, v = np.concatenate([k, ka], axis=1), np.concatenate([v, va], axis=1)
    B, T, H, D = q.shape
    _, Tk, Hkv, _ = k.shape
    group = H // Hkv
    if scale is None:
        scale = float(np.float32(1.0 / math.sqrt(D)))
    else:
        scale = float(np.float32(scale))
    # head-major views so the two contractions are batched BLAS matmuls
    qh = q.transpose(0, 2, 1, 3)
    kh = np.repeat(k, group, axis=2).transpose(0, 2, 1, 3)
    vh = np.repeat(v, group, axis=2).transpose(0, 2, 1, 3)
    s = np.matmul(qh, kh.transpose(0, 1, 3, 2)) * scale
    if bias is not None:
        s = s + np.asarray(bias, dtype=np.float64)
    i = np.arange(T).reshape(1, 1, T, 1)
    j = np.arange(Tk).reshape(1, 1, 1, Tk)
    hidden = np.zeros((B, 1, T, Tk), dtype=bool)
    if causal:
        hidden |= j > i
    if key_lens is not None:
        hidden |= j >= np.asarray(key_lens).reshape(B, 1, 1, 1)
    if window is not None:
        left, right = window
        hidden |= (j + left < i) | (j > i + right)
    if chunk is not None:
        size, left, right = chunk
        hidden |= (j // size) > (i // size + right)
        if left is not None:
            hidden |= (j // size + left) < (i // size)
    if key_mask is not None:
        km = np.asarray(key_mask).reshape(B, 1, 1, cached_keys) == 0
        if n_app:
            km = np.concatenate([km, np.zeros((B, 1, 1, n_app), dtype=bool)], axis=-1)
        hidden |= km
    if seg_start is not None:
        hidden |= j < np.asarray(seg_start).reshape(B, 1, T, 1)
    if n_app:
        # appended keys answer to their own count alone
        seen = np.full(B, n_app) if cache.get("app_lens") is None else np.asarray(cache["app_lens"])
        hidden = np.where(j >= cached_keys, (j - cached_keys) >= seen.reshape(B, 1, 1, 1), hidden)
    s = np.where(hidden, -np.inf, s)
    mx = s.max(axis=-1, keepdims=True)
    empty = ~np.isfinite(mx)
    with np.errstate(invalid="ignore"):
        wts = np.exp(s - np.where(empty, 0.0, mx))
    wts = np.where(hidden, 0.0, wts)
    l = wts.sum(axis=-1, keepdims=True)
    out = np.matmul(wts / np.where(empty, 1.0, l), vh).transpose(0, 2, 1, 3)
    out = round_to(dtype, out)
    if return_lse:
        with np.errstate(divide="ignore"):
            lse = np.where(empty, -np.inf, mx + np.log(np.where(empty, 1.0, l)))[..., 0]
        return out, lse
    return out


def attention_packed(qkv, heads_n, kv_heads, **kw):
    """`ops::attention_packed` (tk/src/ops/attention.rs:107-122): q, k and v
    read from one `[B,T,(H+2Hkv)*D]` projection at head offsets 0 / H / H+Hkv."""
    qkv = np.asarray(qkv, dtype=np.float64)
    B, T, W = qkv.shape
    d = W // (heads_n + 2 * kv_heads)
    x = qkv.reshape(B, T, heads_n + 2 * kv_heads, d)
    return attention(x[:, :, :heads_n], x[:, :, heads_n:heads_n + kv_heads], x[:, :, heads_n + kv_heads:], **kw)


def combine_splits(o_part, m_part, l_part, dtype=BF16):
    """`combine_splits` (tk/src/kernels/attention.rs:948-1014): partial
    `(o, m, l)` states with `m` in log2 units merged as `m = max m_i`,
    `w_i = 2^(m_i - m)`, `o = sum o_i w_i / sum l_i w_i`; `l == 0` -> zeros."""
    o_part = np.asarray(o_part, dtype=np.float64)
    m_part = np.asarray(m_part, dtype=np.float64)
    l_part = np.asarray(l_part, dtype=np.float64)
    m = m_part.max(axis=0)
    w = np.exp2(m_part - m)
    l = (l_part * w).sum(axis=0)
    o = (o_part * w[..., None]).sum(axis=0)
    return round_to(dtype, o / np.where(l == 0.0, 1.0, l)[..., None])


# --------------------------------------------------------------------------
# pooling — model/src/encoder_head.rs:280-286, tensor/src/nn/norm.rs:205-213,
# model/src/qwen3/model.rs:77-99
# --------------------------------------------------------------------------

F32_MIN_POSITIVE = float(np.finfo(np.float32).tiny)


def l2_normalize(x):
    """`lp_normalize(-1, 2)`: divides by `||x||_2 + f32::MIN_POSITIVE`."""
    x = np.asarray(x, dtype=np.float64)
    return x / (np.sqrt((x * x).sum(axis=-1, keepdims=True)) + F32_MIN_POSITIVE)


def pool(hidden, mask, mode: str, lengths=None, normalize=True):
    """`[B,L,D]` -> `[B,D]` float32-valued: CLS (token 0), masked mean in wide
    precision with denominator floor 1e-9, or last real token (index
    `clamp(len-1, 0, L-1)`), then L2."""
    hidden = np.asarray(hidden, dtype=np.float64)
    B, L, _ = hidden.shape
    if mode == "cls":
        p = hidden[:, 0]
    elif mode == "mean":
        m = np.asarray(mask, dtype=np.float64).reshape(B, L, 1)
        p = (hidden * m).sum(axis=1) / np.maximum(m.sum(axis=1), 1e-9)
    elif mode == "last":
        idx = np.clip(np.asarray(lengths) - 1, 0, L - 1)
        p = hidden[np.arange(B), idx]
    else:
        raise ValueError(mode)
    p = l2_normalize(p) if normalize else p
    return round_to(F32, p)


# --------------------------------------------------------------------------
# embeddings — model/src/xlm_roberta/{embeddings.rs:53-63, position_ids.rs:27-32}
# --------------------------------------------------------------------------


def xlmr_position_ids(ids, pad: int):
    """`cumsum(ids != pad) * (ids != pad) + pad`."""
    m = (np.asarray(ids) != pad).astype(np.int64)
    return np.cumsum(m, axis=-1) * m + pad


# --------------------------------------------------------------------------
# the three layer stacks (callers that fix the op sequence)
# --------------------------------------------------------------------------


def xlmr_forward(p, ids, mask, *, heads_n, eps=1e-5, pad=1, dtype=F16, pooling="cls"):
    """XLM-RoBERTa / BGE-M3 encoder: embeddings (word + position + type 0, LN),
    post-LN layers with separate biased Q/K/V projections, key-mask attention,
    erf-GELU FFN, residuals added in the projection before each norm
    (model/src/xlm_roberta/{attention.rs:63-77, feed_forward.rs:40-45,
    encoder_layer.rs:45-49}); pooled by `encoder_head::pool`."""
    ids = np.asarray(ids)
    B, L = ids.shape
    pos = xlmr_position_ids(ids, pad)
    h = round_to(dtype, round_to(dtype, p["word"][ids] + p["pos"][pos]) + p["type"][0])
    h, _ = norm_rows("layer", h, p["emb_ln_w"], p["emb_ln_b"], eps=eps, dtype=dtype)
    D = h.shape[-1]
    hd = D // heads_n
    for lp in p["layers"]:
        q = linear(h, lp["q_w"], lp["q_b"], dtype=dtype).reshape(B, L, heads_n, hd)
        k = linear(h, lp["k_w"], lp["k_b"], dtype=dtype).reshape(B, L, heads_n, hd)
        v = linear(h, lp["v_w"], lp["v_b"], dtype=dtype).reshape(B, L, heads_n, hd)
        a = attention(q, k, v, key_mask=mask, dtype=dtype).reshape(B, L, D)
        x = linear(a, lp["o_w"], lp["o_b"], residual=h, dtype=dtype)
        h, _ = norm_rows("layer", x, lp["ln1_w"], lp["ln1_b"], eps=eps, dtype=dtype)
        y = linear(h, lp["fi_w"], lp["fi_b"], act=ACT_GELU, dtype=dtype)
        x = linear(y, lp["fo_w"], lp["fo_b"], residual=h, dtype=dtype)
        h, _ = norm_rows("layer", x, lp["ln2_w"], lp["ln2_b"], eps=eps, dtype=dtype)
    return pool(h, mask, pooling), h


def qwen3_forward(p, ids, lengths, *, heads_n, kv_heads, head_dim, theta=1e6, eps=1e-6, dtype=BF16):
    """Qwen3 embedding decoder: pre-RMSNorm layers, fused QKV without bias,
    `heads` (q/k RMSNorm + RoPE), causal attention, o_proj with the residual,
    gated SiLU MLP with the residual (model/src/qwen3/{attention.rs:69-113,
    feed_forward.rs:38-42, decoder_layer.rs:55-65}); final RMSNorm, last-token
    pooling, L2 (qwen3/embedder.rs:37-52)."""
    ids = np.asarray(ids)
    B, L = ids.shape
    h = p["embed"][ids]
    cos, sin = rope_table(theta, np.arange(L), head_dim, dtype)
    for lp in p["layers"]:
        xn, _ = norm_rows("rms", h, lp["in_w"], eps=eps, dtype=dtype)
        qkv = linear(xn, lp["qkv_w"], dtype=dtype)
        q, k, v = heads(qkv, heads_n, kv_heads, head_dim, lp["qn_w"], lp["kn_w"], eps, cos, sin, dtype)
        a = attention(q, k, v, causal=True, dtype=dtype).reshape(B, L, heads_n * head_dim)
        h = linear(a, lp["o_w"], residual=h, dtype=dtype)
        hn, _ = norm_rows("rms", h, lp["post_w"], eps=eps, dtype=dtype)
        g = linear(hn, lp["gu_w"], act=ACT_SILU, gated=True, dtype=dtype)
        h = linear(g, lp["down_w"], residual=h, dtype=dtype)
    h, _ = norm_rows("rms", h, p["norm_w"], eps=eps, dtype=dtype)
    return pool(h, None, "last", lengths=lengths), h


def modernbert_forward(p, ids, mask, *, heads_n, global_every=3, global_theta=160000.0, local_theta=10000.0,
                       local_window=(64, 64), eps=1e-5, dtype=BF16, pooling="mean"):
    """ModernBERT encoder: token embedding + LN; pre-LN layers (layer 0 has no
    attention norm), fused QKV with RoPE turned in the projection's store,
    packed attention with the key mask and a per-layer window, GeGLU MLP
    (model/src/modernbert/{attention.rs:52-68, mlp.rs:41-46,
    encoder_layer.rs:52-60, encoder.rs:33-54}); final LN, pooling, L2."""
    ids = np.asarray(ids)
    B, L = ids.shape
    h, _ = norm_rows("layer", p["embed"][ids], p["emb_ln_w"], eps=eps, dtype=dtype)
    D = h.shape[-1]
    hd = D // heads_n
    tables = {True: rope_table(global_theta, np.arange(L), hd, dtype),
              False: rope_table(local_theta, np.arange(L), hd, dtype)}
    for li, lp in enumerate(p["layers"]):
        is_global = li % global_every == 0
        cos, sin = tables[is_global]
        xn = h if lp.get("attn_ln_w") is None else norm_rows("layer", h, lp["attn_ln_w"], eps=eps, dtype=dtype)[0]
        qkv = linear(xn, lp["qkv_w"], rope=(cos, sin, 2 * heads_n, hd), dtype=dtype)
        a = attention_packed(qkv, heads_n, heads_n, key_mask=mask,
                             window=None if is_global else local_window, dtype=dtype).reshape(B, L, D)
        h = linear(a, lp["o_w"], residual=h, dtype=dtype)
        hn, _ = norm_rows("layer", h, lp["mlp_ln_w"], eps=eps, dtype=dtype)
        g = linear(hn, lp["wi_w"], act=ACT_GELU, gated=True, dtype=dtype)
        h = linear(g, lp["wo_w"], residual=h, dtype=dtype)
    h, _ = norm_rows("layer", h, p["final_ln_w"], eps=eps, dtype=dtype)
    return pool(h, mask, pooling), h
