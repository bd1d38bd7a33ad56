"""Pins the CPU oracle against the reference's own known-answer tests and seeded
recipes (no GPU needed).

Known answers replayed from tensor/src/test/unit/transformer.rs (rms_norm, SDPA
causal / bool mask / window, rotary) and the seeded generators of
tk/src/test/unit/{mod,rows,heads,attention}.rs with their closed-form f64
references, restated independently here as plain loops.
"""
import math

import numpy as np
import pytest

from oracle import svod_oracle as O


# ---- rounding: tk/src/interp.rs:37-71 --------------------------------------------
def test_bf16_rounding_is_nearest_even_idempotent_and_monotone():
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(4000) * 10.0 ** rng.integers(-6, 6, 4000), [0.0, 1.0, -1.0]])
    r = O.round_bf16(x)
    assert np.array_equal(O.round_bf16(r), r)
    # within half an ulp of bf16 (8 significant bits)
    assert np.all(np.abs(r - x.astype(np.float32)) <= np.abs(x) * 2.0 ** -8 + 1e-45)
    xs = np.sort(x)
    assert np.all(np.diff(O.round_bf16(xs)) >= 0)
    # ties to even: 1 + 2^-8 is halfway between 1 and 1 + 2^-7
    assert O.round_bf16(1.0 + 2.0 ** -8) == 1.0
    assert O.round_bf16(1.0 + 3 * 2.0 ** -8) == 1.0 + 2 * 2.0 ** -7


def test_f16_rounding_saturates_and_keeps_subnormals():
    assert O.round_f16(70000.0) == np.inf          # exponent above 15 -> inf (interp.rs:57-59)
    assert O.round_f16(2.0 ** -24) == 2.0 ** -24   # smallest subnormal survives
    assert O.round_f16(1.0 + 2.0 ** -11) == 1.0    # tie to even
    r = O.round_f16(np.array([0.1, -3.3, 1000.7]))
    assert np.array_equal(O.round_f16(r), r)


# ---- the LCG: tk/src/test/unit/mod.rs:441-445 --------------------------------------
def test_lcg_first_draws():
    s = 5
    want = []
    for _ in range(4):
        s = (s * 6364136223846793005 + 1442695040888963407) % (1 << 64)
        want.append((s >> 33) / float(1 << 31) * 2.0 - 1.0)
    got = O.Lcg(5).draw(4)
    assert np.array_equal(got, np.array(want))
    assert np.all((got >= -1) & (got < 1))


# ---- rms_norm known answers: transformer.rs:13-48 ------------------------------------
def test_rms_norm_basic_known_answer():
    x = np.array([[1.0, 2.0, 3.0, 4.0]])
    got, _ = O.norm_rows("rms", x, np.ones(4), eps=1e-5, dtype=O.F32)
    inv = 1.0 / math.sqrt(7.5 + 1e-5)
    assert np.allclose(got[0], np.arange(1, 5) * inv, atol=1e-4)
    x = np.array([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    got, _ = O.norm_rows("rms", x, np.ones(3), eps=1e-5, dtype=O.F32)
    assert abs(got[0, 1] - 2.0 / math.sqrt(14.0 / 3 + 1e-5)) < 1e-4
    assert abs(got[1, 0] - 4.0 / math.sqrt(77.0 / 3 + 1e-5)) < 1e-4


# ---- SDPA known answers: transformer.rs:117-130,191-250,279-358 -----------------------
def _hm(x):
    """[B,H,T,D] head-major literals of the reference tests -> sequence-major."""
    return np.asarray(x, dtype=np.float64).transpose(0, 2, 1, 3)


def test_sdpa_causal_known_answer():
    q = _hm([[[[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]]]])
    v = _hm([[[[1.0, 0.0], [0.0, 1.0], [0.0, 0.0]]]])
    out = O.attention(q, q, v, causal=True, dtype=O.F32)
    assert abs(out[0, 0, 0, 0] - 1.0) < 1e-4 and abs(out[0, 0, 0, 1]) < 1e-4


def test_sdpa_bool_mask_known_answers():
    q = _hm([[[[1.0, 0.0]]]])
    k = _hm([[[[1.0, 0.0], [0.0, 1.0]]]])
    v = _hm([[[[10.0, 1.0], [1.0, 10.0]]]])
    # reference polarity: True = masked OUT; the op layer's key mask is the inverse
    out = O.attention(q, k, v, key_mask=np.array([[0, 1]]), dtype=O.F32)
    assert abs(out[0, 0, 0, 0] - 1.0) < 1e-4 and abs(out[0, 0, 0, 1] - 10.0) < 1e-4
    out = O.attention(q, k, v, key_mask=np.array([[0, 0]]), dtype=O.F32)
    assert np.all(np.isfinite(out)) and np.all(out == 0.0)
    q2 = _hm([[[[1.0, 0.0], [0.0, 1.0]]]])
    out = O.attention(q2, q2, v, causal=True, key_mask=np.array([[0, 0]]), dtype=O.F32)
    assert np.all(np.isfinite(out))


def test_sdpa_window_known_answers():
    q = _hm([[[[1.0], [1.0], [1.0], [1.0]]]])
    v = _hm([[[[0.0], [10.0], [20.0], [30.0]]]])
    out = O.attention(q, q, v, window=(0, 0), dtype=O.F32)[0, :, 0, 0]
    assert np.allclose(out, [0, 10, 20, 30], atol=1e-4)
    out = O.attention(q, q, v, window=(1, 1), dtype=O.F32)[0, :, 0, 0]
    assert abs(out[0] - 5) < 1e-4 and abs(out[1] - 10) < 1e-4 and abs(out[3] - 25) < 1e-4
    # window (0,1) intersected with a key mask keeping keys {0,1}
    out = O.attention(q, q, v, window=(0, 1), key_mask=np.array([[1, 1, 0, 0]]), dtype=O.F32)[0, :, 0, 0]
    assert abs(out[1] - 10) < 1e-4


# ---- rotary known answers: transformer.rs:364-427 ---------------------------------------
def test_rotary_known_answers():
    x = np.array([[[1.0, 2.0, 3.0, 4.0]]])
    got = O.apply_rotary_split(x, np.array([[[1.0, 0.0]]]), np.array([[[0.0, 0.0]]]))
    assert np.allclose(got[0, 0], [1, 0, 3, 0], atol=1e-5)
    x = np.array([[[1.0, 0.0, 0.0, 1.0]]])
    got = O.apply_rotary_split(x, np.array([[[0.0, 0.0]]]), np.array([[[1.0, 1.0]]]))
    assert np.allclose(got[0, 0], [0, -1, 1, 0], atol=1e-5)


def test_rope_table_matches_a_direct_evaluation():
    cos, sin = O.rope_table(10000.0, np.arange(16), 8, O.F32)
    for p in (0, 3, 15):
        for i in range(4):
            ang = np.float32(p) * np.float32(10000.0) ** np.float32(-2.0 * i / 8)
            assert abs(cos[p, i] - math.cos(ang)) < 1e-5 and abs(sin[p, i] - math.sin(ang)) < 1e-5


# ---- activations: tk/src/kernels/mod.rs:304-335 ---------------------------------------------
def test_in_kernel_gelu_is_within_the_stated_error_of_erf_gelu():
    x = np.linspace(-6, 6, 2001)
    assert np.max(np.abs(O.gelu_as(x) - O.gelu_erf(x))) < 6 * 1.5e-7 * 6  # |x| * erf error
    assert np.allclose(O.silu(x), x / (1 + np.exp(-x)))
    assert abs(float(O.gelu_tanh(np.array(1.0))) - 0.841192) < 1e-5


def test_the_kernels_single_exponential_gelu_stays_within_1e_4_of_the_pinned_form():
    """The CUDA `gelu_f` evaluates x*Phi(x) as max(x,0) - |x| * 2^P(|x|); its
    coefficients are read from the kernel header and the form is replayed here in
    f32 against the pinned Abramowitz-Stegun form and against erf itself."""
    import pathlib
    import re

    src = (pathlib.Path(__file__).resolve().parent.parent / "svod_b200" / "csrc" / "common.cuh").read_text()
    coef = {k: float(v) for k, v in re.findall(r"constexpr float kGelu(\w+) = ([-+0-9.e]+)f;", src)}
    assert set(coef) == {"Clamp", "P1", "P2", "P3", "P4", "P5"}
    x = np.concatenate([np.linspace(-12, 12, 400001), [-1e4, 1e4, 0.0]]).astype(np.float32)
    a = np.minimum(np.abs(x), np.float32(coef["Clamp"]))
    p = np.full_like(x, np.float32(coef["P5"]))
    for k in ("P4", "P3", "P2", "P1"):
        p = (p * a + np.float32(coef[k])).astype(np.float32)
    p = (p * a - np.float32(1.0)).astype(np.float32)
    got = (np.maximum(x, 0) - a * np.exp2(p).astype(np.float32)).astype(np.float32)
    assert np.max(np.abs(got - O.gelu_as(x.astype(np.float64)))) < 1e-4
    inside = np.abs(x) <= 12
    assert np.max(np.abs(got - O.gelu_erf(x.astype(np.float64)))[inside]) < 5e-6
    # far outside the fitted range the result is x or 0 to within 5.5 * Q(5.5)
    assert abs(got[-3]) < 2e-7 and got[-2] == 1e4 and got[-1] == 0


# ---- the GEMM epilogue recipe: tk/src/test/unit/rows.rs:37-104 -------------------------------
EPILOGUES = [
    dict(bias=True), dict(residual=True), dict(bias=True, act=O.ACT_GELU),
    dict(bias=True, residual=True, act=O.ACT_SILU), dict(bias=True, act=O.ACT_SILU, gated=True),
    dict(residual=True, act=O.ACT_GELU, gated=True), dict(bias=True, residual=True, scale=0.5),
    dict(bias=True, act=O.ACT_SILU, gated=True, scale=-1.5),
]


def gemm_recipe(m, n, k, epi):
    """`gemm_inputs` of rows.rs:37-49 (seed 17; bias x2, residual x4)."""
    g = O.Lcg(17)
    halves = 2 if epi.get("gated") else 1
    a = g.rounded(O.BF16, m * k).reshape(m, k)
    w = g.rounded(O.BF16, halves * n * k).reshape(halves * n, k)
    bias = g.rounded(O.BF16, halves * n, lambda x: 2.0 * x) if epi.get("bias") else None
    res = g.rounded(O.BF16, m * n, lambda x: 4.0 * x).reshape(m, n) if epi.get("residual") else None
    return a, w, bias, res


@pytest.mark.parametrize("which", range(8))
def test_gemm_epilogues_match_a_scalar_restatement(which):
    """`gemm_reference` of rows.rs:51-75 written as scalar loops."""
    epi = EPILOGUES[which]
    m = n = k = 16
    a, w, bias, res = gemm_recipe(m, n, k, epi)
    got = O.linear(a, w, bias, epi.get("act", 0), epi.get("gated", False), res, epi.get("scale"), dtype=O.BF16)
    for i in range(m):
        for j in range(n):
            def half(h):
                row = h * n + j
                return float(np.dot(a[i], w[row])) + (bias[row] if bias is not None else 0.0)
            x = half(0)
            act = epi.get("act", 0)
            y = x if act == 0 else (0.5 * x * (1 + math.erf(x / math.sqrt(2))) if act == 1 else x / (1 + math.exp(-x)))
            if epi.get("gated"):
                y *= half(1)
            y *= float(np.float32(epi.get("scale", 1.0)))
            want = O.round_bf16(y + (res[i, j] if res is not None else 0.0))
            assert got[i, j] == want, (i, j)


# ---- the norm recipe: rows.rs:149-197 ---------------------------------------------------------
def norm_recipe(kind, rows, d, residual, bias, seed):
    g = O.Lcg(seed)
    x = g.rounded(O.BF16, rows * d, lambda v: 2.0 * v + 1.5).reshape(rows, d)
    r = g.rounded(O.BF16, rows * d).reshape(rows, d) if residual else None
    w = g.rounded(O.BF16, d, lambda v: 1.0 + 0.5 * v)
    b = g.rounded(O.BF16, d, lambda v: 0.5 * v) if (kind == "layer" and bias) else None
    return x, r, w, b


@pytest.mark.parametrize("kind,residual,bias", [("layer", False, True), ("layer", True, True), ("rms", True, False),
                                                 ("rms", False, False), ("layer", False, False)])
def test_norm_matches_a_scalar_restatement(kind, residual, bias):
    rows, d, eps = 5, 256, 1e-5
    x, r, w, b = norm_recipe(kind, rows, d, residual, bias, 5)
    got, gsum = O.norm_rows(kind, x, w, b, r, eps, O.BF16)
    for i in range(rows):
        row = [float(O.round_bf16(x[i, c] + (r[i, c] if r is not None else 0.0))) for c in range(d)]
        if residual:
            assert np.array_equal(gsum[i], np.array(row))
        mean = sum(row) / d if kind == "layer" else 0.0
        var = sum((v - mean) ** 2 for v in row) / d
        inv = 1.0 / math.sqrt(var + eps)
        for c in range(0, d, 17):
            y = (row[c] - mean) * inv * w[c] + (b[c] if b is not None else 0.0)
            assert got[i, c] == O.round_bf16(y)


# ---- the heads recipe: tk/src/test/unit/heads.rs:37-105 -------------------------------------------
def heads_recipe(cap, t, H, Hkv, d, q_norm, k_norm, rope, seed):
    g = O.Lcg(seed)
    slots, half = H + 2 * Hkv, d // 2
    qkv = g.rounded(O.BF16, cap * t * slots * d, lambda v: 3.0 * v).reshape(cap, t, slots * d)
    qw = g.rounded(O.BF16, d, lambda v: 1.0 + 0.5 * v) if q_norm else None
    kw = g.rounded(O.BF16, d, lambda v: 1.0 + 0.5 * v) if k_norm else None
    cos = sin = None
    if rope is not None:
        rows = cap * t if rope else t
        e = np.arange(rows * half)
        ang = (e // half) * 0.01 * (1.0 + (e % half))
        cos = O.round_bf16(np.cos(ang)).reshape(-1, t, half)
        sin = O.round_bf16(np.sin(ang)).reshape(-1, t, half)
    return qkv, qw, kw, cos, sin


@pytest.mark.parametrize("cap,t,H,Hkv,d,qn,kn,rope", [(2, 9, 4, 2, 64, True, True, False),
                                                      (2, 10, 4, 2, 128, True, True, True),
                                                      (2, 5, 2, 2, 64, False, False, False),
                                                      (2, 8, 4, 1, 64, True, False, None),
                                                      (2, 3, 2, 1, 32, False, False, None)])
def test_heads_matches_a_scalar_restatement(cap, t, H, Hkv, d, qn, kn, rope):
    qkv, qw, kw, cos, sin = heads_recipe(cap, t, H, Hkv, d, qn, kn, rope, 7)
    q, k, v = O.heads(qkv, H, Hkv, d, qw, kw, 1e-6, cos, sin, O.BF16)
    half, slots = d // 2, H + 2 * Hkv
    for b in range(cap):
        for i in range(0, t, 2):
            for slot in range(slots):
                x = [float(z) for z in qkv[b, i, slot * d:(slot + 1) * d]]
                which, head, w = (0, slot, qw) if slot < H else ((1, slot - H, kw) if slot < H + Hkv else (2, slot - H - Hkv, None))
                if w is not None:
                    inv = 1.0 / math.sqrt(sum(z * z for z in x) / d + 1e-6)
                    x = [z * inv * float(wc) for z, wc in zip(x, w)]
                if cos is not None and which < 2:
                    tb = b if cos.shape[0] > 1 else 0
                    x = [x[c] * cos[tb, i, c % half] - x[c + half] * sin[tb, i, c % half] if c < half
                         else x[c - half] * sin[tb, i, c % half] + x[c] * cos[tb, i, c % half] for c in range(d)]
                got = (q, k, v)[which][b, i, head]
                assert np.array_equal(got, O.round_bf16(np.array(x))), (b, i, slot)


# ---- the attention recipe: tk/src/test/unit/attention.rs:69-178 ----------------------------------
def attention_recipe(B, T, Tk, H, Hkv, D):
    g = O.Lcg(5)
    q = g.rounded(O.BF16, B * T * H * D).reshape(B, T, H, D)
    k = g.rounded(O.BF16, B * Tk * Hkv * D).reshape(B, Tk, Hkv, D)
    v = g.rounded(O.BF16, B * Tk * Hkv * D).reshape(B, Tk, Hkv, D)
    return q, k, v


def scalar_attention(q, k, v, hidden, scale):
    B, T, H, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    out = np.zeros((B, T, H, D))
    for b in range(B):
        for h in range(H):
            hk = h // (H // Hkv)
            for i in range(T):
                sc = [(-math.inf if hidden(b, i, j) else float(np.dot(q[b, i, h], k[b, j, hk])) * scale)
                      for j in range(Tk)]
                mx = max(sc)
                if mx == -math.inf:
                    continue
                w = [math.exp(s - mx) for s in sc]
                l = sum(w)
                acc = np.zeros(D)
                for j in range(Tk):
                    acc += w[j] * v[b, j, hk]
                out[b, i, h] = acc / l
    return out


@pytest.mark.parametrize("name", ["plain", "causal", "lens", "window", "key_mask", "segments", "every", "gqa"])
def test_attention_matches_the_reference_tests_direct_softmax(name):
    """The f64 `reference()` of tk/src/test/unit/attention.rs:102-178 as scalar
    loops, on the recipe's inputs (key mask hides (b+j)%5==2, segments of 40)."""
    B, T, Tk, H, Hkv, D = 2, 24, 30, 2, 2, 16
    if name == "gqa":
        H, Hkv = 4, 2
    q, k, v = attention_recipe(B, T, Tk, H, Hkv, D)
    scale = float(np.float32(1.0 / math.sqrt(D)))
    lens = [Tk, 7]
    key_mask = np.array([[(b + j) % 5 != 2 for j in range(Tk)] for b in range(B)])
    seg = np.array([[i - i % 10 for i in range(T)] for _ in range(B)])
    kw, conds = {}, []
    if name in ("causal", "every", "segments"):
        kw["causal"] = True
        conds.append(lambda b, i, j: j > i)
    if name in ("lens", "every"):
        kw["key_lens"] = np.array(lens)
        conds.append(lambda b, i, j: j >= lens[b])
    if name in ("window", "every"):
        kw["window"] = (5, 3)
        conds.append(lambda b, i, j: j + 5 < i or j > i + 3)
    if name in ("key_mask", "every"):
        kw["key_mask"] = key_mask
        conds.append(lambda b, i, j: not key_mask[b, j])
    if name in ("segments", "every"):
        kw["seg_start"] = seg
        conds.append(lambda b, i, j: j < seg[b, i])
    hidden = lambda b, i, j: any(c(b, i, j) for c in conds)
    want = scalar_attention(q, k, v, hidden, scale)
    got = O.attention(q, k, v, dtype=O.F32, **kw)
    assert np.max(np.abs(got - want)) < 1e-6


def test_a_fully_masked_batch_is_zeros_and_lse_is_minus_inf():
    q, k, v = attention_recipe(2, 8, 8, 2, 2, 16)
    m = np.ones((2, 8), dtype=bool)
    m[1] = False
    out, lse = O.attention(q, k, v, key_mask=m, dtype=O.BF16, return_lse=True)
    assert np.any(out[0] != 0) and np.all(out[1] == 0)
    assert np.all(np.isfinite(lse[0])) and np.all(np.isneginf(lse[1]))


def test_combine_splits_equals_unsplit_attention():
    q, k, v = attention_recipe(1, 4, 40, 2, 2, 16)
    want = O.attention(q, k, v, dtype=O.F32)
    scale = float(np.float32(0.25)) * math.log2(math.e)
    parts = []
    for lo, hi in [(0, 16), (16, 32), (32, 40)]:
        s = np.einsum("bihd,bjhd->bihj", q, k[:, lo:hi]) * scale
        m = s.max(-1)
        p = np.exp2(s - m[..., None])
        parts.append((np.einsum("bihj,bjhd->bihd", p, v[:, lo:hi]), m, p.sum(-1)))
    o = O.combine_splits(np.stack([p[0] for p in parts]), np.stack([p[1] for p in parts]),
                         np.stack([p[2] for p in parts]), dtype=O.F32)
    assert np.max(np.abs(o - want)) < 1e-6


def test_xlmr_position_ids():
    ids = np.array([[5, 6, 7, 1, 1], [1, 9, 1, 9, 9]])
    assert np.array_equal(O.xlmr_position_ids(ids, 1), [[2, 3, 4, 1, 1], [1, 2, 1, 3, 4]])


def test_l2_normalize_keeps_a_zero_row_zero():
    x = np.array([[3.0, 4.0], [0.0, 0.0]])
    y = O.l2_normalize(x)
    assert np.allclose(y[0], [0.6, 0.8]) and np.all(y[1] == 0)


# ---- cached reads: tk/src/test/unit/attention.rs:69-178 (`case`, `reference`) -----------------------
@pytest.mark.parametrize("t,tk,hhd,row_map,appended,lens,counted,biased", [
    (1, 100, (4, 2, 64), True, 1, [100, 37], False, False),
    (8, 64, (2, 2, 64), False, 8, [64, 20], True, True),
    (1, 7, (6, 6, 64), False, 1, [0, 7], False, False),
    (5, 96, (2, 2, 128), False, 1, [64, 96], False, True),
])
def test_cached_attention_matches_a_scalar_restatement(t, tk, hhd, row_map, appended, lens, counted, biased):
    """The oracle's `cache=` against loops written from the reference test's own
    f64 `reference`: head_start = kv_heads, lane b on cache row 2-b under a row
    map, masks on cached keys only, appended keys hidden past the lane's count."""
    B, rows = 2, 3
    H, Hkv, D = hhd
    g = O.Lcg(5)
    q = g.rounded(O.BF16, B * t * H * D).reshape(B, t, H, D)
    k = g.rounded(O.BF16, rows * tk * 3 * Hkv * D).reshape(rows, tk, 3 * Hkv, D)
    v = g.rounded(O.BF16, rows * tk * 3 * Hkv * D).reshape(rows, tk, 3 * Hkv, D)
    ka = g.rounded(O.BF16, B * appended * Hkv * D).reshape(B, appended, Hkv, D)
    va = g.rounded(O.BF16, B * appended * Hkv * D).reshape(B, appended, Hkv, D)
    bias = 2.0 * g.rounded(O.BF16, B * H * t * (tk + appended)).reshape(B, H, t, tk + appended) if biased else None
    rm = [rows - 1 - b for b in range(B)] if row_map else None
    seen = [max(appended - b % 3, 1) for b in range(B)] if counted else None
    cache = dict(head_start=Hkv, kv_heads=Hkv, row_map=rm, k_app=ka if appended else None,
                 v_app=va if appended else None, app_lens=seen)
    got = O.attention(q, k, v, key_lens=np.array(lens), bias=bias, cache=cache, dtype=O.F32)
    want = np.zeros_like(got)
    group, scale = H // Hkv, float(np.float32(1.0 / math.sqrt(D)))
    for b in range(B):
        row = rm[b] if rm else b
        sn = seen[b] if seen else appended
        for h in range(H):
            for i in range(t):
                sc, vals = [], []
                for j in range(tk + appended):
                    if j < tk:
                        if j >= lens[b]:
                            continue
                        kk, vv = k[row, j, Hkv + h // group], v[row, j, Hkv + h // group]
                    else:
                        if j - tk >= sn:
                            continue
                        kk, vv = ka[b, j - tk, h // group], va[b, j - tk, h // group]
                    sc.append(float(q[b, i, h] @ kk) * scale + (bias[b, h, i, j] if biased else 0.0))
                    vals.append(vv)
                if sc:
                    w = np.exp(np.array(sc) - max(sc))
                    want[b, i, h] = (w / w.sum()) @ np.array(vals)
    assert np.abs(got - want).max() < 1e-6


# ---- committed fixtures -----------------------------------------------------------------------------
def test_oracle_reproduces_the_committed_fixtures():
    """`tests/golden/ops_golden.npz` (written by tests/golden/make_golden.py):
    the oracle's outputs for seeded inputs, bit for bit."""
    from tests.golden import make_golden as G
    want, got = G.load(), G.build()
    fresh = {}
    for key, val in got.items():
        fresh[key[2:] if key.startswith("i_") else key] = val
    assert set(want) == set(fresh)
    for key in want:
        a = fresh[key]
        a = (a.astype(np.uint32) << 16).view(np.float32).astype(np.float64) if a.dtype == np.uint16 else a
        assert np.array_equal(a, want[key]), key


# --------------------------------------------------------------------------
# More of the reference's own known-answer tests, replayed on the oracle
# --------------------------------------------------------------------------


def ramp(count):
    """`ramp` of tensor/src/test/unit/attention_helpers.rs:80-82 (float32 arithmetic)."""
    i = np.arange(count, dtype=np.float32)
    return (np.sin(i * np.float32(0.37)) + i * np.float32(0.01)).astype(np.float32)


def test_layernorm_known_answer():
    """tensor/src/test/unit/nn.rs:428-446: rows [1,2,3,4] and [5,6,7,8], eps 1e-5:
    every row comes out with mean ~0 and variance ~1."""
    x = np.array([[1.0, 2.0, 3.0, 4.0], [5.0, 6.0, 7.0, 8.0]])
    y, _ = O.norm_rows("layer", x, np.ones(4), np.zeros(4), eps=1e-5, dtype=O.F32)
    for row in y:
        assert abs(row.mean()) < 1e-4 and abs(row.var() - 1.0) < 0.1
    # closed form: (x - 2.5) / sqrt(1.25 + 1e-5)
    assert np.allclose(y[0], (x[0] - 2.5) / np.sqrt(1.25 + 1e-5), atol=1e-6)


@pytest.mark.parametrize("theta,seq,hd", [(10_000.0, 8, 16), (100_000.0, 6, 8), (1_000_000.0, 5, 8), (64.0, 4, 4)])
def test_rope_table_matches_the_reference_host_loop(theta, seq, hd):
    """tensor/src/test/unit/attention_helpers.rs:19-32,88-104: inv_freq = theta^(-2i/d)
    formed in f64 and cast to f32, angle = s * inv_freq in f32, cos/sin in f32; 1e-5."""
    half = hd // 2
    inv = np.array([theta ** (-2.0 * i / hd) for i in range(half)], dtype=np.float32)
    ang = (np.arange(seq, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32)
    cos, sin = O.rope_table(theta, np.arange(seq), hd, O.F32)
    assert np.abs(np.asarray(cos).reshape(seq, half) - np.cos(ang)).max() < 1e-5
    assert np.abs(np.asarray(sin).reshape(seq, half) - np.sin(ang)).max() < 1e-5


@pytest.mark.parametrize("mask", [[1, 1, 1, 1, 1, 0], [1, 0, 0, 0, 0, 0], [1, 1, 1, 1, 1, 1], [0, 0, 0, 1, 1, 1]])
def test_masked_mean_matches_the_reference_host_loop(mask):
    """tensor/src/test/unit/attention_helpers.rs:66-76,487-505: sum over the masked
    tokens / max(count, 1e-9) on the `ramp` data, batch 2 x len 3 x depth 4; 1e-5."""
    data = ramp(2 * 3 * 4).reshape(2, 3, 4)
    m = np.array(mask, dtype=np.float32).reshape(2, 3)
    want = np.zeros((2, 4), dtype=np.float32)
    for b in range(2):
        count = max(float(m[b].sum()), 1e-9)
        for d in range(4):
            want[b, d] = sum(float(data[b, l, d]) * float(m[b, l]) for l in range(3)) / count
    got = O.pool(data, m > 0.5, "mean", normalize=False)
    assert np.abs(got - want).max() < 1e-5
    # cls / last-token pooling of the same tensor (attention_helpers.rs:507-520)
    assert np.array_equal(O.pool(data, None, "cls", normalize=False), data[:, 0].astype(np.float64))
    assert np.array_equal(O.pool(data, None, "last", lengths=np.array([3, 3]), normalize=False),
                          data[:, -1].astype(np.float64))


def test_embedding_known_answers():
    """tensor/src/test/unit/transformer.rs:51-100: rows of the table by index, 1-D,
    2-D and int64 indices (the oracle's lookup is `table[ids]`)."""
    w = np.arange(12, dtype=np.float64).reshape(3, 4)
    got = w[np.array([2, 0])]
    assert got[0, 0] == 8.0 and got[0, 3] == 11.0 and got[1, 0] == 0.0 and got[1, 3] == 3.0
    w2 = np.array([[0.0, 1.0], [2.0, 3.0], [4.0, 5.0], [6.0, 7.0]])
    got = w2[np.array([[0, 1, 2], [3, 2, 1]])]
    assert got.shape == (2, 3, 2) and got[0, 2, 0] == 4.0 and list(got[1, 0]) == [6.0, 7.0]
    got = w2[np.array([[3, 0], [1, 3]], dtype=np.int64)]
    assert list(got.reshape(-1)) == [6.0, 7.0, 0.0, 1.0, 2.0, 3.0, 6.0, 7.0]


def test_f16_scores_are_formed_in_wide_precision():
    """tensor/src/test/unit/transformer.rs:170-190: 64 products of 100*100 pass
    float16's range; scores formed wide keep the softmax finite and key 0 (ahead
    by 800 in score) takes every query to V[0] = 1."""
    q = O.round_to(O.F16, np.full((1, 2, 1, 64), 100.0))
    k = O.round_to(O.F16, np.stack([np.full(64, 100.0), np.full(64, 99.0)]).reshape(1, 2, 1, 64))
    v = O.round_to(O.F16, np.array([1.0, 100.0]).reshape(1, 2, 1, 1))
    # the oracle takes [B,T,H,D]; a 1-wide value head is padded to the key's head dim for the kernels,
    # the oracle itself has no such limit
    out = O.attention(q, k, np.repeat(v, 64, axis=-1), dtype=O.F16)
    assert np.isfinite(out).all() and np.abs(out - 1.0).max() < 1e-3
