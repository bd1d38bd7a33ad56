"""The compiled CPU restatement (`oracle/svod_oracle.c`) held to the pinned numpy
float64 restatement on seeded inputs, and to the reference's known answers
(tensor/src/test/unit/transformer.rs: rms_norm) where they are closed form.
CPU only."""
import numpy as np
import pytest

from oracle import c_oracle as C
from oracle import svod_oracle as O


@pytest.fixture(scope="module", autouse=True)
def built():
    C.build()
    C.load()


def r(rng, shape, dt, scale=1.0):
    return O.round_to(dt, rng.standard_normal(shape) * scale).astype(np.float32)


DT = [(O.BF16, C.BF16), (O.F16, C.F16)]


def test_rounding_matches_the_numpy_rounding_bit_for_bit():
    rng = np.random.default_rng(1)
    x = np.concatenate([rng.standard_normal(4096) * 10.0 ** rng.integers(-9, 5, 4096),
                        np.array([0.0, -0.0, 65504.0, 65520.0, 1e-8, 6e-8, 6.1e-5, 3.0e38])]).astype(np.float32)
    for odt, cdt in DT:
        got = x.copy()
        C.load().so_round(C._p(got), got.size, cdt)
        want = O.round_to(odt, x.astype(np.float64)).astype(np.float32)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("act", ["none", "gelu", "silu", "gelu_tanh"])
@pytest.mark.parametrize("gated", [False, True])
def test_linear_epilogues_match(act, gated):
    rng = np.random.default_rng(2)
    oact = dict(none=O.ACT_NONE, gelu=O.ACT_GELU, silu=O.ACT_SILU, gelu_tanh=O.ACT_GELU_TANH)[act]
    cact = dict(none=C.ACT_NONE, gelu=C.ACT_GELU, silu=C.ACT_SILU, gelu_tanh=C.ACT_GELU_TANH)[act]
    for odt, cdt in DT:
        m, n, k = 70, 52, 100  # ragged against the 4 x 4 blocks and the 8-wide vectors
        x, w, b = r(rng, (m, k), odt), r(rng, ((2 if gated else 1) * n, k), odt, 0.1), r(rng, ((2 if gated else 1) * n,), odt, 0.1)
        res = r(rng, (m, n), odt)
        got = C.linear(x, w, b, act=cact, gated=gated, residual=res, scale=0.5, dtype=cdt)
        want = O.linear(x, w, b, act=oact, gated=gated, residual=res, scale=0.5, dtype=odt)
        # f32 against f64 accumulation: at most one rounding step of the 16-bit type
        assert np.abs(got - want).max() <= 2.0 ** -7 * max(1.0, np.abs(want).max())
        assert np.mean(got == want) > 0.98


@pytest.mark.parametrize("kind", ["layer", "rms"])
@pytest.mark.parametrize("fused", [False, True])
def test_norms_match(kind, fused):
    rng = np.random.default_rng(3)
    for odt, cdt in DT:
        x, w, b = r(rng, (33, 100), odt), r(rng, (100,), odt), r(rng, (100,), odt)
        res = r(rng, (33, 100), odt) if fused else None
        got, gsum = C.norm_rows(kind, x, w, b if kind == "layer" else None, residual=res, eps=1e-5, dtype=cdt)
        want, wsum = O.norm_rows(kind, x, w, b if kind == "layer" else None, residual=res, eps=1e-5, dtype=odt)
        assert np.abs(got - want).max() <= 2.0 ** -6 and np.mean(got == want) > 0.98
        if fused:
            assert np.array_equal(gsum, np.asarray(wsum, dtype=np.float32))  # the rounded sum is exact


def test_rms_norm_known_answer():
    # x = [1,2,3,4], weight 1, eps 0: x / sqrt(7.5)
    x = np.array([[1.0, 2.0, 3.0, 4.0]], dtype=np.float32)
    got, _ = C.norm_rows("rms", x, np.ones(4, np.float32), eps=0.0, dtype=C.F32)
    assert np.allclose(got, x / np.sqrt(7.5), rtol=1e-6)


def test_heads_and_rope_table_match():
    rng = np.random.default_rng(4)
    for odt, cdt in DT:
        cos, sin = C.rope_table(1e6, np.arange(50), 64, cdt)
        ocos, osin = O.rope_table(1e6, np.arange(50), 64, odt)
        assert np.abs(cos - np.asarray(ocos).reshape(50, 32)).max() <= 2.0 ** -8
        assert np.abs(sin - np.asarray(osin).reshape(50, 32)).max() <= 2.0 ** -8
        qkv, qw, kw = r(rng, (2, 50, 8 * 64), odt), r(rng, (64,), odt), r(rng, (64,), odt)
        got = C.heads(qkv, 4, 2, 64, qw, kw, 1e-6, cos, sin, cdt)
        want = O.heads(qkv, 4, 2, 64, qw, kw, 1e-6, cos.reshape(1, 50, 1, 32), sin.reshape(1, 50, 1, 32), odt)
        for g, w_ in zip(got[:2], want[:2]):
            assert np.abs(g - w_).max() <= 2e-2
        assert np.array_equal(got[2], np.asarray(want[2], dtype=np.float32))  # v is a copy


@pytest.mark.parametrize("kw", [dict(), dict(causal=True), dict(key_lens=[50, 0]), dict(window=(5, 3), key_lens=[20, 50]),
                                dict(causal=True, key_lens=[7, 50])],
                         ids=["plain", "causal", "lens+empty", "window+lens", "causal+lens"])
def test_attention_matches_within_the_16_bit_tolerance(kw):
    """The C code rounds the softmax weights to the tensor type before `@ V`, as
    the reference's graph path does (tensor/src/transformer.rs:526-530); the
    numpy restatement keeps them exact, so the comparison is by tolerance."""
    rng = np.random.default_rng(5)
    for odt, cdt in DT:
        q, k, v = r(rng, (2, 50, 4, 64), odt), r(rng, (2, 50, 2, 64), odt), r(rng, (2, 50, 2, 64), odt)
        got = C.attention(q, k, v, dtype=cdt, **kw)
        want = O.attention(q, k, v, dtype=odt, **kw)
        assert np.abs(got - want).max() < 2e-2
        assert np.abs(got - want).mean() / np.abs(want).mean() < 5e-3
        if "key_lens" in kw and 0 in kw["key_lens"]:
            assert not got[kw["key_lens"].index(0)].any()  # no visible key -> zeros


def test_qwen3_layers_match_the_numpy_stack():
    rng = np.random.default_rng(6)
    dt, D, H, Hkv, hd, F, L = O.BF16, 256, 4, 2, 64, 384, 96
    w = lambda *s: r(rng, s, dt, 0.05)
    lps = [dict(in_w=1 + w(D), qkv_w=w((H + 2 * Hkv) * hd, D), qn_w=1 + w(hd), kn_w=1 + w(hd), o_w=w(D, H * hd),
                post_w=1 + w(D), gu_w=w(2 * F, D), down_w=w(D, F)) for _ in range(2)]
    lps = [{k: O.round_to(dt, v).astype(np.float32) for k, v in lp.items()} for lp in lps]
    hidden = r(rng, (2, L, D), dt)
    got = C.qwen3_layers(hidden, lps, heads_n=H, kv_heads=Hkv, head_dim=hd, dtype=C.BF16)
    x = hidden.astype(np.float64)
    cos, sin = O.rope_table(1e6, np.arange(L), hd, dt)
    for lp in lps:
        xn, _ = O.norm_rows("rms", x, lp["in_w"], eps=1e-6, dtype=dt)
        q, k, v = O.heads(O.linear(xn, lp["qkv_w"], dtype=dt), H, Hkv, hd, lp["qn_w"], lp["kn_w"], 1e-6, cos, sin, dt)
        a = O.attention(q, k, v, causal=True, dtype=dt).reshape(2, L, H * hd)
        x = O.linear(a, lp["o_w"], residual=x, dtype=dt)
        hn, _ = O.norm_rows("rms", x, lp["post_w"], eps=1e-6, dtype=dt)
        x = O.linear(O.linear(hn, lp["gu_w"], act=O.ACT_SILU, gated=True, dtype=dt), lp["down_w"], residual=x, dtype=dt)
    assert np.abs(got - x).max() < 4e-2 and np.abs(got - x).mean() / np.abs(x).mean() < 5e-3


def test_attention_with_a_bool_key_mask_matches():
    """`KeyMask::Bool` with holes (the `(b+j)%5 != 2` mask of tk/src/test/unit/attention.rs:69-99)
    and a batch lane with no visible key."""
    rng = np.random.default_rng(7)
    for odt, cdt in DT:
        q, k, v = r(rng, (3, 40, 4, 64), odt), r(rng, (3, 40, 2, 64), odt), r(rng, (3, 40, 2, 64), odt)
        mask = np.array([[(b + j) % 5 != 2 for j in range(40)] for b in range(3)])
        mask[2] = False
        for kw in (dict(), dict(window=(6, 2))):
            got = C.attention(q, k, v, key_mask=mask, dtype=cdt, **kw)
            want = O.attention(q, k, v, key_mask=mask, dtype=odt, **kw)
            assert np.abs(got - want).max() < 2e-2
            assert np.abs(got - want).mean() / np.abs(want).mean() < 5e-3
            assert not got[2].any()


def test_rope_in_the_projection_store_matches():
    rng = np.random.default_rng(8)
    for odt, cdt in DT:
        B, T, K, H, hd = 2, 30, 48, 3, 16
        x, w, b = r(rng, (B, T, K), odt), r(rng, (H * hd + 20, K), odt, 0.2), r(rng, (H * hd + 20,), odt, 0.2)
        cos, sin = C.rope_table(1e4, np.arange(T), hd, cdt)
        got = C.linear_rope(x, w, cos, sin, H, hd, bias=b, dtype=cdt)
        want = O.linear(x, w, b, rope=(cos, sin, H, hd), dtype=odt)
        assert np.abs(got - want).max() <= 2.0 ** -7 * max(1.0, np.abs(want).max())
        assert np.mean(got == want) > 0.97


def test_xlmr_layers_match_the_numpy_stack():
    rng = np.random.default_rng(9)
    dt, D, H, F, L, B = O.F16, 128, 4, 256, 48, 2
    w = lambda *s: r(rng, s, dt, 0.05)
    lps = []
    for _ in range(2):
        lp = {k: w(*s) for k, s in dict(q_w=(D, D), q_b=(D,), k_w=(D, D), k_b=(D,), v_w=(D, D), v_b=(D,), o_w=(D, D),
                                        o_b=(D,), fi_w=(F, D), fi_b=(F,), fo_w=(D, F), fo_b=(D,), ln1_b=(D,),
                                        ln2_b=(D,)).items()}
        lp["ln1_w"], lp["ln2_w"] = O.round_to(dt, 1 + w(D)).astype(np.float32), O.round_to(dt, 1 + w(D)).astype(np.float32)
        lps.append(lp)
    hidden = r(rng, (B, L, D), dt)
    mask = np.arange(L)[None, :] < np.array([L, 19])[:, None]
    got = C.xlmr_layers(hidden, lps, mask, heads_n=H, dtype=C.F16)
    h = hidden.astype(np.float64)
    hd = D // H
    for lp in lps:
        q = O.linear(h, lp["q_w"], lp["q_b"], dtype=dt).reshape(B, L, H, hd)
        k = O.linear(h, lp["k_w"], lp["k_b"], dtype=dt).reshape(B, L, H, hd)
        v = O.linear(h, lp["v_w"], lp["v_b"], dtype=dt).reshape(B, L, H, hd)
        a = O.attention(q, k, v, key_mask=mask, dtype=dt).reshape(B, L, D)
        x = O.linear(a, lp["o_w"], lp["o_b"], residual=h, dtype=dt)
        h, _ = O.norm_rows("layer", x, lp["ln1_w"], lp["ln1_b"], eps=1e-5, dtype=dt)
        y = O.linear(h, lp["fi_w"], lp["fi_b"], act=O.ACT_GELU, dtype=dt)
        x = O.linear(y, lp["fo_w"], lp["fo_b"], residual=h, dtype=dt)
        h, _ = O.norm_rows("layer", x, lp["ln2_w"], lp["ln2_b"], eps=1e-5, dtype=dt)
    live = mask[..., None] & np.ones((1, 1, D), dtype=bool)
    assert np.abs(got - h)[live].max() < 2e-2 and np.abs(got - h)[live].mean() / np.abs(h[live]).mean() < 5e-3


def test_modernbert_layers_match_the_numpy_stack():
    rng = np.random.default_rng(10)
    dt, D, H, F, L, B = O.BF16, 128, 4, 192, 200, 2
    w = lambda *s: r(rng, s, dt, 0.05)
    one = lambda n: O.round_to(dt, 1 + w(n)).astype(np.float32)
    lps = [dict(attn_ln_w=None if i == 0 else one(D), qkv_w=w(3 * D, D), o_w=w(D, D), mlp_ln_w=one(D),
                wi_w=w(2 * F, D), wo_w=w(D, F)) for i in range(4)]
    hidden = r(rng, (B, L, D), dt)
    mask = np.arange(L)[None, :] < np.array([L, 77])[:, None]
    got = C.modernbert_layers(hidden, lps, mask, heads_n=H, dtype=C.BF16)
    h = hidden.astype(np.float64)
    hd = D // H
    tabs = {True: O.rope_table(160000.0, np.arange(L), hd, dt), False: O.rope_table(10000.0, np.arange(L), hd, dt)}
    for li, lp in enumerate(lps):
        glob = li % 3 == 0
        cos, sin = tabs[glob]
        xn = h if lp["attn_ln_w"] is None else O.norm_rows("layer", h, lp["attn_ln_w"], eps=1e-5, dtype=dt)[0]
        qkv = O.linear(xn, lp["qkv_w"], rope=(cos, sin, 2 * H, hd), dtype=dt)
        a = O.attention_packed(qkv, H, H, key_mask=mask, window=None if glob else (64, 64), dtype=dt).reshape(B, L, D)
        h = O.linear(a, lp["o_w"], residual=h, dtype=dt)
        hn, _ = O.norm_rows("layer", h, lp["mlp_ln_w"], eps=1e-5, dtype=dt)
        h = O.linear(O.linear(hn, lp["wi_w"], act=O.ACT_GELU, gated=True, dtype=dt), lp["wo_w"], residual=h, dtype=dt)
    live = mask[..., None] & np.ones((1, 1, D), dtype=bool)
    assert np.abs(got - h)[live].max() < 4e-2 and np.abs(got - h)[live].mean() / np.abs(h[live]).mean() < 5e-3
    # the layer index decides global / local: starting at layer 1 the first layer is windowed
    one_layer = C.modernbert_layers(hidden, lps[1:2], mask, heads_n=H, first_layer=1, dtype=C.BF16)
    as_global = C.modernbert_layers(hidden, lps[1:2], mask, heads_n=H, first_layer=0, dtype=C.BF16)
    assert not np.array_equal(one_layer, as_global)
