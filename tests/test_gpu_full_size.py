"""GPU parity of the three encoder stacks at their full widths and depths: the
benchmark configurations' real layer shapes (hidden size, heads, FFN, layer
count, sequence length, dtype, masks) on a reduced batch, seeded weights shared
bit for bit with the compiled CPU restatement (`oracle/svod_oracle.c`, held to
the pinned numpy restatement by `tests/test_c_oracle_cpu.py`).

Three comparisons per stack:

* op by op, in every layer: each operator of the GPU stack (norm, projection
  with its epilogue, attention prologue, attention, ...) is fed the ORACLE's
  input of that operator and compared with the oracle's output at the 16-bit
  operator tolerance: max-abs 2e-2 relative to `max(1, max|want|)` and mean-rel
  5e-3. Every full-size kernel the benchmark runs is on this path, at the
  benchmark's shapes.
* layer by layer: layer `l` of the GPU stack, as the stack runs it, on the
  oracle's hidden states after layer `l-1`. A layer chains eight roundings to
  16 bits, and two correct implementations differ by a unit in the last place
  on a fraction of the values at each of them: the bound is LAYER_MEAN_REL.
* end to end: embeddings -> all layers -> final norm -> pooling -> L2 with no
  help from the oracle. Over a deep 16-bit stack the drift compounds (the f32 C
  restatement and the float64 numpy one differ by mean-rel 1.2e-2 after 28
  Qwen3 layers at this width), so the bound on hidden states is DRIFT_MEAN_REL;
  the pooled unit-norm rows are held to max-abs 2e-2 and to a cosine distance.

The embedding tables keep the full vocabulary: they are drawn on the device and
only the rows the ids select travel to the host for the oracle.
"""
import numpy as np
import pytest
import torch

from oracle import c_oracle as C
from oracle import svod_oracle as O
from svod_b200 import encoders as E
from svod_b200 import ops
from tests.util import host, max_abs, mean_rel

pytestmark = pytest.mark.gpu

# bounds of a layer's and a whole stack's chain of 16-bit roundings (see the module docstring)
LAYER_MEAN_REL = 1.5e-2
DRIFT_MEAN_REL = 3e-2


@pytest.fixture(scope="module", autouse=True)
def built():
    C.build()
    C.load()
    C.use_all_cores()


class Weights:
    """Seeded N(mean, sigma) tensors rounded to the stack's 16-bit type, as a
    CUDA tensor for the stack and as float32 host values for the oracle."""

    def __init__(self, seed, dtype):
        self.g = torch.Generator().manual_seed(seed)
        self.dtype = dtype

    def __call__(self, *shape, sigma=0.02, mean=0.0):
        t = (torch.randn(*shape, generator=self.g) * sigma + mean).to(self.dtype)
        return t.cuda(), t.float().numpy()


def split(pairs):
    return {k: v[0] for k, v in pairs.items()}, {k: v[1] for k, v in pairs.items()}


class Worst:
    """Keeps the worst errors seen per operator name and asserts each comparison."""

    def __init__(self, stack):
        self.stack, self.seen = stack, {}

    def check(self, op, li, got, want, live=None, mean_rel_bound=5e-3):
        # the error measures of tests.util, taken on the device (the tensors are large):
        # max|got - want| and mean|got - want| / mean|want| over the live rows
        g = got.detach().double()
        w_ = torch.from_numpy(np.ascontiguousarray(want)).cuda().double()
        assert g.shape == w_.shape, (op, tuple(g.shape), tuple(w_.shape))
        if live is not None:
            rows = torch.from_numpy(np.ascontiguousarray(live[..., 0])).cuda()
            g, w_ = g[rows], w_[rows]
        err = (g - w_).abs()
        ma, mr = float(err.max()), float(err.mean() / w_.abs().mean())
        bound = 2e-2 * max(1.0, float(w_.abs().max()))
        assert ma <= bound and mr < mean_rel_bound, \
            f"{self.stack} layer {li} {op}: max-abs {ma:.3e} (bound {bound:.3e}), mean-rel {mr:.3e} (bound {mean_rel_bound})"
        a, b = self.seen.get(op, (0.0, 0.0))
        self.seen[op] = (max(a, ma), max(b, mr))

    def report(self):
        for op, (ma, mr) in self.seen.items():
            print(f"{self.stack} {op}: worst max-abs {ma:.3e}, worst mean-rel {mr:.3e}")


def up(x, dtype):
    """Oracle values (already rounded to the 16-bit type) as a CUDA tensor."""
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(dtype).cuda()


def pooled_check(name, got, want, hidden_got, hidden_want, live=None):
    got, want = host(got), np.asarray(want, dtype=np.float64)
    hg, hw = (host(hidden_got), hidden_want) if live is None else (host(hidden_got)[live], hidden_want[live])
    cos = (got * want).sum(-1) / (np.linalg.norm(got, axis=-1) * np.linalg.norm(want, axis=-1))
    report = (f"{name} end to end: hidden max-abs {max_abs(hg, hw):.3e} mean-rel {mean_rel(hg, hw):.3e}; "
              f"pooled max-abs {max_abs(got, want):.3e} mean-rel {mean_rel(got, want):.3e} min cosine {cos.min():.6f}")
    print(report)
    assert max_abs(got, want) < 2e-2, report
    assert mean_rel(hg, hw) < DRIFT_MEAN_REL, report
    assert cos.min() > 0.999, report
    assert np.allclose(np.linalg.norm(got, axis=-1), 1.0, atol=1e-4)


def test_qwen3_full_width_full_depth_row():
    """Qwen3-0.6B shape: 28 layers, hidden 1024, 16 query / 8 KV heads x 128, FFN 3072, bf16, causal,
    one full-length row of 4096 tokens (the benchmark's row length), last-token pooling."""
    cfg = E.Qwen3Config()
    D, H, Hkv, hd, F, L = 1024, 16, 8, 128, 3072, 4096
    dt, cdt, eps = torch.bfloat16, C.BF16, cfg.rms_norm_eps
    wt = Weights(4000, dt)
    dl, hl = [], []
    for _ in range(cfg.num_hidden_layers):
        d_, h_ = split(dict(in_w=wt(D, mean=1.0), qkv_w=wt((H + 2 * Hkv) * hd, D), qn_w=wt(hd, mean=1.0),
                            kn_w=wt(hd, mean=1.0), o_w=wt(D, H * hd), post_w=wt(D, mean=1.0), gu_w=wt(2 * F, D),
                            down_w=wt(D, F)))
        dl.append(d_), hl.append(h_)
    norm_d, norm_h = wt(D, mean=1.0)
    embed = (torch.randn(cfg.vocab_size, D, generator=torch.Generator(device="cuda").manual_seed(4001), device="cuda")
             * 0.02).to(dt)
    ids = torch.randint(0, cfg.vocab_size, (1, L), generator=wt.g, dtype=torch.int32)
    lengths = np.array([L], dtype=np.int32)
    m = E.Qwen3Embedder(cfg, dict(embed=embed, layers=dl, norm_w=norm_d))
    # the oracle's rotation tables (f32 recipe on the host) on both sides
    cos, sin = C.rope_table(cfg.rope_theta, np.arange(L), hd, cdt)
    rope = tuple(up(t, dt).view(1, L, 1, hd // 2) for t in (cos, sin))

    w = Worst("qwen3")
    x = embed[ids.long().cuda()].float().cpu().numpy()
    for li, (lp, dp) in enumerate(zip(hl, dl)):
        # the oracle's layer, operator by operator (model/src/qwen3/decoder_layer.rs:55-65)
        xn, _ = C.norm_rows("rms", x, lp["in_w"], eps=eps, dtype=cdt)
        qkv = C.linear(xn, lp["qkv_w"], dtype=cdt)
        q, k, v = C.heads(qkv, H, Hkv, hd, lp["qn_w"], lp["kn_w"], eps, cos, sin, cdt)
        a = C.attention(q, k, v, causal=True, dtype=cdt)
        h = C.linear(a.reshape(1, L, H * hd), lp["o_w"], residual=x, dtype=cdt)
        hn, _ = C.norm_rows("rms", h, lp["post_w"], eps=eps, dtype=cdt)
        g = C.linear(hn, lp["gu_w"], act=C.ACT_SILU, gated=True, dtype=cdt)
        x_next = C.linear(g, lp["down_w"], residual=h, dtype=cdt)
        # each GPU operator on the oracle's input of that operator
        X, XN, A, Hh, HN, G = (up(t, dt) for t in (x, xn, a, h, hn, g))
        prologue = ops.Qkv(H, Hkv, hd, dp["qn_w"], dp["kn_w"], eps, rope)
        w.check("rms_norm", li, ops.rms_norm(X, dp["in_w"], eps), xn)
        w.check("linear qkv", li, ops.linear(XN, dp["qkv_w"]), qkv)
        gq, gk, gv = ops.heads(up(qkv, dt), prologue)
        w.check("heads q", li, gq, q), w.check("heads k", li, gk, k)
        assert torch.equal(gv, up(v, dt))
        packed = np.concatenate([t.reshape(1, L, -1) for t in (q, k, v)], axis=-1)
        w.check("linear qkv + prologue in the store", li, ops.linear(XN, dp["qkv_w"], ops.Linear(qkv=prologue)), packed)
        w.check("attention", li, ops.attention(up(q, dt), up(k, dt), up(v, dt), ops.Attn(causal=True)), a)
        w.check("attention_packed", li, ops.attention_packed(up(packed, dt), H, Hkv, ops.Attn(causal=True)), a)
        w.check("linear o + residual", li, ops.linear(A.view(1, L, H * hd), dp["o_w"], ops.Linear(residual=X)), h)
        w.check("rms_norm post", li, ops.rms_norm(Hh, dp["post_w"], eps), hn)
        w.check("linear gate/up silu", li, ops.linear(HN, dp["gu_w"], ops.Linear(act=ops.Act.SILU, gated=True)), g)
        w.check("linear down + residual", li, ops.linear(G, dp["down_w"], ops.Linear(residual=Hh)), x_next)
        # the layer as the stack runs it, both op sequences
        for fused in (True, False):
            m.fused_prologue = fused
            w.check("layer (prologue in the store)" if fused else "layer (reference op sequence)", li,
                    m.run_layers(X, rope=rope, start=li, stop=li + 1), x_next, mean_rel_bound=LAYER_MEAN_REL)
        x = x_next
    w.report()
    ops.device_status()

    m.fused_prologue = True
    want_hidden, _ = C.norm_rows("rms", x, norm_h, eps=eps, dtype=cdt)
    want = O.pool(want_hidden, None, "last", lengths=lengths)
    hgot = m.hidden(ids.cuda(), rope=rope)
    got = ops.pool(hgot, torch.from_numpy(lengths).cuda(), ops.POOL_LAST)
    pooled_check("qwen3", got, want, hgot, want_hidden)
    # the stack's own device-built tables and its one-call forward
    got2 = m.forward(ids.cuda(), torch.from_numpy(lengths).cuda())
    assert max_abs(host(got2), want) < 2e-2
    ops.device_status()


def test_xlm_roberta_large_full_width_full_depth_rows():
    """XLM-RoBERTa-large shape (BGE-M3 layout): 24 post-LN layers, hidden 1024, 16 heads x 64, FFN 4096
    erf-GELU, fp16, rows of 512 with lengths drawn from [64, 512] behind a padding mask, CLS pooling."""
    cfg = E.XlmRobertaConfig()
    D, H, F, L, B = 1024, 16, 4096, 512, 4
    hd = D // H
    dt, cdt, eps = torch.float16, C.F16, cfg.layer_norm_eps
    wt = Weights(3000, dt)
    dl, hl = [], []
    for _ in range(cfg.num_hidden_layers):
        d_, h_ = split(dict(q_w=wt(D, D), q_b=wt(D), k_w=wt(D, D), k_b=wt(D), v_w=wt(D, D), v_b=wt(D), o_w=wt(D, D),
                            o_b=wt(D), ln1_w=wt(D, mean=1.0), ln1_b=wt(D), fi_w=wt(F, D), fi_b=wt(F), fo_w=wt(D, F),
                            fo_b=wt(D), ln2_w=wt(D, mean=1.0), ln2_b=wt(D)))
        dl.append(d_), hl.append(h_)
    gd = torch.Generator(device="cuda").manual_seed(3001)
    word = (torch.randn(cfg.vocab_size, D, generator=gd, device="cuda") * 0.02).to(dt)
    pos_d, pos_h = wt(cfg.max_position_embeddings, D)
    type_d, type_h = wt(1, D)
    elw_d, elw_h = wt(D, mean=1.0)
    elb_d, elb_h = wt(D)
    rng = np.random.default_rng(3002)
    lens = np.concatenate([[L], rng.integers(64, L + 1, B - 1)])
    mask = np.arange(L)[None, :] < lens[:, None]
    ids = rng.integers(2, cfg.vocab_size, (B, L))  # never the padding id inside a row (position ids count non-pad tokens)
    ids[~mask] = cfg.pad_token_id
    m = E.XlmRobertaEncoder(cfg, dict(word=word, pos=pos_d, type=type_d, emb_ln_w=elw_d, emb_ln_b=elb_d, layers=dl))
    I, M = torch.from_numpy(ids).cuda(), torch.from_numpy(mask).cuda()
    live = mask[..., None] & np.ones((1, 1, D), dtype=bool)   # real tokens; `check` selects rows by live[..., 0]
    live_f = live_3 = live

    w = Worst("xlm-r")
    rows = word[I].float().cpu().numpy().astype(np.float64)
    e = O.round_to(O.F16, O.round_to(O.F16, rows + pos_h[O.xlmr_position_ids(ids, cfg.pad_token_id)]) + type_h[0])
    ge = ops.embed(I, word, pos_d, type_d, cfg.pad_token_id)
    assert np.array_equal(host(ge), e)                       # gather + the two rounded adds: exact
    x, _ = C.norm_rows("layer", e, elw_h, elb_h, eps=eps, dtype=cdt)
    w.check("embedding layer_norm", -1, ops.layer_norm(ge, elw_d, elb_d, eps), x)
    keys = ops.KeyMask.Bool(M)
    for li, (lp, dp) in enumerate(zip(hl, dl)):
        # the oracle's layer, operator by operator (model/src/xlm_roberta/encoder_layer.rs:45-49)
        q = C.linear(x, lp["q_w"], lp["q_b"], dtype=cdt)
        k = C.linear(x, lp["k_w"], lp["k_b"], dtype=cdt)
        v = C.linear(x, lp["v_w"], lp["v_b"], dtype=cdt)
        a = C.attention(*(t.reshape(B, L, H, hd) for t in (q, k, v)), key_mask=mask, dtype=cdt).reshape(B, L, D)
        o = C.linear(a, lp["o_w"], lp["o_b"], residual=x, dtype=cdt)
        h1, _ = C.norm_rows("layer", o, lp["ln1_w"], lp["ln1_b"], eps=eps, dtype=cdt)
        f = C.linear(h1, lp["fi_w"], lp["fi_b"], act=C.ACT_GELU, dtype=cdt)
        o2 = C.linear(f, lp["fo_w"], lp["fo_b"], residual=h1, dtype=cdt)
        x_next, _ = C.norm_rows("layer", o2, lp["ln2_w"], lp["ln2_b"], eps=eps, dtype=cdt)
        X, A, O1, H1, Ff, O2 = (up(t, dt) for t in (x, a, o, h1, f, o2))
        packed = np.concatenate([q, k, v], axis=-1)
        w.check("linear qkv + bias (one fused projection)", li, ops.linear(X, dp["qkv_w"], ops.Linear(bias=dp["qkv_b"])),
                packed, live_3)
        w.check("attention_packed, bool key mask", li,
                ops.attention_packed(up(packed, dt), H, H, ops.Attn(keys=keys)).view(B, L, D), a, live)
        w.check("linear o + bias + residual", li, ops.linear(A, dp["o_w"], ops.Linear(bias=dp["o_b"], residual=X)), o, live)
        w.check("layer_norm 1", li, ops.layer_norm(O1, dp["ln1_w"], dp["ln1_b"], eps), h1, live)
        w.check("linear ffn-in + bias + erf-gelu", li,
                ops.linear(H1, dp["fi_w"], ops.Linear(bias=dp["fi_b"], act=ops.Act.GELU)), f, live_f)
        w.check("linear ffn-out + bias + residual", li, ops.linear(Ff, dp["fo_w"], ops.Linear(bias=dp["fo_b"], residual=H1)),
                o2, live)
        w.check("layer_norm 2", li, ops.layer_norm(O2, dp["ln2_w"], dp["ln2_b"], eps), x_next, live)
        w.check("layer", li, m.run_layers(X, M, start=li, stop=li + 1), x_next, live, mean_rel_bound=LAYER_MEAN_REL)
        x = x_next
    w.report()
    ops.device_status()

    want = O.pool(x, mask, "cls")
    hgot = m.hidden(I, M)
    got = m.forward(I, M)
    pooled_check("xlm-r", got, want, hgot, x, live)
    ops.device_status()


def test_modernbert_base_full_width_full_depth_rows():
    """ModernBERT-base shape: 22 pre-LN layers (every third global, the rest a 128-token window), hidden 768,
    12 heads x 64, GeGLU 1152, RoPE in the projection's store, bf16, rows of 8192 with lengths from
    [2048, 8192] behind a padding mask, mean pooling."""
    cfg = E.ModernBertConfig()
    D, H, F, L, B = 768, 12, 1152, 8192, 2
    hd = D // H
    dt, cdt, eps = torch.bfloat16, C.BF16, cfg.norm_eps
    wt = Weights(5000, dt)
    dl, hl = [], []
    for i in range(cfg.num_hidden_layers):
        d_, h_ = split(dict(qkv_w=wt(3 * D, D), o_w=wt(D, D), mlp_ln_w=wt(D, mean=1.0), wi_w=wt(2 * F, D),
                            wo_w=wt(D, F)))
        d_["attn_ln_w"], h_["attn_ln_w"] = (None, None) if i == 0 else wt(D, mean=1.0)
        dl.append(d_), hl.append(h_)
    gd = torch.Generator(device="cuda").manual_seed(5001)
    embed = (torch.randn(cfg.vocab_size, D, generator=gd, device="cuda") * 0.02).to(dt)
    eln_d, eln_h = wt(D, mean=1.0)
    fln_d, fln_h = wt(D, mean=1.0)
    rng = np.random.default_rng(5002)
    lens = np.array([L, int(rng.integers(2048, L + 1))])
    mask = np.arange(L)[None, :] < lens[:, None]
    ids = rng.integers(0, cfg.vocab_size, (B, L)).astype(np.int32)
    m = E.ModernBertEncoder(cfg, dict(embed=embed, emb_ln_w=eln_d, layers=dl, final_ln_w=fln_d))
    tabs_h, tabs = {}, {}
    for is_global, theta in ((True, cfg.global_rope_theta), (False, cfg.local_rope_theta)):
        tabs_h[is_global] = C.rope_table(theta, np.arange(L), hd, cdt)
        tabs[is_global] = tuple(up(t, dt).view(1, L, 1, hd // 2) for t in tabs_h[is_global])
    m._rope[L] = tabs
    I, M = torch.from_numpy(ids).cuda(), torch.from_numpy(mask).cuda()
    live = mask[..., None] & np.ones((1, 1, D), dtype=bool)   # real tokens; `check` selects rows by live[..., 0]
    live_f = live_3 = live
    half = cfg.local_attention // 2

    w = Worst("modernbert")
    x, _ = C.norm_rows("layer", embed[I.long()].float().cpu().numpy(), eln_h, eps=eps, dtype=cdt)
    w.check("embedding layer_norm", -1, ops.layer_norm(ops.embed(I, embed), eln_d, None, eps), x)
    keys = ops.KeyMask.Bool(M)
    for li, (lp, dp) in enumerate(zip(hl, dl)):
        # the oracle's layer, operator by operator (model/src/modernbert/encoder_layer.rs:52-60)
        is_global = li % cfg.global_attn_every_n_layers == 0
        window = None if is_global else (half, half)
        cos, sin = tabs_h[is_global]
        xn = x if lp["attn_ln_w"] is None else C.norm_rows("layer", x, lp["attn_ln_w"], eps=eps, dtype=cdt)[0]
        qkv = C.linear_rope(xn, lp["qkv_w"], cos, sin, 2 * H, hd, dtype=cdt)
        q, k, v = (qkv[..., i * D:(i + 1) * D].reshape(B, L, H, hd) for i in range(3))
        a = C.attention(q, k, v, key_mask=mask, window=window, dtype=cdt).reshape(B, L, D)
        h = C.linear(a, lp["o_w"], residual=x, dtype=cdt)
        hn, _ = C.norm_rows("layer", h, lp["mlp_ln_w"], eps=eps, dtype=cdt)
        g = C.linear(hn, lp["wi_w"], act=C.ACT_GELU, gated=True, dtype=cdt)
        x_next = C.linear(g, lp["wo_w"], residual=h, dtype=cdt)
        X, XN, A, Hh, HN, G = (up(t, dt) for t in (x, xn, a, h, hn, g))
        kind = "global" if is_global else "local"
        if lp["attn_ln_w"] is not None:
            w.check("layer_norm attn", li, ops.layer_norm(X, dp["attn_ln_w"], None, eps), xn, live)
        rot = ops.Rotary(*tabs[is_global], 2 * H, hd)
        w.check("linear qkv + rope in the store", li, ops.linear(XN, dp["qkv_w"], ops.Linear(rope=rot)), qkv, live_3)
        w.check(f"attention_packed, bool key mask, {kind}", li,
                ops.attention_packed(up(qkv, dt), H, H, ops.Attn(keys=keys, window=window)).view(B, L, D), a, live)
        w.check("linear o + residual", li, ops.linear(A, dp["o_w"], ops.Linear(residual=X)), h, live)
        w.check("layer_norm mlp", li, ops.layer_norm(Hh, dp["mlp_ln_w"], None, eps), hn, live)
        w.check("linear wi geglu", li, ops.linear(HN, dp["wi_w"], ops.Linear(act=ops.Act.GELU, gated=True)), g, live_f)
        w.check("linear wo + residual", li, ops.linear(G, dp["wo_w"], ops.Linear(residual=Hh)), x_next, live)
        w.check(f"layer ({kind})", li, m.run_layers(X, M, start=li, stop=li + 1), x_next, live,
                mean_rel_bound=LAYER_MEAN_REL)
        x = x_next
    w.report()
    ops.device_status()

    want_hidden, _ = C.norm_rows("layer", x, fln_h, eps=eps, dtype=cdt)
    want = O.pool(want_hidden, mask, "mean")
    hgot = m.hidden(I, M)
    got = m.forward(I, M)
    pooled_check("modernbert", got, want, hgot, want_hidden, live)
    ops.device_status()
