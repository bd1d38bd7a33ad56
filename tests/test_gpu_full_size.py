"""GPU parity of the three encoder stacks at their full widths and depths: the
benchmark configurations' real layer shapes (hidden size, heads, FFN, layer
count, sequence length, dtype, masks) on a reduced batch, seeded weights shared
bit for bit with the compiled CPU restatement (`oracle/svod_oracle.c`, held to
the pinned numpy restatement by `tests/test_c_oracle_cpu.py`).

Two comparisons per stack:

* layer by layer: layer `l` of the GPU stack is fed the oracle's hidden states
  after layer `l-1` and compared with the oracle's after layer `l`, at the
  16-bit operator tolerance (max-abs 2e-2 relative to `max(1, max|want|)`,
  mean-rel 5e-3). Every full-size kernel the benchmark runs is on this path.
* end to end: embeddings -> all layers -> final norm -> pooling -> L2 with no
  help from the oracle. Two correct implementations drift apart over a deep
  16-bit stack (the f32 C restatement and the float64 numpy one differ by
  mean-rel 1.2e-2 after 28 Qwen3 layers at this width), so the end-to-end bound
  on hidden states is the drift bound below; the pooled unit-norm rows are held
  to max-abs 2e-2 and to a cosine distance.

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

# end-to-end drift bound on hidden states of a deep 16-bit stack (see the module docstring)
DRIFT_MEAN_REL = 2.5e-2


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


def layer_check(name, li, got, want, live=None):
    g, w_ = (host(got), want) if live is None else (host(got)[live], want[live])
    ma, mr = max_abs(g, w_), mean_rel(g, w_)
    bound = 2e-2 * max(1.0, float(np.abs(w_).max()))
    assert ma <= bound and mr < 5e-3, f"{name} layer {li}: max-abs {ma:.3e} (bound {bound:.3e}), mean-rel {mr:.3e}"
    return ma, mr


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
    wt = Weights(4000, torch.bfloat16)
    dl, hl = [], []
    for _ in range(cfg.num_hidden_layers):
        d_, h_ = split(dict(in_w=wt(D, mean=1.0), qkv_w=wt((H + 2 * Hkv) * hd, D), qn_w=wt(hd, mean=1.0),
                            kn_w=wt(hd, mean=1.0), o_w=wt(D, H * hd), post_w=wt(D, mean=1.0), gu_w=wt(2 * F, D),
                            down_w=wt(D, F)))
        dl.append(d_), hl.append(h_)
    norm_d, norm_h = wt(D, mean=1.0)
    embed = (torch.randn(cfg.vocab_size, D, generator=torch.Generator(device="cuda").manual_seed(4001), device="cuda")
             * 0.02).to(torch.bfloat16)
    ids = torch.randint(0, cfg.vocab_size, (1, L), generator=wt.g, dtype=torch.int32)
    lengths = np.array([L], dtype=np.int32)
    m = E.Qwen3Embedder(cfg, dict(embed=embed, layers=dl, norm_w=norm_d))
    # the oracle's rotation tables (f32 recipe on the host) on both sides
    cos, sin = C.rope_table(cfg.rope_theta, np.arange(L), hd, C.BF16)
    rope = tuple(torch.from_numpy(t).to(torch.bfloat16).cuda().view(1, L, 1, hd // 2) for t in (cos, sin))

    hs = [embed[ids.long().cuda()].float().cpu().numpy()]
    for lp in hl:
        hs.append(C.qwen3_layers(hs[-1], [lp], heads_n=H, kv_heads=Hkv, head_dim=hd, theta=cfg.rope_theta,
                                 eps=cfg.rms_norm_eps, dtype=C.BF16))
    worst = (0.0, 0.0)
    for fused in (True, False):
        m.fused_prologue = fused
        for li in range(cfg.num_hidden_layers):
            x = torch.from_numpy(hs[li]).to(torch.bfloat16).cuda()
            got = m.run_layers(x, rope=rope, start=li, stop=li + 1)
            worst = tuple(max(a, b) for a, b in zip(worst, layer_check("qwen3", li, got, hs[li + 1])))
    print(f"qwen3 layer by layer (both op sequences): worst max-abs {worst[0]:.3e}, worst mean-rel {worst[1]:.3e}")
    ops.device_status()

    m.fused_prologue = True
    want_hidden, _ = C.norm_rows("rms", hs[-1], norm_h, eps=cfg.rms_norm_eps, dtype=C.BF16)
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
    wt = Weights(3000, torch.float16)
    dl, hl = [], []
    for _ in range(cfg.num_hidden_layers):
        d_, h_ = split(dict(q_w=wt(D, D), q_b=wt(D), k_w=wt(D, D), k_b=wt(D), v_w=wt(D, D), v_b=wt(D), o_w=wt(D, D),
                            o_b=wt(D), ln1_w=wt(D, mean=1.0), ln1_b=wt(D), fi_w=wt(F, D), fi_b=wt(F), fo_w=wt(D, F),
                            fo_b=wt(D), ln2_w=wt(D, mean=1.0), ln2_b=wt(D)))
        dl.append(d_), hl.append(h_)
    gd = torch.Generator(device="cuda").manual_seed(3001)
    word = (torch.randn(cfg.vocab_size, D, generator=gd, device="cuda") * 0.02).to(torch.float16)
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

    rows = word[I].float().cpu().numpy().astype(np.float64)
    e = O.round_to(O.F16, O.round_to(O.F16, rows + pos_h[O.xlmr_position_ids(ids, cfg.pad_token_id)]) + type_h[0])
    h0, _ = C.norm_rows("layer", e, elw_h, elb_h, eps=cfg.layer_norm_eps, dtype=C.F16)
    hs = [h0]
    for lp in hl:
        hs.append(C.xlmr_layers(hs[-1], [lp], mask, heads_n=H, eps=cfg.layer_norm_eps, dtype=C.F16))
    live = mask[..., None] & np.ones((1, 1, D), dtype=bool)
    worst = (0.0, 0.0)
    for li in range(cfg.num_hidden_layers):
        x = torch.from_numpy(hs[li]).to(torch.float16).cuda()
        got = m.run_layers(x, M, start=li, stop=li + 1)
        worst = tuple(max(a, b) for a, b in zip(worst, layer_check("xlm-r", li, got, hs[li + 1], live)))
    print(f"xlm-r layer by layer: worst max-abs {worst[0]:.3e}, worst mean-rel {worst[1]:.3e}")
    ops.device_status()

    want = O.pool(hs[-1], mask, "cls")
    hgot = m.hidden(I, M)
    got = m.forward(I, M)
    pooled_check("xlm-r", got, want, hgot, hs[-1], live)
    ops.device_status()


def test_modernbert_base_full_width_full_depth_rows():
    """ModernBERT-base shape: 22 pre-LN layers (every third global, the rest a 128-token window), hidden 768,
    12 heads x 64, GeGLU 1152, RoPE in the projection's store, bf16, rows of 8192 with lengths from
    [2048, 8192] behind a padding mask, mean pooling."""
    cfg = E.ModernBertConfig()
    D, H, F, L, B = 768, 12, 1152, 8192, 2
    hd = D // H
    wt = Weights(5000, torch.bfloat16)
    dl, hl = [], []
    for i in range(cfg.num_hidden_layers):
        d_, h_ = split(dict(qkv_w=wt(3 * D, D), o_w=wt(D, D), mlp_ln_w=wt(D, mean=1.0), wi_w=wt(2 * F, D),
                            wo_w=wt(D, F)))
        a = (None, None) if i == 0 else wt(D, mean=1.0)
        d_["attn_ln_w"], h_["attn_ln_w"] = a
        dl.append(d_), hl.append(h_)
    gd = torch.Generator(device="cuda").manual_seed(5001)
    embed = (torch.randn(cfg.vocab_size, D, generator=gd, device="cuda") * 0.02).to(torch.bfloat16)
    eln_d, eln_h = wt(D, mean=1.0)
    fln_d, fln_h = wt(D, mean=1.0)
    rng = np.random.default_rng(5002)
    lens = np.array([L, int(rng.integers(2048, L + 1))])
    mask = np.arange(L)[None, :] < lens[:, None]
    ids = rng.integers(0, cfg.vocab_size, (B, L)).astype(np.int32)
    m = E.ModernBertEncoder(cfg, dict(embed=embed, emb_ln_w=eln_d, layers=dl, final_ln_w=fln_d))
    tabs = {}
    for is_global, theta in ((True, cfg.global_rope_theta), (False, cfg.local_rope_theta)):
        cos, sin = C.rope_table(theta, np.arange(L), hd, C.BF16)
        tabs[is_global] = tuple(torch.from_numpy(t).to(torch.bfloat16).cuda().view(1, L, 1, hd // 2) for t in (cos, sin))
    m._rope[L] = tabs
    I, M = torch.from_numpy(ids).cuda(), torch.from_numpy(mask).cuda()

    half = cfg.local_attention // 2
    kw = dict(heads_n=H, global_every=cfg.global_attn_every_n_layers, global_theta=cfg.global_rope_theta,
              local_theta=cfg.local_rope_theta, local_window=(half, half), eps=cfg.norm_eps, dtype=C.BF16)
    h0, _ = C.norm_rows("layer", embed[I.long()].float().cpu().numpy(), eln_h, eps=cfg.norm_eps, dtype=C.BF16)
    hs = [h0]
    for li, lp in enumerate(hl):
        hs.append(C.modernbert_layers(hs[-1], [lp], mask, first_layer=li, **kw))
    live = mask[..., None] & np.ones((1, 1, D), dtype=bool)
    worst = (0.0, 0.0)
    for li in range(cfg.num_hidden_layers):
        x = torch.from_numpy(hs[li]).to(torch.bfloat16).cuda()
        got = m.run_layers(x, M, start=li, stop=li + 1)
        worst = tuple(max(a, b) for a, b in zip(worst, layer_check("modernbert", li, got, hs[li + 1], live)))
    print(f"modernbert layer by layer: worst max-abs {worst[0]:.3e}, worst mean-rel {worst[1]:.3e}")
    ops.device_status()

    want_hidden, _ = C.norm_rows("layer", hs[-1], fln_h, eps=cfg.norm_eps, dtype=C.BF16)
    want = O.pool(want_hidden, mask, "mean")
    hgot = m.hidden(I, M)
    got = m.forward(I, M)
    pooled_check("modernbert", got, want, hgot, want_hidden, live)
    ops.device_status()
