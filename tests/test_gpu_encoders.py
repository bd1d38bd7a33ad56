"""GPU parity of the three encoder stacks (small shapes of the same
architectures, seeded weights shared bit for bit with the oracle) and of the
captured-plan replay."""
import numpy as np
import pytest
import torch

from oracle import svod_oracle as O
from svod_b200 import encoders as E
from svod_b200 import ops
from tests.util import TORCH_DTYPE, dev, host, max_abs, mean_rel

pytestmark = pytest.mark.gpu


def w(rng, shape, dt, sigma=0.02, mean=0.0):
    return O.round_to(dt, rng.standard_normal(shape) * sigma + mean)


def to_dev(p, dt):
    if isinstance(p, dict):
        return {k: to_dev(v, dt) for k, v in p.items()}
    if isinstance(p, list):
        return [to_dev(v, dt) for v in p]
    return None if p is None else dev(p, dt)


def check_pooled(got, want, hidden_got, hidden_want):
    # 16-bit bounds on both the hidden states and the pooled, L2-normalised f32
    # embeddings: max-abs 2e-2 / mean-rel 5e-3
    report = (f"hidden max-abs {max_abs(hidden_got, hidden_want):.3e} mean-rel {mean_rel(hidden_got, hidden_want):.3e}; "
              f"pooled max-abs {max_abs(got, want):.3e} mean-rel {mean_rel(got, want):.3e}")
    print(report)
    assert max_abs(got, want) < 2e-2 and mean_rel(got, want) < 5e-3, report
    assert mean_rel(hidden_got, hidden_want) < 5e-3, report
    assert max_abs(hidden_got, hidden_want) < 2e-2 * max(1.0, float(np.abs(hidden_want).max())), report


def test_xlm_roberta_stack_matches_the_oracle():
    dt = O.F16
    rng = np.random.default_rng(3000)
    V, D, H, F, L, B, NL = 500, 256, 4, 512, 160, 3, 2
    layers = []
    for _ in range(NL):
        layers.append({k: w(rng, s, dt) for k, s in dict(q_w=(D, D), q_b=(D,), k_w=(D, D), k_b=(D,), v_w=(D, D),
                       v_b=(D,), o_w=(D, D), o_b=(D,), fi_w=(F, D), fi_b=(F,), fo_w=(D, F), fo_b=(D,),
                       ln1_b=(D,), ln2_b=(D,)).items()})
        layers[-1]["ln1_w"] = w(rng, (D,), dt, 0.02, 1.0)
        layers[-1]["ln2_w"] = w(rng, (D,), dt, 0.02, 1.0)
    # embedding rows are O(1) after the LayerNorm either way; sigma 0.5 keeps the sum well conditioned
    p = dict(word=w(rng, (V, D), dt, 0.5), pos=w(rng, (L + 2, D), dt, 0.5), type=w(rng, (1, D), dt, 0.5),
             emb_ln_w=w(rng, (D,), dt, 0.02, 1.0), emb_ln_b=w(rng, (D,), dt), layers=layers)
    lens = [160, 64, 97]
    ids = rng.integers(2, V, (B, L))
    mask = np.arange(L)[None, :] < np.array(lens)[:, None]
    ids[~mask] = 1
    want, hwant = O.xlmr_forward(p, ids, mask, heads_n=H, dtype=dt)
    cfg = E.XlmRobertaConfig(vocab_size=V, hidden_size=D, num_hidden_layers=NL, num_attention_heads=H,
                             intermediate_size=F, max_position_embeddings=L + 2)
    m = E.XlmRobertaEncoder(cfg, to_dev(p, dt))
    I, M = torch.from_numpy(ids).cuda(), torch.from_numpy(mask).cuda()
    hgot = m.hidden(I, M)
    got = m.forward(I, M)
    live = mask[..., None] * np.ones((1, 1, D), dtype=bool)
    check_pooled(host(got), want, host(hgot)[live], hwant[live])


def test_qwen3_stack_matches_the_oracle():
    dt = O.BF16
    rng = np.random.default_rng(4000)
    V, D, H, Hkv, hd, F, L, B, NL = 300, 256, 4, 2, 128, 384, 256, 2, 2
    layers = []
    for _ in range(NL):
        layers.append(dict(in_w=w(rng, (D,), dt, 0.02, 1.0), qkv_w=w(rng, ((H + 2 * Hkv) * hd, D), dt),
                           qn_w=w(rng, (hd,), dt, 0.02, 1.0), kn_w=w(rng, (hd,), dt, 0.02, 1.0),
                           o_w=w(rng, (D, H * hd), dt), post_w=w(rng, (D,), dt, 0.02, 1.0),
                           gu_w=w(rng, (2 * F, D), dt), down_w=w(rng, (D, F), dt)))
    p = dict(embed=w(rng, (V, D), dt, 0.5), layers=layers, norm_w=w(rng, (D,), dt, 0.02, 1.0))
    ids = rng.integers(0, V, (B, L))
    lengths = np.array([256, 100])
    want, hwant = O.qwen3_forward(p, ids, lengths, heads_n=H, kv_heads=Hkv, head_dim=hd, dtype=dt)
    cfg = E.Qwen3Config(vocab_size=V, hidden_size=D, num_hidden_layers=NL, num_attention_heads=H,
                        num_key_value_heads=Hkv, head_dim=hd, intermediate_size=F)
    m = E.Qwen3Embedder(cfg, to_dev(p, dt))
    I = torch.from_numpy(ids.astype(np.int32)).cuda()
    # the oracle's tables (f32 recipe on the host) are shared so both sides rotate by identical values
    cos, sin = O.rope_table(cfg.rope_theta, np.arange(L), hd, dt)
    rope = (dev(cos, dt).view(1, L, 1, hd // 2), dev(sin, dt).view(1, L, 1, hd // 2))
    hgot = m.hidden(I, rope=rope)
    got = ops.pool(hgot, torch.from_numpy(lengths.astype(np.int32)).cuda(), ops.POOL_LAST)
    check_pooled(host(got), want, host(hgot), hwant)
    # the stack's own device-built tables agree with it too
    got2 = m.forward(I, torch.from_numpy(lengths.astype(np.int32)).cuda())
    assert max_abs(host(got2), want) < 2e-2


def test_modernbert_stack_matches_the_oracle():
    dt = O.BF16
    rng = np.random.default_rng(5000)
    V, D, H, F, L, B, NL = 400, 256, 4, 384, 320, 2, 4
    layers = []
    for i in range(NL):
        layers.append(dict(attn_ln_w=None if i == 0 else w(rng, (D,), dt, 0.02, 1.0), qkv_w=w(rng, (3 * D, D), dt),
                           o_w=w(rng, (D, D), dt), mlp_ln_w=w(rng, (D,), dt, 0.02, 1.0),
                           wi_w=w(rng, (2 * F, D), dt), wo_w=w(rng, (D, F), dt)))
    p = dict(embed=w(rng, (V, D), dt, 0.5), emb_ln_w=w(rng, (D,), dt, 0.02, 1.0), layers=layers,
             final_ln_w=w(rng, (D,), dt, 0.02, 1.0))
    lens = [320, 150]
    ids = rng.integers(0, V, (B, L))
    mask = np.arange(L)[None, :] < np.array(lens)[:, None]
    want, hwant = O.modernbert_forward(p, ids, mask, heads_n=H, dtype=dt)
    cfg = E.ModernBertConfig(vocab_size=V, hidden_size=D, num_hidden_layers=NL, num_attention_heads=H,
                             intermediate_size=F)
    m = E.ModernBertEncoder(cfg, to_dev(p, dt))
    hd = D // H
    tabs = {}
    for is_global, theta in ((True, cfg.global_rope_theta), (False, cfg.local_rope_theta)):
        cos, sin = O.rope_table(theta, np.arange(L), hd, dt)
        tabs[is_global] = (dev(cos, dt).view(1, L, 1, hd // 2), dev(sin, dt).view(1, L, 1, hd // 2))
    m._rope[L] = tabs
    I, M = torch.from_numpy(ids.astype(np.int32)).cuda(), torch.from_numpy(mask).cuda()
    hgot = m.hidden(I, M)
    got = m.forward(I, M)
    live = mask[..., None] * np.ones((1, 1, D), dtype=bool)
    check_pooled(host(got), want, host(hgot)[live], hwant[live])


def test_a_captured_plan_replays_the_eager_result_with_new_inputs():
    cfg = E.Qwen3Config(vocab_size=1000, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, head_dim=64, intermediate_size=512)
    m = E.Qwen3Embedder.random_init(cfg, seed=1)
    rows, L = 4, 256
    plan = E.Plan(m, rows, L, "lengths").capture()
    g = torch.Generator().manual_seed(0)
    for trial in range(2):
        ids = torch.randint(0, 1000, (rows, L), generator=g, dtype=torch.int32).pin_memory()
        lengths = torch.tensor([256, 17, 200, 1 + trial], dtype=torch.int32).pin_memory()
        out_host = torch.empty(rows, 256, dtype=torch.float32).pin_memory()
        plan.run(ids, lengths, out_host)
        plan.stream.synchronize()
        eager = m.forward(ids.cuda(), lengths.cuda())
        torch.cuda.synchronize()
        assert torch.equal(out_host, eager.cpu())
    ops.device_status()


def test_padding_rows_do_not_change_live_rows():
    """Right-padding invariance (model/src/test/unit/qwen3/model.rs:71): a row's
    embedding does not depend on the tokens after its length."""
    cfg = E.Qwen3Config(vocab_size=1000, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, head_dim=64, intermediate_size=512)
    m = E.Qwen3Embedder.random_init(cfg, seed=2)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 1000, (2, 256), generator=g, dtype=torch.int32).cuda()
    lengths = torch.tensor([100, 256], dtype=torch.int32).cuda()
    a = m.forward(ids, lengths)
    ids2 = ids.clone()
    ids2[0, 100:] = 7
    b = m.forward(ids2, lengths)
    assert torch.equal(a[0], b[0])


def test_packed_rows_match_separate_forwards():
    """`packed_rows_match_separate_forwards` (model/src/test/unit/qwen3/model.rs:104):
    rows packed end to end with segment starts and per-token positions embed as
    each row alone does."""
    from svod_b200 import encoder_head as EH
    cfg = E.Qwen3Config(vocab_size=1000, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, head_dim=64, intermediate_size=512)
    m = E.Qwen3Embedder.random_init(cfg, seed=3)
    rng = np.random.default_rng(0)
    rows = [rng.integers(1, 1000, n).tolist() for n in (200, 17, 90, 128, 1, 60)]
    packed = EH.Qwen3PackedEmbedder(m, max_batch=2, max_len=512).embed(rows)
    for r, got in zip(rows, packed):
        ids = torch.tensor([r], dtype=torch.int32).cuda()
        alone = m.forward(ids, torch.tensor([len(r)], dtype=torch.int32).cuda())
        assert max_abs(got, host(alone)[0]) < 2e-2
        assert abs(float(np.linalg.norm(got)) - 1.0) < 1e-3


def test_head_plans_bucket_capture_once_and_return_live_rows():
    from svod_b200 import encoder_head as EH
    cfg = E.XlmRobertaConfig(vocab_size=500, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                             intermediate_size=512, max_position_embeddings=514)
    m = E.XlmRobertaEncoder.random_init(cfg, seed=4)
    plans = EH.HeadPlans(m, max_batch=8, max_seq=512, pad_id=1)
    rng = np.random.default_rng(1)
    chunks = [rng.integers(2, 500, n).tolist() for n in (100, 30, 128, 5, 77)]
    out = EH.embed_chunks(plans, chunks)
    assert out.shape == (5, 256) and len(plans.plans) == 1 and (8, 128) in plans.plans
    for c, got in zip(chunks, out):
        ids = torch.tensor([c], dtype=torch.int32).cuda()
        mask = torch.ones(1, len(c), dtype=torch.bool).cuda()
        alone = m.forward(ids, mask)
        assert max_abs(got, host(alone)[0]) < 2e-2
    out2 = EH.embed_chunks(plans, chunks[:2])          # another bucket: (2, 128)
    assert len(plans.plans) == 2 and max_abs(out2, out[:2]) < 2e-2


@pytest.mark.parametrize("reference_ops", [False, True])
def test_native_runner_equals_the_python_stack(reference_ops):
    """`svodb_qwen3_*` / `svodb_plan_run`: the same ops in the same order issued
    from compiled code under one captured graph give the same bits as the Python
    stack, for host inputs changed between replays."""
    from svod_b200.native import NativeQwen3
    V, D, H, Hkv, hd, F, L, B, NL = 500, 256, 4, 2, 128, 384, 256, 3, 2
    cfg = E.Qwen3Config(vocab_size=V, hidden_size=D, num_hidden_layers=NL, num_attention_heads=H,
                        num_key_value_heads=Hkv, head_dim=hd, intermediate_size=F)
    m = E.Qwen3Embedder.random_init(cfg, seed=3)
    for lp in m.p["layers"]:  # non-trivial norm weights
        for name in ("in_w", "post_w", "qn_w", "kn_w"):
            lp[name].add_(torch.randn_like(lp[name]) * 0.05)
    m.fused_prologue = not reference_ops
    runner = NativeQwen3(m, reference_ops=reference_ops)
    rng = np.random.default_rng(9)
    for trial in range(2):
        ids = rng.integers(0, V, (B, L)).astype(np.int32)
        lengths = np.array([L, 17 + trial, 200], dtype=np.int32)
        got = runner.run(ids, lengths)
        want = m.forward(torch.from_numpy(ids).cuda(), torch.from_numpy(lengths).cuda()).cpu().numpy()
        assert got.shape == (B, D) and np.array_equal(got, want)
        assert np.allclose(np.linalg.norm(got, axis=1), 1.0, atol=1e-5)
    runner.replay(B, L)
    ops.device_status()
    with pytest.raises(ops.OpsError):
        NativeQwen3(m).plan(0, 16)
    runner.close()


def test_native_xlm_roberta_and_modernbert_runners_equal_the_python_stacks():
    """`svodb_xlmr_create` / `svodb_modernbert_create` + `svodb_model_plan` / `svodb_plan_run`: the same
    ops in the same order issued from compiled code under one captured graph give the same bits as the
    Python stacks, for host ids and padding masks changed between replays."""
    from svod_b200.native import NativeModernBert, NativeXlmRoberta
    rng = np.random.default_rng(12)
    B, L = 3, 256
    xc = E.XlmRobertaConfig(vocab_size=600, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                            intermediate_size=512, max_position_embeddings=L + 2)
    mc = E.ModernBertConfig(vocab_size=600, hidden_size=256, num_hidden_layers=4, num_attention_heads=4,
                            intermediate_size=384)
    for model, Runner in ((E.XlmRobertaEncoder.random_init(xc, seed=5), NativeXlmRoberta),
                          (E.ModernBertEncoder.random_init(mc, seed=6), NativeModernBert)):
        for lp in model.p["layers"]:  # non-trivial norm weights
            for name, t in lp.items():
                if t is not None and t.dim() == 1 and name.endswith("_w"):
                    t.add_(torch.randn_like(t) * 0.05)
        runner = Runner(model)
        for trial in range(2):
            lens = np.array([L, 40 + trial, 199])
            mask = np.arange(L)[None, :] < lens[:, None]
            ids = rng.integers(2, 600, (B, L)).astype(np.int32)
            ids[~mask] = 1
            got = runner.run(ids, mask)
            want = model.forward(torch.from_numpy(ids).cuda(), torch.from_numpy(mask).cuda()).cpu().numpy()
            assert got.shape == want.shape and np.array_equal(got, want), type(model).__name__
            assert np.allclose(np.linalg.norm(got, axis=1), 1.0, atol=1e-5)
        runner.replay(B, L)
        ops.device_status()
        runner.close()
