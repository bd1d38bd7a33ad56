"""GPU parity of `ops.attention` / `attention_packed` against the oracle: the
reference's kernel cases (tk/src/test/unit/attention.rs:349-455: LCG seed 5,
key mask hiding (b+j)%5==2, segments of 40, max-abs 2e-2) and its op-level cases
(tk/src/test/unit/ops.rs:436-470, 507-523, 1004-1024), through the C ABI."""
import math

import numpy as np
import pytest
import torch

from oracle import svod_oracle as O
from svod_b200 import ops
from tests.util import dev, host, max_abs, mean_rel, normal

pytestmark = pytest.mark.gpu

SEGMENT = 40


def recipe(B, T, Tk, H, Hkv, D, dt=O.BF16, seed=5):
    g = O.Lcg(seed)
    q = g.rounded(dt, B * T * H * D).reshape(B, T, H, D)
    k = g.rounded(dt, B * Tk * Hkv * D).reshape(B, Tk, Hkv, D)
    v = g.rounded(dt, B * Tk * Hkv * D).reshape(B, Tk, Hkv, D)
    return q, k, v


def run_case(q, k, v, dt, packed=False, lse=False, **kw):
    B, T, H, D = q.shape
    a = ops.Attn(want_lse=lse, causal=bool(kw.get("causal")), window=kw.get("window"), scale=kw.get("scale"),
                 splits=kw.get("splits"))
    okw = {key: kw[key] for key in ("causal", "window", "scale") if kw.get(key) is not None}
    if "lens" in kw:
        okw["key_lens"] = np.array(kw["lens"])
        a.keys = ops.KeyMask.Lens(torch.tensor(kw["lens"], dtype=torch.int64).cuda())
    if "mask" in kw:
        okw["key_mask"] = kw["mask"]
        a.keys = ops.KeyMask.Bool(torch.from_numpy(np.asarray(kw["mask"])).cuda())
    if "seg" in kw:
        okw["seg_start"] = kw["seg"]
        a.seg_start = torch.from_numpy(np.asarray(kw["seg"], dtype=np.int64)).cuda()
    if "chunk" in kw:
        okw["chunk"] = kw["chunk"]
        a.chunk = ops.Chunk(*kw["chunk"])
    if "bias" in kw:
        okw["bias"] = kw["bias"]
        a.bias = dev(kw["bias"], dt)
    want = O.attention(q, k, v, dtype=dt, return_lse=lse, **okw)
    if packed:
        qkv = np.concatenate([q.reshape(B, T, -1), k.reshape(B, T, -1), v.reshape(B, T, -1)], axis=-1)
        got = ops.attention_packed(dev(qkv, dt), H, k.shape[2], a)
    else:
        got = ops.attention(dev(q, dt), dev(k, dt), dev(v, dt), a)
    if lse:
        return host(got[0]), host(got[1]), want[0], want[1]
    return host(got), want


def key_mask(B, Tk):
    return np.array([[(b + j) % 5 != 2 for j in range(Tk)] for b in range(B)])


def segments(B, T, seg=SEGMENT):
    return np.array([[i - i % seg for i in range(T)] for _ in range(B)])


KERNEL_CASES = [
    # name, T, Tk, D, kwargs            (B = 2, H = Hkv = 2 as in the reference's `spec`)
    ("one block", 64, 64, 64, {}),
    ("three key blocks", 128, 192, 64, {}),
    ("causal", 128, 128, 64, dict(causal=True)),
    ("key lengths", 128, 128, 64, dict(lens=[100, 7])),
    ("causal with lengths", 128, 128, 64, dict(causal=True, lens=[128, 50])),
    ("window with lengths", 128, 128, 64, dict(window=(16, 8), lens=[128, 90])),
    ("key mask", 128, 128, 64, dict(mask="km")),
    ("causal segments", 128, 128, 64, dict(causal=True, seg="seg")),
    ("chunks with lengths", 128, 128, 64, dict(chunk=(32, 1, 0), lens=[128, 90])),
    ("chunks, every earlier one and one ahead, ragged", 100, 100, 64, dict(chunk=(32, None, 1))),
    ("every mask", 128, 128, 64, dict(causal=True, window=(64, 64), lens=[128, 100], mask="km", seg="seg")),
    ("a lane with no keys", 128, 128, 64, dict(lens=[100, 0])),
    ("causal, a lane with no keys", 128, 128, 64, dict(causal=True, lens=[0, 50])),
    ("a larger scale", 128, 128, 64, dict(causal=True, lens=[128, 50], scale=0.3)),
    ("plain", 128, 128, 64, {}),
    ("causal, 256 queries", 256, 256, 64, dict(causal=True)),
    ("key lengths, 256 keys", 128, 256, 64, dict(lens=[200, 33])),
    ("d 128, causal with lengths", 128, 128, 128, dict(causal=True, lens=[128, 64])),
    ("bq 128, three stages", 256, 192, 64, dict(causal=True, lens=[192, 70])),
    ("d 128, ragged", 200, 130, 128, dict(lens=[130, 99])),
    ("d 128, bq 256, ragged", 600, 420, 128, dict(lens=[420, 299])),
    ("key mask, ragged", 100, 100, 64, dict(mask="km")),
    ("every mask, d 128", 128, 128, 128, dict(causal=True, window=(64, 64), lens=[128, 100], mask="km", seg="seg")),
    ("wide core, d 128", 200, 300, 128, {}),
    ("wide core, d 64, bq 256", 300, 300, 64, {}),
    ("odd keys", 99, 99, 64, dict(lens=[99, 41])),
    # head dims between the two tiled ones run zero-padded on the next (the reference plans 32 and 48 too:
    # tk/src/test/unit/attention.rs:349-455 has d 48)
    ("d 48, causal segments", 96, 96, 48, dict(causal=True, seg="seg")),
    ("d 32, key lengths", 128, 192, 32, dict(lens=[192, 77])),
    ("d 96, ragged, key mask", 200, 130, 96, dict(mask="km")),
    ("d 48, a lane with no keys", 100, 100, 48, dict(lens=[100, 0])),
]


@pytest.mark.parametrize("name,T,Tk,D,kw", KERNEL_CASES, ids=[c[0] for c in KERNEL_CASES])
def test_flash_attention_matches_a_direct_softmax(name, T, Tk, D, kw):
    B, H = 2, 2
    kw = dict(kw)
    if kw.get("mask") == "km":
        kw["mask"] = key_mask(B, Tk)
    if kw.get("seg") == "seg":
        kw["seg"] = segments(B, T)
    if "lens" in kw and "mask" in kw:
        # KeyMask is one or the other: fold the lengths into the bool mask
        kw["mask"] = kw["mask"] & (np.arange(Tk)[None, :] < np.array(kw.pop("lens"))[:, None])
    q, k, v = recipe(B, T, Tk, H, H, D)
    got, want = run_case(q, k, v, O.BF16, **kw)
    assert "kernel flash_attention" in ops.chosen()
    assert not np.isnan(got).any()
    assert max_abs(got, want) < 2e-2


def test_a_fully_masked_batch_is_zeros():
    B, T, D = 2, 128, 64
    q, k, v = recipe(B, T, T, 2, 2, D)
    m = key_mask(B, T)
    m[1] = False
    got, want = run_case(q, k, v, O.BF16, mask=m)
    assert np.any(got[0] != 0) and np.all(got[1] == 0)
    assert max_abs(got, want) < 2e-2


OP_CASES = [
    ("lens", 2, 100, 100, 4, 4, 64, O.BF16, dict(lens=[100, 61])),
    ("causal T200", 2, 200, 200, 4, 4, 64, O.BF16, dict(causal=True)),
    ("gqa 8/2", 2, 100, 100, 8, 2, 64, O.BF16, {}),
    ("d128 gqa causal", 2, 100, 100, 8, 2, 128, O.BF16, dict(causal=True)),
    ("cross 37x150", 2, 37, 150, 4, 4, 64, O.BF16, {}),
    ("window (64,64) T300", 2, 300, 300, 4, 4, 64, O.BF16, dict(window=(64, 64))),
    ("bool mask", 2, 100, 100, 4, 4, 64, O.BF16, dict(mask="km")),
    ("segments of 30", 2, 100, 100, 4, 4, 64, O.BF16, dict(causal=True, seg=30)),
    ("f16", 2, 100, 100, 4, 4, 64, O.F16, dict(lens=[100, 61])),
    ("f16 d128 causal 700", 1, 700, 700, 4, 2, 128, O.F16, dict(causal=True)),
]


@pytest.mark.parametrize("name,B,T,Tk,H,Hkv,D,dt,kw", OP_CASES, ids=[c[0] for c in OP_CASES])
def test_attention_op_matches_the_oracle(name, B, T, Tk, H, Hkv, D, dt, kw):
    kw = dict(kw)
    if kw.get("mask") == "km":
        kw["mask"] = key_mask(B, Tk)
    if "seg" in kw:
        kw["seg"] = segments(B, T, kw["seg"])
    rng = np.random.default_rng(11)
    q = O.round_to(dt, rng.uniform(-1, 1, (B, T, H, D)))
    k = O.round_to(dt, rng.uniform(-1, 1, (B, Tk, Hkv, D)))
    v = O.round_to(dt, rng.uniform(-1, 1, (B, Tk, Hkv, D)))
    got, want = run_case(q, k, v, dt, **kw)
    assert "kernel flash_attention" in ops.chosen()
    assert max_abs(got, want) < 2e-2


@pytest.mark.parametrize("kw", [dict(window=(64, 64)), dict(mask="km"), dict(causal=True)])
def test_packed_attention_is_bit_identical_to_the_split_operands(kw):
    """`packed_attention_matches_the_split_kernel` (ops.rs:507-523)."""
    kw = dict(kw)
    B, T, H, D = 2, 300, 4, 64
    if kw.get("mask") == "km":
        kw["mask"] = key_mask(B, T)
    q, k, v = recipe(B, T, T, H, H, D)
    a, want = run_case(q, k, v, O.BF16, **kw)
    b, _ = run_case(q, k, v, O.BF16, packed=True, **kw)
    assert "flash_attention_packed" in ops.chosen()
    assert np.array_equal(a, b)
    assert max_abs(a, want) < 2e-2


def test_config_1_f32_attention_with_key_lengths_output_and_logsumexp():
    """f32, batch 2, 8 heads, seq 512, head_dim 64, N(0,1) from seed, key-padding
    lengths uniform in [256, 512], scale 1/sqrt(64): output and log-sum-exp
    within 1e-4 of the CPU oracle."""
    rng = np.random.default_rng(1000)
    B, T, H, D = 2, 512, 8, 64
    q = O.round_to(O.F32, rng.standard_normal((B, T, H, D)))
    k = O.round_to(O.F32, rng.standard_normal((B, T, H, D)))
    v = O.round_to(O.F32, rng.standard_normal((B, T, H, D)))
    lens = rng.integers(256, 513, B).tolist()
    got, glse, want, wlse = run_case(q, k, v, O.F32, lse=True, lens=lens, scale=1.0 / math.sqrt(64))
    assert ops.chosen() == "attention: graph dtype"
    assert max_abs(got, want) < 1e-4
    assert max_abs(glse, wlse) < 1e-4
    # the same inputs rounded to bf16 run the tcgen05 kernel: 2e-2 / 5e-3
    qb, kb, vb = (O.round_to(O.BF16, t) for t in (q, k, v))
    got, glse, want, wlse = run_case(qb, kb, vb, O.BF16, lse=True, lens=lens)
    assert "kernel flash_attention" in ops.chosen()
    assert max_abs(got, want) < 2e-2 and mean_rel(got, want) < 5e-3
    assert max_abs(glse, wlse) < 2e-2


# Additive bias and key splits run on the persistent tensor-core kernel (partials merged by
# `combine_splits`); the exact kernel keeps f32, a non-positive scale and rows off the 16-byte grid.
BIAS_SPLIT_CASES = [
    ("bias per batch", 2, 128, 128, 2, 2, 64, O.BF16, dict(bias=(2, 2, 128, 128))),
    ("shared bias, ragged", 2, 100, 130, 2, 2, 64, O.BF16, dict(bias=(1, 2, 100, 130))),
    ("bias with key lengths", 2, 99, 99, 2, 2, 64, O.BF16, dict(bias=(2, 2, 99, 99), lens=[99, 41])),
    ("causal bias, d 128, 300 queries", 2, 300, 300, 4, 2, 128, O.BF16, dict(bias=(2, 4, 300, 300), causal=True)),
    ("four splits", 1, 1, 200, 4, 4, 64, O.BF16, dict(lens=[70], splits=4)),
    ("two splits, five queries, d128", 2, 5, 96, 2, 2, 128, O.BF16, dict(lens=[64, 96], splits=2)),
    ("more splits than blocks", 2, 1, 64, 2, 2, 64, O.BF16, dict(lens=[64, 40], splits=4)),
    ("splits, a lane with no keys", 2, 1, 200, 4, 4, 64, O.BF16, dict(lens=[0, 70], splits=4)),
    ("three splits, causal, 300 queries, gqa", 2, 300, 300, 4, 2, 128, O.BF16, dict(causal=True, splits=3)),
    ("five splits with a bias, f16", 2, 40, 700, 2, 2, 64, O.F16, dict(bias=(1, 2, 40, 700), splits=5, lens=[700, 333])),
]


@pytest.mark.parametrize("name,B,T,Tk,H,Hkv,D,dt,kw", BIAS_SPLIT_CASES, ids=[c[0] for c in BIAS_SPLIT_CASES])
def test_bias_and_key_splits_run_on_the_tensor_core_kernel(name, B, T, Tk, H, Hkv, D, dt, kw):
    kw = dict(kw)
    q, k, v = recipe(B, T, Tk, H, Hkv, D, dt)
    if "bias" in kw:
        kw["bias"] = O.Lcg(99).rounded(dt, int(np.prod(kw["bias"])), lambda x: 2.0 * x).reshape(kw["bias"])
    got, want = run_case(q, k, v, dt, **kw)
    ran = min(kw.get("splits", 1), (Tk + 31) // 32)   # a request is capped at the 32-key tile count
    assert "kernel flash_attention" in ops.chosen() and f"splits:{ran}" in ops.chosen(), ops.chosen()
    assert max_abs(got, want) < 2e-2
    if "lens" in kw and 0 in kw["lens"]:
        assert np.all(got[kw["lens"].index(0)] == 0.0)


GENERIC_CASES = [
    ("d 44 (rows off the 16-byte grid)", 2, 96, 96, 2, 2, 44, O.BF16, dict(causal=True, seg=40)),
    ("negative scale", 2, 128, 128, 2, 2, 64, O.BF16, dict(causal=True, lens=[128, 50], scale=-0.1)),
    ("negative scale with splits and a bias", 2, 8, 128, 2, 2, 64, O.BF16,
     dict(lens=[128, 50], scale=-0.1, splits=2, bias=(2, 2, 8, 128))),
    ("f32 causal ragged gqa", 2, 100, 130, 4, 2, 48, O.F32, dict(causal=True)),
    ("f32 splits", 2, 3, 200, 4, 2, 48, O.F32, dict(lens=[200, 70], splits=4)),
]


@pytest.mark.parametrize("name,B,T,Tk,H,Hkv,D,dt,kw", GENERIC_CASES, ids=[c[0] for c in GENERIC_CASES])
def test_cases_outside_the_tile_kernel_run_the_exact_kernel(name, B, T, Tk, H, Hkv, D, dt, kw):
    kw = dict(kw)
    if "seg" in kw:
        kw["seg"] = segments(B, T, kw["seg"])
    q, k, v = recipe(B, T, Tk, H, Hkv, D, dt)
    if "bias" in kw:
        kw["bias"] = O.Lcg(99).rounded(dt, int(np.prod(kw["bias"])), lambda x: 2.0 * x).reshape(kw["bias"])
    got, want = run_case(q, k, v, dt, **kw)
    assert ops.chosen().startswith("attention: graph")
    assert max_abs(got, want) < (1e-4 if dt == O.F32 else 2e-2)


def test_combine_splits_merges_partial_states():
    rng = np.random.default_rng(4)
    S, B, T, H, D = 3, 2, 5, 2, 64
    o = rng.standard_normal((S, B, T, H, D)).astype(np.float32)
    m = (rng.standard_normal((S, B, T, H)) * 3).astype(np.float32)
    l = rng.uniform(0.5, 4, (S, B, T, H)).astype(np.float32)
    l[:, 1, 2] = 0.0
    o[:, 1, 2] = 0.0
    m[:, 1, 2] = -1e30
    want = O.combine_splits(o, m, l, O.BF16)
    got = ops.combine_splits(torch.from_numpy(o).cuda(), torch.from_numpy(m).cuda(), torch.from_numpy(l).cuda(),
                             torch.bfloat16)
    assert max_abs(host(got), want) < 2e-2
    assert np.all(host(got)[1, 2] == 0)


def test_full_size_attention_properties_at_seq_4096_d128():
    """Size-independent checks at the headline shape (heads 16/8, seq 4096, d 128,
    causal), batch 2: (1) v = ones gives ones on every row that sees a key;
    (2) the first 256 queries equal attention over the first 256 keys alone;
    (3) a replay is bit-identical; (4) sampled rows match an f32 softmax."""
    g = torch.Generator(device="cuda").manual_seed(4)
    B, T, H, Hkv, D = 2, 4096, 16, 8, 128
    q = torch.randn(B, T, H, D, generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn(B, T, Hkv, D, generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn(B, T, Hkv, D, generator=g, device="cuda").to(torch.bfloat16)
    a = ops.Attn(causal=True)
    o = ops.attention(q, k, v, a)
    assert "kernel flash_attention" in ops.chosen()
    ones = ops.attention(q, k, torch.ones_like(v), a)
    assert float((ones.float() - 1).abs().max()) < 1e-2
    head = ops.attention(q[:, :256].contiguous(), k[:, :256].contiguous(), v[:, :256].contiguous(), a)
    assert torch.equal(head, o[:, :256])
    assert torch.equal(ops.attention(q, k, v, a), o)
    for (b, h, i) in [(0, 0, 0), (1, 5, 1000), (0, 15, 4095), (1, 9, 2177)]:
        kk, vv = k[b, :i + 1, h // 2].float(), v[b, :i + 1, h // 2].float()
        s = (kk @ q[b, i, h].float()) / math.sqrt(D)
        ref = torch.softmax(s, 0) @ vv
        assert float((o[b, i, h].float() - ref).abs().max()) < 2e-2


# ---- decode-path reads: `ops::Cache` (tk/src/ops/attention.rs:39-55) -------------------------------
# The reference's cached cases (tk/src/test/unit/attention.rs:395-410,488-505): batch 2, a cache of 3
# rows holding 3*kv_heads heads of which this attention reads those from `kv_heads` on, lane b on
# cache row 2-b under a row map, `appended` rows after the cached prefix of which lane b sees
# `max(appended - b % 3, 1)` when counted, a per-batch bias of 2*x when biased; data from the LCG
# (seed 5) in the order q, k, v, appended k, appended v, bias.
CACHED_CASES = [
    # name, t, tk, (heads, kv_heads, d), row_map, appended, splits, lens, counted, biased
    ("cache slice", 1, 100, (4, 4, 64), False, 0, 1, [100, 37], False, False),
    ("row map, appended, gqa", 1, 100, (4, 2, 64), True, 1, 1, [100, 37], False, False),
    ("four splits", 1, 200, (4, 4, 64), True, 1, 4, [200, 70], False, False),
    ("d 128, two splits, five queries", 5, 96, (2, 2, 128), False, 1, 2, [64, 96], False, False),
    ("more splits than blocks for a row", 1, 64, (2, 2, 64), False, 0, 4, [64, 40], False, False),
    ("appended row only, one split", 1, 7, (6, 6, 64), False, 1, 1, [0, 7], False, False),
    ("appended row only, two splits", 1, 7, (6, 6, 64), False, 1, 2, [0, 3], False, False),
    ("eight queries, eight appended, d 48", 8, 128, (4, 4, 48), False, 8, 1, [128, 40], False, False),
    ("sixteen appended, two splits", 16, 128, (2, 2, 64), True, 16, 2, [128, 0], False, False),
    ("counted appended rows", 8, 128, (4, 4, 48), False, 8, 1, [128, 40], True, False),
    ("counted appended rows only, three splits", 16, 96, (2, 2, 64), False, 16, 3, [0, 96], True, False),
    ("biased: row map, appended, gqa", 1, 100, (4, 2, 64), True, 1, 1, [100, 37], False, True),
    ("biased: d 128, two splits", 5, 96, (2, 2, 128), False, 1, 2, [64, 96], False, True),
    ("biased: four splits", 1, 200, (4, 4, 64), False, 0, 4, [200, 70], False, True),
    ("biased: counted appended rows", 8, 64, (2, 2, 64), False, 8, 2, [64, 20], True, True),
    ("a cached lane with no keys", 1, 100, (4, 4, 64), False, 0, 1, [100, 0], False, False),
]


@pytest.mark.parametrize("name,t,tk,hhd,row_map,appended,splits,lens,counted,biased", CACHED_CASES,
                         ids=[c[0] for c in CACHED_CASES])
def test_cached_attention_matches_the_reference_recipe(name, t, tk, hhd, row_map, appended, splits, lens, counted,
                                                       biased):
    dt, B, rows = O.BF16, 2, 3
    H, Hkv, D = hhd
    g = O.Lcg(5)
    q = g.rounded(dt, B * t * H * D).reshape(B, t, H, D)
    k = g.rounded(dt, rows * tk * 3 * Hkv * D).reshape(rows, tk, 3 * Hkv, D)
    v = g.rounded(dt, rows * tk * 3 * Hkv * D).reshape(rows, tk, 3 * Hkv, D)
    k_app = g.rounded(dt, B * appended * Hkv * D).reshape(B, appended, Hkv, D)
    v_app = g.rounded(dt, B * appended * Hkv * D).reshape(B, appended, Hkv, D)
    bias = 2.0 * g.rounded(dt, B * H * t * (tk + appended)).reshape(B, H, t, tk + appended) if biased else None
    rm = np.array([rows - 1 - b for b in range(B)]) if row_map else None
    seen = np.array([max(appended - b % 3, 1) for b in range(B)]) if counted else None
    cache = dict(head_start=Hkv, kv_heads=Hkv, row_map=rm, k_app=k_app if appended else None,
                 v_app=v_app if appended else None, app_lens=seen)
    want = O.attention(q, k, v, key_lens=np.array(lens), bias=bias, cache=cache, dtype=dt)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32).cuda()
    c = ops.Cache(Hkv, Hkv, i32(rm) if row_map else None,
                  (dev(k_app, dt), dev(v_app, dt)) if appended else None, i32(seen) if counted else None)
    a = ops.Attn(keys=ops.KeyMask.Lens(i32(lens)), cache=c, splits=splits if splits > 1 else None,
                 bias=dev(bias, dt) if biased else None)
    if not row_map:  # lane b reads cache row b: the op takes the batch's own rows
        k, v = k[:B], v[:B]
    got = host(ops.attention(dev(q, dt), dev(k, dt), dev(v, dt), a))
    assert max_abs(got, want) < 2e-2
    if name == "a cached lane with no keys":
        assert np.all(got[1] == 0.0) and np.any(got[0] != 0.0)


@pytest.mark.parametrize("D,T,Tk", [(128, 256, 320), (64, 130, 200)])
def test_cache_slices_and_row_maps_stay_on_the_tensor_core_kernel(D, T, Tk):
    """Without appended rows a cache read is a strided view plus a row lookup in
    the loader: same kernel, same numbers as attention over the gathered rows."""
    dt, B, rows, H, Hkv = O.BF16, 3, 5, 4, 2
    rng = np.random.default_rng(D + T)
    q = normal(rng, (B, T, H, D), 1.0, dt)
    k = normal(rng, (rows, Tk, 3 * Hkv, D), 1.0, dt)
    v = normal(rng, (rows, Tk, 3 * Hkv, D), 1.0, dt)
    rm = np.array([4, 0, 2])
    lens = np.array([Tk, 77, Tk - 1])
    cache = dict(head_start=2 * Hkv, kv_heads=Hkv, row_map=rm)
    want = O.attention(q, k, v, causal=True, key_lens=lens, cache=cache, dtype=dt)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32).cuda()
    a = ops.Attn(causal=True, keys=ops.KeyMask.Lens(i32(lens)), cache=ops.Cache(2 * Hkv, Hkv, i32(rm)))
    got = host(ops.attention(dev(q, dt), dev(k, dt), dev(v, dt), a))
    assert "kernel flash_attention" in ops.chosen()
    assert max_abs(got, want) < 2e-2 and mean_rel(got, want) < 5e-3


def test_cache_options_are_validated():
    dt = O.BF16
    z = lambda *s: dev(np.zeros(s), dt)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32).cuda()
    q, k = z(2, 1, 4, 64), z(3, 16, 6, 64)
    lens = ops.KeyMask.Lens(i32([16, 16]))
    with pytest.raises(ops.OpsError) as e:  # rows != B without a row map
        ops.attention(q, k, k, ops.Attn(cache=ops.Cache(0, 2)))
    assert e.value.kind == "Shape"
    with pytest.raises(ops.OpsError) as e:  # heads past the cache row
        ops.attention(q, k, k, ops.Attn(cache=ops.Cache(5, 2, i32([0, 1]))))
    assert e.value.kind == "Shape"
    with pytest.raises(ops.OpsError) as e:  # appended rows need key lengths
        ops.attention(q, k, k, ops.Attn(cache=ops.Cache(0, 2, i32([0, 1]), (z(2, 1, 2, 64), z(2, 1, 2, 64)))))
    assert e.value.kind == "Shape"
    with pytest.raises(ops.OpsError) as e:  # counted rows without appended rows
        ops.attention(q, k, k, ops.Attn(keys=lens, cache=ops.Cache(0, 2, i32([0, 1]), None, i32([1, 1]))))
    assert e.value.kind == "Shape"
    with pytest.raises(ops.OpsError) as e:  # 4 query heads over 3 kv heads
        ops.attention(q, k, k, ops.Attn(keys=lens, cache=ops.Cache(0, 3, i32([0, 1]))))
    assert e.value.kind == "Heads"


# ---- the persistent kernel (more work items than SMs) ---------------------------------------------
def padding_mask(B, Tk, lens):
    return np.array([[j < lens[b] for j in range(Tk)] for b in range(B)])



PERSISTENT_CASES = [
    ("causal", 128, dict(causal=True)),
    ("causal d64", 64, dict(causal=True)),
    ("plain", 128, dict()),
    ("key lengths with empty rows", 128, dict(lens=[1300, 700, 0, 130])),
    ("causal + lengths", 64, dict(causal=True, lens=[1300, 5, 900, 257])),
    ("window", 128, dict(window=(100, 30), lens=[1300, 1000, 1300, 64])),
    ("causal segments", 64, dict(causal=True, seg="seg")),
    ("chunks", 128, dict(chunk=(96, 2, 0), lens=[1300, 1300, 400, 1300])),
    ("bool mask with holes", 128, dict(mask=key_mask(4, 1300))),
    ("bool mask with holes d64 causal", 64, dict(mask=key_mask(4, 1300), causal=True)),
    ("bool padding mask", 64, dict(mask=padding_mask(4, 1300, [1300, 64, 0, 777]))),
    ("bool padding mask + window", 128, dict(mask=padding_mask(4, 1300, [900, 1300, 1, 300]), window=(128, 128))),
]


@pytest.mark.parametrize("name,D,kw", PERSISTENT_CASES, ids=[c[0] for c in PERSISTENT_CASES])
def test_persistent_attention_matches_the_oracle_and_the_one_item_kernel(name, D, kw):
    """176 work items (B4 x 4 head pairs x 11 tiles of a ragged T = 1300: with two
    query heads a KV head an item is one 128-row tile of both) on 148 SMs run the
    persistent kernel: same numbers as the oracle within tolerance and as the
    one-item kernel bit for bit."""
    from svod_b200 import _lib as L
    dt, B, T, H, Hkv = O.BF16, 4, 1300, 8, 4
    rng = np.random.default_rng(len(name) + D)
    q, k, v = normal(rng, (B, T, H, D), 1.0, dt), normal(rng, (B, T, Hkv, D), 1.0, dt), normal(rng, (B, T, Hkv, D), 1.0, dt)
    okw = dict(kw)
    a = ops.Attn(causal=bool(kw.get("causal")), window=kw.get("window"))
    if "lens" in kw:
        okw["key_lens"] = np.array(okw.pop("lens"))
        a.keys = ops.KeyMask.Lens(torch.tensor(kw["lens"], dtype=torch.int32).cuda())
    if "mask" in kw:
        okw["key_mask"] = okw.pop("mask")
        a.keys = ops.KeyMask.Bool(torch.from_numpy(np.asarray(kw["mask"])).cuda())
    if "seg" in kw:
        seg = segments(B, T, 300)
        okw["seg_start"] = seg
        okw.pop("seg")
        a.seg_start = torch.from_numpy(seg.astype(np.int32)).cuda()
    if "chunk" in kw:
        a.chunk = ops.Chunk(*kw["chunk"])
    want = O.attention(q, k, v, dtype=dt, **okw)
    Q, K, V = dev(q, dt), dev(k, dt), dev(v, dt)
    got = host(ops.attention(Q, K, V, a))
    assert "persistent" in ops.chosen() and "head_pairs:1" in ops.chosen(), ops.chosen()
    ops.device_status()
    assert max_abs(got, want) < 2e-2 and mean_rel(got, want) < 5e-3
    lib = L.load()
    lib.svodb_config_set(b"attention|one_item", 1)
    try:
        one = host(ops.attention(Q, K, V, a))
        assert "persistent" not in ops.chosen()
    finally:
        lib.svodb_config_set(b"attention|one_item", 0)
    assert np.array_equal(got, one)
    again = host(ops.attention(Q, K, V, a))  # a second launch takes another queue slot
    assert np.array_equal(got, again)


@pytest.mark.parametrize("H,Hkv,pairs", [(6, 6, False), (6, 2, False), (8, 2, True)])
def test_persistent_attention_pairs_rows_or_heads(H, Hkv, pairs):
    """An item's two query tiles are consecutive tiles of one head, or — when every
    KV head serves an even number of query heads — the same tile of two heads.
    Either way the rows come out as the one-item kernel computes them."""
    from svod_b200 import _lib as L
    dt, B, T, D = O.BF16, 6, 1100, 64
    rng = np.random.default_rng(H * 10 + Hkv)
    q, k, v = normal(rng, (B, T, H, D), 1.0, dt), normal(rng, (B, T, Hkv, D), 1.0, dt), normal(rng, (B, T, Hkv, D), 1.0, dt)
    a = ops.Attn(causal=True, window=(300, 0))
    Q, K, V = dev(q, dt), dev(k, dt), dev(v, dt)
    got = host(ops.attention(Q, K, V, a))
    assert "persistent" in ops.chosen() and ("head_pairs:1" in ops.chosen()) == pairs, ops.chosen()
    want = O.attention(q, k, v, dtype=dt, causal=True, window=(300, 0))
    assert max_abs(got, want) < 2e-2 and mean_rel(got, want) < 5e-3
    lib = L.load()
    lib.svodb_config_set(b"attention|one_item", 1)
    try:
        one = host(ops.attention(Q, K, V, a))
    finally:
        lib.svodb_config_set(b"attention|one_item", 0)
    assert np.array_equal(got, one)


def test_persistent_attention_launches_overlapping_on_two_streams_keep_their_own_queues():
    """Each (device, stream) pair has its own work-queue head, so launches in
    flight at once on two streams hand out every item exactly once: the outputs
    equal those of the same calls made one after the other."""
    dt, B, T, H, Hkv, D = O.BF16, 4, 1300, 8, 4, 128
    rng = np.random.default_rng(77)
    sets = []
    for _ in range(2):
        q, k, v = normal(rng, (B, T, H, D), 1.0, dt), normal(rng, (B, T, Hkv, D), 1.0, dt), normal(rng, (B, T, Hkv, D), 1.0, dt)
        sets.append((dev(q, dt), dev(k, dt), dev(v, dt)))
    a = ops.Attn(causal=True)
    want = [host(ops.attention(*s_, a)) for s_ in sets]
    assert "persistent" in ops.chosen()
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    got = [[], []]
    for _ in range(6):
        for i in range(2):
            with torch.cuda.stream(streams[i]):
                got[i].append(ops.attention(*sets[i], a))
    torch.cuda.synchronize()
    ops.device_status()
    for i in range(2):
        for g in got[i]:
            assert np.array_equal(host(g), want[i])


def test_persistent_attention_reads_cache_slices_through_a_row_map():
    """More items than SMs with a cache (head slice + row map): the persistent
    kernel's loader looks the cache row up per item; same numbers as the oracle
    and as the one-item kernel."""
    from svod_b200 import _lib as L
    dt, B, rows, H, Hkv, D, T, Tk = O.BF16, 6, 8, 8, 4, 64, 1000, 1100
    rng = np.random.default_rng(31)
    q = normal(rng, (B, T, H, D), 1.0, dt)
    k = normal(rng, (rows, Tk, 2 * Hkv, D), 1.0, dt)
    v = normal(rng, (rows, Tk, 2 * Hkv, D), 1.0, dt)
    rm = np.array([7, 0, 3, 3, 5, 1])
    lens = np.array([Tk, 77, Tk - 1, 640, 0, 1024])
    cache = dict(head_start=Hkv, kv_heads=Hkv, row_map=rm)
    want = O.attention(q, k, v, key_lens=lens, cache=cache, dtype=dt)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32).cuda()
    a = ops.Attn(keys=ops.KeyMask.Lens(i32(lens)), cache=ops.Cache(Hkv, Hkv, i32(rm)))
    Q, K, V = dev(q, dt), dev(k, dt), dev(v, dt)
    got = host(ops.attention(Q, K, V, a))
    assert "persistent" in ops.chosen(), ops.chosen()
    ops.device_status()
    assert max_abs(got, want) < 2e-2 and mean_rel(got, want) < 5e-3
    assert not got[4].any()  # a lane without keys
    lib = L.load()
    lib.svodb_config_set(b"attention|one_item", 1)
    try:
        one = host(ops.attention(Q, K, V, a))
        assert "persistent" not in ops.chosen()
    finally:
        lib.svodb_config_set(b"attention|one_item", 0)
    assert np.array_equal(got, one)


@pytest.mark.parametrize("window", [None, (64, 64)], ids=["global", "local +-64"])
def test_full_size_masked_attention_properties_at_seq_8192_d64(window):
    """Size-independent checks at the ModernBERT layer shape (12 heads of 64, seq
    8192, bool prefix mask of ragged lengths, global or +-64 window), batch 4:
    (1) v = ones gives ones on every row that sees a key and zeros on a lane
    without keys; (2) keys past a lane's length do not matter (they are replaced
    by garbage); (3) sampled rows match an f32 softmax; (4) a replay is
    bit-identical."""
    g = torch.Generator(device="cuda").manual_seed(9)
    B, T, H, D = 4, 8192, 12, 64
    lens = [8192, 5000, 0, 2049]
    qkv = torch.randn(B, T, 3 * H * D, generator=g, device="cuda").to(torch.bfloat16)
    mask = (torch.arange(T, device="cuda")[None, :] < torch.tensor(lens, device="cuda")[:, None])
    a = ops.Attn(keys=ops.KeyMask.Bool(mask), window=window)
    o = ops.attention_packed(qkv, H, H, a)
    assert "persistent" in ops.chosen(), ops.chosen()
    ops.device_status()
    assert torch.equal(ops.attention_packed(qkv, H, H, a), o)
    q, k, v = (t_.reshape(B, T, H, D) for t_ in qkv.split(H * D, dim=-1))
    ones = ops.attention(q.contiguous(), k.contiguous(), torch.ones_like(v).contiguous(), a)
    left = window[0] if window else T
    for b, n in enumerate(lens):
        seen = torch.arange(T, device="cuda") - left < n if n > 0 else torch.zeros(T, dtype=torch.bool, device="cuda")
        assert float((ones[b][seen].float() - 1).abs().max() if seen.any() else 0.0) < 1e-2
        assert float(ones[b][~seen].float().abs().max() if (~seen).any() else 0.0) == 0.0
    noisy = qkv.clone().reshape(B, T, 3, H, D)
    for b, n in enumerate(lens):
        noisy[b, n:, 1:] = 77.0  # keys and values past the length
    o2 = ops.attention_packed(noisy.reshape(B, T, 3 * H * D), H, H, a)
    assert torch.equal(o2, o)
    for (b, h, i) in [(0, 0, 0), (1, 5, 4999), (1, 11, 6000), (3, 7, 2048), (0, 3, 8191)]:
        lo = max(0, i - window[0]) if window else 0
        hi = min(lens[b], i + window[1] + 1) if window else lens[b]
        if hi <= lo:
            assert float(o[b, i, h].float().abs().max()) == 0.0
            continue
        s = (k[b, lo:hi, h].float() @ q[b, i, h].float()) / math.sqrt(D)
        ref = torch.softmax(s, 0) @ v[b, lo:hi, h].float()
        assert float((o[b, i, h].float() - ref).abs().max()) < 2e-2


@pytest.mark.parametrize("kind", ["holes", "padding"])
def test_persistent_attention_scans_aligned_byte_masks_in_16_byte_pieces(kind):
    """A key count that is a multiple of 16 takes the vector scan of the mask row
    (T = 1300 above takes the byte loop): same numbers as the oracle and as the
    one-item kernel, with holes (the softmax reads the bits) and as padding."""
    from svod_b200 import _lib as L
    dt, B, T, H, Hkv, D = O.BF16, 4, 1280, 8, 4, 64
    rng = np.random.default_rng(5)
    q, k, v = normal(rng, (B, T, H, D), 1.0, dt), normal(rng, (B, T, Hkv, D), 1.0, dt), normal(rng, (B, T, Hkv, D), 1.0, dt)
    mask = key_mask(B, T) if kind == "holes" else padding_mask(B, T, [1280, 17, 0, 1279])
    if kind == "holes":
        mask[1, 900:] = False   # holes and a tail
        mask[2, :] = False      # a lane without keys
    want = O.attention(q, k, v, key_mask=mask, dtype=dt)
    a = ops.Attn(keys=ops.KeyMask.Bool(torch.from_numpy(np.asarray(mask)).cuda()))
    Q, K, V = dev(q, dt), dev(k, dt), dev(v, dt)
    got = host(ops.attention(Q, K, V, a))
    assert "persistent" in ops.chosen(), ops.chosen()
    ops.device_status()
    assert max_abs(got, want) < 2e-2 and mean_rel(got, want) < 5e-3
    lib = L.load()
    lib.svodb_config_set(b"attention|one_item", 1)
    try:
        one = host(ops.attention(Q, K, V, a))
    finally:
        lib.svodb_config_set(b"attention|one_item", 0)
    assert np.array_equal(got, one)


def test_f16_scores_stay_in_f32_on_the_tensor_core_kernel():
    """tensor/src/test/unit/transformer.rs:170-190 on the GPU: 64 products of
    100*100 overflow float16; the kernel's f32 accumulator keeps the scores finite
    and key 0, ahead by 800 in score, takes every query to V[0] = 1."""
    dt = O.F16
    q = np.full((1, 2, 1, 64), 100.0)
    k = np.stack([np.full(64, 100.0), np.full(64, 99.0)]).reshape(1, 2, 1, 64)
    v = np.repeat(np.array([1.0, 100.0]).reshape(1, 2, 1, 1), 64, axis=-1)
    got = host(ops.attention(dev(q, dt), dev(k, dt), dev(v, dt)))
    assert "kernel flash_attention" in ops.chosen()
    assert np.isfinite(got).all() and np.abs(got - 1.0).max() < 1e-3
