"""GPU parity of `ops.linear` (tcgen05 GEMM + fused epilogue, and the generic
path) against the oracle: the reference's epilogue recipe
(tk/src/test/unit/rows.rs:77-145, seed 17, 64^3 and 256^3, rel 1.6e-2), its
op-vs-graph cases (ops.rs:163-205, rel 2e-2) and the benchmark sweep shapes."""
import numpy as np
import pytest
import torch

from oracle import svod_oracle as O
from svod_b200 import ops
from tests.test_oracle_pins import EPILOGUES, gemm_recipe
from tests.util import dev, host, max_abs, mean_rel, rel_close

pytestmark = pytest.mark.gpu


def run_linear(x, w, dt, bias=None, act=0, gated=False, residual=None, scale=None, rope=None):
    o = ops.Linear(bias=dev(bias, dt) if bias is not None else None, act=ops.Act(act), gated=gated,
                   residual=dev(residual, dt) if residual is not None else None, scale=scale)
    if rope is not None:
        cos, sin, nh, hd = rope
        T = x.shape[1]
        o.rope = ops.Rotary(dev(cos, dt).view(1, T, 1, hd // 2), dev(sin, dt).view(1, T, 1, hd // 2), nh, hd)
    return host(ops.linear(dev(x, dt), dev(w, dt), o))


@pytest.mark.parametrize("size", [64, 256])
@pytest.mark.parametrize("which", range(8))
def test_epilogues_match_the_reference_recipe(size, which):
    epi = EPILOGUES[which]
    a, w, bias, res = gemm_recipe(size, size, size, epi)
    want = O.linear(a, w, bias, epi.get("act", 0), epi.get("gated", False), res, epi.get("scale"), dtype=O.BF16)
    got = run_linear(a, w, O.BF16, bias, epi.get("act", 0), epi.get("gated", False), res, epi.get("scale"))
    assert "kernel gemm" in ops.chosen()
    assert rel_close(got, want, 1.6e-2)


OP_CASES = [
    # (lead, n, k, dtype, bias, act, gated, residual)  -- tk/src/test/unit/ops.rs:163-171
    ((37,), 96, 64, O.BF16, True, O.ACT_GELU, False, True),
    ((3, 50), 96, 64, O.BF16, True, 0, False, False),
    ((300,), 200, 48, O.BF16, False, O.ACT_SILU, False, False),
    ((2048,), 512, 512, O.BF16, True, 0, False, True),
    ((77,), 96, 128, O.BF16, True, O.ACT_SILU, True, False),
    ((77,), 96, 128, O.BF16, False, O.ACT_GELU, True, True),
    ((129,), 264, 80, O.F16, True, O.ACT_GELU, False, True),
    ((1, 1), 8, 16, O.BF16, True, 0, False, False),
    ((1000,), 1152, 768, O.BF16, False, O.ACT_GELU, True, True),
]


@pytest.mark.parametrize("lead,n,k,dt,bias,act,gated,residual", OP_CASES)
def test_linear_matches_the_oracle(lead, n, k, dt, bias, act, gated, residual):
    rng = np.random.default_rng(n * 7 + k)
    halves = 2 if gated else 1
    x = O.round_to(dt, rng.uniform(-1, 1, lead + (k,)))
    w = O.round_to(dt, rng.uniform(-1, 1, (halves * n, k)) * 0.3)
    b = O.round_to(dt, rng.uniform(-1, 1, halves * n)) if bias else None
    r = O.round_to(dt, rng.uniform(-1, 1, lead + (n,))) if residual else None
    want = O.linear(x, w, b, act, gated, r, dtype=dt)
    got = run_linear(x, w, dt, b, act, gated, r)
    assert "kernel gemm" in ops.chosen()
    assert got.shape == want.shape
    assert rel_close(got, want, 2e-2)


@pytest.mark.parametrize("dt,m,n,k", [(O.F32, 37, 96, 64), (O.BF16, 50, 100, 64), (O.BF16, 77, 96, 40), (O.F32, 5, 7, 3)])
def test_shapes_and_dtypes_without_a_tile_kernel_take_the_generic_path(dt, m, n, k):
    rng = np.random.default_rng(1)
    x = O.round_to(dt, rng.standard_normal((m, k)))
    w = O.round_to(dt, rng.standard_normal((2 * n, k)) * 0.2)
    b = O.round_to(dt, rng.standard_normal(2 * n))
    r = O.round_to(dt, rng.standard_normal((m, n)))
    want = O.linear(x, w, b, O.ACT_SILU, True, r, 0.5, dtype=dt)
    got = run_linear(x, w, dt, b, O.ACT_SILU, True, r, 0.5)
    assert ops.chosen().startswith("linear: graph")
    assert rel_close(got, want, 1e-4 if dt == O.F32 else 2e-2)


@pytest.mark.parametrize("B,T,k,heads,hd,extra,bias", [(2, 200, 768, 24, 64, 768, False), (2, 37, 128, 4, 64, 64, True),
                                                        (1, 130, 128, 2, 128, 256, False), (2, 50, 64, 2, 32, 16, False)])
def test_rope_in_the_projection_store(B, T, k, heads, hd, extra, bias):
    """`Rotary` (tk/src/ops/linear.rs:45-56): the first heads*hd columns turned
    by position, the rest stored as they are. hd 32 has no turning tile and
    takes the generic rotation."""
    dt = O.BF16
    rng = np.random.default_rng(T)
    n = heads * hd + extra
    x = O.round_to(dt, rng.standard_normal((B, T, k)))
    w = O.round_to(dt, rng.standard_normal((n, k)) / np.sqrt(k))
    b = O.round_to(dt, rng.standard_normal(n)) if bias else None
    cos, sin = O.rope_table(10000.0, np.arange(T), hd, dt)
    want = O.linear(x, w, b, rope=(cos, sin, heads, hd), dtype=dt)
    got = run_linear(x, w, dt, b, rope=(cos, sin, heads, hd))
    assert ("kernel gemm" in ops.chosen()) == (hd in (64, 128))
    assert rel_close(got, want, 2e-2)


def test_into_stores_a_channel_window():
    """`into` (tk/src/ops/mod.rs:431-477): the output stored into channels
    [at, at+N) of a wider buffer, the other channels untouched."""
    dt = O.BF16
    rng = np.random.default_rng(9)
    x = O.round_to(dt, rng.standard_normal((70, 64)))
    w = O.round_to(dt, rng.standard_normal((32, 64)) * 0.2)
    wide = torch.full((70, 96), 3.0, dtype=torch.bfloat16, device="cuda")
    out = ops.linear(dev(x, dt), dev(w, dt), ops.Linear(into=(wide, 32)))
    assert out.data_ptr() == wide.data_ptr()
    got = host(wide)
    assert rel_close(got[:, 32:64], O.linear(x, w, dtype=dt), 2e-2)
    assert np.all(got[:, :32] == 3.0) and np.all(got[:, 64:] == 3.0)


@pytest.mark.parametrize("m", [512, 4096, 32768])
@pytest.mark.parametrize("nk", [768, 1024, 4096])
@pytest.mark.parametrize("epi", ["gelu", "gelu_tanh", "swiglu"])
def test_sweep_shapes_of_the_gemm_benchmark(m, nk, epi):
    """Every shape of the benchmark sweep (M in {512, 4096, 32768}, N = K in
    {768, 1024, 4096}): bf16 N(0,0.02) inputs and bias, erf-GELU, GELU (tanh) and
    SwiGLU (gate rows over up rows) epilogues. The whole product runs on the
    GPU; 64 seeded output rows (the first and last among them) are compared
    with the oracle on the same rows: max-abs 2e-2 / mean-rel 5e-3."""
    dt = O.BF16
    g = torch.Generator(device="cuda").manual_seed(2000 + m + nk)
    gated = epi == "swiglu"
    halves = 2 if gated else 1
    x = (torch.randn(m, nk, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    w = (torch.randn(halves * nk, nk, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    b = (torch.randn(halves * nk, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    act = dict(gelu=O.ACT_GELU, gelu_tanh=O.ACT_GELU_TANH, swiglu=O.ACT_SILU)[epi]
    y = ops.linear(x, w, ops.Linear(bias=b, act=ops.Act(act), gated=gated))
    assert "kernel gemm" in ops.chosen()
    rows = np.unique(np.concatenate([[0, m - 1], np.random.default_rng(m + nk).integers(0, m, 62)]))
    idx = torch.from_numpy(rows).cuda()
    want = O.linear(host(x[idx]), host(w), host(b), act, gated, dtype=dt)
    got = host(y[idx])
    assert got.shape == want.shape == (len(rows), nk)
    assert max_abs(got, want) <= 2e-2 and mean_rel(got, want) <= 5e-3, (max_abs(got, want), mean_rel(got, want))


def test_full_size_gemm_is_linear_in_its_input():
    """Size-independent property at the sweep's largest shape (M 32768, N = K =
    4096): with a power-of-two factor, linear(2x) == 2*linear(x) exactly and
    a second run is bit-identical."""
    g = torch.Generator(device="cuda").manual_seed(3)
    x = (torch.randn(32768, 4096, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    w = (torch.randn(4096, 4096, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    y1 = ops.linear(x, w)
    y2 = ops.linear(x * 2, w)
    assert torch.equal(y2, y1 * 2)
    assert torch.equal(ops.linear(x, w), y1)
    # spot rows against an f32 product of the same inputs
    rows = torch.tensor([0, 777, 32767], device="cuda")
    ref = x[rows].float() @ w.float().t()
    assert float((y1[rows].float() - ref).abs().max()) <= 2e-2


@pytest.mark.parametrize("dt,B,T,k,H,Hkv,hd,qn,kn,rope,kernel", [
    (O.BF16, 2, 200, 256, 4, 2, 128, True, True, "shared", True),     # Qwen3's layout: in the store
    (O.BF16, 2, 130, 128, 2, 1, 128, True, False, "per_batch", True),  # per-row tables, no k norm
    (O.F16, 1, 77, 128, 2, 2, 128, False, False, "shared", True),      # rotation only
    (O.BF16, 1, 64, 128, 2, 2, 128, True, True, None, True),           # norm only
    (O.F16, 2, 50, 128, 4, 2, 64, True, True, "shared", False),        # 64-wide heads: projection, then in place
    (O.F32, 1, 9, 40, 2, 1, 16, True, True, "shared", False),          # f32: exact projection, then in place
])
def test_qkv_prologue_in_the_projection_store(dt, B, T, k, H, Hkv, hd, qn, kn, rope, kernel):
    """`Linear(qkv=...)`: the `ops::heads` prologue applied to the projection's
    accumulator; the packed result equals `heads(linear(x, w))` laid back side
    by side (the oracle rounds between the two ops, the fused store does not:
    the tolerance of the heads recipe covers it)."""
    rng = np.random.default_rng(B * 1000 + T)
    n = (H + 2 * Hkv) * hd
    x = O.round_to(dt, rng.standard_normal((B, T, k)))
    w = O.round_to(dt, rng.standard_normal((n, k)) / np.sqrt(k))
    qw = O.round_to(dt, 1 + 0.2 * rng.standard_normal(hd)) if qn else None
    kw = O.round_to(dt, 1 + 0.2 * rng.standard_normal(hd)) if kn else None
    cos = sin = None
    if rope == "shared":
        cos, sin = O.rope_table(1e6, np.arange(T), hd, dt)
    elif rope == "per_batch":
        pos = np.stack([(np.arange(T) * (b + 2)) % 97 for b in range(B)])
        cos, sin = O.rope_table(1e6, pos.reshape(-1), hd, dt)
        cos, sin = cos.reshape(B, T, hd // 2), sin.reshape(B, T, hd // 2)
    q, kk, v = O.heads(O.linear(x, w, dtype=dt), H, Hkv, hd, qw, kw, 1e-6, cos, sin, dt)
    want = np.concatenate([q.reshape(B, T, -1), kk.reshape(B, T, -1), v.reshape(B, T, -1)], axis=-1)
    tabs = None
    if cos is not None:
        tabs = (dev(cos, dt).view(-1, T, 1, hd // 2), dev(sin, dt).view(-1, T, 1, hd // 2))
    o = ops.Linear(qkv=ops.Qkv(H, Hkv, hd, dev(qw, dt) if qn else None, dev(kw, dt) if kn else None, 1e-6, tabs))
    got = host(ops.linear(dev(x, dt), dev(w, dt), o))
    assert ("kernel gemm" in ops.chosen()) == (dt != O.F32)
    tol = 1e-4 if dt == O.F32 else 2e-2
    assert rel_close(got, want, 1e-3 if dt == O.F32 else 2e-2)
    assert mean_rel(got, want) < (1e-5 if dt == O.F32 else 5e-3)
    assert rel_close(got[..., (H + Hkv) * hd:], want[..., (H + Hkv) * hd:], tol)  # v: the plain projection
    # attention reads the packed projection in place
    a = host(ops.attention_packed(dev(got, dt), H, Hkv, ops.Attn(causal=True)))
    a_want = O.attention(q, kk, v, causal=True, dtype=dt)
    assert max_abs(a, a_want) < (1e-3 if dt == O.F32 else 2e-2)


def test_qkv_prologue_excludes_the_other_epilogues():
    dt = O.BF16
    x, w = dev(np.zeros((1, 8, 64)), dt), dev(np.zeros((4 * 64, 64)), dt)
    for bad in (dict(gated=True), dict(act=ops.Act.SILU), dict(scale=2.0), dict(residual=dev(np.zeros((1, 8, 256)), dt))):
        with pytest.raises(ops.OpsError) as e:
            ops.linear(x, w, ops.Linear(qkv=ops.Qkv(2, 1, 64), **bad))
        assert e.value.kind in ("Graph", "Shape")
    with pytest.raises(ops.OpsError) as e:
        ops.linear(x, w, ops.Linear(qkv=ops.Qkv(3, 1, 64)))
    assert e.value.kind == "Shape"


@pytest.mark.parametrize("m,n,k,kw", [
    (4864, 1024, 256, dict()),                                   # 19 x 4 pair tiles
    (4864, 1024, 320, dict(bias=True, act=1)),                   # bias + GELU, k not a multiple of 64... of 128
    (4964, 1000, 256, dict(bias=True, residual=True, scale=0.5)),  # ragged rows (the odd CTA of the last tile is empty) and columns
    (4864, 512, 256, dict(act=2, gated=True)),                   # SwiGLU: gate rows in the even CTA, up rows in the odd one
    (9728, 512, 192, dict(bias=True, act=2, gated=True, residual=True)),
    (4964, 1000, 512, dict(bias=True, act=1, residual=True, scale=0.5)),  # activation with a residual: eight epilogue warps
    (4964, 1000, 512, dict(bias=True, act=1, scale=0.5)),  # sixteen epilogue warps (per-warp slabs), ragged rows and columns
    (4900, 1096, 2048, dict(act=1)),                       # sixteen warps without a bias, rows ragged inside a 32-row slab
    (4864, 1024, 512, dict(act=3)),                                        # tanh GELU, four column groups
])
def test_cta_pair_gemm_matches_the_oracle(m, n, k, kw):
    """Shapes with at least one 256 x 256 tile per CTA pair run the
    `cta_group::2` kernel; same epilogue, same tolerance as the one-CTA kernel
    (tk/src/test/unit/rows.rs:77-145: rel 1.6e-2)."""
    dt = O.BF16
    rng = np.random.default_rng(m + n + k)
    gated = kw.get("gated", False)
    x = O.round_to(dt, rng.standard_normal((m, k)))
    w = O.round_to(dt, rng.standard_normal(((2 if gated else 1) * n, k)) / np.sqrt(k))
    b = O.round_to(dt, rng.standard_normal((2 if gated else 1) * n)) if kw.get("bias") else None
    r = O.round_to(dt, rng.standard_normal((m, n))) if kw.get("residual") else None
    want = O.linear(x, w, b, act=kw.get("act", 0), gated=gated, residual=r, scale=kw.get("scale"), dtype=dt)
    # the one-CTA kernel (config code 256): same k order, same epilogue
    from svod_b200 import _lib as L
    lib = L.load()
    run_linear(x, w, dt, b, kw.get("act", 0), gated, r, kw.get("scale"))
    key = lib.svodb_last_config_key()
    lib.svodb_config_set(key, 256)
    one = run_linear(x, w, dt, b, kw.get("act", 0), gated, r, kw.get("scale"))
    assert "cta_pair" not in ops.chosen()
    lib.svodb_config_set(key, 512)  # the config store's code for the pair kernel
    try:
        got = run_linear(x, w, dt, b, kw.get("act", 0), gated, r, kw.get("scale"))
        assert "cta_pair:1" in ops.chosen(), ops.chosen()
    finally:
        lib.svodb_config_set(key, 0)
    assert rel_close(got, want, 1.6e-2)
    assert mean_rel(got, want) < 5e-3
    assert max_abs(got, one) == 0.0


def test_long_k_projections_take_the_cta_pair_kernel_by_default():
    dt = O.BF16
    rng = np.random.default_rng(11)
    m, n, k = 5120, 1024, 1024
    x = O.round_to(dt, rng.standard_normal((m, k)))
    w = O.round_to(dt, rng.standard_normal((n, k)) / np.sqrt(k))
    got = run_linear(x, w, dt)
    assert "cta_pair:1" in ops.chosen()
    assert rel_close(got, O.linear(x, w, dtype=dt), 1.6e-2)


@pytest.mark.parametrize("dt,B,T,k,H,Hkv,qn,kn,rope", [
    (O.BF16, 4, 1280, 1024, 4, 2, True, True, "shared"),      # 20 x 4 pair tiles, Qwen3's layout
    (O.F16, 3, 2560, 1024, 2, 2, True, False, "per_batch"),   # tables per row of the batch
    (O.BF16, 4, 1280, 1024, 4, 2, True, True, None),           # norm only
    (O.BF16, 3, 1664, 1024, 4, 2, False, False, "shared"),     # rotation only, ragged last row tile
])
def test_qkv_prologue_on_the_cta_pair_kernel(dt, B, T, k, H, Hkv, qn, kn, rope):
    """The attention prologue in the store of the CTA-pair kernel (rotation tables
    TMA-loaded per tile) against `heads(linear(x, w))`, and against the one-CTA
    head epilogue bit for bit."""
    hd = 128
    rng = np.random.default_rng(T + k)
    n = (H + 2 * Hkv) * hd
    x = O.round_to(dt, rng.standard_normal((B, T, k)))
    w = O.round_to(dt, rng.standard_normal((n, k)) / np.sqrt(k))
    qw = O.round_to(dt, 1 + 0.2 * rng.standard_normal(hd)) if qn else None
    kw = O.round_to(dt, 1 + 0.2 * rng.standard_normal(hd)) if kn else None
    cos = sin = None
    if rope == "shared":
        cos, sin = O.rope_table(1e6, np.arange(T), hd, dt)
    elif rope == "per_batch":
        pos = np.stack([(np.arange(T) * (b + 2)) % 997 for b in range(B)])
        cos, sin = O.rope_table(1e6, pos.reshape(-1), hd, dt)
        cos, sin = cos.reshape(B, T, hd // 2), sin.reshape(B, T, hd // 2)
    q, kk, v = O.heads(O.linear(x, w, dtype=dt), H, Hkv, hd, qw, kw, 1e-6, cos, sin, dt)
    want = np.concatenate([q.reshape(B, T, -1), kk.reshape(B, T, -1), v.reshape(B, T, -1)], axis=-1)
    tabs = None
    if cos is not None:
        tabs = (dev(cos, dt).view(-1, T, 1, hd // 2), dev(sin, dt).view(-1, T, 1, hd // 2))
    o = ops.Linear(qkv=ops.Qkv(H, Hkv, hd, dev(qw, dt) if qn else None, dev(kw, dt) if kn else None, 1e-6, tabs))
    X, W = dev(x, dt), dev(w, dt)
    got = host(ops.linear(X, W, o))
    assert "cta_pair:1" in ops.chosen(), ops.chosen()
    assert rel_close(got, want, 2e-2) and mean_rel(got, want) < 5e-3
    from svod_b200 import _lib as L
    lib = L.load()
    key = lib.svodb_last_config_key()
    lib.svodb_config_set(key, 256)
    try:
        one = host(ops.linear(X, W, o))
        assert "cta_pair" not in ops.chosen() and "kernel gemm" in ops.chosen()
    finally:
        lib.svodb_config_set(key, 0)
    assert max_abs(got, one) == 0.0


@pytest.mark.parametrize("dt,B,T,k,heads,extra", [
    (O.BF16, 4, 1664, 768, 8, 256),    # ModernBERT's layout in small: q,k heads turned, v columns stored as they are
    (O.F16, 5, 1408, 512, 12, 0),      # every column turned, ragged last row tile (27.5 pair tiles of rows)
])
def test_rope_of_64_wide_heads_on_the_cta_pair_kernel(dt, B, T, k, heads, extra):
    """`Rotary` with 64-wide heads in the CTA-pair kernel's store (table slabs of
    64-byte rows by TMA) against the oracle and, bit for bit, against the
    one-CTA kernel's direct-store rotation."""
    hd = 64
    rng = np.random.default_rng(T + k)
    n = heads * hd + extra
    x = O.round_to(dt, rng.standard_normal((B, T, k)))
    w = O.round_to(dt, rng.standard_normal((n, k)) / np.sqrt(k))
    cos, sin = O.rope_table(160000.0, np.arange(T), hd, dt)
    want = O.linear(x, w, None, rope=(cos, sin, heads, hd), dtype=dt)
    o = ops.Linear(rope=ops.Rotary(dev(cos, dt).view(1, T, 1, hd // 2), dev(sin, dt).view(1, T, 1, hd // 2), heads, hd))
    X, W = dev(x, dt), dev(w, dt)
    got = host(ops.linear(X, W, o))
    assert "cta_pair:1" in ops.chosen(), ops.chosen()
    ops.device_status()
    assert rel_close(got, want, 2e-2) and mean_rel(got, want) < 5e-3
    from svod_b200 import _lib as L
    lib = L.load()
    key = lib.svodb_last_config_key()
    lib.svodb_config_set(key, 256)
    try:
        one = host(ops.linear(X, W, o))
        assert "cta_pair" not in ops.chosen() and "kernel gemm" in ops.chosen()
    finally:
        lib.svodb_config_set(key, 0)
    assert max_abs(got, one) == 0.0


SPLIT_K_CASES = [
    # (m, n, k, dtype, k_splits (None = the op layer's choice), epilogue)
    (512, 4096, 4096, O.BF16, 2, dict(bias=True, act=1)),               # the sweep's one-wave shape: 32 tiles x 2 pieces
    (512, 1024, 2048, O.BF16, 4, dict(bias=True, residual=True, scale=0.5)),
    (700, 1000, 2240, O.BF16, 3, dict(bias=True, act=3, residual=True)),  # ragged rows and columns, 35 k-blocks in 3 uneven pieces
    (256, 512, 4096, O.F16, 8, dict()),                                   # one pair tile a column block, 8 pieces
    (1024, 768, 3072, O.F16, 6, dict(act=2, residual=True)),              # 4 x 3 tiles x 6 pieces = 72 items on 74 pairs
]


@pytest.mark.parametrize("m,n,k,dt,splits,kw", SPLIT_K_CASES)
def test_split_k_matches_the_oracle_and_the_unsplit_kernel(m, n, k, dt, splits, kw):
    """The reference's tail split + merge (tk/src/kernels/gemm.rs:454-466,750-808):
    f32 partials of pieces of the k loop, merged in piece order with the epilogue
    applied once. Same tolerance as the unsplit GEMM; two runs are bit-equal."""
    rng = np.random.default_rng(m + n + k)
    x = O.round_to(dt, rng.standard_normal((m, k)))
    w = O.round_to(dt, rng.standard_normal((n, k)) / np.sqrt(k))
    b = O.round_to(dt, rng.standard_normal(n)) if kw.get("bias") else None
    r = O.round_to(dt, rng.standard_normal((m, n))) if kw.get("residual") else None
    want = O.linear(x, w, b, act=kw.get("act", 0), residual=r, scale=kw.get("scale"), dtype=dt)

    def run(k_splits):
        o = ops.Linear(bias=dev(b, dt) if b is not None else None, act=ops.Act(kw.get("act", 0)),
                       residual=dev(r, dt) if r is not None else None, scale=kw.get("scale"), k_splits=k_splits)
        return host(ops.linear(dev(x, dt), dev(w, dt), o))

    got = run(splits)
    chosen = ops.chosen()
    assert f"k_splits:{splits}" in chosen, chosen
    assert rel_close(got, want, 1.6e-2)
    assert mean_rel(got, want) < 5e-3
    assert max_abs(run(splits), got) == 0.0          # the merge order does not depend on who came last
    one = run(1)
    assert "k_splits" not in ops.chosen()
    assert rel_close(got, one, 1.6e-2)


def test_split_k_is_the_callers_choice_and_never_splits_a_gated_projection():
    dt = torch.bfloat16
    # left to the op layer, the k loop stays in one piece (the split kernel measured slower)
    assert ops.auto_k_splits(512, 4096, 4096, ops.Linear(), dt) == 1
    x = torch.randn(512, 2048, device="cuda").to(dt)
    w = (torch.randn(1024, 2048, device="cuda") * 0.02).to(dt)
    ops.linear(x, w, ops.Linear())
    assert "k_splits" not in ops.chosen()
    # asked for on a gated projection: the call runs unsplit (tk/src/kernels/gemm.rs:459-462)
    ops.linear(x, w, ops.Linear(gated=True, act=ops.Act.SILU, k_splits=4))
    assert "k_splits" not in ops.chosen()
    # asked for without a workspace through the C ABI: refused, not run
    from svod_b200 import _lib as L
    import ctypes as C
    y = torch.empty(512, 1024, device="cuda", dtype=dt)
    o = L.LinearOpts()
    o.k_splits = 2
    xd, wd, yd = ops._desc(x), ops._desc(w), ops._desc(y)
    rc = L.load().svodb_linear(ops._p(xd), ops._p(wd), C.byref(o), ops._p(yd), ops._stream())
    assert rc == L.ERR_WORKSPACE


def test_device_gelu_is_within_5e_6_of_erf_gelu_on_a_dense_grid():
    """The device's erf-GELU (`max(x,0) - a*2^P(a)`, one exponential) seen at f32
    precision: an f32 linear with an identity weight returns gelu(x) unrounded
    (the exact generic kernel shares `gelu_f` with the tile kernels' epilogues)."""
    n = 256
    x = np.linspace(-9.0, 9.0, 64 * n, dtype=np.float32).reshape(64, n)
    w = np.eye(n, dtype=np.float32)
    got = ops.linear(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), ops.Linear(act=ops.Act.GELU))
    assert "graph" in ops.chosen()
    err = np.abs(got.cpu().numpy().astype(np.float64) - O.gelu_erf(x.astype(np.float64)))
    assert err.max() < 5e-6
    # and the tile kernel's epilogue, through bf16 rounding: within half a bf16 step of the pinned form
    xb = O.round_to(O.BF16, x)
    gb = host(ops.linear(dev(xb, O.BF16), dev(w, O.BF16), ops.Linear(act=ops.Act.GELU)))
    assert "kernel gemm" in ops.chosen()
    want = O.round_to(O.BF16, O.gelu_as(xb))
    assert np.max(np.abs(gb - want) / np.maximum(np.abs(want), 1e-2)) < 2.0 ** -7
