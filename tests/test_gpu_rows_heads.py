"""GPU parity of the row kernels and the attention prologue against the oracle,
on the reference's own recipes (tk/src/test/unit/rows.rs:205-256,
heads.rs:112-161, ops.rs:645-731) and through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import svod_oracle as O
from svod_b200 import ops
from tests.test_oracle_pins import heads_recipe, norm_recipe
from tests.util import dev, host, max_abs, rel_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind,d,residual,bias", [
    ("layer", 512, False, True), ("layer", 512, False, False), ("layer", 1024, True, True),
    ("rms", 512, True, False), ("rms", 1024, False, False), ("layer", 512, True, True),
    ("rms", 2048, False, False), ("layer", 768, False, False), ("layer", 256, True, True), ("rms", 1536, True, False)])
def test_norms_match_the_reference_recipe(kind, d, residual, bias):
    """`norms_match_on_device`: rows 37 (partial block), eps 1e-5, seed 5; out
    within rel 1e-2, the fused sum exact."""
    rows, eps, dt = 37, 1e-5, O.BF16
    x, r, w, b = norm_recipe(kind, rows, d, residual, bias, 5)
    want, wsum = O.norm_rows(kind, x, w, b, r, eps, dt)
    X, W = dev(x, dt), dev(w, dt)
    Bt = dev(b, dt) if b is not None else None
    if kind == "layer":
        got = ops.add_layer_norm(X, dev(r, dt), W, Bt, eps) if residual else (None, ops.layer_norm(X, W, Bt, eps))
    else:
        got = ops.add_rms_norm(X, dev(r, dt), W, eps) if residual else (None, ops.rms_norm(X, W, eps))
    assert ops.chosen().startswith(("layer_norm: kernel", "rms_norm: kernel"))
    assert rel_close(host(got[1]), want, 1e-2)
    if residual:
        assert np.array_equal(host(got[0]), wsum)


@pytest.mark.parametrize("dt,d", [(O.F16, 1024), (O.BF16, 100), (O.F32, 300), (O.F16, 4096)])
def test_norms_outside_the_kernel_shape_take_the_generic_path(dt, d):
    rng = np.random.default_rng(d)
    x = O.round_to(dt, rng.standard_normal((3, 7, d)) * 2 + 1.5)
    w = O.round_to(dt, 1 + 0.5 * rng.standard_normal(d))
    b = O.round_to(dt, 0.5 * rng.standard_normal(d))
    r = O.round_to(dt, rng.standard_normal((3, 7, d)))
    want, wsum = O.norm_rows("layer", x, w, b, r, 1e-5, dt)
    s, got = ops.add_layer_norm(dev(x, dt), dev(r, dt), dev(w, dt), dev(b, dt), 1e-5)
    tol = 1e-4 if dt == O.F32 else 1e-2
    assert rel_close(host(got), want, tol)
    assert max_abs(host(s), wsum) <= (1e-6 if dt == O.F32 else 0.0)
    if d in (100, 300, 4096):
        assert "graph" in ops.chosen()


@pytest.mark.parametrize("cap,t,H,Hkv,d,qn,kn,rope", [
    (2, 9, 4, 2, 64, True, True, False), (2, 10, 4, 2, 128, True, True, True), (2, 5, 2, 2, 64, False, False, False),
    (2, 8, 4, 1, 64, True, False, None), (2, 3, 2, 1, 32, False, False, None), (2, 37, 4, 2, 64, True, True, False),
    (2, 40, 8, 2, 128, True, True, True), (2, 16, 2, 2, 64, False, False, None), (1, 7, 2, 2, 256, True, True, False),
    (1, 7, 3, 1, 16, True, True, False), (2, 6, 2, 2, 48, True, True, False)])
def test_heads_match_the_reference_recipe(cap, t, H, Hkv, d, qn, kn, rope):
    """`program_matches_the_reference` / `kernel_matches_the_program`: q, k
    within abs 2e-2, v exact."""
    dt = O.BF16
    qkv, qw, kw, cos, sin = heads_recipe(cap, t, H, Hkv, d, qn, kn, rope, 7)
    want = O.heads(qkv, H, Hkv, d, qw, kw, 1e-6, cos, sin, dt)
    tabs = None
    if cos is not None:
        tabs = (dev(cos, dt).view(-1, t, 1, d // 2), dev(sin, dt).view(-1, t, 1, d // 2))
    got = ops.heads(dev(qkv, dt), ops.Qkv(H, Hkv, d, dev(qw, dt) if qn else None, dev(kw, dt) if kn else None,
                                         1e-6, tabs))
    assert ("kernel heads" in ops.chosen()) == (d in (16, 32, 64, 128, 256))
    assert max_abs(host(got[0]), want[0]) < 2e-2
    assert max_abs(host(got[1]), want[1]) < 2e-2
    assert np.array_equal(host(got[2]), want[2])


def test_heads_f16_and_full_size_row_is_a_copy_for_v():
    dt = O.F16
    rng = np.random.default_rng(0)
    B, T, H, Hkv, d = 2, 130, 16, 8, 128
    qkv = O.round_to(dt, rng.standard_normal((B, T, (H + 2 * Hkv) * d)))
    w = O.round_to(dt, 1 + 0.1 * rng.standard_normal(d))
    cos, sin = O.rope_table(1e6, np.arange(T), d, dt)
    want = O.heads(qkv, H, Hkv, d, w, w, 1e-6, cos, sin, dt)
    W = dev(w, dt)
    got = ops.heads(dev(qkv, dt), ops.Qkv(H, Hkv, d, W, W, 1e-6, (dev(cos, dt).view(1, T, 1, d // 2),
                                                                   dev(sin, dt).view(1, T, 1, d // 2))))
    for g, w_ in zip(got[:2], want[:2]):
        assert max_abs(host(g), w_) < 1e-2
    assert np.array_equal(host(got[2]), want[2])


def test_rope_table_matches_the_f32_recipe():
    for theta, hd in ((1e6, 128), (160000.0, 64), (10000.0, 64)):
        cos, sin = ops.rope_table(theta, 4096, hd, torch.float32)
        wc, ws = O.rope_table(theta, np.arange(4096), hd, O.F32)
        # position * frequency reaches thousands of radians: f32 pow/mul ulps
        # move the angle by ~1e-3 at the high positions, hence the bound.
        assert max_abs(host(cos), wc) < 5e-3 and max_abs(host(sin), ws) < 5e-3
        cos, sin = ops.rope_table(theta, 512, hd, torch.bfloat16)
        wc, ws = O.rope_table(theta, np.arange(512), hd, O.BF16)
        assert max_abs(host(cos), wc) < 8e-3 and max_abs(host(sin), ws) < 8e-3


def test_embed_and_pool_are_exact():
    rng = np.random.default_rng(3)
    V, D, B, T, dt = 1000, 256, 3, 50, O.F16
    table = O.round_to(dt, rng.standard_normal((V, D)) * 0.02)
    pos = O.round_to(dt, rng.standard_normal((T + 2, D)) * 0.02)
    typ = O.round_to(dt, rng.standard_normal((1, D)) * 0.02)
    ids = rng.integers(2, V, (B, T))
    lens = [50, 20, 1]
    for b, l in enumerate(lens):
        ids[b, l:] = 1
    pid = O.xlmr_position_ids(ids, 1)
    want = O.round_to(dt, O.round_to(dt, table[ids] + pos[pid]) + typ[0])
    got = ops.embed(torch.from_numpy(ids).cuda(), dev(table, dt), dev(pos, dt), dev(typ, dt), 1)
    assert np.array_equal(host(got), want)
    got = ops.embed(torch.from_numpy(ids.astype(np.int32)).cuda(), dev(table, dt))
    assert np.array_equal(host(got), table[ids])
    h = O.round_to(dt, rng.standard_normal((B, T, D)))
    mask = np.arange(T)[None, :] < np.array(lens)[:, None]
    H = dev(h, dt)
    assert max_abs(host(ops.pool(H, None, ops.POOL_CLS)), O.pool(h, mask, "cls")) < 1e-6
    assert max_abs(host(ops.pool(H, torch.from_numpy(mask).cuda(), ops.POOL_MEAN)), O.pool(h, mask, "mean")) < 1e-6
    L = torch.tensor(lens, dtype=torch.int32).cuda()
    assert max_abs(host(ops.pool(H, L, ops.POOL_LAST)), O.pool(h, None, "last", lengths=np.array(lens))) < 1e-6
    # an all-pad row pools to the zero vector and stays zero; the slot of a wider buffer is honoured
    mask[2] = False
    buf = torch.full((B, 2 * D), 7.0, device="cuda")
    out = ops.pool(H, torch.from_numpy(mask).cuda(), ops.POOL_MEAN, True, buf[:, :D])
    assert np.all(host(out)[2] == 0) and np.all(host(buf[:, D:]) == 7.0)


def off_boundary(x, dt, shift=3):
    """The same values as a contiguous device view that starts `shift` elements
    (6 bytes for a 16-bit type) past an allocation boundary."""
    flat = dev(np.asarray(x).reshape(-1), dt)
    buf = torch.zeros(flat.numel() + 16, dtype=flat.dtype, device="cuda")
    buf[shift:shift + flat.numel()] = flat
    view = buf[shift:shift + flat.numel()].view(np.asarray(x).shape)
    assert view.data_ptr() % 16 != 0 and view.is_contiguous()
    return view


def test_views_off_the_16_byte_boundary_take_the_generic_kernels():
    """The vector kernels move 16 bytes per access; a dense view that starts at
    an odd element is valid input and must run (on the element-wise kernels),
    not fault."""
    dt = O.BF16
    rng = np.random.default_rng(11)
    # norms: x, then the weight, off the boundary
    d = 512
    x = O.round_to(dt, rng.standard_normal((5, d)) * 2 + 1.5)
    w = O.round_to(dt, 1 + 0.5 * rng.standard_normal(d))
    r = O.round_to(dt, rng.standard_normal((5, d)))
    want, wsum = O.norm_rows("rms", x, w, None, r, 1e-6, dt)
    for X, W in ((off_boundary(x, dt), dev(w, dt)), (dev(x, dt), off_boundary(w, dt))):
        s, got = ops.add_rms_norm(X, dev(r, dt), W, 1e-6)
        assert "graph" in ops.chosen()
        assert rel_close(host(got), want, 1e-2) and np.array_equal(host(s), wsum)
    # heads: the packed projection off the boundary
    B, T, H, Hkv, hd = 1, 9, 4, 2, 64
    qkv, qw, kw, cos, sin = heads_recipe(B, T, H, Hkv, hd, True, True, False, 7)
    want = O.heads(qkv, H, Hkv, hd, qw, kw, 1e-6, cos, sin, dt)
    tabs = (dev(cos, dt).view(-1, T, 1, hd // 2), dev(sin, dt).view(-1, T, 1, hd // 2))
    got = ops.heads(off_boundary(qkv, dt), ops.Qkv(H, Hkv, hd, dev(qw, dt), dev(kw, dt), 1e-6, tabs))
    assert "graph" in ops.chosen()
    assert max_abs(host(got[0]), want[0]) < 2e-2 and max_abs(host(got[1]), want[1]) < 2e-2
    assert np.array_equal(host(got[2]), want[2])
    # embedding: the table off the boundary, same bits as the aligned lookup
    V, D = 50, 64
    table = O.round_to(dt, rng.standard_normal((V, D)))
    pos = O.round_to(dt, rng.standard_normal((12, D)))
    ids = rng.integers(2, V, (2, 7))
    pid = O.xlmr_position_ids(ids, 1)
    got = ops.embed(torch.from_numpy(ids).cuda(), off_boundary(table, dt), off_boundary(pos, dt, 5), None, 1)
    assert np.array_equal(host(got), O.round_to(dt, table[ids] + pos[pid]))
    ops.device_status()


@pytest.mark.parametrize("dt,D", [(O.F16, 1024), (O.BF16, 768), (O.BF16, 320)])
def test_embedding_lookup_with_the_norm_in_one_kernel(dt, D):
    """`embed_norm`: word + position + type rows (each add rounded) and the
    LayerNorm of the rounded sum, against the oracle and bit for bit against the
    two separate ops; D = 320 has no fused kernel and takes the two-pass path."""
    rng = np.random.default_rng(D)
    V, B, T = 500, 3, 70
    table = O.round_to(dt, rng.standard_normal((V, D)) * 0.02)
    pos = O.round_to(dt, rng.standard_normal((T + 2, D)) * 0.02)
    typ = O.round_to(dt, rng.standard_normal((1, D)) * 0.02)
    w = O.round_to(dt, 1 + 0.1 * rng.standard_normal(D))
    b = O.round_to(dt, 0.1 * rng.standard_normal(D))
    ids = rng.integers(2, V, (B, T))
    for r, l in enumerate([70, 33, 1]):
        ids[r, l:] = 1
    I = torch.from_numpy(ids).cuda()
    e = O.round_to(dt, O.round_to(dt, table[ids] + pos[O.xlmr_position_ids(ids, 1)]) + typ[0])
    want, _ = O.norm_rows("layer", e, w, b, eps=1e-5, dtype=dt)
    got = ops.embed_norm(I, dev(table, dt), dev(w, dt), dev(b, dt), 1e-5, dev(pos, dt), dev(typ, dt), 1)
    assert ("kernel embed_norm" in ops.chosen()) == (D % 256 == 0)
    assert rel_close(host(got), want, 1e-2)
    two = ops.layer_norm(ops.embed(I, dev(table, dt), dev(pos, dt), dev(typ, dt), 1), dev(w, dt), dev(b, dt), 1e-5)
    assert torch.equal(got, two)
    # ModernBERT's form: the table row alone, LayerNorm without bias, i32 ids
    want2, _ = O.norm_rows("layer", table[ids], w, None, eps=1e-5, dtype=dt)
    got2 = ops.embed_norm(I.to(torch.int32), dev(table, dt), dev(w, dt), None, 1e-5)
    assert rel_close(host(got2), want2, 1e-2)
    ops.device_status()


@pytest.mark.parametrize("dt,D,kind", [(O.BF16, 1024, "rms"), (O.BF16, 768, "layer"), (O.F16, 1024, None),
                                       (O.BF16, 320, "layer")])
def test_final_norm_pooling_and_l2_in_one_kernel(dt, D, kind):
    """`norm_pool` against the oracle's norm -> pool -> L2 for every pooling mode;
    D = 320 has no fused kernel and takes the unfused sequence through a scratch."""
    rng = np.random.default_rng(D + 1)
    B, T = 3, 90
    h = O.round_to(dt, rng.standard_normal((B, T, D)) * 2 + 0.5)
    w = O.round_to(dt, 1 + 0.1 * rng.standard_normal(D))
    lens = [90, 41, 0]
    mask = np.arange(T)[None, :] < np.array(lens)[:, None]
    normed = h if kind is None else O.norm_rows(kind, h, w, None, eps=1e-6, dtype=dt)[0]
    H, W = dev(h, dt), (None if kind is None else dev(w, dt))
    kw = dict(norm_w=W, eps=1e-6, layer=kind != "rms")
    M, Ln = torch.from_numpy(mask).cuda(), torch.tensor(lens, dtype=torch.int32).cuda()
    got = ops.norm_pool(H, aux=None, mode=ops.POOL_CLS, **kw)
    assert ("kernel norm_pool" in ops.chosen()) == (D % 256 == 0)
    assert max_abs(host(got), O.pool(normed, mask, "cls")) < 2e-4
    got = ops.norm_pool(H, aux=M, mode=ops.POOL_MEAN, **kw)
    want = O.pool(normed, mask, "mean")
    assert max_abs(host(got), want) < 2e-4 and np.all(host(got)[2] == 0)       # an all-pad row stays the zero vector
    got = ops.norm_pool(H, aux=Ln, mode=ops.POOL_LAST, **kw)
    assert max_abs(host(got), O.pool(normed, None, "last", lengths=np.array(lens))) < 2e-4
    idx = np.array([[0, 5], [40, 40], [89, 3]])
    got = ops.norm_pool(H, aux=torch.from_numpy(idx.astype(np.int32)).cuda(), mode=ops.POOL_GATHER, **kw)
    want = O.l2_normalize(np.stack([normed[b, t] for b in range(B) for t in idx[b]]))
    assert max_abs(host(got), want) < 2e-4
    # the slot of a wider buffer is honoured, unnormalised pooling too
    buf = torch.full((B, 2 * D), 7.0, device="cuda")
    out = ops.norm_pool(H, aux=M, mode=ops.POOL_MEAN, normalize=False, out=buf[:, :D], **kw)
    assert max_abs(host(out), O.pool(normed, mask, "mean", normalize=False)) < 2e-3
    assert np.all(host(buf[:, D:]) == 7.0)
    ops.device_status()
