"""The config store on a GPU: a `linear` shape's tile width and a decode
attention's key-split count are measured once, kept, replayed from the file, and
never change the numbers (the stand-in for tk/src/tune.rs)."""
import numpy as np
import pytest
import torch

from oracle import svod_oracle as O
from svod_b200 import _lib as L
from svod_b200 import ops, tune
from tests.util import dev, host, max_abs, normal

pytestmark = pytest.mark.gpu


def test_linear_tile_width_is_measured_once_and_replayed(tmp_path):
    lib = L.load()
    lib.svodb_config_clear()
    dt = O.BF16
    rng = np.random.default_rng(3)
    x, w = dev(normal(rng, (2048, 512), 1.0, dt), dt), dev(normal(rng, (1024, 512), 0.05, dt), dt)
    base = host(ops.linear(x, w))
    key = lib.svodb_last_config_key().decode()
    assert key == "gemm|BFloat16|2048|1024|512|plain"
    store = tune.TuneStore(torch.cuda.get_device_name(0), directory=tmp_path)
    bn = store.tune_linear(x, w)
    assert bn in tune.GEMM_WIDTHS and store.get(key) == bn and lib.svodb_config_get(key.encode()) == bn
    got = host(ops.linear(x, w))
    assert f"bn:{bn}" in ops.chosen()
    assert max_abs(got, base) == 0.0  # the k order does not depend on the tile width
    # every width gives the same numbers
    for cand in (64, 128, 256):
        lib.svodb_config_set(key.encode(), cand)
        assert max_abs(host(ops.linear(x, w)), base) == 0.0 and f"bn:{cand}" in ops.chosen()
    # the CTA-pair kernel needs a 256 x 256 tile per pair of SMs: ignored for this shape
    lib.svodb_config_set(key.encode(), 512)
    assert max_abs(host(ops.linear(x, w)), base) == 0.0 and "cta_pair" not in ops.chosen()
    # a fresh process state reads the choice back from the file
    lib.svodb_config_clear()
    again = tune.TuneStore(torch.cuda.get_device_name(0), directory=tmp_path)
    assert again.load() == 1 and lib.svodb_config_get(key.encode()) == bn
    assert again.tune_linear(x, w) == bn  # a hit: nothing is timed
    # a width the epilogue cannot take is ignored (a gated tile needs 128)
    wg = dev(normal(rng, (2048, 512), 0.05, dt), dt)
    ops.linear(x, wg, ops.Linear(act=ops.Act.SILU, gated=True))
    gkey = lib.svodb_last_config_key()
    lib.svodb_config_set(gkey, 64)
    ops.linear(x, wg, ops.Linear(act=ops.Act.SILU, gated=True))
    assert "bn:64" not in ops.chosen()
    # shapes on the generic kernel have no key
    ops.linear(dev(np.zeros((4, 7)), O.F32), dev(np.zeros((5, 7)), O.F32))
    assert lib.svodb_last_config_key() == b""
    lib.svodb_config_clear()


def test_decode_attention_splits_come_from_the_store(tmp_path):
    dt = O.BF16
    rng = np.random.default_rng(5)
    B, T, Tk, H, D = 2, 1, 2048, 8, 128
    q = normal(rng, (B, T, H, D), 1.0, dt)
    k = normal(rng, (B, Tk, H, D), 1.0, dt)
    v = normal(rng, (B, Tk, H, D), 1.0, dt)
    ka, va = normal(rng, (B, 1, H, D), 1.0, dt), normal(rng, (B, 1, H, D), 1.0, dt)
    lens = np.array([Tk, 700])
    want = O.attention(q, k, v, key_lens=lens, cache=dict(head_start=0, kv_heads=H, k_app=ka, v_app=va), dtype=dt)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32).cuda()
    a = ops.Attn(keys=ops.KeyMask.Lens(i32(lens)), cache=ops.Cache(0, H, None, (dev(ka, dt), dev(va, dt))))
    Q, K, V = dev(q, dt), dev(k, dt), dev(v, dt)
    store = tune.TuneStore(torch.cuda.get_device_name(0), directory=tmp_path)
    splits = store.tune_attention_splits(Q, K, V, a)
    assert 1 <= splits <= (Tk + 1 + 31) // 32 and store.get(store.attention_key(Q, K, a)) == splits
    tune.activate(store)
    try:
        got = host(ops.attention(Q, K, V, a))  # `splits=None`: the store's count
    finally:
        tune.activate(None)
    assert max_abs(got, want) < 2e-2
    assert max_abs(host(ops.attention(Q, K, V, a)), want) < 2e-2  # and without the store
