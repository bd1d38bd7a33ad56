"""A batch bound below its capacity (tk/src/test/unit/ops.rs:260-345,526-560).

The reference binds a symbolic batch variable to a live count at run time: one
kernel over the live batches only, the output shrunk to the live dim, rows past
it never written. This library's ops take explicit pointers and sizes, so the
live count IS the batch the caller passes: operands sit in capacity-sized
buffers, the op runs on their leading `live` rows in place (no copy), and a
capacity-sized output keeps its sentinel in the rows past the live count."""
import numpy as np
import pytest
import torch

from oracle import svod_oracle as O
from svod_b200 import ops
from tests.test_gpu_attention import key_mask, recipe
from tests.util import dev, host, rel_close

pytestmark = pytest.mark.gpu

SENTINEL = 7.0


def test_linear_under_a_live_batch_count():
    """ops.rs:260-316: cap 4, live 3, 37 rows a batch, 64 -> 64 with bias and residual."""
    cap, live, rows, n, k = 4, 3, 37, 64, 64
    dt = O.BF16
    rng = np.random.default_rng(3)
    x = O.round_to(dt, rng.uniform(-1, 1, (cap, rows, k)))
    r = O.round_to(dt, rng.uniform(-1, 1, (cap, rows, n)))
    w = O.round_to(dt, rng.uniform(-1, 1, (n, k)) * 0.3)
    b = O.round_to(dt, rng.uniform(-1, 1, n))
    xd, rd = dev(x, dt), dev(r, dt)
    y = torch.full((cap, rows, n), SENTINEL, dtype=torch.bfloat16, device="cuda")
    out = ops.linear(xd[:live], dev(w, dt), ops.Linear(bias=dev(b, dt), residual=rd[:live], into=(y[:live], 0)))
    assert "kernel gemm" in ops.chosen()
    assert out.data_ptr() == y.data_ptr() and tuple(out.shape) == (live, rows, n)
    got = host(y)
    assert rel_close(got[:live], O.linear(x[:live], w, b, residual=r[:live], dtype=dt), 2e-2)
    assert np.all(got[live:] == SENTINEL)


def test_rotated_linear_under_a_live_batch_count():
    """ops.rs:318-345: the rotation in the store, tables shared by the batch lanes."""
    cap, live, t, h, hkv, d, k = 4, 3, 37, 4, 2, 64, 128
    dt = O.BF16
    rng = np.random.default_rng(4)
    n = (h + 2 * hkv) * d
    x = O.round_to(dt, rng.uniform(-1, 1, (cap, t, k)))
    w = O.round_to(dt, rng.uniform(-1, 1, (n, k)) * 0.2)
    cos, sin = O.rope_table(10000.0, np.arange(t), d, dt)
    rope = ops.Rotary(dev(cos, dt).view(1, t, 1, d // 2), dev(sin, dt).view(1, t, 1, d // 2), h + hkv, d)
    y = torch.full((cap, t, n), SENTINEL, dtype=torch.bfloat16, device="cuda")
    ops.linear(dev(x, dt)[:live], dev(w, dt), ops.Linear(rope=rope, into=(y[:live], 0)))
    got = host(y)
    want = O.linear(x[:live], w, rope=(cos, sin, h + hkv, d), dtype=dt)
    assert rel_close(got[:live], want, 2e-2)
    assert np.all(got[live:] == SENTINEL)


def test_attention_under_a_live_batch_count():
    """ops.rs:544-560: cap 3, live 2, key lengths [96, 40, 5], scale 0.2."""
    cap, live = 3, 2
    dt = O.BF16
    q, k, v = recipe(cap, 96, 96, 4, 2, 64, dt)
    lens = np.array([96, 40, 5])
    lens_d = torch.tensor(lens, dtype=torch.int64).cuda()
    a = ops.Attn(keys=ops.KeyMask.Lens(lens_d[:live]), scale=0.2)
    got = ops.attention(dev(q, dt)[:live], dev(k, dt)[:live], dev(v, dt)[:live], a)
    assert "kernel flash_attention" in ops.chosen()
    assert tuple(got.shape) == (live, 96, 4, 64)
    want = O.attention(q[:live], k[:live], v[:live], key_lens=lens[:live], scale=0.2, dtype=dt)
    assert rel_close(host(got), want, 2e-2)


def test_packed_attention_under_a_live_batch_count():
    """ops.rs:526-541: packed projection, bool key mask, window (16, 16)."""
    cap, live = 3, 2
    dt = O.BF16
    q, k, v = recipe(cap, 96, 96, 4, 2, 64, dt)
    mask = key_mask(cap, 96)
    qkv = np.concatenate([q.reshape(cap, 96, -1), k.reshape(cap, 96, -1), v.reshape(cap, 96, -1)], axis=-1)
    mask_d = torch.from_numpy(mask).cuda()
    a = ops.Attn(keys=ops.KeyMask.Bool(mask_d[:live]), window=(16, 16))
    got = ops.attention_packed(dev(qkv, dt)[:live], 4, 2, a)
    assert "flash_attention" in ops.chosen()
    want = O.attention(q[:live], k[:live], v[:live], key_mask=mask[:live], window=(16, 16), dtype=dt)
    assert rel_close(host(got), want, 2e-2)
