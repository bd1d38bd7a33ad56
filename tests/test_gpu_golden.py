"""The CUDA path against the committed fixtures (`tests/golden/ops_golden.npz`,
written from the oracle by `tests/golden/make_golden.py`): seeded inputs and
expected outputs read from the file, nothing computed on the host."""
import numpy as np
import pytest
import torch

from oracle import svod_oracle as O
from svod_b200 import ops
from tests.golden import make_golden as G
from tests.util import dev, host, max_abs, mean_rel

pytestmark = pytest.mark.gpu
DT = O.BF16


@pytest.fixture(scope="module")
def g():
    return G.load()


def i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32).cuda()


def close(got, want, tol=2e-2):
    assert max_abs(got, want) < tol and mean_rel(got, want) < 5e-3


def test_attention_fixtures(g):
    o = ops.attention(dev(g["attn_q"], DT), dev(g["attn_k"], DT), dev(g["attn_v"], DT),
                      ops.Attn(causal=True, keys=ops.KeyMask.Lens(i32(g["attn_lens"]))))
    assert "kernel flash_attention" in ops.chosen()
    close(host(o), g["attn_o"])
    o = ops.attention(dev(g["attn2_q"], DT), dev(g["attn2_k"], DT), dev(g["attn2_v"], DT),
                      ops.Attn(causal=True, window=(30, 0), seg_start=i32(g["attn2_seg"])))
    close(host(o), g["attn2_o"])
    cache = ops.Cache(2, 2, i32([2, 0]), (dev(g["cache_ka"], DT), dev(g["cache_va"], DT)), i32([4, 2]))
    o = ops.attention(dev(g["cache_q"], DT), dev(g["cache_k"], DT), dev(g["cache_v"], DT),
                      ops.Attn(keys=ops.KeyMask.Lens(i32([32, 11])), cache=cache))
    close(host(o), g["cache_o"])


def test_linear_fixtures(g):
    x = dev(g["lin_x"], DT)
    y = ops.linear(x, dev(g["lin_w"], DT), ops.Linear(bias=dev(g["lin_b"], DT), act=ops.Act.GELU))
    assert "kernel gemm" in ops.chosen()
    close(host(y), g["lin_gelu"])
    y = ops.linear(x, dev(g["lin_wg"], DT), ops.Linear(bias=dev(g["lin_bg"], DT), act=ops.Act.SILU, gated=True,
                                                        residual=dev(g["lin_r"], DT), scale=0.5))
    close(host(y), g["lin_swiglu"])


def test_heads_and_norm_fixtures(g):
    tabs = (dev(g["heads_cos"], DT).view(1, 24, 1, 32), dev(g["heads_sin"], DT).view(1, 24, 1, 32))
    q, k, v = ops.heads(dev(g["heads_qkv"], DT), ops.Qkv(2, 1, 64, dev(g["heads_qw"], DT), dev(g["heads_kw"], DT),
                                                          1e-6, tabs))
    close(host(q), g["heads_q"])
    close(host(k), g["heads_k"])
    assert np.array_equal(host(v), g["heads_v"])
    s, y = ops.add_rms_norm(dev(g["norm_x"], DT), dev(g["norm_r"], DT), dev(g["norm_w"], DT), 1e-6)
    assert np.array_equal(host(s), g["norm_sum"])  # the fused sum is exact
    close(host(y), g["norm_rms"], 2e-2)
    y = ops.layer_norm(dev(g["norm_x"], DT), dev(g["norm_w"], DT), dev(g["norm_b"], DT), 1e-5)
    close(host(y), g["norm_layer"], 3e-2)
