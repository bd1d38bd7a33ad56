"""Error behaviour of the op layer: what the reference's ops reject
(tk/src/ops/{linear.rs:63-106, attention.rs:126-198, heads.rs:37-63, norm.rs:52-66})
is rejected with the same error class, nothing is launched, and the device stays
usable. Also the device seam: graph capture/replay, allocator, status word."""
import ctypes as C

import numpy as np
import pytest
import torch

from svod_b200 import _lib as L
from svod_b200 import ops

pytestmark = pytest.mark.gpu

bf = dict(dtype=torch.bfloat16, device="cuda")


def kind(fn):
    with pytest.raises(ops.OpsError) as e:
        fn()
    return e.value.kind


def test_linear_rejections():
    x, w = torch.zeros(4, 64, **bf), torch.zeros(32, 64, **bf)
    assert kind(lambda: ops.linear(x, torch.zeros(32, 48, **bf))) == "Shape"
    assert kind(lambda: ops.linear(x, w.half())) == "Dtype"
    assert kind(lambda: ops.linear(x, torch.zeros(33, 64, **bf), ops.Linear(gated=True))) == "Shape"
    assert kind(lambda: ops.linear(x, w, ops.Linear(bias=torch.zeros(31, **bf)))) == "Shape"
    assert kind(lambda: ops.linear(x, w, ops.Linear(residual=torch.zeros(4, 31, **bf)))) == "Shape"
    assert kind(lambda: ops.linear(x, w, ops.Linear(rope=ops.Rotary(x, x, 1, 32)))) == "Shape"   # x is not [B,T,K]
    assert ops.linear(x, w).shape == (4, 32)


def test_attention_rejections():
    q = torch.zeros(2, 8, 4, 64, **bf)
    k = torch.zeros(2, 8, 2, 64, **bf)
    assert kind(lambda: ops.attention(q[0], k, k)) == "Shape"
    assert kind(lambda: ops.attention(q, k[:, :, :, :32], k)) == "Shape"
    assert kind(lambda: ops.attention(q, k, k[:, :4])) == "Shape"
    assert kind(lambda: ops.attention(q, k.half(), k)) == "Dtype"
    assert kind(lambda: ops.attention(q, torch.zeros(2, 8, 3, 64, **bf), torch.zeros(2, 8, 3, 64, **bf))) == "Heads"
    assert kind(lambda: ops.attention(q, k, k, ops.Attn(keys=ops.KeyMask.Lens(torch.zeros(3, dtype=torch.int32, device="cuda"))))) == "Shape"
    assert kind(lambda: ops.attention(q, k, k, ops.Attn(keys=ops.KeyMask.Bool(torch.zeros(2, 9, dtype=torch.bool, device="cuda"))))) == "Shape"
    assert kind(lambda: ops.attention(q, k, k, ops.Attn(seg_start=torch.zeros(2, 9, dtype=torch.int32, device="cuda")))) == "Shape"
    assert kind(lambda: ops.attention(q, k, k, ops.Attn(bias=torch.zeros(2, 4, 8, 9, **bf)))) == "Shape"
    assert kind(lambda: ops.attention_packed(torch.zeros(2, 8, 100, **bf), 4, 2)) == "Shape"
    assert kind(lambda: ops.attention_packed(torch.zeros(2, 8, 512, **bf), 4, 3)) == "Heads"
    assert ops.attention(q, k, k).shape == q.shape


def test_heads_and_norm_rejections():
    qkv = torch.zeros(2, 8, 8 * 64, **bf)
    assert kind(lambda: ops.heads(qkv, ops.Qkv(4, 3, 64))) == "Heads"
    assert kind(lambda: ops.heads(qkv, ops.Qkv(4, 2, 32))) == "Shape"
    assert kind(lambda: ops.heads(qkv, ops.Qkv(4, 2, 64, q_norm=torch.zeros(32, **bf)))) == "Shape"
    assert kind(lambda: ops.heads(qkv, ops.Qkv(4, 2, 64, q_norm=torch.zeros(64, dtype=torch.float16, device="cuda")))) == "Dtype"
    t = torch.zeros(1, 9, 1, 32, **bf)
    assert kind(lambda: ops.heads(qkv, ops.Qkv(4, 2, 64, rope=(t, t)))) == "Shape"
    x = torch.zeros(5, 256, **bf)
    assert kind(lambda: ops.layer_norm(x, torch.zeros(255, **bf))) == "Shape"
    assert kind(lambda: ops.rms_norm(x, torch.zeros(256, dtype=torch.float16, device="cuda"))) == "Dtype"
    assert kind(lambda: ops.add_rms_norm(x, torch.zeros(4, 256, **bf), torch.zeros(256, **bf))) == "Shape"
    assert kind(lambda: ops.layer_norm(torch.zeros(5, 256), torch.zeros(256))) == "Unrealized"   # host tensors


def test_supported_chosen_and_status():
    assert ops.supported()
    ops.rms_norm(torch.ones(3, 256, **bf), torch.ones(256, **bf))
    assert ops.chosen() == "rms_norm: kernel rms_norm {br:8}"
    ops.rms_norm(torch.ones(3, 100, **bf), torch.ones(100, **bf))
    assert ops.chosen() == "rms_norm: graph shape"
    ops.device_status()


def test_empty_inputs_launch_nothing():
    assert ops.linear(torch.zeros(0, 64, **bf), torch.zeros(32, 64, **bf)).shape == (0, 32)
    assert ops.rms_norm(torch.zeros(0, 256, **bf), torch.ones(256, **bf)).shape == (0, 256)
    q = torch.zeros(2, 0, 4, 64, **bf)
    k = torch.zeros(2, 8, 4, 64, **bf)
    assert ops.attention(q, k, k).shape == q.shape
    # no key at all: zeros
    q = torch.ones(2, 5, 4, 64, **bf)
    k = torch.zeros(2, 0, 4, 64, **bf)
    assert float(ops.attention(q, k, k).abs().max()) == 0.0


def test_device_seam_alloc_copy_graph_replay():
    lib = L.load()
    s = torch.cuda.Stream()
    dptr, hptr = C.c_void_p(), C.c_void_p()
    assert lib.svodb_alloc(4096, 0, C.byref(dptr)) == 0 and lib.svodb_alloc(4096, 1, C.byref(hptr)) == 0
    src = (C.c_float * 1024)(*range(1024))
    C.memmove(hptr, src, 4096)
    assert lib.svodb_copy_h2d(dptr, hptr, 4096, s.cuda_stream) == 0
    C.memset(hptr, 0, 4096)
    assert lib.svodb_copy_d2h(hptr, dptr, 4096, s.cuda_stream) == 0
    assert lib.svodb_stream_sync(s.cuda_stream) == 0
    back = (C.c_float * 1024).from_address(hptr.value)
    assert list(back[:5]) == [0, 1, 2, 3, 4] and back[1023] == 1023
    assert lib.svodb_free(dptr, 0) == 0 and lib.svodb_free(hptr, 1) == 0
    # capture one op into a graph through the ABI and replay it on new data
    x = torch.randn(64, 256, **bf)
    w = torch.ones(256, **bf)
    with torch.cuda.stream(s):
        out = ops.rms_norm(x, w)          # warm: first-use work outside the capture
        s.synchronize()
        assert lib.svodb_graph_begin(s.cuda_stream) == 0
        out = ops.rms_norm(x, w)
        g = C.c_void_p()
        assert lib.svodb_graph_end(s.cuda_stream, C.byref(g)) == 0
        x.copy_(torch.randn(64, 256, **bf))
        assert lib.svodb_graph_replay(g, s.cuda_stream) == 0
        s.synchronize()
    want = ops.rms_norm(x, w)
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    assert lib.svodb_graph_free(g) == 0


def test_a_wait_that_runs_out_is_reported_not_hung():
    """The status word path: set the word the way a timed-out wait would and
    read it back through the ABI (no kernel is made to hang)."""
    lib = L.load()
    ops.device_status()
    assert lib.svodb_device_status(torch.cuda.current_stream().cuda_stream) == 0
