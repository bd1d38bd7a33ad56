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


def code(fn):
    with pytest.raises(ops.OpsError) as e:
        fn()
    return e.value.code


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
    """A bounded wait that really runs out: a one-warp kernel waits on a barrier
    nothing arrives on, gives up after a few thousand tries, sets the status word
    and returns. The host sees SVODB_ERR_TIMEOUT exactly once, the word is
    cleared, and the next op runs normally on the same context."""
    lib = L.load()
    s = torch.cuda.current_stream().cuda_stream
    ops.device_status()
    assert lib.svodb_selftest_wait_timeout(0, s) == L.ERR_SHAPE          # the cap itself is bounded
    assert lib.svodb_selftest_wait_timeout(3000, s) == 0
    assert lib.svodb_device_status(s) == L.ERR_TIMEOUT
    assert b"wait ran out" in lib.svodb_last_error()
    assert lib.svodb_device_status(s) == 0                               # read once, then clear
    assert lib.svodb_selftest_wait_timeout(3000, s) == 0
    assert code(ops.device_status) == L.ERR_TIMEOUT                      # the Python mirror raises it
    x = torch.randn(8, 256, **bf)
    got = ops.rms_norm(x, torch.ones(256, **bf))
    want = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)
    assert float((got.float() - want).abs().max()) < 2e-2
    ops.device_status()


def test_a_sticky_error_code_poisons_every_later_call_until_cleared():
    """The error latch (device/src/cuda/sys.rs:78-96) with a faked code: no device
    fault is raised. 700 = cudaErrorIllegalAddress (sticky), 1 = cudaErrorInvalidValue (not)."""
    lib = L.load()
    x, w = torch.ones(3, 256, **bf), torch.ones(256, **bf)
    assert lib.svodb_selftest_latch_error(1) == L.ERR_LAUNCH
    assert ops.rms_norm(x, w).shape == x.shape                           # not sticky: nothing latched
    assert lib.svodb_selftest_latch_error(700) == L.ERR_LAUNCH
    try:
        assert code(lambda: ops.rms_norm(x, w)) == L.ERR_POISONED
        assert code(lambda: ops.linear(x, torch.ones(8, 256, **bf))) == L.ERR_POISONED
        assert lib.svodb_device_status(torch.cuda.current_stream().cuda_stream) == L.ERR_POISONED
    finally:
        lib.svodb_selftest_clear_latch()
    assert ops.rms_norm(x, w).shape == x.shape
    ops.device_status()


ADD_SCALAR_PTX = b"""
.version 7.8
.target sm_80
.address_size 64
.visible .entry add_scalar(.param .u64 p_in, .param .u64 p_out, .param .u32 p_n, .param .u32 p_val)
{
  .reg .pred %p;
  .reg .b32 %r<6>;
  .reg .b64 %rd<6>;
  ld.param.u64 %rd0, [p_in];
  ld.param.u64 %rd1, [p_out];
  ld.param.u32 %r0, [p_n];
  ld.param.u32 %r1, [p_val];
  mov.u32 %r2, %ctaid.x;
  mov.u32 %r3, %ntid.x;
  mov.u32 %r4, %tid.x;
  mad.lo.s32 %r2, %r2, %r3, %r4;
  setp.ge.s32 %p, %r2, %r0;
  @%p bra DONE;
  cvta.to.global.u64 %rd0, %rd0;
  cvta.to.global.u64 %rd1, %rd1;
  mul.wide.s32 %rd2, %r2, 4;
  add.s64 %rd3, %rd0, %rd2;
  add.s64 %rd4, %rd1, %rd2;
  ld.global.s32 %r5, [%rd3];
  add.s32 %r5, %r5, %r1;
  st.global.s32 [%rd4], %r5;
DONE:
  ret;
}
\0"""


def test_module_load_program_launch_and_free_round_trip():
    """`CudaProgram::load` -> `Program::execute` (device/src/cuda/program.rs:116-219,264-274): a PTX
    image, an entry name, parameters as two storage slots then two i32 scalars, grid in blocks and
    block in threads."""
    lib = L.load()
    params = (L.AbiParam * 4)(L.AbiParam(0, 0), L.AbiParam(1, 0), L.AbiParam(2, 1), L.AbiParam(3, 1))
    prog = C.c_void_p()
    assert lib.svodb_module_load(ADD_SCALAR_PTX, len(ADD_SCALAR_PTX), b"no_such_entry", params, 4, C.byref(prog)) == L.ERR_LAUNCH
    assert lib.svodb_module_load(ADD_SCALAR_PTX, len(ADD_SCALAR_PTX), b"add_scalar", params, 4, C.byref(prog)) == 0, \
        lib.svodb_last_error()
    n = 1000
    src = torch.arange(n, dtype=torch.int32, device="cuda")
    dst = torch.zeros(n + 8, dtype=torch.int32, device="cuda")
    bufs = (C.c_void_p * 2)(src.data_ptr(), dst.data_ptr())
    vals = (C.c_int32 * 2)(n, 42)
    grid, block = (C.c_uint32 * 3)((n + 127) // 128, 1, 1), (C.c_uint32 * 3)(128, 1, 1)
    s = torch.cuda.current_stream().cuda_stream
    assert lib.svodb_program_launch(prog, s, bufs, 2, vals, 2, grid, block, 0) == 0, lib.svodb_last_error()
    torch.cuda.synchronize()
    assert torch.equal(dst[:n], src + 42) and int(dst[n:].abs().sum()) == 0
    assert lib.svodb_program_launch(None, s, bufs, 2, vals, 2, grid, block, 0) == L.ERR_UNREALIZED
    assert lib.svodb_program_free(prog) == 0


def test_a_cache_row_map_entry_outside_the_cache_is_reported_not_followed():
    """The exact kernel reads K/V through `row_map[b]`; an entry outside the cache
    rows reads nothing: that lane sees no key (zeros) and the status word says so."""
    dt = dict(dtype=torch.float32, device="cuda")       # f32: the exact CUDA-core kernel
    B, T, Tk, H, D, rows = 2, 4, 16, 2, 32, 3
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn(B, T, H, D, generator=g, **dt)
    k = torch.randn(rows, Tk, H, D, generator=g, **dt)
    v = torch.randn(rows, Tk, H, D, generator=g, **dt)
    lens = torch.tensor([Tk, Tk], dtype=torch.int32, device="cuda")
    good = ops.attention(q, k, v, ops.Attn(keys=ops.KeyMask.Lens(lens), cache=ops.Cache(0, H, torch.tensor([2, 1], dtype=torch.int32, device="cuda"))))
    ops.device_status()
    bad = ops.attention(q, k, v, ops.Attn(keys=ops.KeyMask.Lens(lens), cache=ops.Cache(0, H, torch.tensor([2, 7], dtype=torch.int32, device="cuda"))))
    assert "graph" in ops.chosen()
    assert code(ops.device_status) == L.ERR_SHAPE
    assert torch.equal(bad[0], good[0]) and float(bad[1].abs().max()) == 0.0
    ops.device_status()
