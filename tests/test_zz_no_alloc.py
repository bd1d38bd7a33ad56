"""The split attention that brings its own scratch.

`svodb_attention_splits_noalloc` exists for callers that must not allocate
device memory at call time: a host replaying a prepared plan (all buffers were
laid out when the plan was built) or issuing work while a stream is being
captured, where cudaMalloc is not permitted. It keeps the f32 partials of a
key-split attention in a fixed array inside the library instead of a workspace
the caller supplies.

Checked through the C ABI against the regular entry point (caller-supplied
workspace) on the same inputs, twice in a row with different data so stale
partials of the first call would show, and for the refusal of shapes the array
cannot hold. Collected last on purpose: a run that stops at the first failure
has then already run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import svod_oracle as O
from svod_b200 import _lib as L
from svod_b200 import ops
from tests.util import host, max_abs

pytestmark = pytest.mark.gpu


def call(entry, q, k, v, splits, lens, workspace=None):
    lib = L.load()
    out = torch.empty_like(q)
    o = L.AttnOpts()
    o.splits = splits
    lens_d = ops._desc(lens)
    o.key_lens = C.pointer(lens_d)
    if workspace is not None:
        o.workspace = workspace.data_ptr()
        o.workspace_bytes = workspace.numel()
    qd, kd, vd, od = ops._desc(q), ops._desc(k), ops._desc(v), ops._desc(out)
    rc = getattr(lib, entry)(C.byref(qd), C.byref(kd), C.byref(vd), C.byref(o), C.byref(od),
                             torch.cuda.current_stream().cuda_stream)
    return rc, out


def test_noalloc_split_attention_matches_the_workspace_entry_point_twice():
    lib = L.load()
    g = torch.Generator(device="cuda").manual_seed(7)
    B, T, Tk, H, Hkv, D, splits = 2, 3, 400, 8, 4, 128, 5
    need = lib.svodb_attention_workspace_bytes(B, T, H, D, splits)
    assert 0 < need <= L.NOALLOC_SCRATCH_BYTES
    for trial, lens in enumerate(([400, 123], [0, 77])):
        q = torch.randn(B, T, H, D, generator=g, device="cuda").to(torch.bfloat16)
        k = torch.randn(B, Tk, Hkv, D, generator=g, device="cuda").to(torch.bfloat16)
        v = torch.randn(B, Tk, Hkv, D, generator=g, device="cuda").to(torch.bfloat16)
        lens_t = torch.tensor(lens, dtype=torch.int32, device="cuda")
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        rc_ref, want = call("svodb_attention", q, k, v, splits, lens_t, ws)
        rc_new, got = call("svodb_attention_splits_noalloc", q, k, v, splits, lens_t)
        torch.cuda.synchronize()
        assert rc_ref == 0 and rc_new == 0, lib.svodb_last_error()
        # the tolerance the attention tests use; the two paths run the same kernels
        assert float((got.float() - want.float()).abs().max()) <= 2e-2
        assert torch.equal(got, want)
        # and the oracle on the same inputs (16-bit bound)
        ref = O.attention(host(q), host(k), host(v), key_lens=np.array(lens), dtype=O.BF16)
        assert max_abs(host(got), ref) < 2e-2
        if trial == 1:
            assert float(got[0].abs().max()) == 0.0   # a lane with no keys attends to nothing
    ops.device_status()


def test_noalloc_refuses_partials_that_do_not_fit():
    lib = L.load()
    B, T, Tk, H, D, splits = 8, 64, 256, 16, 128, 8
    assert lib.svodb_attention_workspace_bytes(B, T, H, D, splits) > L.NOALLOC_SCRATCH_BYTES
    q = torch.zeros(B, T, H, D, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(B, Tk, H, D, dtype=torch.bfloat16, device="cuda")
    lens = torch.full((B,), Tk, dtype=torch.int32, device="cuda")
    rc, _ = call("svodb_attention_splits_noalloc", q, k, k, splits, lens)
    assert rc == L.ERR_WORKSPACE
    assert b"built-in scratch" in lib.svodb_last_error()
    # a request above the key tile count is capped before the size check: 64 keys are two
    # tiles, and two splits of this shape fit although the 64 requested would not
    q4 = torch.zeros(4, T, H, D, dtype=torch.bfloat16, device="cuda")
    k64 = torch.zeros(4, 64, H, D, dtype=torch.bfloat16, device="cuda")
    assert lib.svodb_attention_workspace_bytes(4, T, H, D, 64) > L.NOALLOC_SCRATCH_BYTES
    assert lib.svodb_attention_workspace_bytes(4, T, H, D, 2) <= L.NOALLOC_SCRATCH_BYTES
    rc, out = call("svodb_attention_splits_noalloc", q4, k64, k64, 64, torch.full((4,), 64, dtype=torch.int32, device="cuda"))
    assert rc == 0, lib.svodb_last_error()
    # without splits no scratch is needed and the call is the regular attention
    rc, out = call("svodb_attention_splits_noalloc", q, k, k, 1, lens)
    assert rc == 0 and float(out.abs().max()) == 0.0
