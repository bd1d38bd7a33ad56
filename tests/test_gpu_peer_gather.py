"""The all-gather of pooled rows over peer memory (`svodb_peer_all_gather`).

On one GPU the protocol is walked with the ranks emulated as buffer sets of one
process: every rank's push is launched, then every rank's unstage — so no launch
ever waits for one that has not run (the flags are already set when the waits
look). With two or more GPUs the same step runs as one process per GPU over CUDA
IPC and is compared with the NCCL all-gather."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from svod_b200 import _lib as L
from svod_b200 import ops

pytestmark = pytest.mark.gpu


def _alloc(nbytes):
    lib = L.load()
    p = C.c_void_p()
    assert lib.svodb_alloc(nbytes, 0, C.byref(p)) == L.OK
    assert lib.svodb_memset(p, 0, nbytes, ops._stream()) == L.OK
    return p.value


@pytest.mark.parametrize("world,rows,d", [(2, 5, 1024), (4, 32, 768), (8, 3, 256)])
def test_the_protocol_with_every_rank_in_one_process(world, rows, d):
    lib = L.load()
    stage = [_alloc(lib.svodb_peer_stage_bytes(world, rows, d)) for _ in range(world)]
    flags = [_alloc(256) for _ in range(world)]
    local = [_alloc(256) for _ in range(world)]
    ctxs = []
    for r in range(world):
        c = L.PeerGather()
        c.world, c.rank, c.wait_polls = world, r, 1000
        for q in range(world):
            c.stage[q], c.flags[q] = stage[q], flags[q]
        c.local = local[r]
        ctxs.append(c)
    gen = torch.Generator(device="cuda").manual_seed(world)
    gathered = [torch.zeros(world * rows, d, device="cuda") for _ in range(world)]
    # With every rank on one GPU no launch may wait for one that has not run: all the pushes
    # of a step are launched first (`phases = 1`), then all the unstages (`phases = 2`), whose
    # waits find every flag already set.
    for step in range(3):
        want = torch.randn(world * rows, d, generator=gen, device="cuda")
        for r in range(world):
            gathered[r].zero_()
            gathered[r][r * rows:(r + 1) * rows] = want[r * rows:(r + 1) * rows]
        for phase in (1, 2):
            for r in range(world):
                ctxs[r].phases = phase
                rc = lib.svodb_peer_all_gather(C.byref(ctxs[r]), gathered[r][r * rows:].data_ptr(),
                                               gathered[r].data_ptr(), rows, d, ops._stream())
                assert rc == L.OK
        torch.cuda.synchronize()
        assert lib.svodb_device_status(None) == L.OK
        for r in range(world):
            assert torch.equal(gathered[r], want), (step, r)
    for p in stage + flags + local:
        lib.svodb_free(p, 0)


def test_a_peer_that_never_delivers_ends_in_a_reported_timeout():
    """The unstage of a step whose peer never pushed: the bounded wait (a flag nothing
    sets, two thousand polls) runs out, the status word says so once, nothing is
    copied, and the context goes on working."""
    lib = L.load()
    world, rows, d = 2, 4, 256
    stage = [_alloc(lib.svodb_peer_stage_bytes(world, rows, d)) for _ in range(world)]
    flags = [_alloc(256) for _ in range(world)]
    local = _alloc(256)
    c = L.PeerGather()
    c.world, c.rank, c.wait_polls, c.phases = world, 0, 2000, 2
    for q in range(world):
        c.stage[q], c.flags[q] = stage[q], flags[q]
    c.local = local
    gathered = torch.full((world * rows, d), 5.0, device="cuda")
    assert lib.svodb_peer_all_gather(C.byref(c), gathered.data_ptr(), gathered.data_ptr(), rows, d, ops._stream()) == L.OK
    torch.cuda.synchronize()
    assert lib.svodb_device_status(None) == L.ERR_TIMEOUT
    assert lib.svodb_device_status(None) == L.OK
    assert bool((gathered == 5.0).all())
    x = torch.randn(8, 256, device="cuda").to(torch.bfloat16)
    w = torch.ones(256, device="cuda", dtype=torch.bfloat16)
    assert torch.isfinite(ops.rms_norm(x, w).float()).all()
    for p in stage + flags + [local]:
        lib.svodb_free(p, 0)


WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from svod_b200 import ops
from svod_b200.peer import PeerGather
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
rows, d = 7, 1024
pg = PeerGather(rows, d)
ok = True
for step in range(5):
    g = torch.Generator(device="cuda").manual_seed(100 * step + rank)
    mine = torch.randn(rows, d, generator=g, device="cuda")
    a = torch.zeros(world * rows, d, device="cuda"); b = torch.zeros_like(a)
    a[rank * rows:(rank + 1) * rows] = mine
    pg.all_gather(a[rank * rows:(rank + 1) * rows], a)
    dist.all_gather_into_tensor(b, mine)
    torch.cuda.synchronize()
    ops.device_status()
    ok = ok and torch.equal(a, b)
# inside a captured graph, replayed
a = torch.zeros(world * rows, d, device="cuda"); mine = a[rank * rows:(rank + 1) * rows]
s = torch.cuda.Stream()
with torch.cuda.stream(s):
    mine.fill_(float(rank)); pg.all_gather(mine, a)
    torch.cuda.synchronize(); dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=s):
        pg.all_gather(mine, a)
    for k in range(4):
        mine.fill_(10.0 * k + rank)
        graph.replay()
        s.synchronize()
        want = torch.cat([torch.full((rows, d), 10.0 * k + r, device="cuda") for r in range(world)])
        ok = ok and torch.equal(a, want)
ops.device_status()
# the send half inside the pooling kernel (`svodb_norm_pool_gather`), eagerly and from a graph
L_, D_ = 40, 1024
fused = PeerGather(rows, D_)
gbuf = torch.zeros(world * rows, D_, device="cuda")
fused.bind(gbuf)
wn = torch.ones(D_, device="cuda", dtype=torch.bfloat16)
for step in range(3):
    g = torch.Generator(device="cuda").manual_seed(7 * step + rank)
    hid = torch.randn(rows, L_, D_, generator=g, device="cuda").to(torch.bfloat16)
    lens = torch.randint(1, L_ + 1, (rows,), generator=g, device="cuda", dtype=torch.int32)
    mine = ops.norm_pool(hid, wn, None, 1e-6, layer=False, aux=lens, mode=ops.POOL_LAST)
    want = torch.zeros_like(gbuf)
    dist.all_gather_into_tensor(want, mine)
    got = ops.norm_pool(hid, wn, None, 1e-6, layer=False, aux=lens, mode=ops.POOL_LAST, gather=fused)
    ok = ok and "push:peers" in ops.chosen()
    torch.cuda.synchronize()
    ok = ok and torch.equal(got, want)
ops.device_status()
dist.barrier()
print("PEER_OK" if ok else "PEER_MISMATCH", flush=True)
pg.close()
os._exit(0)
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_per_gpu_matches_the_nccl_all_gather(tmp_path):
    world = min(4, torch.cuda.device_count())
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, REPO=str(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
               NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert r.stdout.count("PEER_OK") == world, r.stdout[-2000:] + r.stderr[-2000:]
