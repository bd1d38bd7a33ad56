"""The all-gather of pooled rows as this library's own kernels over NVLink peer
memory (`svodb_peer_all_gather`): one process per GPU, every rank's staging
buffer and flags mapped into the others through CUDA IPC handles that travel
over the process group. A drop-in for `encoders.gather_pooled` (NCCL) as a
`Plan` epilogue; both launches are captured in the plan's graph."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from . import _lib as L
from . import ops


def _alloc_zeroed(nbytes: int) -> int:
    """A device allocation of its own (an IPC handle names a whole allocation, so
    these do not come from torch's caching allocator), zeroed."""
    lib = L.load()
    ptr = C.c_void_p()
    ops._check(lib.svodb_alloc(max(nbytes, 256), 0, C.byref(ptr)), 0)
    ops._check(lib.svodb_memset(ptr, 0, max(nbytes, 256), ops._stream()), 0)
    return ptr.value


class PeerGather:
    """Buffers and mappings of one rank for gathers of `[rows, d]` f32 blocks.

    `group` is the `torch.distributed` group whose ranks take part (at most 8, one
    GPU each); it only carries the 64-byte handles at construction. With
    `world == 1` nothing is allocated and `all_gather` is a no-op."""

    def __init__(self, rows: int, d: int, group=None, wait_polls: int = 0):
        import torch.distributed as dist
        self.rows, self.d = rows, d
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > 8:
            raise ops.OpsError(L.ERR_SHAPE, f"peer gather: {self.world} ranks (at most 8)")
        self._opened: List[int] = []
        self._owned: List[int] = []
        self.ctx = L.PeerGather()
        self.ctx.world, self.ctx.rank, self.ctx.wait_polls = self.world, self.rank, wait_polls
        if self.world == 1:
            return
        lib = L.load()
        # Every rank must come out of this constructor the same way (with the mappings, or with
        # an error): what can fail on one rank alone is tried first and the outcome is exchanged
        # with the handles, so that nobody is left waiting for a rank that gave up.
        handles, err = None, None
        try:
            stage = _alloc_zeroed(lib.svodb_peer_stage_bytes(self.world, rows, d))
            flags = _alloc_zeroed(256)
            local = _alloc_zeroed(256)
            self._owned = [stage, flags, local]
            torch.cuda.current_stream().synchronize()
            handles = []
            for ptr in (stage, flags):
                h = (C.c_uint8 * 64)()
                ops._check(lib.svodb_ipc_export(ptr, h), 0)
                handles.append(bytes(h))
        except ops.OpsError as e:
            err = str(e)
        everyone: List[Optional[tuple]] = [None] * self.world
        dist.all_gather_object(everyone, tuple(handles) if err is None else None, group=group)
        if err is None and all(h is not None for h in everyone):
            try:
                for r in range(self.world):
                    if r == self.rank:
                        self.ctx.stage[r], self.ctx.flags[r] = stage, flags
                        continue
                    for k, field in enumerate((self.ctx.stage, self.ctx.flags)):
                        out = C.c_void_p()
                        buf = (C.c_uint8 * 64).from_buffer_copy(everyone[r][k])
                        ops._check(lib.svodb_ipc_open(buf, C.byref(out)), 0)
                        self._opened.append(out.value)
                        field[r] = out.value
                self.ctx.local = local
            except ops.OpsError as e:
                err = str(e)
        elif err is None:
            err = "a peer could not export its buffers"
        # the second exchange doubles as the barrier: nobody pushes into a stage before every
        # rank has mapped and zeroed its own
        outcomes: List[Optional[str]] = [None] * self.world
        dist.all_gather_object(outcomes, err, group=group)
        failed = [f"rank {r}: {o}" for r, o in enumerate(outcomes) if o is not None]
        if failed:
            self.close()
            raise ops.OpsError(L.ERR_LAUNCH, "peer gather: " + "; ".join(failed))

    def bind(self, gathered: torch.Tensor) -> "PeerGather":
        """Names the `[world*rows, d]` f32 buffer the gathers fill: `ops.norm_pool(...,
        gather=self)` then pools into this rank's slot of it and sends the rows from the
        pooling kernel itself."""
        if tuple(gathered.shape) != (self.world * self.rows, self.d) or gathered.dtype != torch.float32 \
                or not gathered.is_contiguous():
            raise ops.OpsError(L.ERR_SHAPE, f"peer gather: gathered {list(gathered.shape)}, expected contiguous f32 "
                                            f"[{self.world * self.rows}, {self.d}]")
        self.gathered = gathered
        self.mine = gathered[self.rank * self.rows:(self.rank + 1) * self.rows]
        return self

    def all_gather(self, local: torch.Tensor, gathered: torch.Tensor) -> torch.Tensor:
        """`local` `[rows, d]` f32 (normally slot `rank` of `gathered`) into slot `rank`
        of every rank's `gathered` `[world*rows, d]`, on torch's current stream."""
        if tuple(local.shape) != (self.rows, self.d) or tuple(gathered.shape) != (self.world * self.rows, self.d):
            raise ops.OpsError(L.ERR_SHAPE, f"peer gather: local {list(local.shape)}, gathered {list(gathered.shape)}, "
                                            f"expected [{self.rows}, {self.d}] and [{self.world * self.rows}, {self.d}]")
        if local.dtype != torch.float32 or gathered.dtype != torch.float32 or not local.is_contiguous() \
                or not gathered.is_contiguous():
            raise ops.OpsError(L.ERR_DTYPE, "peer gather: contiguous f32 rows")
        mine = gathered[self.rank * self.rows:(self.rank + 1) * self.rows]
        if local.data_ptr() != mine.data_ptr():
            mine.copy_(local)
        ops._check(L.load().svodb_peer_all_gather(C.byref(self.ctx), mine.data_ptr(), gathered.data_ptr(), self.rows,
                                                  self.d, ops._stream()), 2 if self.world > 1 else 0)
        return gathered

    def close(self):
        lib = L.load()
        for ptr in self._opened:
            lib.svodb_ipc_close(ptr)
        self._opened = []
        for ptr in self._owned:
            lib.svodb_free(ptr, 0)
        self._owned = []
