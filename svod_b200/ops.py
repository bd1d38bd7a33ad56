"""The op layer: a Python mirror of `svod_tk::ops` (tk/src/ops/mod.rs:30-38).

Same names, argument meaning and error behaviour as the reference's Rust
functions: every op takes tensors and returns tensors, runs a hand-written
sm_100a kernel when dtype and shape fit and an exact generic CUDA kernel where
the reference would build its graph, and raises `OpsError` only for what the
graph op would also reject. `chosen()` reports what the last op ran.

Tensors are `torch.Tensor`s on a CUDA device; torch supplies device memory and
the current stream, every computation goes through the C ABI of libsvodb.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _lib as L


class Act(enum.IntEnum):
    """`kernels::Act` (tk/src/kernels/mod.rs:272-280)."""
    NONE = 0
    GELU = 1       # erf GELU
    SILU = 2
    GELU_TANH = 3  # `Tensor::gelu`, outside the reference's op layer


class OpsError(RuntimeError):
    """`ops::Error` (tk/src/ops/mod.rs:132-159); `kind` names the variant."""

    KINDS = {
        L.ERR_SHAPE: "Shape", L.ERR_DTYPE: "Dtype", L.ERR_HEADS: "Heads", L.ERR_GRAPH: "Graph",
        L.ERR_LAUNCH: "Launch", L.ERR_UNREALIZED: "Unrealized", L.ERR_ALIAS: "Launch",
        L.ERR_TIMEOUT: "Launch", L.ERR_POISONED: "Launch", L.ERR_WORKSPACE: "Graph",
        L.ERR_UNSUPPORTED: "Graph",
    }

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code
        self.kind = self.KINDS.get(code, "Launch")


@dataclass
class Rotary:
    """`ops::Rotary` (tk/src/ops/linear.rs:45-56): tables `[1, T, 1, head_dim/2]`."""
    cos: torch.Tensor
    sin: torch.Tensor
    heads: int
    head_dim: int


@dataclass
class Linear:
    """`ops::Linear` (tk/src/ops/linear.rs:24-43)."""
    bias: Optional[torch.Tensor] = None
    act: Act = Act.NONE
    gated: bool = False
    residual: Optional[torch.Tensor] = None
    scale: Optional[float] = None
    rope: Optional[Rotary] = None
    into: Optional[Tuple[torch.Tensor, int]] = None
    # Not in the reference's `Linear`: the `ops::heads` prologue (per-head RMSNorm
    # of q and k, rotation) applied in this projection's store; the result stays
    # the packed `[B, T, (H + 2*Hkv)*D]` projection for `attention_packed`.
    qkv: Optional["Qkv"] = None
    # Split-K (the reference's tail split + merge, tk/src/kernels/gemm.rs:454-466,750-808):
    # None = this module's choice (`auto_k_splits`: one piece), 0 / 1 = the k loop in one
    # piece, > 1 = that many pieces on the CTA-pair kernel. The f32 workspace is allocated here.
    k_splits: Optional[int] = None


@dataclass
class KeyMask:
    """`ops::KeyMask` (tk/src/ops/attention.rs:29-37): `lens` `[B]` valid-key
    counts or `mask` `[B, Tk]` bool/integer, nonzero where attended."""
    lens: Optional[torch.Tensor] = None
    mask: Optional[torch.Tensor] = None

    @staticmethod
    def Lens(t: torch.Tensor) -> "KeyMask":
        return KeyMask(lens=t)

    @staticmethod
    def Bool(t: torch.Tensor) -> "KeyMask":
        return KeyMask(mask=t)


@dataclass
class Chunk:
    """`kernels::attention::Chunk`: query `i` sees chunk `i/size`, `left`
    chunks before it (None = all) and `right` after."""
    size: int
    left: Optional[int] = None
    right: int = 0


@dataclass
class Cache:
    """`ops::Cache` (tk/src/ops/attention.rs:39-55): `k`, `v` are caches
    `[rows, Tk, H_all, D]`; `appended = (k, v)` of `[B, n, kv_heads, D]` are
    scored after the cached prefix that `KeyMask.Lens` names."""
    head_start: int
    kv_heads: int
    row_map: Optional[torch.Tensor] = None
    appended: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
    app_lens: Optional[torch.Tensor] = None


@dataclass
class Attn:
    """`ops::Attn` (tk/src/ops/attention.rs:59-86)."""
    causal: bool = False
    keys: Optional[KeyMask] = None
    window: Optional[Tuple[int, int]] = None
    chunk: Optional[Chunk] = None
    seg_start: Optional[torch.Tensor] = None
    splits: Optional[int] = None
    scale: Optional[float] = None
    bias: Optional[torch.Tensor] = None
    cache: Optional[Cache] = None
    want_lse: bool = False  # also return ln-sum-exp `[B, H, T]` f32


@dataclass
class Qkv:
    """`ops::Qkv` (tk/src/ops/heads.rs:18-32)."""
    heads: int
    kv_heads: int
    head_dim: int
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    eps: float = 1e-6
    rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None


_DTYPES = {
    torch.float32: L.F32, torch.float16: L.F16, torch.bfloat16: L.BF16,
    torch.int32: L.I32, torch.int64: L.I64, torch.uint8: L.U8, torch.bool: L.U8,
}


def _desc(t: Optional[torch.Tensor]):
    """The `svodb_tensor` of a CUDA tensor, or a null pointer."""
    if t is None:
        return None
    if not t.is_cuda:
        raise OpsError(L.ERR_UNREALIZED, "operand is not a realized device buffer")
    if t.dtype not in _DTYPES:
        raise OpsError(L.ERR_DTYPE, f"unsupported element type {t.dtype}")
    if t.dim() > L.MAX_RANK:
        raise OpsError(L.ERR_SHAPE, f"rank {t.dim()} is above {L.MAX_RANK}")
    d = L.Tensor()
    d.data = t.data_ptr()
    d.dtype = _DTYPES[t.dtype]
    d.rank = t.dim()
    for i, (s, st) in enumerate(zip(t.shape, t.stride())):
        d.shape[i] = s
        d.stride[i] = st
    return d


def _p(d):
    return C.byref(d) if d is not None else None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


# Kernel launches issued through this module since import (an op that runs two
# kernels, e.g. pooling + L2 or a split attention + merge, counts both).
launches = 0


def _check(rc: int, kernels: int = 1):
    global launches
    if rc != L.OK:
        raise OpsError(rc, L.load().svodb_last_error().decode())
    launches += kernels


def supported(device=None) -> bool:
    """`ops::supported` (tk/src/ops/mod.rs:161-166)."""
    if not torch.cuda.is_available():
        return False
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    return bool(L.load().svodb_supported(idx))


def chosen() -> Optional[str]:
    """`ops::chosen()` (tk/src/ops/mod.rs:101-118): what the last op on this
    thread ran — `"<op>: kernel <family> <cfg>"` or `"<op>: graph <why>"`."""
    s = L.load().svodb_last_chosen().decode()
    return s or None


def device_status() -> None:
    """Raises if a bounded device-side wait ran out since the last check."""
    _check(L.load().svodb_device_status(_stream()), 0)


# --------------------------------------------------------------------------- linear
def auto_k_splits(m: int, n: int, k: int, opts: "Linear", dtype) -> int:
    """Pieces of the k loop when the caller leaves the choice here: always one.
    Measured on every one-wave shape of the GEMM sweep, the split kernel is slower
    than the unsplit one (512 x 4096 x 4096: 29 us in two pieces against 21 us;
    512 x 1024 x 4096: 25 us in four against 19 us): what a piece saves in its k
    loop, the f32 blocks' trip through L2 and the merge cost again. A caller (or a
    tuned config) that knows better passes `k_splits`."""
    return 1


def linear(x: torch.Tensor, w: torch.Tensor, opts: Optional[Linear] = None) -> torch.Tensor:
    """`ops::linear` (tk/src/ops/linear.rs:63-191): `x [lead..., K] . w [N, K]^T`
    with the epilogue `opts`."""
    opts = opts or Linear()
    lib = L.load()
    if w.dim() != 2:
        raise OpsError(L.ERR_SHAPE, f"linear: w has shape {list(w.shape)}, expected [N, K]")
    n = w.shape[0] // 2 if opts.gated else w.shape[0]
    if opts.into is not None:
        into, at = opts.into
        if into.shape[:-1] != x.shape[:-1] or at + n > into.shape[-1] or into.dtype != x.dtype:
            raise OpsError(L.ERR_SHAPE, f"linear: into has shape {list(into.shape)}, expected "
                                        f"{list(x.shape[:-1])} + [>= {at + n}]")
        y = into[..., at:at + n]
    else:
        y = torch.empty(*x.shape[:-1], n, dtype=x.dtype, device=x.device)
    o = L.LinearOpts()
    keep = [_desc(opts.bias), _desc(opts.residual),
            _desc(opts.rope.cos) if opts.rope else None, _desc(opts.rope.sin) if opts.rope else None]
    o.bias = C.pointer(keep[0]) if keep[0] is not None else None
    o.act = int(opts.act)
    o.gated = int(opts.gated)
    o.residual = C.pointer(keep[1]) if keep[1] is not None else None
    o.has_scale = int(opts.scale is not None)
    o.scale = float(opts.scale or 0.0)
    if opts.rope:
        o.rope_cos = C.pointer(keep[2])
        o.rope_sin = C.pointer(keep[3])
        o.rope_heads = opts.rope.heads
        o.rope_head_dim = opts.rope.head_dim
    o.into_at = opts.into[1] if opts.into else 0
    if opts.qkv is not None:
        qo = _qkv_opts(opts.qkv, keep)
        keep.append(qo)
        o.qkv = C.cast(C.pointer(qo), C.c_void_p)
    m = x.numel() // max(1, x.shape[-1])
    splits = opts.k_splits if opts.k_splits is not None else auto_k_splits(m, n, x.shape[-1], opts, x.dtype)
    if splits and splits > 1:
        need = lib.svodb_linear_workspace_bytes(m, n, splits)
        ws = torch.empty(max(need, 1), dtype=torch.uint8, device=x.device)
        keep.append(ws)
        o.k_splits, o.workspace, o.workspace_bytes = splits, ws.data_ptr(), need
    xd, wd, yd = _desc(x), _desc(w), _desc(y)
    _check(lib.svodb_linear(_p(xd), _p(wd), C.byref(o), _p(yd), _stream()))
    return opts.into[0] if opts.into is not None else y


# ------------------------------------------------------------------------ attention
def _attn_opts(opts: Attn, q_shape, dtype, device, keep: list):
    o = L.AttnOpts()
    o.causal = int(opts.causal)
    if opts.keys is not None and opts.keys.lens is not None:
        t = opts.keys.lens
        t = t if t.dtype == torch.int32 else t.to(torch.int32)
        keep.append(_desc(t)), keep.append(t)
        o.key_lens = C.pointer(keep[-2])
    if opts.keys is not None and opts.keys.mask is not None:
        t = opts.keys.mask
        if t.dtype not in (torch.bool, torch.uint8, torch.int32):
            t = (t != 0)
        t = t.contiguous()
        keep.append(_desc(t)), keep.append(t)
        o.key_mask = C.pointer(keep[-2])
    if opts.window is not None:
        o.has_window, o.window_left, o.window_right = 1, int(opts.window[0]), int(opts.window[1])
    if opts.chunk is not None:
        o.has_chunk, o.chunk_size = 1, int(opts.chunk.size)
        o.chunk_left = -1 if opts.chunk.left is None else int(opts.chunk.left)
        o.chunk_right = int(opts.chunk.right)
    if opts.seg_start is not None:
        t = opts.seg_start
        t = (t if t.dtype == torch.int32 else t.to(torch.int32)).contiguous()
        keep.append(_desc(t)), keep.append(t)
        o.seg_start = C.pointer(keep[-2])
    o.splits = int(opts.splits or 0)
    o.has_scale = int(opts.scale is not None)
    o.scale = float(opts.scale or 0.0)
    if opts.bias is not None:
        t = opts.bias.contiguous()
        keep.append(_desc(t)), keep.append(t)
        o.bias = C.pointer(keep[-2])
    if opts.cache is not None:
        c = opts.cache
        o.has_cache, o.cache_head_start, o.cache_kv_heads = 1, int(c.head_start), int(c.kv_heads)
        i32 = lambda t: (t if t.dtype == torch.int32 else t.to(torch.int32)).contiguous()
        if c.row_map is not None:
            t = i32(c.row_map)
            keep.append(_desc(t)), keep.append(t)
            o.cache_row_map = C.pointer(keep[-2])
        if c.appended is not None:
            for name, t in (("cache_app_k", c.appended[0]), ("cache_app_v", c.appended[1])):
                t = t.contiguous()
                keep.append(_desc(t)), keep.append(t)
                setattr(o, name, C.pointer(keep[-2]))
        if c.app_lens is not None:
            t = i32(c.app_lens)
            keep.append(_desc(t)), keep.append(t)
            o.cache_app_lens = C.pointer(keep[-2])
    lse = None
    B, T, H, D = q_shape
    if opts.want_lse:
        lse = torch.empty(B, H, T, dtype=torch.float32, device=device)
        keep.append(_desc(lse))
        o.lse = C.pointer(keep[-1])
    if opts.splits and opts.splits > 1:
        nbytes = L.load().svodb_attention_workspace_bytes(B, T, H, D, int(opts.splits))
        ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=device)
        keep.append(ws)
        o.workspace = ws.data_ptr()
        o.workspace_bytes = nbytes
    return o, lse


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, opts: Optional[Attn] = None):
    """`ops::attention` (tk/src/ops/attention.rs:100-102): `q [B,T,H,D]`,
    `k,v [B,Tk,Hkv,D]` -> `[B,T,H,D]` (and `lse` when `opts.want_lse`)."""
    opts = opts or Attn()
    if q.dim() != 4:
        raise OpsError(L.ERR_SHAPE, f"attention: q has shape {list(q.shape)}, expected [B, T, H, D]")
    if opts.splits is None and not opts.want_lse:
        # `splits: None` lets the tune store choose (tk/src/ops/attention.rs:74-80)
        from . import tune
        store = tune.active()
        if store is not None:
            hit = store.get(store.attention_key(q, k, opts))
            if hit and hit > 1:
                from dataclasses import replace
                opts = replace(opts, splits=hit)
    out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    keep: list = []
    o, lse = _attn_opts(opts, q.shape, q.dtype, q.device, keep)
    qd, kd, vd, od = _desc(q), _desc(k), _desc(v), _desc(out)
    _check(L.load().svodb_attention(_p(qd), _p(kd), _p(vd), C.byref(o), _p(od), _stream()))
    return (out, lse) if opts.want_lse else out


def attention_packed(qkv: torch.Tensor, heads: int, kv_heads: int, opts: Optional[Attn] = None):
    """`ops::attention_packed` (tk/src/ops/attention.rs:107-122): the kernel
    reads q, k and v in place from `qkv [B, T, (heads + 2 kv_heads) D]`."""
    opts = opts or Attn()
    if kv_heads <= 0 or heads % kv_heads != 0:
        raise OpsError(L.ERR_HEADS, f"attention: {heads} query heads are not a multiple of {kv_heads} key/value heads")
    slots = heads + 2 * kv_heads
    if qkv.dim() != 3 or slots <= 0 or qkv.shape[2] % slots != 0:
        raise OpsError(L.ERR_SHAPE, f"attention: qkv has shape {list(qkv.shape)}, expected [B, T, slots*D]")
    d = qkv.shape[2] // slots
    B, T = qkv.shape[:2]
    out = torch.empty(B, T, heads, d, dtype=qkv.dtype, device=qkv.device)
    keep: list = []
    o, lse = _attn_opts(opts, (B, T, heads, d), qkv.dtype, qkv.device, keep)
    xd, od = _desc(qkv), _desc(out)
    _check(L.load().svodb_attention_packed(_p(xd), heads, kv_heads, C.byref(o), _p(od), _stream()))
    return (out, lse) if opts.want_lse else out


def combine_splits(o_part: torch.Tensor, m_part: torch.Tensor, l_part: torch.Tensor, dtype) -> torch.Tensor:
    """`kernels::attention::combine` (tk/src/kernels/attention.rs:984-1014)."""
    out = torch.empty(o_part.shape[1:], dtype=dtype, device=o_part.device)
    a, b, c, d = _desc(o_part), _desc(m_part), _desc(l_part), _desc(out)
    _check(L.load().svodb_combine_splits(_p(a), _p(b), _p(c), _p(d), _stream()))
    return out


# ---------------------------------------------------------------------------- heads
def _qkv_opts(opts: Qkv, keep: list):
    o = L.QkvOpts()
    o.heads, o.kv_heads, o.head_dim, o.eps = opts.heads, opts.kv_heads, opts.head_dim, float(opts.eps)
    descs = [_desc(opts.q_norm), _desc(opts.k_norm),
             _desc(opts.rope[0]) if opts.rope else None, _desc(opts.rope[1]) if opts.rope else None]
    keep.extend(descs)
    if descs[0] is not None:
        o.q_norm = C.pointer(descs[0])
    if descs[1] is not None:
        o.k_norm = C.pointer(descs[1])
    if opts.rope:
        o.rope_cos, o.rope_sin = C.pointer(descs[2]), C.pointer(descs[3])
    return o


def heads(qkv: torch.Tensor, opts: Qkv):
    """`ops::heads` (tk/src/ops/heads.rs:37-102): `(q, k, v)`."""
    if qkv.dim() != 3:
        raise OpsError(L.ERR_SHAPE, f"heads: qkv has shape {list(qkv.shape)}, expected [B, T, slots*head_dim]")
    B, T = qkv.shape[:2]
    mk = lambda h: torch.empty(B, T, h, opts.head_dim, dtype=qkv.dtype, device=qkv.device)
    q, k, v = mk(opts.heads), mk(opts.kv_heads), mk(opts.kv_heads)
    keep: list = []
    o = _qkv_opts(opts, keep)
    xd, qd, kd, vd = _desc(qkv), _desc(q), _desc(k), _desc(v)
    _check(L.load().svodb_heads(_p(xd), C.byref(o), _p(qd), _p(kd), _p(vd), _stream()))
    return q, k, v


# ---------------------------------------------------------------------------- norms
def layer_norm(x, w, b=None, eps: float = 1e-5):
    """`ops::layer_norm` (tk/src/ops/norm.rs:17-19)."""
    out = torch.empty_like(x)
    xd, wd, bd, od = _desc(x), _desc(w), _desc(b), _desc(out)
    _check(L.load().svodb_layer_norm(_p(xd), _p(wd), _p(bd), float(eps), _p(od), _stream()))
    return out


def add_layer_norm(x, residual, w, b=None, eps: float = 1e-5):
    """`ops::add_layer_norm` (tk/src/ops/norm.rs:22-32): `(x + residual, norm)`."""
    out, s = torch.empty_like(x), torch.empty_like(x)
    xd, rd, wd, bd, sd, od = _desc(x), _desc(residual), _desc(w), _desc(b), _desc(s), _desc(out)
    _check(L.load().svodb_add_layer_norm(_p(xd), _p(rd), _p(wd), _p(bd), float(eps), _p(sd), _p(od), _stream()))
    return s, out


def rms_norm(x, w, eps: float = 1e-6):
    """`ops::rms_norm` (tk/src/ops/norm.rs:35-37)."""
    out = torch.empty_like(x)
    xd, wd, od = _desc(x), _desc(w), _desc(out)
    _check(L.load().svodb_rms_norm(_p(xd), _p(wd), float(eps), _p(od), _stream()))
    return out


def add_rms_norm(x, residual, w, eps: float = 1e-6):
    """`ops::add_rms_norm` (tk/src/ops/norm.rs:40-43): `(x + residual, norm)`."""
    out, s = torch.empty_like(x), torch.empty_like(x)
    xd, rd, wd, sd, od = _desc(x), _desc(residual), _desc(w), _desc(s), _desc(out)
    _check(L.load().svodb_add_rms_norm(_p(xd), _p(rd), _p(wd), float(eps), _p(sd), _p(od), _stream()))
    return s, out


# ----------------------------------------------------------------------------- glue
def embed(ids, table, pos_table=None, type_row=None, pad_id: int = -1):
    """Token embedding lookup; with `pos_table` and `pad_id >= 0` the XLM-R
    form (model/src/xlm_roberta/embeddings.rs:53-63)."""
    B, T = ids.shape
    out = torch.empty(B, T, table.shape[1], dtype=table.dtype, device=table.device)
    a, b, c, d, e = _desc(ids), _desc(table), _desc(pos_table), _desc(type_row), _desc(out)
    _check(L.load().svodb_embed(_p(a), _p(b), _p(c), _p(d), int(pad_id), _p(e), _stream()))
    return out


def embed_norm(ids, table, norm_w, norm_b=None, eps: float = 1e-5, pos_table=None, type_row=None, pad_id: int = -1,
               layer: bool = True):
    """The lookup of `embed` and the embedding norm in one kernel
    (model/src/xlm_roberta/embeddings.rs:53-63: word + position + type, LayerNorm)."""
    B, T = ids.shape
    out = torch.empty(B, T, table.shape[1], dtype=table.dtype, device=table.device)
    a, b, c, d, e = _desc(ids), _desc(table), _desc(pos_table), _desc(type_row), _desc(out)
    w, bb = _desc(norm_w), _desc(norm_b)
    _check(L.load().svodb_embed_norm(_p(a), _p(b), _p(c), _p(d), int(pad_id), _p(w), _p(bb), float(eps), int(layer),
                                     _p(e), _stream()), 1)
    return out


POOL_CLS, POOL_MEAN, POOL_LAST, POOL_GATHER = 0, 1, 2, 3


def norm_pool(hidden, norm_w=None, norm_b=None, eps: float = 1e-5, layer: bool = True, aux=None, mode: int = POOL_CLS,
              normalize: bool = True, out=None, gather=None):
    """The stack's final norm (none when `norm_w` is None), the pooling and the
    L2 normalisation in one kernel (model/src/encoder_head.rs:280-286;
    model/src/qwen3/model.rs:77-99): `hidden [B,L,D]` before its final norm ->
    f32 `[B,D]`. Only the pooled tokens are normalised (every real token for the
    masked mean).

    `gather` (a `peer.PeerGather` bound to a gather buffer): the rows are written
    into this rank's slot of that buffer and gathered from the other GPUs — the
    pooling kernel itself stores each row into the peers' staging buffers, then the
    unstage kernel follows (`svodb_norm_pool_gather`). Returns the whole buffer."""
    B, _, D = hidden.shape
    if gather is not None:
        out = gather.gathered
    elif out is None:
        rows = B * aux.shape[1] if mode == POOL_GATHER else B
        out = torch.empty(rows, D, dtype=torch.float32, device=hidden.device)
    if aux is not None and aux.dtype not in (torch.bool, torch.uint8, torch.int32):
        aux = aux.to(torch.int32)
    a, b, c, w, bb = _desc(hidden), _desc(aux), _desc(out), _desc(norm_w), _desc(norm_b)
    lib = L.load()

    def call(scratch):
        if gather is not None:
            return lib.svodb_norm_pool_gather(_p(a), _p(w), _p(bb), float(eps), int(layer), scratch, _p(b), int(mode),
                                              int(normalize), C.byref(gather.ctx), _p(c), _stream())
        return lib.svodb_norm_pool(_p(a), _p(w), _p(bb), float(eps), int(layer), scratch, _p(b), int(mode), int(normalize),
                                   _p(c), _stream())

    rc = call(None)
    if rc == L.ERR_WORKSPACE:
        # rows outside the fused kernel: the unfused sequence wants room for the normalised hidden states
        scratch = torch.empty_like(hidden)
        sd = _desc(scratch)
        rc = call(_p(sd))
    _check(rc, 1 if gather is None or gather.world == 1 else 2)
    return out


def pool(hidden, aux=None, mode: int = POOL_CLS, normalize: bool = True, out=None):
    """`encoder_head::pool` + L2 (model/src/encoder_head.rs:280-286): `[B,L,D]`
    -> f32 `[B,D]`; `out` may be a row slice of a wider gather buffer."""
    B, _, D = hidden.shape
    if out is None:
        rows = B * aux.shape[1] if mode == POOL_GATHER else B
        out = torch.empty(rows, D, dtype=torch.float32, device=hidden.device)
    if aux is not None and aux.dtype not in (torch.bool, torch.uint8, torch.int32):
        aux = aux.to(torch.int32)
    a, b, c = _desc(hidden), _desc(aux), _desc(out)
    _check(L.load().svodb_pool(_p(a), _p(b), int(mode), int(normalize), _p(c), _stream()), 2 if normalize else 1)
    return out


def rope_table(theta: float, positions, head_dim: int, dtype, device="cuda"):
    """`Tensor::rope_table` (tensor/src/transformer.rs:130-164): `(cos, sin)` of
    `[P, head_dim/2]`; `positions` an int or an int32 tensor `[P]`."""
    if isinstance(positions, int):
        n, pos = positions, None
    else:
        pos = positions.to(torch.int32).contiguous().view(-1)
        n = pos.numel()
    cos = torch.empty(n, head_dim // 2, dtype=dtype, device=device)
    sin = torch.empty_like(cos)
    a, b, c = _desc(pos), _desc(cos), _desc(sin)
    _check(L.load().svodb_rope_table(float(theta), _p(a), int(head_dim), _p(b), _p(c), _stream()))
    return cos, sin
