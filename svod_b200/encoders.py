"""The three encoder stacks that call the op layer, wired as the reference's
model crate wires them, plus CUDA-graph replay of a fixed plan shape and the
batch sharding used on several GPUs.

  XLM-RoBERTa / BGE-M3   model/src/xlm_roberta/{attention.rs:63-77, feed_forward.rs:40-45,
                         encoder_layer.rs:45-49, embeddings.rs:53-63}
  Qwen3 embedding        model/src/qwen3/{attention.rs:69-113, feed_forward.rs:38-42,
                         decoder_layer.rs:55-65, embedder.rs:37-52}
  ModernBERT             model/src/modernbert/{attention.rs:52-68, mlp.rs:41-46,
                         encoder_layer.rs:52-60, encoder.rs:33-54}
  pooling                model/src/encoder_head.rs:280-286

Weights are plain dicts of CUDA tensors (random-init helpers below); every
computation goes through `svod_b200.ops`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from . import ops
from .ops import Act, Attn, KeyMask, Linear, Qkv, Rotary


# --------------------------------------------------------------------------- configs
@dataclass
class XlmRobertaConfig:
    """model/src/xlm_roberta/config.rs:119-136 (XLM-RoBERTa-large defaults)."""
    vocab_size: int = 250002
    hidden_size: int = 1024
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    intermediate_size: int = 4096
    max_position_embeddings: int = 514
    type_vocab_size: int = 1
    layer_norm_eps: float = 1e-5
    pad_token_id: int = 1
    dtype: torch.dtype = torch.float16
    pooling: str = "cls"


@dataclass
class Qwen3Config:
    """model/src/qwen3/config.rs:62-81 (Qwen3-0.6B defaults)."""
    vocab_size: int = 151669
    hidden_size: int = 1024
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 3072
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    dtype: torch.dtype = torch.bfloat16


@dataclass
class ModernBertConfig:
    """model/src/modernbert/config.rs:72-92 (ModernBERT-base defaults)."""
    vocab_size: int = 50368
    hidden_size: int = 768
    num_hidden_layers: int = 22
    num_attention_heads: int = 12
    intermediate_size: int = 1152
    norm_eps: float = 1e-5
    global_attn_every_n_layers: int = 3
    global_rope_theta: float = 160000.0
    local_rope_theta: float = 10000.0
    local_attention: int = 128
    dtype: torch.dtype = torch.bfloat16
    pooling: str = "mean"


def _randn(gen, shape, dtype, device, sigma=0.02):
    return (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * sigma).to(dtype)


# --------------------------------------------------------------------------- XLM-R
class XlmRobertaEncoder:
    def __init__(self, cfg: XlmRobertaConfig, params: Dict):
        self.cfg, self.p = cfg, params
        # One fused [3D, D] projection computes the same columns as the
        # reference's three GEMMs; attention then reads q, k, v in place.
        for lp in params["layers"]:
            if "qkv_w" not in lp:
                lp["qkv_w"] = torch.cat([lp["q_w"], lp["k_w"], lp["v_w"]], 0).contiguous()
                lp["qkv_b"] = torch.cat([lp["q_b"], lp["k_b"], lp["v_b"]], 0).contiguous()

    @staticmethod
    def random_init(cfg: XlmRobertaConfig, seed: int = 0, device="cuda") -> "XlmRobertaEncoder":
        g = torch.Generator(device=device).manual_seed(seed)
        D, F, dt = cfg.hidden_size, cfg.intermediate_size, cfg.dtype
        r = lambda *s: _randn(g, s, dt, device)
        ones = lambda n: torch.ones(n, dtype=dt, device=device)
        zeros = lambda n: torch.zeros(n, dtype=dt, device=device)
        layers = []
        for _ in range(cfg.num_hidden_layers):
            layers.append(dict(q_w=r(D, D), q_b=r(D), k_w=r(D, D), k_b=r(D), v_w=r(D, D), v_b=r(D),
                               o_w=r(D, D), o_b=r(D), ln1_w=ones(D), ln1_b=zeros(D),
                               fi_w=r(F, D), fi_b=r(F), fo_w=r(D, F), fo_b=r(D), ln2_w=ones(D), ln2_b=zeros(D)))
        p = dict(word=r(cfg.vocab_size, D), pos=r(cfg.max_position_embeddings, D), type=r(cfg.type_vocab_size, D),
                 emb_ln_w=ones(D), emb_ln_b=zeros(D), layers=layers)
        return XlmRobertaEncoder(cfg, p)

    def hidden(self, ids: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        c, p = self.cfg, self.p
        H = c.num_attention_heads
        # lookup (word + position + type) and the embedding LayerNorm: one kernel
        x = ops.embed_norm(ids, p["word"], p["emb_ln_w"], p["emb_ln_b"], c.layer_norm_eps, p["pos"], p["type"],
                           c.pad_token_id)
        return self.run_layers(x, mask)

    def run_layers(self, x: torch.Tensor, mask: torch.Tensor, start: int = 0, stop: Optional[int] = None):
        """Layers `start .. stop` over the hidden states `x [B,L,D]`."""
        c, p = self.cfg, self.p
        H = c.num_attention_heads
        B, L, D = x.shape
        keys = KeyMask.Bool(mask)
        for lp in p["layers"][start:stop]:
            qkv = ops.linear(x, lp["qkv_w"], Linear(bias=lp["qkv_b"]))
            a = ops.attention_packed(qkv, H, H, Attn(keys=keys)).view(B, L, D)
            y = ops.linear(a, lp["o_w"], Linear(bias=lp["o_b"], residual=x))
            x = ops.layer_norm(y, lp["ln1_w"], lp["ln1_b"], c.layer_norm_eps)
            f = ops.linear(x, lp["fi_w"], Linear(bias=lp["fi_b"], act=Act.GELU))
            y = ops.linear(f, lp["fo_w"], Linear(bias=lp["fo_b"], residual=x))
            x = ops.layer_norm(y, lp["ln2_w"], lp["ln2_b"], c.layer_norm_eps)
        return x

    def forward(self, ids, mask, out=None, gather=None):
        h = self.hidden(ids, mask)
        mode = ops.POOL_CLS if self.cfg.pooling == "cls" else ops.POOL_MEAN
        # post-LN stack: the last layer's norm is the final one; pooling + L2 in one kernel
        return ops.norm_pool(h, aux=mask if mode == ops.POOL_MEAN else None, mode=mode, out=out, gather=gather)


# --------------------------------------------------------------------------- Qwen3
class Qwen3Embedder:
    def __init__(self, cfg: Qwen3Config, params: Dict, fused_prologue: bool = True):
        self.cfg, self.p = cfg, params
        self._rope = {}
        self.fused_prologue = fused_prologue

    @staticmethod
    def random_init(cfg: Qwen3Config, seed: int = 0, device="cuda") -> "Qwen3Embedder":
        g = torch.Generator(device=device).manual_seed(seed)
        D, F, dt = cfg.hidden_size, cfg.intermediate_size, cfg.dtype
        H, Hkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        r = lambda *s: _randn(g, s, dt, device)
        ones = lambda n: torch.ones(n, dtype=dt, device=device)
        layers = []
        for _ in range(cfg.num_hidden_layers):
            layers.append(dict(in_w=ones(D), qkv_w=r((H + 2 * Hkv) * hd, D), qn_w=ones(hd), kn_w=ones(hd),
                               o_w=r(D, H * hd), post_w=ones(D), gu_w=r(2 * F, D), down_w=r(D, F)))
        return Qwen3Embedder(cfg, dict(embed=r(cfg.vocab_size, D), layers=layers, norm_w=ones(D)))

    def rope(self, L: int, device):
        if L not in self._rope:
            hd = self.cfg.head_dim
            cos, sin = ops.rope_table(self.cfg.rope_theta, L, hd, self.cfg.dtype, device)
            self._rope[L] = (cos.view(1, L, 1, hd // 2), sin.view(1, L, 1, hd // 2))
        return self._rope[L]

    def hidden(self, ids: torch.Tensor, seg_start: Optional[torch.Tensor] = None,
               rope=None) -> torch.Tensor:
        c, p = self.cfg, self.p
        H, Hkv, hd = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        x = self.run_layers(ops.embed(ids, p["embed"]), seg_start, rope)
        return ops.rms_norm(x, p["norm_w"], c.rms_norm_eps)

    def run_layers(self, x: torch.Tensor, seg_start: Optional[torch.Tensor] = None, rope=None, start: int = 0,
                   stop: Optional[int] = None) -> torch.Tensor:
        """Layers `start .. stop` over the hidden states `x [B,L,D]` (no final norm)."""
        c, p = self.cfg, self.p
        H, Hkv, hd = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        B, L, D = x.shape
        rope = rope or self.rope(L, x.device)
        for lp in p["layers"][start:stop]:
            xn = ops.rms_norm(x, lp["in_w"], c.rms_norm_eps)
            prologue = Qkv(H, Hkv, hd, lp["qn_w"], lp["kn_w"], c.rms_norm_eps, rope)
            if self.fused_prologue:
                # q/k norm and rotation in the projection's store; attention reads
                # the packed projection in place (no q, k, v copies).
                qkv = ops.linear(xn, lp["qkv_w"], Linear(qkv=prologue))
                a = ops.attention_packed(qkv, H, Hkv, Attn(causal=True, seg_start=seg_start)).view(B, L, H * hd)
            else:
                # the reference's op sequence (model/src/qwen3/attention.rs:69-113)
                q, k, v = ops.heads(ops.linear(xn, lp["qkv_w"]), prologue)
                a = ops.attention(q, k, v, Attn(causal=True, seg_start=seg_start)).view(B, L, H * hd)
            h = ops.linear(a, lp["o_w"], Linear(residual=x))
            hn = ops.rms_norm(h, lp["post_w"], c.rms_norm_eps)
            g = ops.linear(hn, lp["gu_w"], Linear(act=Act.SILU, gated=True))
            x = ops.linear(g, lp["down_w"], Linear(residual=h))
        return x

    def forward(self, ids, lengths, out=None, gather=None):
        # final RMSNorm of the pooled (last real) tokens alone, pooling and L2: one kernel
        x = self.run_layers(ops.embed(ids, self.p["embed"]))
        return ops.norm_pool(x, self.p["norm_w"], None, self.cfg.rms_norm_eps, layer=False, aux=lengths,
                             mode=ops.POOL_LAST, out=out, gather=gather)


# --------------------------------------------------------------------------- ModernBERT
class ModernBertEncoder:
    def __init__(self, cfg: ModernBertConfig, params: Dict):
        self.cfg, self.p = cfg, params
        self._rope = {}

    @staticmethod
    def random_init(cfg: ModernBertConfig, seed: int = 0, device="cuda") -> "ModernBertEncoder":
        g = torch.Generator(device=device).manual_seed(seed)
        D, F, dt = cfg.hidden_size, cfg.intermediate_size, cfg.dtype
        r = lambda *s: _randn(g, s, dt, device)
        ones = lambda n: torch.ones(n, dtype=dt, device=device)
        layers = []
        for i in range(cfg.num_hidden_layers):
            layers.append(dict(attn_ln_w=None if i == 0 else ones(D), qkv_w=r(3 * D, D), o_w=r(D, D),
                               mlp_ln_w=ones(D), wi_w=r(2 * F, D), wo_w=r(D, F)))
        return ModernBertEncoder(cfg, dict(embed=r(cfg.vocab_size, D), emb_ln_w=ones(D), layers=layers,
                                           final_ln_w=ones(D)))

    def rope(self, L: int, device):
        if L not in self._rope:
            hd = self.cfg.hidden_size // self.cfg.num_attention_heads
            t = {}
            for is_global, theta in ((True, self.cfg.global_rope_theta), (False, self.cfg.local_rope_theta)):
                cos, sin = ops.rope_table(theta, L, hd, self.cfg.dtype, device)
                t[is_global] = (cos.view(1, L, 1, hd // 2), sin.view(1, L, 1, hd // 2))
            self._rope[L] = t
        return self._rope[L]

    def hidden(self, ids: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        c, p = self.cfg, self.p
        H = c.num_attention_heads
        hd = c.hidden_size // H
        x = ops.embed_norm(ids, p["embed"], p["emb_ln_w"], None, c.norm_eps)
        return ops.layer_norm(self.run_layers(x, mask), p["final_ln_w"], None, c.norm_eps)

    def run_layers(self, x: torch.Tensor, mask: torch.Tensor, start: int = 0, stop: Optional[int] = None):
        """Layers `start .. stop` over the hidden states `x [B,L,D]` (no final norm)."""
        c, p = self.cfg, self.p
        H = c.num_attention_heads
        hd = c.hidden_size // H
        B, L, D = x.shape
        tables = self.rope(L, x.device)
        keys = KeyMask.Bool(mask)
        half = c.local_attention // 2
        for li, lp in list(enumerate(p["layers"]))[start:stop]:
            is_global = li % c.global_attn_every_n_layers == 0
            cos, sin = tables[is_global]
            xn = x if lp["attn_ln_w"] is None else ops.layer_norm(x, lp["attn_ln_w"], None, c.norm_eps)
            qkv = ops.linear(xn, lp["qkv_w"], Linear(rope=Rotary(cos, sin, 2 * H, hd)))
            a = ops.attention_packed(qkv, H, H, Attn(keys=keys, window=None if is_global else (half, half)))
            h = ops.linear(a.view(B, L, D), lp["o_w"], Linear(residual=x))
            hn = ops.layer_norm(h, lp["mlp_ln_w"], None, c.norm_eps)
            g = ops.linear(hn, lp["wi_w"], Linear(act=Act.GELU, gated=True))
            x = ops.linear(g, lp["wo_w"], Linear(residual=h))
        return x

    def forward(self, ids, mask, out=None, gather=None):
        c, p = self.cfg, self.p
        x = self.run_layers(ops.embed_norm(ids, p["embed"], p["emb_ln_w"], None, c.norm_eps), mask)
        mode = ops.POOL_CLS if c.pooling == "cls" else ops.POOL_MEAN
        # final LayerNorm (of the tokens that are pooled), pooling and L2: one kernel
        return ops.norm_pool(x, p["final_ln_w"], None, c.norm_eps, aux=mask if mode == ops.POOL_MEAN else None,
                             mode=mode, out=out, gather=gather)


# --------------------------------------------------------------------------- plan replay
class Plan:
    """One plan shape `(rows, len)` captured once and replayed, as the
    reference's `HeadPlans::execute` does (model/src/encoder_head.rs:464-500):
    inputs are written into fixed device buffers, the whole stack is one CUDA
    graph launch, the pooled `[rows, D]` f32 output is read back.

    `aux` is the padding mask `[rows, len]` (bool) or the lengths `[rows]` (i32),
    whichever the model's `forward` takes. `out` may be this rank's slice of a
    gather buffer; `epilogue` (no arguments) is issued on the plan's stream right
    after the stack and becomes part of the captured graph: the all-gather of the
    pooled rows on several GPUs, so that a replay is the whole step. `gather` (a
    `peer.PeerGather` bound to the gather buffer) instead makes the stack's pooling
    kernel send its rows to the other GPUs itself, with the unstage kernel behind it.
    """

    def __init__(self, model, rows: int, length: int, aux_kind: str, out: Optional[torch.Tensor] = None,
                 ids_dtype=torch.int32, device="cuda", epilogue=None, gather=None):
        self.model = model
        self.epilogue = epilogue
        self.gather = gather
        self.ids = torch.zeros(rows, length, dtype=ids_dtype, device=device)
        self.aux = (torch.ones(rows, length, dtype=torch.bool, device=device) if aux_kind == "mask"
                    else torch.full((rows,), length, dtype=torch.int32, device=device))
        D = model.cfg.hidden_size
        self.out = out if out is not None else torch.empty(rows, D, dtype=torch.float32, device=device)
        self.graph = None
        self.stream = torch.cuda.Stream(device=device)

    def capture(self):
        # One eager run first: first-use work (kernel attributes, RoPE tables)
        # happens outside the capture.
        with torch.cuda.stream(self.stream):
            self._step()
        self.stream.synchronize()
        ops.device_status()
        g = torch.cuda.CUDAGraph()
        # thread-local capture mode: helper threads of the process (a collective
        # library's watchdog) may query events while this thread captures
        with torch.cuda.graph(g, stream=self.stream, capture_error_mode="thread_local"):
            self._step()
        self.graph = g
        return self

    def _step(self):
        if self.gather is not None:
            self.model.forward(self.ids, self.aux, self.out, gather=self.gather)
        else:
            self.model.forward(self.ids, self.aux, self.out)
        if self.epilogue is not None:
            self.epilogue()

    def run(self, ids_host: torch.Tensor, aux_host: torch.Tensor, out_host: Optional[torch.Tensor] = None):
        """Host (pinned) inputs -> device, replay, pooled output -> host."""
        with torch.cuda.stream(self.stream):
            self.ids.copy_(ids_host, non_blocking=True)
            self.aux.copy_(aux_host, non_blocking=True)
            self.graph.replay()
            if out_host is not None:
                out_host.copy_(self.out, non_blocking=True)
        return self.out

    def replay(self):
        with torch.cuda.stream(self.stream):
            self.graph.replay()

    def check(self):
        """Waits for the plan's stream and raises if a bounded device-side wait ran
        out during the replays since the last check (the status word is cleared, so
        a stale value never reaches later launches)."""
        with torch.cuda.stream(self.stream):
            ops.device_status()


# --------------------------------------------------------------------------- sharding
def shard_rows(lengths: List[int], world: int) -> List[List[int]]:
    """Deals rows to `world` ranks longest-first, round-robin, so padded token
    counts balance (the reference runs chunks longest-first:
    arch/src/pipelines/text.rs:968-985). Returns the row indices of each rank."""
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    return [order[r::world] for r in range(world)]


def unshard_rows(gathered: torch.Tensor, shards: List[List[int]]) -> torch.Tensor:
    """Undoes `shard_rows` on the gathered `[rows, D]` output: gathered row
    `r * per + i` is input row `shards[r][i]`; returns the rows in input order."""
    order = torch.tensor([i for sh in shards for i in sh], device=gathered.device)
    out = torch.empty_like(gathered)
    out[order] = gathered
    return out


def gather_pooled(local: torch.Tensor, gathered: torch.Tensor, group=None):
    """The path's one collective: an all-gather of pooled `[rows, D]` f32 over
    NCCL. `local` should be this rank's slice of `gathered` (in-place gather)."""
    import torch.distributed as dist
    dist.all_gather_into_tensor(gathered, local, group=group)
    return gathered
