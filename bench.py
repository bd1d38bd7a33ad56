#!/usr/bin/env python
"""Benchmark of the encoder hot path.

    python bench.py --gpus N --steps K --warmup W            (this library)
    python bench.py --impl reference --steps K --warmup W    (CPU restatement on the host cores)

One step = one pass of the hot path over one batch of synthetic input: the
Qwen3-0.6B-shaped embedding stack (28 layers, hidden 1024, 16/8 heads x 128,
SwiGLU 3072, causal, seq 4096, batch 32 per GPU, bf16, random-init weights,
uniform token ids), i.e. the configuration that carries the flash-attention
target (seq 4096 / head_dim 128). Each rank holds a weight replica and runs a
full batch (weak scaling); the one collective is an NCCL all-gather of the
pooled `[32, 1024]` f32 rows, which each rank writes straight into its slot of
the gather buffer.

Prints ONE JSON line on rank 0. `value` is device-timed with inputs resident in
HBM (one CUDA-graph replay per step, the all-gather captured inside the graph,
CUDA events on the launching stream, max over ranks); `e2e` adds the pinned-host
-> device copy of every step's inputs and the device -> host read of the pooled
result inside the timed region. `roofline` is measured live for the dominant
kernel (timed alone against the burst peak, and inside a step against the
sustained one); `cpu_baseline` times the compiled C + OpenMP restatement on a
bounded sample of the same workload on this box's host cores. `strong` deals ONE
batch of 32 ragged rows over the ranks (`shard_rows`) and times that; at N = 1
`workloads` adds the two other encoder configurations (XLM-RoBERTa-large
B64 x 512 fp16, ModernBERT-base B16 x 8192 bf16).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "encoder tokens/sec"
UNIT = "tokens/s"

WORKLOADS = {
    # name: (kind, batch per GPU, seq)
    "qwen3-0.6b-embed": ("qwen3", 32, 4096),
    "xlm-roberta-large": ("xlmr", 64, 512),
    "modernbert-base": ("modernbert", 16, 8192),
}


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per launch and batch
# row, from the ncu captures summarised under profiles/: the captures run the
# bench's per-launch shape at batch 4 (a full launch is too large to capture
# under a profiler), and the traffic of both kernels grows in proportion to the
# rows (every CTA works on one batch row's tiles).
NCU_DRAM_BYTES_PER_ROW = {
    ("qwen3", "flash_attention"): 803.5e6 / 16,  # batch 16: 562.0 MB read + 241.4 MB written against 402.7 MB algorithmic
                                                 # (batch 4: 203.1 MB, the same 50 MB a row; K/V fetched again, L2 hit rate 73-78 %)
    ("qwen3", "gemm"): 101.7e6 / 4,              # algorithmic 96.5 MB at batch 4 (M = 16384)
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], burst=d["bf16_tflops"], sustained=d["bf16_tflops_sustained"], source="measured")
    return dict(hbm_gbs=6650.0, burst=1590.0, sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only) while the
    timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.1)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def visible_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except ValueError:
            return local_rank
    return local_rank


# --------------------------------------------------------------------------- CPU legs
CPU_SAMPLES = {
    # kind: (rows, seq, layers timed, layers of the full stack)
    "qwen3": (1, 4096, 4, 28),
    "xlmr": (4, 512, 4, 24),
    "modernbert": (1, 8192, 3, 22),
}


def oracle_sample(kind: str, seed: int = 7):
    """A bounded sample of the workload for the compiled CPU restatement
    (`oracle/svod_oracle.c`: f32, OpenMP over all host threads): a few rows of the
    workload's sequence length through a few layers of the same architecture.
    Returns a closure that runs it (and returns the seconds the FULL depth would
    take, by layer count) and the number of tokens it processes."""
    import numpy as np
    import torch
    from oracle import c_oracle as C
    try:
        C.build()
    except Exception:
        pass  # a library built earlier still loads; `load()` reports a missing one
    C.load()
    C.use_all_cores()  # launchers export OMP_NUM_THREADS=1; the baseline uses every core it may run on
    rows, seq, layers, full = CPU_SAMPLES[kind]
    g = torch.Generator().manual_seed(seed)
    dt16 = torch.float16 if kind == "xlmr" else torch.bfloat16
    w = lambda *sh: (torch.randn(*sh, generator=g) * 0.02).to(dt16).float().numpy()
    ones = lambda n: np.ones(n, dtype=np.float32)
    zeros = lambda n: np.zeros(n, dtype=np.float32)
    if kind == "qwen3":
        D, H, Hkv, hd, F = 1024, 16, 8, 128, 3072
        lp = dict(in_w=ones(D), qkv_w=w((H + 2 * Hkv) * hd, D), qn_w=ones(hd), kn_w=ones(hd), o_w=w(D, H * hd),
                  post_w=ones(D), gu_w=w(2 * F, D), down_w=w(D, F))
        hidden = w(rows, seq, D)

        def run():
            t0 = time.perf_counter()
            C.qwen3_layers(hidden, [lp] * layers, heads_n=H, kv_heads=Hkv, head_dim=hd, dtype=C.BF16)
            return (time.perf_counter() - t0) * full / layers
    elif kind == "xlmr":
        D, H, F = 1024, 16, 4096
        lp = dict(q_w=w(D, D), q_b=w(D), k_w=w(D, D), k_b=w(D), v_w=w(D, D), v_b=w(D), o_w=w(D, D), o_b=w(D),
                  ln1_w=ones(D), ln1_b=zeros(D), fi_w=w(F, D), fi_b=w(F), fo_w=w(D, F), fo_b=w(D), ln2_w=ones(D),
                  ln2_b=zeros(D))
        hidden = w(rows, seq, D)
        lens = np.array([512, 64, 288, 400][:rows])
        mask = np.arange(seq)[None, :] < lens[:, None]

        def run():
            t0 = time.perf_counter()
            C.xlmr_layers(hidden, [lp] * layers, mask, heads_n=H, dtype=C.F16)
            return (time.perf_counter() - t0) * full / layers
    else:
        D, H, F = 768, 12, 1152
        lp = dict(attn_ln_w=ones(D), qkv_w=w(3 * D, D), o_w=w(D, D), mlp_ln_w=ones(D), wi_w=w(2 * F, D), wo_w=w(D, F))
        hidden = w(rows, seq, D)
        mask = np.ones((rows, seq), dtype=bool)

        def run():
            # one global layer and two windowed ones timed apart: the stack has 8 and 14 of them
            t0 = time.perf_counter()
            C.modernbert_layers(hidden, [lp], mask, heads_n=H, first_layer=0, dtype=C.BF16)
            t1 = time.perf_counter()
            C.modernbert_layers(hidden, [lp] * 2, mask, heads_n=H, first_layer=1, dtype=C.BF16)
            t2 = time.perf_counter()
            n_global = (full + 2) // 3
            return (t1 - t0) * n_global + (t2 - t1) / 2 * (full - n_global)

    return run, rows * seq


def cpu_threads() -> int:
    from oracle import c_oracle as C
    return C.threads()


def time_cpu(kind: str, steps: int, warmup: int):
    """Times the compiled CPU restatement on a few layers of a few rows and scales
    to the full depth (every layer of a kind does identical work; the embedding
    lookup and the pooling are negligible)."""
    run, tokens = oracle_sample(kind)
    rows, seq, layers, full_layers = CPU_SAMPLES[kind]
    for _ in range(warmup):
        run()
    full = sum(run() for _ in range(steps)) / steps
    sample = (f"C + OpenMP f32 restatement, {rows} row(s) x {seq} tokens, {layers} of {full_layers} layers timed "
              f"and scaled to {full_layers}, {steps} step(s)")
    return tokens / full, full * 1e3, sample


def time_torch_cpu(seq: int = 4096, layers: int = 4, full_layers: int = 28, steps: int = 1):
    """A second, separately labelled CPU reference point (not svod, not the
    oracle): the Qwen3-shaped layer in plain PyTorch f32 CPU ops
    (`F.linear`, `F.scaled_dot_product_attention`) on the same bounded sample,
    with all the threads torch will use."""
    import torch
    import torch.nn.functional as F
    try:
        torch.set_num_threads(len(os.sched_getaffinity(0)))  # launchers export OMP_NUM_THREADS=1
    except (AttributeError, RuntimeError):
        pass
    g = torch.Generator().manual_seed(7)
    D, H, Hkv, hd, Fn = 1024, 16, 8, 128, 3072
    r = lambda *sh: torch.randn(*sh, generator=g) * 0.02
    ws = [dict(qkv=r((H + 2 * Hkv) * hd, D), o=r(D, H * hd), gu=r(2 * Fn, D), down=r(D, Fn)) for _ in range(layers)]
    x0 = torch.randn(1, seq, D, generator=g)
    ang = torch.arange(seq)[:, None] * (1e6 ** (-torch.arange(0, hd, 2) / hd))[None, :]
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    rms = lambda t: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-6)

    def rot(t):
        a, b = t[..., :hd // 2], t[..., hd // 2:]
        return torch.cat([a * cos - b * sin, a * sin + b * cos], -1)

    def run():
        x = x0
        with torch.no_grad():
            for w in ws:
                qkv = F.linear(rms(x), w["qkv"]).view(1, seq, H + 2 * Hkv, hd)
                q, k, v = qkv[:, :, :H], qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:]
                q, k = rot(rms(q)), rot(rms(k))
                k, v = k.repeat_interleave(H // Hkv, 2), v.repeat_interleave(H // Hkv, 2)
                a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                   is_causal=True).transpose(1, 2).reshape(1, seq, H * hd)
                h = x + F.linear(a, w["o"])
                gu = F.linear(rms(h), w["gu"])
                x = h + F.linear(F.silu(gu[..., :Fn]) * gu[..., Fn:], w["down"])
        return x

    run()
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = (time.perf_counter() - t0) / steps * full_layers / layers
    return {"value": seq / dt, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "torch f32 CPU ops (not svod)",
            "sample": f"1 sequence x {seq} tokens, {layers} of {full_layers} layers timed and scaled"}


def reference_arm(args):
    """`--impl reference`: the reference's own CPU path cannot be built here (no
    Rust toolchain), so the arm times the CPU restatement of the same path on
    the host cores (C + OpenMP, f32, every host thread) on a bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    kind, batch, seq = WORKLOADS[args.workload]
    value, ms, sample = time_cpu(kind, max(1, args.steps), max(0, args.warmup))
    cores = cpu_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16" if kind == "xlmr" else "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "batch_per_gpu": batch, "seq_len": seq, "parallelism": "cpu"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def build_model(kind: str, device, reference_ops: bool = False):
    from svod_b200 import encoders as E
    if kind == "qwen3":
        m = E.Qwen3Embedder.random_init(E.Qwen3Config(), seed=0, device=device)
        m.fused_prologue = not reference_ops
        return m, "lengths"
    if kind == "xlmr":
        return E.XlmRobertaEncoder.random_init(E.XlmRobertaConfig(), seed=0, device=device), "mask"
    return E.ModernBertEncoder.random_init(E.ModernBertConfig(), seed=0, device=device), "mask"


def step_flops(kind: str, batch: int, seq: int):
    """Algorithmic FLOPs of one step: GEMM 2*M*N*K, attention 4*B*H*T*T*D halved
    when causal (the reference printer's conventions, tk/examples/tk_bench.rs:221,277)."""
    M = batch * seq
    if kind == "qwen3":
        gemm = 28 * 2 * M * (4096 * 1024 + 1024 * 2048 + 2 * 3072 * 1024 + 1024 * 3072)
        attn = 28 * 4 * batch * 16 * seq * seq * 128 // 2
    elif kind == "xlmr":
        gemm = 24 * 2 * M * (4 * 1024 * 1024 + 2 * 1024 * 4096)
        attn = 24 * 4 * batch * 16 * seq * seq * 64
    else:
        gemm = 22 * 2 * M * (2304 * 768 + 768 * 768 + 2 * 1152 * 768 + 768 * 1152)
        attn = 8 * 4 * batch * 12 * seq * seq * 64 + 14 * 4 * batch * 12 * seq * 129 * 64
    return gemm, attn


def time_kernel(fn, stream, reps: int):
    import torch
    for _ in range(3):
        fn()
    stream.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        fn()
    e1.record(stream)
    stream.synchronize()
    return e0.elapsed_time(e1) / reps


def kernel_rooflines(kind: str, batch: int, seq: int, peaks):
    """Live per-launch timing of the two contraction kernels at the workload's
    shapes: the flash-attention launch and the largest GEMM launch, 20 launches
    captured into one CUDA graph (the host call path stays out of the timed
    region) and timed with CUDA events on the replaying stream."""
    import torch
    from svod_b200 import ops
    out = {}
    g = torch.Generator(device="cuda").manual_seed(1)
    if kind == "qwen3":
        H, Hkv, D, causal = 16, 8, 128, True
    elif kind == "xlmr":
        H, Hkv, D, causal = 16, 16, 64, False
    else:
        H, Hkv, D, causal = 12, 12, 64, False
    dt16 = torch.float16 if kind == "xlmr" else torch.bfloat16
    q = torch.randn(batch, seq, H, D, generator=g, device="cuda").to(dt16)
    k = torch.randn(batch, seq, Hkv, D, generator=g, device="cuda").to(dt16)
    v = torch.randn(batch, seq, Hkv, D, generator=g, device="cuda").to(dt16)
    a = ops.Attn(causal=causal)
    ms = time_graphed(lambda: ops.attention(q, k, v, a), 20)
    fl = 4 * batch * H * seq * seq * D / (2 if causal else 1)
    out["flash_attention"] = {"ms": ms, "tflops": fl / ms / 1e9, "flops_per_launch": fl,
                              "launches_per_step": {"qwen3": 28, "xlmr": 24, "modernbert": 8}[kind]}
    del q, k, v
    M = batch * seq
    if kind == "qwen3":
        N, K, opts, gated = 3072, 1024, ops.Linear(act=ops.Act.SILU, gated=True), True
    elif kind == "xlmr":
        N, K, opts, gated = 4096, 1024, ops.Linear(act=ops.Act.GELU), False
    else:
        N, K, opts, gated = 1152, 768, ops.Linear(act=ops.Act.GELU, gated=True), True
    x = (torch.randn(M, K, generator=g, device="cuda") * 0.5).to(dt16)
    w = (torch.randn((2 if gated else 1) * N, K, generator=g, device="cuda") * 0.02).to(dt16)
    ms = time_graphed(lambda: ops.linear(x, w, opts), 20)
    fl = 2 * M * N * K * (2 if gated else 1)
    out["gemm"] = {"ms": ms, "tflops": fl / ms / 1e9, "flops_per_launch": fl,
                   "launches_per_step": {"qwen3": 28, "xlmr": 24, "modernbert": 22}[kind]}
    for v_ in out.values():
        v_["frac_of_sustained"] = v_["tflops"] / peaks["sustained"]
        v_["frac_of_burst"] = v_["tflops"] / peaks["burst"]
        v_["frac_of_nominal_2250"] = v_["tflops"] / 2250.0
    return out


def synthetic_batch(kind: str, rows: int, seq: int, vocab: int, seed: int, ragged: bool):
    """Pinned host inputs of one batch: uniform ids (the pad id avoided) and the
    padding mask `[rows, seq]` (XLM-R lengths in [seq/8, seq], ModernBERT in
    [seq/4, seq], as the configurations state) or the lengths `[rows]` (Qwen3:
    full rows, or ragged ones when asked). Returns ids, aux, lengths."""
    import torch
    gen = torch.Generator().manual_seed(seed)
    ids = torch.randint(2, vocab, (rows, seq), generator=gen, dtype=torch.int32)
    if kind == "qwen3":
        lens = torch.randint(seq // 4, seq + 1, (rows,), generator=gen) if ragged else torch.full((rows,), seq)
        return ids, lens.to(torch.int32), lens
    lens = torch.randint(seq // 8 if kind == "xlmr" else seq // 4, seq + 1, (rows,), generator=gen)
    return ids, torch.arange(seq)[None, :] < lens[:, None], lens


class StackRun:
    """One plan of one stack on this rank: rows x seq, pooled rows written into this
    rank's slot of `gathered`, the all-gather captured inside the plan's graph."""

    def __init__(self, model, aux_kind, rows, seq, world, rank, device, gather="nccl"):
        import torch
        from svod_b200 import encoders as E
        from svod_b200 import ops
        self.world, self.rows, self.seq = world, rows, seq
        D = model.cfg.hidden_size
        self.gathered = torch.zeros(world * rows, D, dtype=torch.float32, device=device)
        self.mine = self.gathered[rank * rows:(rank + 1) * rows]
        self.out_host = torch.empty(rows, D, dtype=torch.float32).pin_memory()
        epilogue = None
        self.peer = None
        self.collective = "none"
        if world > 1 and gather == "peer":
            # the library's own all-gather: plain stores into the peers' staging buffers over NVLink;
            # if the peers' memory cannot be mapped here, every rank hears of it and all take NCCL
            from svod_b200.peer import PeerGather
            try:
                self.peer = PeerGather(rows, D).bind(self.gathered)
                self.collective = "peer"
            except ops.OpsError as e:
                sys.stderr.write(f"peer gather unavailable ({e}); using NCCL\n")
        if world > 1 and self.collective != "peer":
            epilogue = lambda: E.gather_pooled(self.mine, self.gathered)
            self.collective = "nccl"
        before = ops.launches
        self.plan = E.Plan(model, rows, seq, aux_kind, out=self.mine, device=device, epilogue=epilogue,
                           gather=self.peer if self.collective == "peer" else None)
        self._capture = lambda: self.plan.capture()
        self._before = before

    def load(self, ids_host, aux_host):
        import torch
        from svod_b200 import ops
        self.ids_host, self.aux_host = ids_host.pin_memory(), aux_host.pin_memory()
        self.plan.ids.copy_(self.ids_host)
        self.plan.aux.copy_(self.aux_host)
        torch.cuda.synchronize()
        self._capture()
        self.launches_per_step = (ops.launches - self._before) // 2   # capture() runs the stack twice (eager + capture)
        return self

    def step_resident(self):
        self.plan.replay()

    def step_e2e(self):
        import torch
        self.plan.run(self.ids_host, self.aux_host, None)
        with torch.cuda.stream(self.plan.stream):
            self.out_host.copy_(self.mine, non_blocking=True)

    def timed(self, fn, steps):
        import torch
        import torch.distributed as dist
        stream = self.plan.stream
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        stream.synchronize()
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=self.gathered.device)
        if self.world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    def h2d_bytes(self):
        return (self.ids_host.numel() * self.ids_host.element_size()
                + self.aux_host.numel() * self.aux_host.element_size())


def attention_in_step_ms(model, run):
    """The attention launches of one eager step, each bracketed by a CUDA-event
    pair on the step's stream, right after the timed steps (so under the same
    clocks): the mean per launch and the launch count."""
    import torch
    from svod_b200 import ops
    pairs = []
    real = {"attention": ops.attention, "attention_packed": ops.attention_packed}

    def wrap(fn):
        def inner(*a, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(torch.cuda.current_stream())
            out = fn(*a, **kw)
            e1.record(torch.cuda.current_stream())
            pairs.append((e0, e1))
            return out
        return inner

    plan = run.plan
    try:
        ops.attention, ops.attention_packed = wrap(real["attention"]), wrap(real["attention_packed"])
        with torch.cuda.stream(plan.stream):
            for it in range(2):
                pairs.clear()
                model.forward(plan.ids, plan.aux, plan.out)
        plan.stream.synchronize()
    finally:
        ops.attention, ops.attention_packed = real["attention"], real["attention_packed"]
    ms = [a.elapsed_time(b) for a, b in pairs]
    return (sum(ms) / len(ms), len(ms), max(ms)) if ms else (None, 0, None)


def measure_stack(kind, model, aux_kind, rows, seq, world, rank, device, args, ids_host, aux_host, sample_clocks):
    """Warm-up, K timed resident steps, K timed end-to-end steps of one plan."""
    import torch
    from svod_b200 import ops
    local = int(os.environ.get("LOCAL_RANK", "0"))
    run = StackRun(model, aux_kind, rows, seq, world, rank, device, getattr(args, "gather", "nccl")).load(ids_host,
                                                                                                        aux_host)
    for _ in range(max(3, args.warmup)):
        run.step_resident()
    run.plan.check()
    sampler = ClockSampler(visible_index(local)) if sample_clocks else None
    if sampler:
        sampler.start()
    ms_step = run.timed(run.step_resident, args.steps) / args.steps
    clocks = sampler.stop() if sampler else None
    for _ in range(2):
        run.step_e2e()
    run.plan.stream.synchronize()
    e2e_ms = run.timed(run.step_e2e, args.steps) / args.steps
    run.plan.check()
    return run, dict(ms_per_step=ms_step, e2e_ms=e2e_ms, clocks=clocks, finite=bool(torch.isfinite(run.mine).all()))


def gpu_arm(args):
    import torch
    import torch.distributed as dist
    from svod_b200 import encoders as E
    from svod_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the op layer has no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    kind, batch, seq = WORKLOADS[args.workload]
    peaks = measured_peaks()
    dtype_name = "f16" if kind == "xlmr" else "bf16"

    model, aux_kind = build_model(kind, device, args.reference_ops)
    D = model.cfg.hidden_size
    vocab = model.cfg.vocab_size

    # ---- weak pass: every rank its own full batch (the headline `value`) ----
    ids_host, aux_host, lens = synthetic_batch(kind, batch, seq, vocab, 1234 + rank, ragged=False)
    run, m = measure_stack(kind, model, aux_kind, batch, seq, world, rank, device, args, ids_host, aux_host, True)
    ms_step, e2e_ms, clocks = m["ms_per_step"], m["e2e_ms"], m["clocks"]
    tokens_step = batch * seq * world
    value = tokens_step / (ms_step * 1e-3)
    e2e_value = tokens_step / (e2e_ms * 1e-3)
    real_tokens = int(lens.sum())
    launches_per_step = run.launches_per_step
    run_collective = run.collective
    h2d, d2h = run.h2d_bytes(), run.out_host.numel() * 4
    attn_ms, attn_launches, attn_ms_max = attention_in_step_ms(model, run) if rank == 0 else (None, 0, None)
    ops.device_status()
    ref_rows = run.mine.detach().cpu().numpy().copy() if rank == 0 else None

    # ---- strong pass: ONE batch of `batch` ragged rows dealt over the ranks ----
    strong = None
    if world > 1 and batch % world == 0:
        g_ids, g_aux, g_lens = synthetic_batch(kind, batch, seq, vocab, 4321, ragged=True)   # same on every rank
        shards = E.shard_rows([int(x) for x in g_lens], world)
        my_rows = torch.tensor(shards[rank])
        per = batch // world
        del run
        torch.cuda.empty_cache()
        # rank 0 also embeds the whole batch by itself (eagerly, no collective): the rows the shards must reproduce
        full_rows = None
        if rank == 0:
            full_rows = model.forward(g_ids.to(device), g_aux.to(device)).clone()
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
        srun, sm = measure_stack(kind, model, aux_kind, per, seq, world, rank, device, args, g_ids[my_rows],
                                 g_aux[my_rows], False)
        s_ms = sm["ms_per_step"]
        strong = {"tokens_per_s": batch * seq / (s_ms * 1e-3), "ms_per_step": s_ms, "rows_per_gpu": per,
                  "global_batch": batch, "e2e_tokens_per_s": batch * seq / (sm["e2e_ms"] * 1e-3),
                  "n1_ms_per_step": ms_step, "speedup_vs_n1": ms_step / s_ms, "efficiency_vs_n1": ms_step / s_ms / world,
                  "note": ("one batch of ragged rows dealt longest-first round-robin (shard_rows); n1 = this run's "
                           "own full-batch step on one GPU (the weak pass: the same work, since a Qwen3 row's length "
                           "only moves its pooled position); all-gather inside the captured graph")}
        if rank == 0:
            undone = E.unshard_rows(srun.gathered, shards)   # back to the batch's own row order
            strong["matches_one_gpu_rows"] = bool(torch.equal(undone, full_rows))
            strong["max_abs_diff_vs_one_gpu_rows"] = float((undone - full_rows).abs().max())
        del srun
        torch.cuda.empty_cache()
    else:
        del run
        torch.cuda.empty_cache()

    # The same step through the library's native runner (C ABI, host buffers in,
    # host pooled rows out): no Python between the copies and the graph launch.
    native = None
    if kind == "qwen3" and rank == 0:
        from svod_b200.native import NativeQwen3
        runner = NativeQwen3(model, reference_ops=args.reference_ops)
        out_np = torch.empty(batch, D, dtype=torch.float32).pin_memory().numpy()
        ids_np, len_np = ids_host.pin_memory().numpy(), aux_host.pin_memory().numpy()
        for _ in range(2):
            runner.run(ids_np, len_np, out_np)
        nstream = runner.stream(batch, seq)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(nstream)
        for _ in range(args.steps):
            runner.run(ids_np, len_np, out_np)
        e1.record(nstream)
        nstream.synchronize()
        nms = e0.elapsed_time(e1) / args.steps
        native = {"value": batch * seq / (nms * 1e-3), "unit": UNIT, "ms_per_step": nms,
                  "api": "svodb_plan_run: host ids/lengths -> captured graph -> host pooled rows",
                  "matches_python_stack": bool((out_np == ref_rows).all())}
        runner.close()
        ops.device_status()

    line = None
    if rank == 0:
        gemm_fl, attn_fl = step_flops(kind, batch, seq)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": dtype_name, "data": "synthetic",
            "config": {"workload": args.workload, "batch_per_gpu": batch, "global_batch": batch * world,
                       "seq_len": seq, "parallelism": f"dp{world}",
                       "l2": "activations per step (GBs) exceed the 126 MB L2; no explicit flush",
                       "real_tokens_per_step": real_tokens * world,
                       "collective": ("all-gather of pooled rows by the library's own kernels: the pooling kernel stores "
                                      "its rows into the peers' staging buffers over NVLink, an unstage kernel "
                                      "follows; both inside the step's CUDA graph") if world > 1 and run_collective == "peer"
                       else "NCCL all-gather of pooled rows, captured inside the step's CUDA graph" if world > 1
                       else "none at one GPU"},
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches_per_step * args.steps,
            "gpu_launches_per_step": launches_per_step,
            "clocks": clocks,
            "step_tflops": (gemm_fl + attn_fl) / ms_step / 1e9,
            "output_finite": m["finite"],
        }
        if native is not None:
            line["e2e_native"] = native
        if strong is not None:
            line["strong"] = strong
    if world > 1:
        dist.barrier()
    if rank == 0:
        torch.cuda.empty_cache()
        ks = kernel_rooflines(kind, batch, seq, peaks)
        top = max(ks, key=lambda n: ks[n]["ms"] * ks[n]["launches_per_step"])
        line["roofline"] = {
            "kernel": top, "bound": "tensor", "achieved": ks[top]["tflops"], "peak": peaks["burst"],
            "unit": "TFLOP/s", "frac": ks[top]["tflops"] / peaks["burst"],
            "traffic": NCU_DRAM_BYTES_PER_ROW.get((kind, top), 0) * batch or None,
            "traffic_note": "dram read+write bytes of one ncu capture of the kernel at batch 16, scaled by rows (profiles/)",
            "peak_source": f"{peaks['source']} bf16 burst: the kernel is timed alone (20 launches in one graph)",
        }
        if attn_ms:
            fl = ks["flash_attention"]["flops_per_launch"]
            line["roofline"]["in_step"] = {
                "kernel": "flash_attention", "ms": attn_ms, "ms_max": attn_ms_max, "launches": attn_launches,
                "achieved": fl / attn_ms / 1e9, "peak": peaks["sustained"], "frac": fl / attn_ms / 1e9 / peaks["sustained"],
                "peak_source": f"{peaks['source']} bf16 sustained: event pairs around the attention launches of one "
                               "eager step under the step's clocks"}
            if top == "flash_attention":
                line["roofline"]["frac_in_step"] = line["roofline"]["in_step"]["frac"]
        line["kernels"] = ks
        line["attention_fwd_tflops"] = ks["flash_attention"]["tflops"]
        if world == 1 and not args.no_workloads and kind == "qwen3":
            del model
            torch.cuda.empty_cache()
            line["workloads"] = other_workloads(args, device, peaks)
        if world == 1 and not args.no_cpu:
            v, ms, sample = time_cpu(kind, 2, 1)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cpu_threads(), "kind": "port", "sample": sample}
            if kind == "qwen3":
                line["cpu_baseline"]["second_point"] = time_torch_cpu()
        print(json.dumps(line), flush=True)
    if world > 1:
        # The line is out. Leave without tearing the process group down: destroying a
        # communicator whose collectives live in captured graphs can wait forever, and
        # nothing after this point is worth a hang (a timer covers the barrier too).
        sys.stdout.flush()
        threading.Timer(30.0, lambda: os._exit(0)).start()
        torch.cuda.synchronize()
        dist.barrier()
        os._exit(0)


def other_workloads(args, device, peaks):
    """The two other encoder configurations on one GPU, a few steps each: padded
    and real tokens/s (real = the tokens under the padding mask), step TFLOP/s and
    the per-launch timing of their attention and largest GEMM."""
    import torch
    from svod_b200 import ops
    out = {}
    for name in ("xlm-roberta-large", "modernbert-base"):
        kind, batch, seq = WORKLOADS[name]
        model, aux_kind = build_model(kind, device)
        ids_host, aux_host, lens = synthetic_batch(kind, batch, seq, model.cfg.vocab_size, 1234, ragged=False)
        run, m = measure_stack(kind, model, aux_kind, batch, seq, 1, 0, device, args, ids_host, aux_host, True)
        ms = m["ms_per_step"]
        gemm_fl, attn_fl = step_flops(kind, batch, seq)
        rec = {"batch": batch, "seq_len": seq, "dtype": "f16" if kind == "xlmr" else "bf16", "ms_per_step": ms,
               "tokens_per_s": batch * seq / (ms * 1e-3), "real_tokens_per_s": int(lens.sum()) / (ms * 1e-3),
               "real_tokens_per_step": int(lens.sum()),
               "e2e_tokens_per_s": batch * seq / (m["e2e_ms"] * 1e-3), "step_tflops_padded": (gemm_fl + attn_fl) / ms / 1e9,
               "gpu_launches_per_step": run.launches_per_step, "clocks": m["clocks"], "output_finite": m["finite"]}
        del run, model
        torch.cuda.empty_cache()
        rec["kernels"] = kernel_rooflines(kind, batch, seq, peaks)
        ops.device_status()
        out[name] = rec
        torch.cuda.empty_cache()
    return out


def kernel_case(args):
    """A small single-kernel case for profiler captures: a few launches of one
    kernel at the workload's per-launch shape with a reduced batch (inputs above
    the 126 MB L2, a few hundred MB on the device)."""
    import torch
    from svod_b200 import ops
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(1)
    B, T = args.case_batch, 4096
    if args.kernel_case == "flash_attention":
        q = torch.randn(B, T, 16, 128, generator=g, device="cuda").to(torch.bfloat16)
        k = torch.randn(B, T, 8, 128, generator=g, device="cuda").to(torch.bfloat16)
        v = torch.randn(B, T, 8, 128, generator=g, device="cuda").to(torch.bfloat16)
        a = ops.Attn(causal=True)
        fn = lambda: ops.attention(q, k, v, a)
        flops = 4 * B * 16 * T * T * 128 / 2
    elif args.kernel_case == "gemm":
        M, N, K = B * T, 3072, 1024
        x = (torch.randn(M, K, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
        w = (torch.randn(2 * N, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        o = ops.Linear(act=ops.Act.SILU, gated=True)
        fn = lambda: ops.linear(x, w, o)
        flops = 2 * M * 2 * N * K
    elif args.kernel_case == "gemm_gelu":
        # XLM-R's FFN-in shape at a reduced row count: bias + erf-GELU, K = 1024
        M, N, K = B * T, 4096, 1024
        x = (torch.randn(M, K, generator=g, device="cuda") * 0.5).to(torch.float16)
        w = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(torch.float16)
        bias = (torch.randn(N, generator=g, device="cuda") * 0.02).to(torch.float16)
        o = ops.Linear(bias=bias, act=ops.Act.GELU)
        fn = lambda: ops.linear(x, w, o)
        flops = 2 * M * N * K
    elif args.kernel_case == "rms_norm":
        x = torch.randn(B * T * 4, 1024, generator=g, device="cuda").to(torch.bfloat16)
        w = torch.ones(1024, device="cuda", dtype=torch.bfloat16)
        fn = lambda: ops.rms_norm(x, w)
        flops = 0
    else:
        qkv = torch.randn(B, T, 4096, generator=g, device="cuda").to(torch.bfloat16)
        w = torch.ones(128, device="cuda", dtype=torch.bfloat16)
        cos, sin = ops.rope_table(1e6, T, 128, torch.bfloat16)
        o = ops.Qkv(16, 8, 128, w, w, 1e-6, (cos.view(1, T, 1, 64), sin.view(1, T, 1, 64)))
        fn = lambda: ops.heads(qkv, o)
        flops = 0
    ms = time_kernel(fn, torch.cuda.current_stream(), 3)
    ops.device_status()
    print(json.dumps({"kernel_case": args.kernel_case, "batch": B, "ms": ms,
                      "tflops": flops / ms / 1e9 if flops else None, "chosen": ops.chosen()}), flush=True)


def time_graphed(fn, reps: int = 20):
    """ms per call of `fn` with the host call path taken out: `reps` calls are
    captured into one CUDA graph (after an eager warm-up) and the replay is timed."""
    import torch
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        for _ in range(3):
            fn()
    st.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=st):
        for _ in range(reps):
            fn()
    with torch.cuda.stream(st):
        g.replay()
        st.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        g.replay()
        e1.record(st)
    st.synchronize()
    return e0.elapsed_time(e1) / reps


def sweep(args):
    """The two kernel-level configurations of the baseline that are not model
    steps: the f32 attention case (the exact CUDA-core path, with log-sum-exp)
    and the GEMM sweep M in {512, 4096, 32768} x N=K in {768, 1024, 4096} with the
    bias+GELU, bias+tanh-GELU and bias+SwiGLU epilogues. One JSON line per case."""
    import torch
    from svod_b200 import ops
    torch.cuda.set_device(0)
    peaks = measured_peaks()
    g = torch.Generator(device="cuda").manual_seed(2)
    stream = torch.cuda.current_stream()
    if args.sweep == "decode":
        # decode-shaped attention: few queries per lane against a long cache, key splits on the
        # tensor-core kernel against the exact kernel (config key `attention|exact`)
        from svod_b200 import _lib as L
        lib = L.load()
        for (B, T, Tk, H, Hk, D) in [(8, 1, 32768, 16, 8, 128), (8, 16, 32768, 16, 8, 128), (64, 1, 4096, 16, 8, 128)]:
            q = torch.randn(B, T, H, D, generator=g, device="cuda").to(torch.bfloat16)
            k = torch.randn(B, Tk, Hk, D, generator=g, device="cuda").to(torch.bfloat16)
            v = torch.randn(B, Tk, Hk, D, generator=g, device="cuda").to(torch.bfloat16)
            lens = torch.full((B,), Tk, dtype=torch.int32, device="cuda")
            kv_bytes = 2 * B * Tk * Hk * D * 2
            ref = None
            for splits in (1, 4, 8, 16, 32):
                row = {}
                for mode in ("tensor", "exact"):
                    lib.svodb_config_set(b"attention|exact", 1 if mode == "exact" else 0)
                    a = ops.Attn(keys=ops.KeyMask.Lens(lens), splits=splits if splits > 1 else None)
                    out = ops.attention(q, k, v, a)
                    ch = ops.chosen()
                    ms = time_graphed(lambda: ops.attention(q, k, v, a), 10)
                    ref = out.float() if ref is None else ref
                    row[mode] = {"ms": round(ms, 4), "kv_gbs": round(kv_bytes / ms / 1e6, 1),
                                 "max_abs_vs_first": float((out.float() - ref).abs().max()),
                                 "kernel": "flash_attention" if "kernel" in ch else "exact"}
                lib.svodb_config_set(b"attention|exact", 0)
                print(json.dumps({"case": f"decode B{B} T{T} Tk{Tk} H{H}/{Hk} D{D}", "splits": splits, **row}), flush=True)
        ops.device_status()
        return
    if args.sweep == "split-k":
        # the one-wave shapes with a long k loop: the k loop in one piece (the default) against 2 / 4 / 8 pieces
        for (m, n, k) in [(512, 4096, 4096), (512, 1024, 4096), (1024, 4096, 4096), (2048, 1024, 3072)]:
            x = (torch.randn(m, k, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
            w = (torch.randn(n, k, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
            b = (torch.randn(n, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
            ref = None
            for pieces in (1, 2, 4, 8):
                o = ops.Linear(bias=b, act=ops.Act.GELU, k_splits=pieces)
                out = ops.linear(x, w, o)
                ch = ops.chosen()
                ref = out.float() if ref is None else ref
                ms = time_graphed(lambda: ops.linear(x, w, o), 10)
                print(json.dumps({"case": f"gemm bias+gelu M{m} N{n} K{k}", "k_splits": pieces, "us": round(ms * 1e3, 1),
                                  "tflops": round(2 * m * n * k / ms / 1e9, 1),
                                  "max_abs_vs_unsplit": float((out.float() - ref).abs().max()),
                                  "chosen": ch.split("kernel gemm ")[-1]}), flush=True)
        ops.device_status()
        return
    if args.sweep == "attention-f32":
        B, H, T, D = 2, 8, 512, 64
        q, k, v = (torch.randn(B, T, H, D, generator=g, device="cuda") for _ in range(3))
        lens = torch.randint(256, 513, (B,), generator=g, device="cuda", dtype=torch.int32)
        a = ops.Attn(keys=ops.KeyMask.Lens(lens), scale=0.125, want_lse=True)
        ms = time_graphed(lambda: ops.attention(q, k, v, a))
        flops = 4 * H * D * T * int(lens.sum().item())
        print(json.dumps({"case": "attention f32 B2 H8 T512 D64 key_lens + lse", "ms": ms,
                          "gflops": flops / ms / 1e6, "chosen": ops.chosen()}), flush=True)
        return
    for m in (512, 4096, 32768):
        for nk in (768, 1024, 4096):
            x = (torch.randn(m, nk, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
            for name, act, gated in (("bias+gelu", ops.Act.GELU, False), ("bias+gelu_tanh", ops.Act.GELU_TANH, False),
                                     ("bias+swiglu", ops.Act.SILU, True)):
                rows = 2 * nk if gated else nk
                w = (torch.randn(rows, nk, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
                b = (torch.randn(rows, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
                o = ops.Linear(bias=b, act=act, gated=gated)
                ms = time_graphed(lambda: ops.linear(x, w, o))
                flops = 2 * m * rows * nk
                nbytes = 2 * (m * nk + rows * nk + m * nk) + 2 * rows
                tf = flops / ms / 1e9
                print(json.dumps({"case": f"gemm {name} M{m} N{nk} K{nk}", "ms": round(ms, 4), "tflops": round(tf, 1),
                                  "min_gbs": round(nbytes / ms / 1e6, 1),
                                  "frac_of_burst": round(tf / peaks["burst"], 3),
                                  "frac_of_nominal_2250": round(tf / 2250.0, 3),
                                  "chosen": ops.chosen().split("kernel gemm ")[-1]}), flush=True)
    ops.device_status()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="qwen3-0.6b-embed", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--gather", default="peer", choices=["nccl", "peer"],
                    help="the all-gather of pooled rows at N > 1: the library's own peer-memory kernels (NCCL if the "
                         "peers' memory cannot be mapped), or NCCL")
    ap.add_argument("--no-workloads", action="store_true",
                    help="skip the short XLM-RoBERTa-large and ModernBERT-base runs of the default one-GPU line")
    ap.add_argument("--reference-ops", action="store_true",
                    help="Qwen3: the reference's op sequence (linear, heads, attention) instead of the "
                         "q/k prologue fused into the projection's store")
    ap.add_argument("--kernel-case", default=None, choices=["flash_attention", "gemm", "gemm_gelu", "rms_norm", "heads"],
                    help="run a few launches of one kernel on a small case (for profiler captures) and exit")
    ap.add_argument("--case-batch", type=int, default=4)
    ap.add_argument("--sweep", default=None, choices=["gemm", "attention-f32", "decode", "split-k"],
                    help="time the kernel-level baseline configurations (one JSON line per case) and exit")
    args = ap.parse_args()
    if args.kernel_case:
        return kernel_case(args)
    if args.sweep:
        return sweep(args)
    if args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
