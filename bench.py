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
HBM (CUDA-graph replay + all-gather, CUDA events on the launching stream, max
over ranks); `e2e` adds the pinned-host -> device copy of every step's inputs
and the device -> host read of the pooled result inside the timed region.
`roofline` is measured live for the dominant kernel; `cpu_baseline` times the
compiled C + OpenMP restatement on a bounded sample of the same workload on this
box's host cores.
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
    ("qwen3", "flash_attention"): 173.6e6 / 4,   # algorithmic 100.7 MB at batch 4
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
def oracle_sample(kind: str, seq: int, layers: int, seed: int = 7):
    """A bounded sample of the workload for the compiled CPU restatement
    (`oracle/svod_oracle.c`: f32, OpenMP over all host threads): one sequence of
    `seq` tokens through `layers` decoder layers of the same architecture.
    Returns a closure that runs it and the number of tokens it processes."""
    import numpy as np
    from oracle import c_oracle as C
    from oracle import svod_oracle as O
    try:
        C.build()
    except Exception:
        pass  # a library built earlier still loads; `load()` reports a missing one
    rng = np.random.default_rng(seed)
    dt = O.BF16
    w = lambda *s: O.round_to(dt, rng.standard_normal(s) * 0.02).astype(np.float32)
    if kind != "qwen3":
        raise SystemExit("the CPU leg samples the default (qwen3) workload")
    D, H, Hkv, hd, F = 1024, 16, 8, 128, 3072
    ones = lambda n: np.ones(n, dtype=np.float32)
    lp = dict(in_w=ones(D), qkv_w=w((H + 2 * Hkv) * hd, D), qn_w=ones(hd), kn_w=ones(hd), o_w=w(D, H * hd),
              post_w=ones(D), gu_w=w(2 * F, D), down_w=w(D, F))
    hidden = w(1, seq, D)
    C.load()

    def run():
        return C.qwen3_layers(hidden, [lp] * layers, heads_n=H, kv_heads=Hkv, head_dim=hd, dtype=C.BF16)

    return run, seq


def cpu_threads() -> int:
    from oracle import c_oracle as C
    return C.threads()


def time_cpu(kind: str, steps: int, warmup: int, seq: int = 4096, layers: int = 4, full_layers: int = 28):
    """Times the compiled CPU restatement on `layers` of the `full_layers` layers
    of one full-length sequence and scales to the full depth (every layer does
    identical work; the embedding lookup and the pooling are negligible)."""
    run, tokens = oracle_sample(kind, seq, layers)
    for _ in range(warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = (time.perf_counter() - t0) / steps
    full = dt * full_layers / layers
    sample = (f"C + OpenMP f32 restatement, 1 sequence x {seq} tokens, {layers} of {full_layers} layers timed "
              f"and scaled to {full_layers}, {steps} step(s)")
    return tokens / full, full * 1e3, sample


def time_torch_cpu(seq: int = 4096, layers: int = 4, full_layers: int = 28, steps: int = 1):
    """A second, separately labelled CPU reference point (not svod, not the
    oracle): the Qwen3-shaped layer in plain PyTorch f32 CPU ops
    (`F.linear`, `F.scaled_dot_product_attention`) on the same bounded sample,
    with all the threads torch will use."""
    import torch
    import torch.nn.functional as F
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
        "dtype": "bf16", "data": "synthetic",
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
    q = torch.randn(batch, seq, H, D, generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn(batch, seq, Hkv, D, generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn(batch, seq, Hkv, D, generator=g, device="cuda").to(torch.bfloat16)
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
    x = (torch.randn(M, K, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn((2 if gated else 1) * N, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    ms = time_graphed(lambda: ops.linear(x, w, opts), 20)
    fl = 2 * M * N * K * (2 if gated else 1)
    out["gemm"] = {"ms": ms, "tflops": fl / ms / 1e9, "flops_per_launch": fl,
                   "launches_per_step": {"qwen3": 28, "xlmr": 24, "modernbert": 22}[kind]}
    for v_ in out.values():
        v_["frac_of_sustained"] = v_["tflops"] / peaks["sustained"]
        v_["frac_of_burst"] = v_["tflops"] / peaks["burst"]
        v_["frac_of_nominal_2250"] = v_["tflops"] / 2250.0
    return out


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

    model, aux_kind = build_model(kind, device, args.reference_ops)
    D = model.cfg.hidden_size
    gathered = torch.zeros(world * batch, D, dtype=torch.float32, device=device)
    mine = gathered[rank * batch:(rank + 1) * batch]
    before = ops.launches
    plan = E.Plan(model, batch, seq, aux_kind, out=mine, device=device)
    # synthetic inputs: uniform ids (pad id avoided), full-length rows
    gen = torch.Generator().manual_seed(1234 + rank)
    vocab = model.cfg.vocab_size
    ids_host = torch.randint(2, vocab, (batch, seq), generator=gen, dtype=torch.int32).pin_memory()
    if aux_kind == "mask":
        lens = torch.randint(seq // 8 if kind == "xlmr" else seq // 4, seq + 1, (batch,), generator=gen)
        aux_host = (torch.arange(seq)[None, :] < lens[:, None]).pin_memory()
        real_tokens = int(lens.sum())
    else:
        aux_host = torch.full((batch,), seq, dtype=torch.int32).pin_memory()
        real_tokens = batch * seq
    out_host = torch.empty(batch, D, dtype=torch.float32).pin_memory()
    plan.ids.copy_(ids_host)
    plan.aux.copy_(aux_host)
    torch.cuda.synchronize()
    plan.capture()
    launches_per_step = (ops.launches - before) // 2   # capture() runs the stack twice (eager + capture)
    stream = plan.stream

    def step_resident():
        plan.replay()
        if world > 1:
            with torch.cuda.stream(stream):
                E.gather_pooled(mine, gathered)

    def step_e2e():
        plan.run(ids_host, aux_host, None)
        with torch.cuda.stream(stream):
            if world > 1:
                E.gather_pooled(mine, gathered)
            out_host.copy_(mine, non_blocking=True)

    def timed(fn, steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(3, args.warmup)):
        step_resident()
    stream.synchronize()
    ops.device_status()
    sampler = ClockSampler(visible_index(local))
    sampler.start()
    total_ms = timed(step_resident, args.steps)
    clocks = sampler.stop()
    ms_step = total_ms / args.steps
    tokens_step = batch * seq * world
    value = tokens_step / (ms_step * 1e-3)

    for _ in range(2):
        step_e2e()
    stream.synchronize()
    e2e_ms = timed(step_e2e, args.steps) / args.steps
    e2e_value = tokens_step / (e2e_ms * 1e-3)
    ops.device_status()
    finite = bool(torch.isfinite(mine).all())

    # The same step through the library's native runner (C ABI, host buffers in,
    # host pooled rows out): no Python between the copies and the graph launch.
    native = None
    if kind == "qwen3" and rank == 0:
        from svod_b200.native import NativeQwen3
        ref_rows = mine.detach().cpu().numpy().copy()
        del plan
        plan = None
        torch.cuda.empty_cache()
        runner = NativeQwen3(model, reference_ops=args.reference_ops)
        ids_np, len_np, out_np = ids_host.numpy(), aux_host.numpy(), out_host.numpy()
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
            "vs_baseline": None, "dtype": "bf16" if kind != "xlmr" else "f16", "data": "synthetic",
            "config": {"workload": args.workload, "batch_per_gpu": batch, "global_batch": batch * world,
                       "seq_len": seq, "parallelism": f"dp{world}",
                       "l2": "activations per step (GBs) exceed the 126 MB L2; no explicit flush",
                       "real_tokens_per_step": real_tokens * world},
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": ids_host.numel() * ids_host.element_size() + aux_host.numel() * aux_host.element_size(),
                    "d2h_bytes_per_step": out_host.numel() * 4},
            "gpu_launches": launches_per_step * args.steps,
            "gpu_launches_per_step": launches_per_step,
            "clocks": clocks,
            "step_tflops": (gemm_fl + attn_fl) / ms_step / 1e9,
            "output_finite": finite,
        }
        if native is not None:
            line["e2e_native"] = native
    del plan
    if world > 1:
        dist.barrier()
    if rank == 0:
        torch.cuda.empty_cache()
        ks = kernel_rooflines(kind, batch, seq, peaks)
        top = max(ks, key=lambda n: ks[n]["ms"] * ks[n]["launches_per_step"])
        line["roofline"] = {
            "kernel": top, "bound": "tensor", "achieved": ks[top]["tflops"], "peak": peaks["sustained"],
            "unit": "TFLOP/s", "frac": ks[top]["tflops"] / peaks["sustained"],
            "traffic": NCU_DRAM_BYTES_PER_ROW.get((kind, top), 0) * batch or None,
            "traffic_note": "dram read+write bytes of one ncu capture at batch 4, scaled by rows (profiles/)",
            "peak_source": f"{peaks['source']} bf16 sustained (kernel timed back to back)",
        }
        line["kernels"] = ks
        line["attention_fwd_tflops"] = ks["flash_attention"]["tflops"]
        if world == 1 and not args.no_cpu:
            v, ms, sample = time_cpu("qwen3", 2, 1) if kind == "qwen3" else (None, None, None)
            if v is not None:
                line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cpu_threads(), "kind": "port",
                                        "sample": sample, "second_point": time_torch_cpu()}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


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
    ap.add_argument("--reference-ops", action="store_true",
                    help="Qwen3: the reference's op sequence (linear, heads, attention) instead of the "
                         "q/k prologue fused into the projection's store")
    ap.add_argument("--kernel-case", default=None, choices=["flash_attention", "gemm", "rms_norm", "heads"],
                    help="run a few launches of one kernel on a small case (for profiler captures) and exit")
    ap.add_argument("--case-batch", type=int, default=4)
    ap.add_argument("--sweep", default=None, choices=["gemm", "attention-f32"],
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
