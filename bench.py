#!/usr/bin/env python3
"""Benchmark of the decode linear stack (the hot path) on B200.

A "step" is one decode step of the Qwen3-0.6B-shaped linear stack: the four
projections (fused QKV, O, fused gate/up, down) of all 28 layers, block-quantised
weights, each projection with its own seeded activation matrix, executed by the
grouped persistent launch of libizwi_b200.so.  All inputs are synthetic and
seeded.  One JSON line is printed by rank 0.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
  python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

`value` is tokens/s with everything resident in HBM; `e2e` is the same metric
through the C ABI with host activations copied in and host results copied out
every step; `roofline` is algorithmic bytes per launch over the measured launch
time against the measured HBM copy bandwidth; `cpu_baseline` / `--impl
reference` time the CPU restatement of the same stack on the host cores.
At N > 1 the stack does not shard (0.6B decode): each rank runs a replica.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "decode_linear_stack_tokens_per_s"
WORKLOADS = {
    # name: (format, tokens per step)
    "qwen3-0.6b-q8_0-m1": ("q8_0", 1),
    "qwen3-0.6b-q8_0-m4": ("q8_0", 4),
    "qwen3-0.6b-q8_0-m16": ("q8_0", 16),
    "qwen3-0.6b-q8_0-m32": ("q8_0", 32),
    "qwen3-0.6b-q8_0-m64": ("q8_0", 64),
    "qwen3-0.6b-q4_k-m1": ("q4_k", 1),
    "qwen3-0.6b-q4_k-m4": ("q4_k", 4),
    "qwen3-0.6b-q4_k-m16": ("q4_k", 16),
    "qwen3-0.6b-q4_k-m32": ("q4_k", 32),
    "qwen3-0.6b-q4_k-m64": ("q4_k", 64),
    "qwen3-0.6b-bf16-m1": ("bf16", 1),
}
DEFAULT_WORKLOAD = "qwen3-0.6b-q8_0-m1"
WEIGHT_SEED, ACT_SEED = 0, 2

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the grouped kernel, from the ncu
# capture summarised under profiles/ (None until a capture exists for that workload).
NCU_DRAM_BYTES_PER_LAUNCH = {
    # (134.27 MB read + 3.9 MB written) on an 8-layer stack, scaled to 28 layers: profiles/skinny_gemv_q8_0_m1_qwen3-0.6b-stack.md
    "qwen3-0.6b-q8_0-m1": 483_600_000,
    # (70.93 + 1.1) MB x 28/8: profiles/skinny_gemv_q4_k_m1_qwen3-0.6b-stack.md
    "qwen3-0.6b-q4_k-m1": 252_100_000,
    # (141.1 + 8.7) MB x 28/8 and (78.2 + 4.4) MB x 28/8: profiles/skinny_tc_m64_qwen3-0.6b-stack.md
    "qwen3-0.6b-q8_0-m64": 524_300_000,
    "qwen3-0.6b-q4_k-m64": 289_100_000,
}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock, power and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples = []  # (time, sm_mhz, power_w, reasons bitmask)
        self.stop_flag = threading.Event()
        self.max_mhz = None
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.nv = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self.stop_flag.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                power = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                self.samples.append((time.perf_counter(), mhz, power, reasons))
            except Exception:
                pass
            time.sleep(self.period)

    def summary(self, t0: float, t1: float):
        if not self.ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml_unavailable"]}
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        where = "timed_region"
        if len(inside) < 3:  # a very short timed region: fall back to every sample taken under load
            inside, where = self.samples, "warmup_and_timed_region"
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
                 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting"}
        mask = 0
        for s in inside:
            mask |= s[3]
        return {"sm_mhz": statistics.median(s[1] for s in inside) if inside else None,
                "sm_max_mhz": self.max_mhz,
                "power_w_max": max((s[2] for s in inside), default=None),
                "reasons": [n for b, n in names.items() if mask & b],
                "samples": len(inside), "sampled_during": where}


def dist_setup(n_gpus: int):
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    return world, rank, local


def barrier(world):
    import torch
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(ms: float, world: int) -> float:
    if world == 1:
        return ms
    import torch
    import torch.distributed as dist
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_steps(fn, steps: int, world: int):
    """Exactly `steps` calls of fn between CUDA events on the launching stream, barrier + sync on both sides."""
    import torch
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    barrier(world)
    return max_over_ranks(e0.elapsed_time(e1), world), t0, t1


def oracle_lib():
    import subprocess
    so = ROOT / "oracle" / "liboracle_c.so"
    if not so.exists():
        subprocess.run(["make", "-C", str(ROOT / "oracle")], check=True, capture_output=True)
    lib = ctypes.CDLL(str(so))
    lib.orc_num_threads.restype = ctypes.c_int
    return lib


class CpuStack:
    """The same stack on the host: raw weight bytes (or fp32 for bf16) + fp32 activations, run by the C port."""

    def __init__(self, stack):
        import numpy as np
        import torch
        self.lib = oracle_lib()
        self.fmt, self.m = stack.fmt, stack.m
        self.items = []
        for wl, al in zip(stack.weights, stack.acts):
            for (_, n, k), w, x in zip(stack.shape.projections, wl, al):
                wh = (w.float() if self.fmt == "bf16" else w).cpu().numpy()
                xh = x.float().cpu().numpy()
                self.items.append((np.ascontiguousarray(wh), np.ascontiguousarray(xh), np.empty((self.m, n), np.float32), n, k))
        self.cores = self.lib.orc_num_threads()

    def step(self):
        vp = ctypes.c_void_p
        for wh, xh, yh, n, k in self.items:
            if self.fmt == "bf16":
                self.lib.orc_linear_f32(xh.ctypes.data_as(vp), wh.ctypes.data_as(vp), None, yh.ctypes.data_as(vp),
                                        ctypes.c_int64(self.m), ctypes.c_int64(n), ctypes.c_int64(k))
            else:
                self.lib.orc_qlinear_f32(0 if self.fmt == "q8_0" else 1, xh.ctypes.data_as(vp), wh.ctypes.data_as(vp),
                                         yh.ctypes.data_as(vp), ctypes.c_int64(self.m), ctypes.c_int64(n),
                                         ctypes.c_int64(k))

    def timed(self, budget_s: float, max_steps: int = 400):
        self.step()  # warm-up (page in, thread pool)
        t0 = time.perf_counter()
        self.step()
        one = time.perf_counter() - t0
        n = int(max(1, min(max_steps, budget_s / max(one, 1e-6))))
        t0 = time.perf_counter()
        for _ in range(n):
            self.step()
        dt = time.perf_counter() - t0
        return n, dt


LAYERS_OVERRIDE = None  # --layers: a shorter stack, for profiler captures only


def make_stack(workload: str, device):
    from izwi_b200 import workloads as wl
    fmt, m = WORKLOADS[workload]
    return wl.make_linear_stack(wl.QWEN3_0_6B, fmt, m, device, WEIGHT_SEED, ACT_SEED, layers=LAYERS_OVERRIDE)


def measure_case(workload: str, device, steps: int, warmup: int, peak: float):
    """Short device-resident measurement of one more configuration (not the headline line)."""
    import torch
    from izwi_b200 import workloads as wl
    stack = make_stack(workload, device)
    group = wl.stack_group(stack)
    for _ in range(warmup):
        group.launch()
    ms, _, _ = time_steps(group.launch, steps, 1)
    group.ctx.check()
    per = ms / steps
    gbs = stack.algorithmic_bytes / (per * 1e-3) / 1e9
    out = {"workload": workload, "ms_per_step": round(per, 5), "tokens_per_s": round(stack.m / (per * 1e-3), 1),
           "hbm_gbs": round(gbs, 1), "hbm_frac_of_measured": round(gbs / peak, 4),
           "tflops": round(stack.flops / (per * 1e-3) / 1e12, 2)}
    del group, stack
    torch.cuda.empty_cache()
    return out


def load_tensor_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), "measured burst"
    return 1590.0, "fallback"


def _time_call(fn, iters: int, warmup: int = 3):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def measure_gemm_cases(device, only=None, iters=20):
    """Prefill (Qwen3-8B shape, M = 2048) and ASR-encoder GEMMs through izb_linear: TFLOP/s against the
    measured bf16 tensor peak.  Operands are a few hundred MB, so successive calls do not reuse L2 for
    the large ones; the small ones are reported as measured (L2-resident, as they would be in a layer loop)."""
    import torch
    from izwi_b200 import ops
    peak, kind = load_tensor_peak()
    gen = torch.Generator(device=device).manual_seed(3)
    shapes = [
        ("qwen3-8b-prefill-qkv", 2048, 6144, 4096, None, False),
        ("qwen3-8b-prefill-o", 2048, 4096, 4096, None, False),
        ("qwen3-8b-prefill-gate_up+swiglu", 2048, 24576, 4096, "swiglu", False),
        ("qwen3-8b-prefill-down", 2048, 4096, 12288, None, False),
        ("fastconformer-b32-ffn1+silu", 12000, 4096, 1024, "silu", False),
        ("fastconformer-b32-ffn2", 12000, 1024, 4096, None, False),
        ("fastconformer-b32-attn", 12000, 1024, 1024, None, False),
        ("whisper-b32-qkv+bias", 48000, 3840, 1280, None, True),
        ("whisper-b32-fc1+bias+gelu", 48000, 5120, 1280, "gelu", True),
        ("whisper-b32-fc2+bias", 48000, 1280, 5120, None, True),
        ("whisper-b1-fc1+bias+gelu", 1500, 5120, 1280, "gelu", True),
        ("fastconformer-b1-ffn1+silu", 375, 4096, 1024, "silu", False),
    ]
    out = []
    for name, m, n, k, epi, has_bias in shapes:
        if only is not None and name != only:
            continue
        x = torch.randn(m, k, device=device, generator=gen).to(torch.bfloat16)
        w = (torch.randn(n, k, device=device, generator=gen) * 0.02).to(torch.bfloat16)
        b = (torch.randn(n, device=device, generator=gen) * 0.1).to(torch.bfloat16) if has_bias else None
        y = torch.empty(m, n // 2 if epi == "swiglu" else n, device=device, dtype=torch.bfloat16)
        ms = _time_call(lambda: ops.linear(x, w, bias=b, out=y, epilogue=epi), iters)
        tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        out.append({"workload": name, "M": m, "N": n, "K": k, "ms": round(ms, 4), "tflops": round(tf, 1),
                    "tensor_frac": round(tf / peak, 4), "peak_kind": f"of {kind} {peak}"})
        del x, w, y
    ops.Context.get(device.index).check()
    torch.cuda.empty_cache()
    return out


def measure_attention_cases(device):
    """Single-query GQA attention over a head-major KV cache (Qwen3-8B heads: 32 query, 8 KV, d 128)
    through izb_decode_gqa_attention: K + V bytes per second against the measured HBM rate.  Caches of
    36 layers are rotated so that successive calls do not find theirs in L2."""
    import torch
    from izwi_b200 import ops
    peak_bw, _ = load_peaks()
    gen = torch.Generator(device=device).manual_seed(5)
    h, kvh, d = 32, 8, 128
    out = []
    for batch, kv_len in ((1, 4096), (1, 32768), (16, 4096)):
        n_layers = max(2, min(36, int(4e9 // (2 * batch * kvh * kv_len * d * 2))))
        caches = [(torch.randn(batch, kvh, kv_len, d, device=device, generator=gen).to(torch.bfloat16),
                   torch.randn(batch, kvh, kv_len, d, device=device, generator=gen).to(torch.bfloat16))
                  for _ in range(n_layers)]
        q = torch.randn(batch, h, d, device=device, generator=gen).to(torch.bfloat16)
        y = torch.empty(batch, h, d, device=device, dtype=torch.bfloat16)
        ws = torch.empty(64 << 20, device=device, dtype=torch.uint8)
        state = {"i": 0}

        def step():
            k, v = caches[state["i"] % n_layers]
            ops.decode_gqa_attention(q, k, v, kv_len, out=y, workspace=ws)
            state["i"] += 1
        ms = _time_call(step, 50)
        kv_bytes = 2 * batch * kvh * kv_len * d * 2
        gbs = kv_bytes / (ms * 1e-3) / 1e9
        out.append({"workload": f"qwen3-8b-decode-attention-b{batch}-kv{kv_len}", "ms": round(ms, 4),
                    "kv_gbs": round(gbs, 1), "hbm_frac_of_measured": round(gbs / peak_bw, 4),
                    "layers_rotated": n_layers, "kv_bytes_per_call": kv_bytes})
        del caches
        torch.cuda.empty_cache()
    ops.Context.get(device.index).check()
    return out


def measure_decode_token_cases(device):
    """A whole greedy decode token of a Qwen3-0.6B-shaped model with Q8_0 projections (embedding, 28
    layers of norm / fused QKV / q,k norm / RoPE / KV append / GQA attention / O / norm / gate-up /
    SiLU-multiply / down, final norm, lm_head over 151,936 tokens, arg-max), captured once in a CUDA
    graph at a fixed context length and replayed: what the linear stack of the headline sits in."""
    import torch
    from izwi_b200 import decoder, ops
    from izwi_b200 import workloads as wl
    peak_bw, _ = load_peaks()
    shape = wl.QWEN3_0_6B
    gen = torch.Generator(device=device).manual_seed(6)
    vocab, hid, qd, kd = 151936, shape.hidden, shape.q_heads * shape.head_dim, shape.kv_heads * shape.head_dim
    ones = lambda n: (1.0 + 0.1 * torch.randn(n, device=device, generator=gen)).to(torch.bfloat16)  # noqa: E731
    layers = []
    for _ in range(shape.layers):
        layers.append(decoder.Qwen3DecoderLayer(decoder.Qwen3LayerWeights(
            "q8_0", hid, shape.q_heads, shape.kv_heads, shape.head_dim, shape.intermediate, ones(hid), ones(hid),
            ones(shape.head_dim), ones(shape.head_dim), wl.make_q8_0_weight(qd + 2 * kd, hid, gen),
            wl.make_q8_0_weight(hid, qd, gen), wl.make_q8_0_weight(2 * shape.intermediate, hid, gen),
            wl.make_q8_0_weight(hid, shape.intermediate, gen))))
    embed = (torch.randn(vocab, hid, device=device, generator=gen) * 0.5).to(torch.bfloat16)
    model = decoder.Qwen3Decoder(embed, layers, ones(hid), wl.make_q8_0_weight(vocab, hid, gen), "q8_0")
    weight_bytes = sum(w.numel() for l in layers for w in (l.w.qkv, l.w.o, l.w.gate_up, l.w.down)) + model.lm_head.numel()
    out = []
    for ctx_len, fused in ((512, True), (4096, True), (512, False)):
        # fused: norms, SiLU-multiply and residual adds ride inside the one-token projections
        for l in layers:
            l.fused_linear = fused
            l.fusion_max_tokens = ops.linear_fusion_max_tokens("q8_0") if fused else 0
        caches = [decoder.KvCache(1, shape.kv_heads, ctx_len + 8, shape.head_dim, device) for _ in layers]
        for c in caches:
            c.k.normal_(generator=gen)
            c.v.normal_(generator=gen)
        tok = torch.tensor([17], device=device)
        cos, sin = model.rope_tables(ctx_len, 1)
        launches0 = ops.Context.get(device.index).launch_count
        for _ in range(2):
            nxt = model.step(tok, caches, ctx_len, cos, sin)
        torch.cuda.synchronize()
        launches = (ops.Context.get(device.index).launch_count - launches0) // 2
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            nxt = model.step(tok, caches, ctx_len, cos, sin)
        ms = _time_call(graph.replay, 30)
        ops.Context.get(device.index).check()
        kv_bytes = shape.layers * 2 * shape.kv_heads * (ctx_len + 1) * shape.head_dim * 2
        gbs = (weight_bytes + kv_bytes) / (ms * 1e-3) / 1e9
        out.append({"workload": f"qwen3-0.6b-q8_0-greedy-token-ctx{ctx_len}", "ms_per_token": round(ms, 4),
                    "tokens_per_s": round(1e3 / ms, 1), "kernels_per_token": int(launches), "fused_projections": fused,
                    "weight_and_kv_gbs": round(gbs, 1), "hbm_frac_of_measured": round(gbs / peak_bw, 4),
                    "next_token": int(nxt[0])})
        del caches, graph
        torch.cuda.empty_cache()
    del model, layers, embed
    torch.cuda.empty_cache()
    return out


def measure_moe_cases(device):
    """One Qwen3-30B-A3B-shaped MoE layer (H 2048, I 768, 128 experts, top-8, router bias ~N(0, 0.5))
    through izb_moe_forward at T = 1, 64, 4096; rotating over 3 layers' weights (3.6 GB) so the
    small-T cases stream expert weights from HBM rather than L2."""
    import torch
    from izwi_b200 import moe, ops
    peak_tf, _ = load_tensor_peak()
    peak_bw, _ = load_peaks()
    gen = torch.Generator(device=device).manual_seed(4)
    h, i, e, k = 2048, 768, 128, 8
    rn = lambda *s, std=1.0: (torch.randn(*s, device=device, generator=gen) * std).to(torch.bfloat16)  # noqa: E731
    layers = [moe.MoeLayer(rn(e, h, std=h ** -0.5), rn(e, std=0.5), rn(e, 2 * i, h, std=0.02), rn(e, h, i, std=0.02), k)
              for _ in range(3)]
    out = []
    for t in (1, 64, 4096):
        x = rn(t, h)
        state = {"i": 0}

        def step():
            layers[state["i"] % 3].forward(x)
            state["i"] += 1
        ms = _time_call(step, 30)
        _, _, idx, _ = layers[0].forward(x)
        touched = int(torch.unique(idx).numel())
        flops = 2.0 * t * k * 3 * i * h + 2.0 * t * e * h
        wbytes = touched * 3 * i * h * 2 + e * h * 2
        out.append({"workload": f"qwen3-30b-a3b-moe-layer-T{t}", "ms": round(ms, 4), "experts_touched": touched,
                    "tflops": round(flops / (ms * 1e-3) / 1e12, 2), "tensor_frac": round(flops / (ms * 1e-3) / 1e12 / peak_tf, 4),
                    "weight_gbs": round(wbytes / (ms * 1e-3) / 1e9, 1), "hbm_frac_of_measured": round(wbytes / (ms * 1e-3) / 1e9 / peak_bw, 4),
                    "kernels_per_layer": 8})
    ops.Context.get(device.index).check()
    del layers
    torch.cuda.empty_cache()
    return out


def run_ours(args):
    import torch
    from izwi_b200 import workloads as wl

    world, rank, local = dist_setup(args.gpus)
    device = torch.device("cuda", local)
    peak, peak_kind = load_peaks()
    fmt, m = WORKLOADS[args.workload]

    stack = make_stack(args.workload, device)
    group = wl.stack_group(stack)
    ctx = group.ctx

    for _ in range(max(args.warmup, 3)):
        group.launch()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = ctx.launch_count
    ms, t0, t1 = time_steps(group.launch, args.steps, world)
    launches = ctx.launch_count - launches0
    sampler.stop_flag.set()
    sampler.join(timeout=2)
    ctx.check()  # raises if any bounded device-side wait gave up

    per_ms = ms / args.steps
    tokens_per_s = world * m / (per_ms * 1e-3)
    achieved = stack.algorithmic_bytes / (per_ms * 1e-3) / 1e9

    # ---- end to end through the C ABI: host activations in, host results out, every step ----
    h_in = torch.empty_like(stack.acts_buf, device="cpu").pin_memory()
    h_in.copy_(stack.acts_buf)
    h_out = torch.empty_like(stack.outs_buf, device="cpu").pin_memory()

    def e2e_step():
        stack.acts_buf.copy_(h_in, non_blocking=True)
        group.launch()
        h_out.copy_(stack.outs_buf, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller reads the result before the next token

    e2e_steps = max(3, min(args.steps, 2000))
    for _ in range(3):
        e2e_step()
    e2e_ms, _, _ = time_steps(e2e_step, e2e_steps, world)
    e2e_tokens = world * m / (e2e_ms / e2e_steps * 1e-3)
    ctx.check()

    line = {
        "metric": METRIC, "value": round(tokens_per_s, 2), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(per_ms, 6),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "weights": fmt, "tokens_per_step": m,
                   "layers": stack.shape.layers, "projections_per_layer": 4,
                   "weight_bytes": stack.weight_bytes, "launch": "one grouped persistent launch per step",
                   "l2": f"inputs larger than L2 ({stack.weight_bytes / 1e6:.0f} MB streamed per step vs 126 MB)",
                   "multi_gpu": "replicas only (the 0.6B decode stack does not shard)" if world > 1 else "single GPU"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "peak_kind": f"of {peak_kind}",
                     "frac_of_nominal_8000": round(achieved / 8000.0, 4),
                     "algorithmic_bytes_per_launch": stack.algorithmic_bytes,
                     "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(args.workload)},
        "e2e": {"value": round(e2e_tokens, 2), "unit": "tokens/s",
                "h2d_bytes_per_step": h_in.numel() * 2, "d2h_bytes_per_step": h_out.numel() * 2,
                "steps": e2e_steps},
        "gpu_launches": int(launches),
        "clocks": sampler.summary(t0, t1),
    }

    if rank == 0 and world == 1:
        if not args.no_cpu_baseline:
            cpu = CpuStack(stack)
            # parity of the timed path against the checker, on the spot
            import numpy as np
            cpu.step()
            worst_rel, worst_cos = 0.0, 1.0
            flat_out = [y for ol in stack.outs for y in ol]
            for (wh, xh, yh, n, k), yd in list(zip(cpu.items, flat_out))[:8]:
                g = yd.float().cpu().numpy()
                denom = np.abs(yh).max(axis=1, keepdims=True)
                worst_rel = max(worst_rel, float((np.abs(g - yh) / np.where(denom == 0, 1, denom)).max()))
                worst_cos = min(worst_cos, float((g * yh).sum() / (np.linalg.norm(g) * np.linalg.norm(yh))))
            line["parity"] = {"max_rel_err": round(worst_rel, 6), "min_cosine": round(worst_cos, 7),
                              "checked": "first 2 layers vs CPU port", "gate": "rel<=2e-2, cos>=0.9999"}
            n, dt = cpu.timed(args.cpu_seconds)
            line["cpu_baseline"] = {"value": round(n * m / dt, 3), "unit": "tokens/s", "cores": cpu.cores,
                                    "kind": "port",
                                    "sample": f"{n} full decode steps of the same stack (dequantise + fp32 dot, "
                                              f"OpenMP over weight rows), {dt:.1f} s"}
            del cpu
        if not args.no_cases:
            del group
            cases = []
            for wname in WORKLOADS:
                if wname == args.workload:
                    continue
                cases.append(measure_case(wname, device, args.case_steps, 5, peak))
            line["cases"] = cases
            line["gemm_cases"] = measure_gemm_cases(device)
            line["moe_cases"] = measure_moe_cases(device)
            line["attention_cases"] = measure_attention_cases(device)
            line["decode_token_cases"] = measure_decode_token_cases(device)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------------------
# sharded workloads (run with --gpus N under torch.distributed.run; N = 1 gives the baseline point)
# ----------------------------------------------------------------------------------------------
SHARDED = {
    # name: (kind, parameter)
    "qwen3-8b-tp-decode-m1": ("tp", 1), "qwen3-8b-tp-decode-m8": ("tp", 8), "qwen3-8b-tp-decode-m32": ("tp", 32),
    "qwen3-8b-tp-prefill-m2048": ("tp", 2048),
    "qwen3-30b-a3b-ep-t64": ("ep", 64), "qwen3-30b-a3b-ep-t4096": ("ep", 4096),
    "fastconformer-b32": ("enc", ("fastconformer", 24, 1024, 4096, 375, 32, False, "silu")),
    "whisper-large-v3-b32": ("enc", ("whisper", 32, 1280, 5120, 1500, 32, True, "gelu")),
}


def run_sharded(args):
    import torch
    from izwi_b200 import moe, ops, parallel
    from izwi_b200 import workloads as wl

    world, rank, local = dist_setup(args.gpus)
    device = torch.device("cuda", local)
    kind, param = SHARDED[args.workload]
    comm = parallel.Comm(local) if world > 1 else None
    if comm is not None and kind == "tp":
        # sums go through NVLink peer memory, not NCCL: one-shot up to 1 MB, two-shot up to 64 MB
        comm.enable_peer_allreduce(1 << 20 if args.nccl_ep else 64 << 20)
    gen = torch.Generator(device=device).manual_seed(3)       # same stream of weights on every rank
    rn = lambda *s, std=1.0: (torch.randn(*s, device=device, generator=gen) * std).to(torch.bfloat16)  # noqa: E731
    cfg = {"workload": args.workload, "l2": "weights larger than L2"}
    flops = 0.0

    if kind == "tp":
        shape, m = wl.QWEN3_8B, param
        (_, n_qkv, h), (_, _, k_o), (_, n_gu, _), (_, _, k_d) = shape.projections
        layers = []
        for _ in range(shape.layers):
            full = (rn(n_qkv, h, std=0.02), rn(h, k_o, std=0.02), rn(n_gu, h, std=0.02), rn(h, k_d, std=0.02))
            layers.append(parallel.TpDecoderLayer.from_full(comm, shape, *full, world, rank) if world > 1
                          else parallel.TpDecoderLayer(None, *full))
            del full
        lo, hi = parallel.tp_row_split_cols(k_o, world, rank)
        x_a, x_o, x_m = rn(m, h), rn(m, hi - lo), rn(m, h)

        def step():
            for layer in layers:
                layer.forward(x_a, x_o, x_m)
        units, unit_name = m, "tokens/s"
        flops = 2.0 * m * shape.layers * shape.weights_per_layer
        cfg.update(model="qwen3-8b linear stack", tokens_per_step=m, layers=shape.layers,
                   parallelism=f"tp{world}: column-split QKV and gate/up, row-split O and down, 2 all-reduces per layer")
    elif kind == "ep":
        t_total, n_layers = param, 8
        h, inter, e, k = 2048, 768, 128, 8
        lo_e, hi_e = parallel.ep_expert_range(e, world, rank)
        layers = []
        for _ in range(n_layers):
            wr, br = rn(e, h, std=h ** -0.5), rn(e, std=0.5)
            wgu, wd = rn(e, 2 * inter, h, std=0.02), rn(e, h, inter, std=0.02)
            if world > 1:
                layers.append(parallel.EpMoeLayer(comm, wr, br, wgu[lo_e:hi_e].clone(), wd[lo_e:hi_e].clone(), e, k))
            else:
                layers.append(moe.MoeLayer(wr, br, wgu, wd, k))
            del wgu, wd
        lo_t, hi_t = parallel.split_range(t_total, world, rank)
        x = rn(t_total, h)[lo_t:hi_t].contiguous()
        if world > 1 and not args.nccl_ep:
            # rows travel through NVLink peer memory with device-side counts (no host read per layer)
            comm.enable_peer_ep(e, h, (t_total + world - 1) // world, k)

        def step():
            for layer in layers:
                layer.forward(x)
        units, unit_name = t_total, "tokens/s"
        flops = 2.0 * t_total * k * 3 * inter * h * n_layers
        cfg.update(model="qwen3-30b-a3b MoE FFN layers", tokens_per_step=t_total, layers=n_layers,
                   note="8 of the 48 layers (each layer is 1.2 GB of expert weights)",
                   parallelism=f"ep{world}: {e // world} experts per rank, tokens split, dispatch and return each way "
                               + ("over NCCL with host-side counts" if args.nccl_ep or world == 1 else "over peer memory"))
    else:
        name, n_layers, d, ff, frames, batch, has_bias, act = param
        lo_b, hi_b = parallel.batch_split(batch, world, rank)
        m = (hi_b - lo_b) * frames
        layers = []
        for _ in range(n_layers):
            ws = {"qkv": rn(3 * d, d, std=0.02), "o": rn(d, d, std=0.02), "fc1": rn(ff, d, std=0.02), "fc2": rn(d, ff, std=0.02)}
            bs = {kk: (rn(v.shape[0], std=0.1) if has_bias else None) for kk, v in ws.items()}
            layers.append((ws, bs))
        n_ffn = 2 if name == "fastconformer" else 1                   # two macaron feed-forwards per layer
        x = rn(max(m, 1), d)
        bufs = {"qkv": torch.empty(max(m, 1), 3 * d, device=device, dtype=torch.bfloat16),
                "d": torch.empty(max(m, 1), d, device=device, dtype=torch.bfloat16),
                "ff": torch.empty(max(m, 1), ff, device=device, dtype=torch.bfloat16)}

        def step():
            if m == 0:
                return
            for ws, bs in layers:
                ops.linear(x, ws["qkv"], bias=bs["qkv"], out=bufs["qkv"])
                ops.linear(x, ws["o"], bias=bs["o"], out=bufs["d"])
                for _ in range(n_ffn):
                    ops.linear(x, ws["fc1"], bias=bs["fc1"], out=bufs["ff"], epilogue=act)
                    ops.linear(bufs["ff"], ws["fc2"], bias=bs["fc2"], out=bufs["d"])
        units, unit_name = batch, "utterances/s"
        flops = 2.0 * batch * frames * n_layers * (4 * d * d + n_ffn * 2 * d * ff)
        cfg.update(model=f"{name} encoder GEMMs (QKV, O, FFN)", batch=batch, frames=frames, layers=n_layers,
                   parallelism=f"batch split over {world} ranks, weights replicated, no collective")

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if kind == "tp" and param <= 32 and not args.no_graph:
        # the decode step is a fixed sequence of launches: replay it as one CUDA graph
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        eager_step, step = step, graph.replay
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        cfg["launch"] = "CUDA graph replay of the whole step"
    sampler = ClockSampler(local)
    sampler.start()
    ctx = ops.Context.get(local)
    launches0 = ctx.launch_count
    ms, t0, t1 = time_steps(step, args.steps, world)
    launches = ctx.launch_count - launches0
    sampler.stop_flag.set()
    sampler.join(timeout=2)
    ctx.check()
    per_ms = ms / args.steps
    peak_tf, kind_tf = load_tensor_peak()
    line = {"metric": f"{args.workload}_{unit_name.split('/')[0]}_per_s", "value": round(units / (per_ms * 1e-3), 2),
            "unit": unit_name, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(per_ms, 5), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": cfg,
            "tflops_total": round(flops / (per_ms * 1e-3) / 1e12, 1),
            "tensor_frac_per_gpu": round(flops / (per_ms * 1e-3) / 1e12 / world / peak_tf, 4),
            "gpu_launches": int(launches), "clocks": sampler.summary(t0, t1)}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        comm.close()
        dist.destroy_process_group()


def run_reference(args):
    """The reference arm: the CPU restatement of the same stack on the host cores (the reference's
    own Candle CPU path cannot be built without a Rust toolchain)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    dev = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    fmt, m = WORKLOADS[args.workload]
    stack = make_stack(args.workload, dev)
    cpu = CpuStack(stack)
    weight_bytes = stack.weight_bytes
    del stack
    for _ in range(max(1, min(args.warmup, 3))):
        cpu.step()
    steps = max(1, min(args.steps, 50))  # each step is a full CPU decode step; bounded so the run ends in minutes
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu.step()
    dt = time.perf_counter() - t0
    v = round(steps * m / dt, 3)
    sample = f"{steps} full decode steps of the stack on the host cores"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": max(1, min(args.warmup, 3)), "ms_per_step": round(dt / steps * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "weights": fmt, "tokens_per_step": m, "weight_bytes": weight_bytes},
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": cpu.cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS) + sorted(SHARDED))
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--case-steps", type=int, default=300)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-cases", action="store_true")
    ap.add_argument("--nccl-ep", action="store_true", help="expert-parallel workloads: exchange rows with NCCL instead of peer memory")
    ap.add_argument("--no-graph", action="store_true", help="sharded decode workloads: launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--attention-cases", action="store_true",
                    help="profiler captures: run only the decode-attention cases and exit")
    ap.add_argument("--decode-token-cases", action="store_true",
                    help="only the whole-greedy-token cases (eager steps, then a CUDA graph replayed)")
    ap.add_argument("--gemm-case", default=None,
                    help="profiler captures: run only this prefill / encoder GEMM shape (a name from gemm_cases) and exit")
    ap.add_argument("--layers", type=int, default=None,
                    help="shorter stack for profiler captures (the reported line is then not the benchmark)")
    args = ap.parse_args()
    global LAYERS_OVERRIDE
    LAYERS_OVERRIDE = args.layers
    if args.attention_cases:
        import torch
        print(json.dumps({"attention_cases": measure_attention_cases(torch.device("cuda", 0))}), flush=True)
        return
    if args.decode_token_cases:
        import torch
        print(json.dumps({"decode_token_cases": measure_decode_token_cases(torch.device("cuda", 0))}), flush=True)
        return
    if args.gemm_case:
        import torch
        res = measure_gemm_cases(torch.device("cuda", 0), only=args.gemm_case, iters=max(1, min(args.steps, 20)))
        print(json.dumps({"gemm_case": res}), flush=True)
        return
    if args.workload in SHARDED:
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the CPU reference arm covers the default workload only"}))
            return
        if args.steps == 20000:
            args.steps = 20
        run_sharded(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
