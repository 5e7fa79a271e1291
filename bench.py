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
through the C ABI with host activations copied in and the results stored into
host memory every step (izb_linear_group_launch_host); `roofline` is algorithmic bytes per launch over the measured launch
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


def time_blocks(fn, steps: int, world: int, min_ms: float, max_blocks: int = 400):
    """Blocks of exactly `steps` calls each (timed as time_steps does), repeated until the blocks add up
    to `min_ms` of device time, so that a short `--steps` does not leave the number hanging on a
    millisecond of measurement.  Returns (median block ms, all block ms, wall start, wall end); every
    rank sees the same max-over-ranks block times and therefore stops after the same block."""
    blocks, t_first, t_last = [], None, None
    while True:
        ms, t0, t1 = time_steps(fn, steps, world)
        blocks.append(ms)
        t_first = t0 if t_first is None else t_first
        t_last = t1
        if sum(blocks) >= min_ms or len(blocks) >= max_blocks:
            break
    return statistics.median(blocks), blocks, t_first, t_last


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def oracle_lib():
    """The C restatement (CPU baseline leg and on-the-spot checker only).  The OpenMP team is sized here
    from the cores this process may run on: a launcher such as torch.distributed.run exports
    OMP_NUM_THREADS=1, which would otherwise leave the baseline on one core."""
    import subprocess
    so = ROOT / "oracle" / "liboracle_c.so"
    if not so.exists():
        subprocess.run(["make", "-C", str(ROOT / "oracle")], check=True, capture_output=True)
    lib = ctypes.CDLL(str(so))
    lib.orc_num_threads.restype = ctypes.c_int
    lib.orc_set_num_threads.argtypes = [ctypes.c_int]
    lib.orc_set_num_threads(host_cores())
    return lib


class CpuStack:
    """The same stack on the host: raw weight bytes (or fp32 for bf16) + fp32 activations, run by the C
    port.  `layers` restricts it to some layers (the checker of the secondary cases)."""

    def __init__(self, stack, layers=None):
        import numpy as np
        self.lib = oracle_lib()
        self.fmt, self.m = stack.fmt, stack.m
        self.items, self.outs = [], []
        for li, (wl, al, ol) in enumerate(zip(stack.weights, stack.acts, stack.outs)):
            if layers is not None and li not in layers:
                continue
            for (_, n, k), w, x, y in zip(stack.shape.projections, wl, al, ol):
                wh = (w.float() if self.fmt == "bf16" else w).cpu().numpy()
                xh = x.float().cpu().numpy()
                self.items.append((np.ascontiguousarray(wh), np.ascontiguousarray(xh), np.empty((self.m, n), np.float32), n, k))
                self.outs.append(y)
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

    def parity(self):
        """Worst max-relative error (to the row's largest magnitude) and cosine of the device outputs of the
        projections held here against one CPU step."""
        self.step()
        worst = Parity()
        for (wh, xh, yh, n, k), yd in zip(self.items, self.outs):
            worst.add(yd.float().cpu().numpy(), yh)
        return worst

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


class Parity:
    """Accumulates the two gated figures over several outputs: max |got - want| relative to the largest
    |want| of the row, and the cosine of the flattened outputs.  Gate: rel <= 2e-2, cosine >= 0.9999."""
    GATE = "rel<=2e-2, cos>=0.9999"

    def __init__(self):
        self.rel, self.cos, self.n = 0.0, 1.0, 0

    def add(self, got, want):
        import numpy as np
        got = np.asarray(got, dtype=np.float64).reshape(-1, got.shape[-1])
        want = np.asarray(want, dtype=np.float64).reshape(-1, want.shape[-1])
        denom = np.abs(want).max(axis=1, keepdims=True)
        self.rel = max(self.rel, float((np.abs(got - want) / np.where(denom == 0, 1, denom)).max()))
        nrm = np.linalg.norm(got) * np.linalg.norm(want)
        self.cos = min(self.cos, float((got * want).sum() / nrm) if nrm > 0 else 1.0)
        self.n += 1

    def result(self, checked: str, **extra):
        ok = self.rel <= 2e-2 and self.cos >= 0.9999 and all(v is not False for v in extra.values())
        return {"max_rel_err": round(self.rel, 6), "min_cosine": round(self.cos, 7), "outputs_checked": self.n,
                "checked": checked, "gate": self.GATE, "pass": bool(ok), **extra}


def bf16_round_np(x):
    """fp32/fp64 values rounded to the nearest bf16 (ties to even), returned as float64."""
    import numpy as np
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32).astype(np.float64).reshape(np.shape(x))


def host64(t):
    """A device tensor as a float64 host array."""
    return t.detach().float().cpu().numpy().astype("float64")


def act_np(name, v):
    """The fused epilogue functions in float64 (erf GELU, tanh-form GELU, SiLU)."""
    import math
    import numpy as np
    if name == "gelu":
        return 0.5 * v * (1.0 + np.vectorize(math.erf)(v * 0.7071067811865476))
    if name == "gelu_tanh":
        return 0.5 * v * (1.0 + np.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3)))
    if name == "silu":
        return v / (1.0 + np.exp(-v))
    return v


LAYERS_OVERRIDE = None  # --layers: a shorter stack, for profiler captures only


def make_stack(workload: str, device):
    from izwi_b200 import workloads as wl
    fmt, m = WORKLOADS[workload]
    return wl.make_linear_stack(wl.QWEN3_0_6B, fmt, m, device, WEIGHT_SEED, ACT_SEED, layers=LAYERS_OVERRIDE)


def measure_case(workload: str, device, steps: int, warmup: int, peak: float, check: bool = True):
    """Short device-resident measurement of one more configuration (not the headline line), checked on
    its first and last layer against the CPU port."""
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
    if check:
        last = stack.shape.layers - 1
        out["parity"] = CpuStack(stack, layers={0, last}).parity().result(f"layers 0 and {last} vs CPU port")
    del group, stack
    torch.cuda.empty_cache()
    return out


def load_tensor_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), "measured burst"
    return 1590.0, "fallback"


def _time_call(fn, iters: int, warmup: int = 3, graph_batch: int = 0):
    """Average device time of one call.  With graph_batch > 0 that many calls are captured into one CUDA
    graph and the graph is replayed, so a kernel of a few microseconds is timed at the rate the GPU can
    run it back to back rather than at the rate Python can issue it."""
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    run, per = fn, 1
    if graph_batch > 0:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(graph_batch):
                fn()
        run, per = g.replay, graph_batch
        iters = max(1, iters // graph_batch)
        run()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (iters * per)


def sampled_rows(m: int):
    return sorted({0, m // 3, m // 2, m - 1})


def linear_rows_ref(x, w, bias, rows, epilogue=None):
    """float64 product of the sampled activation rows with the whole weight on the host."""
    import numpy as np
    v = host64(x[rows]) @ host64(w).T
    if bias is not None:
        v = v + host64(bias)[None, :]
    if epilogue == "swiglu":
        half = v.shape[1] // 2
        return act_np("silu", v[:, :half]) * v[:, half:]
    return act_np(epilogue, v)


def measure_gemm_cases(device, only=None, iters=20):
    """Prefill (Qwen3-8B shape, M = 2048) and ASR-encoder GEMMs through izb_linear: TFLOP/s against the
    measured bf16 tensor peak.  The single-shape entries re-run one operand set (the large ones exceed
    L2, the small ones are L2-resident as they would be inside a layer loop); the `-stack` entries run
    every layer of the model with its own weights, so each weight comes from HBM once per pass.  Every
    entry is checked on sampled rows against a float64 product on the host."""
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
        ("whisper-b32-fc1+bias+gelu", 48000, 5120, 1280, "gelu_tanh", True),
        ("whisper-b32-fc2+bias", 48000, 1280, 5120, None, True),
        ("whisper-b1-fc1+bias+gelu", 1500, 5120, 1280, "gelu_tanh", True),
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
        # calls replayed from a CUDA graph (10 per graph): the launch rate of the caller's language is not the subject
        ms = _time_call(lambda: ops.linear(x, w, bias=b, out=y, epilogue=epi), max(iters, 10), graph_batch=10 if iters >= 10 else 0)
        tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        rows = sampled_rows(m)
        par = Parity()
        par.add(host64(y[rows]), linear_rows_ref(x, w, b, rows, epi))
        out.append({"workload": name, "M": m, "N": n, "K": k, "ms": round(ms, 4), "tflops": round(tf, 1),
                    "tensor_frac": round(tf / peak, 4), "peak_kind": f"of {kind} {peak}",
                    "parity": par.result(f"{len(rows)} sampled rows x all columns vs float64 on the host")})
        del x, w, y
    if only is None:
        out += measure_stack_gemm_cases(device, peak, kind)
    ops.Context.get(device.index).check()
    torch.cuda.empty_cache()
    return out


def measure_stack_gemm_cases(device, peak, kind):
    """Whole-model passes (every layer with its own weights, HBM-cold): Qwen3-8B prefill M = 2048,
    Whisper-large-v3 and FastConformer encoder GEMMs at batch 1 and 32."""
    import torch
    out = []
    tp = TpStack(None, 1, 0, device)
    out.append(stack_entry("qwen3-8b-prefill-m2048-stack", tp.case(2048, 5, 3), peak, kind))
    del tp
    torch.cuda.empty_cache()
    for name in ("whisper-large-v3", "fastconformer"):
        enc = EncStack(name, 1, 0, device)
        for batch in (1, 32):
            out.append(stack_entry(f"{name}-b{batch}-stack", enc.case(batch, 5, 3), peak, kind))
        del enc
        torch.cuda.empty_cache()
    return out


def stack_entry(name, case, peak, kind):
    return {"workload": name, "ms": case["ms_per_step"], "tflops": case["tflops_total"],
            "tensor_frac": round(case["tflops_total"] / peak, 4), "peak_kind": f"of {kind} {peak}",
            "launches_per_pass": case["launches_per_step"], "parity": case["parity"]}


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


def measure_decode_token_cases(device, shape=None, variants=None, fmt="q8_0"):
    """A whole greedy decode token of a Qwen3-0.6B-shaped model with Q8_0 (or Q4_K) projections (embedding, 28
    layers of norm / fused QKV / q,k norm / RoPE / KV append / GQA attention / O / norm / gate-up /
    SiLU-multiply / down, final norm, lm_head over 151,936 tokens, arg-max), captured once in a CUDA
    graph at a fixed context length and replayed: what the linear stack of the headline sits in."""
    import torch
    from izwi_b200 import decoder, ops
    from izwi_b200 import workloads as wl
    peak_bw, _ = load_peaks()
    if shape is None:
        # the 0.6B shape (launch- and latency-bound: 0.64 GB of weights per token) and, for the one-launch kernel and
        # the fused chain, the 8B shape (8.7 GB per token: bandwidth starts to matter)
        return (measure_decode_token_cases(device, wl.QWEN3_0_6B, ((512, "one_launch"), (4096, "one_launch"), (512, True), (4096, True), (512, False)))
                + measure_decode_token_cases(device, wl.QWEN3_0_6B, ((512, "one_launch"), (512, True)), fmt="q4_k")
                + measure_decode_token_cases(device, wl.QWEN3_8B, ((512, "one_launch"), (512, True))))
    gen = torch.Generator(device=device).manual_seed(6)
    vocab, hid, qd, kd = 151936, shape.hidden, shape.q_heads * shape.head_dim, shape.kv_heads * shape.head_dim
    ones = lambda n: (1.0 + 0.1 * torch.randn(n, device=device, generator=gen)).to(torch.bfloat16)  # noqa: E731
    layers = []
    make_w = wl.make_q8_0_weight if fmt == "q8_0" else wl.make_q4_k_weight
    for _ in range(shape.layers):
        layers.append(decoder.Qwen3DecoderLayer(decoder.Qwen3LayerWeights(
            fmt, hid, shape.q_heads, shape.kv_heads, shape.head_dim, shape.intermediate, ones(hid), ones(hid),
            ones(shape.head_dim), ones(shape.head_dim), make_w(qd + 2 * kd, hid, gen),
            make_w(hid, qd, gen), make_w(2 * shape.intermediate, hid, gen),
            make_w(hid, shape.intermediate, gen))))
    embed = (torch.randn(vocab, hid, device=device, generator=gen) * 0.5).to(torch.bfloat16)
    model = decoder.Qwen3Decoder(embed, layers, ones(hid), make_w(vocab, hid, gen), fmt)
    weight_bytes = sum(w.numel() for l in layers for w in (l.w.qkv, l.w.o, l.w.gate_up, l.w.down)) + model.lm_head.numel()
    out = []
    for ctx_len, fused in variants:
        # fused: norms, SiLU-multiply and residual adds ride inside the one-token projections;
        # "one_launch": the whole token in one cooperative launch (izb_qwen3_decode_token)
        one_launch = fused == "one_launch"
        for l in layers:
            l.fused_linear = fused
            l.fusion_max_tokens = ops.linear_fusion_max_tokens(fmt) if fused else 0
        # the cache contents depend on the context length only, so the fused and unfused builds of one
        # length see the same model state and must pick the same token
        cgen = torch.Generator(device=device).manual_seed(7000 + ctx_len)
        caches = [decoder.KvCache(1, shape.kv_heads, ctx_len + 8, shape.head_dim, device) for _ in layers]
        for c in caches:
            c.k.normal_(generator=cgen)
            c.v.normal_(generator=cgen)
        tok = torch.tensor([17], device=device, dtype=torch.int32 if one_launch else torch.int64)
        cos, sin = model.rope_tables(ctx_len, 1)
        if one_launch:
            kernel = decoder.Qwen3TokenKernel(model, caches)
            step = lambda: kernel.step(tok, ctx_len, cos, sin)  # noqa: E731
        else:
            step = lambda: model.step(tok, caches, ctx_len, cos, sin)  # noqa: E731
        launches0 = ops.Context.get(device.index).launch_count
        for _ in range(2):
            nxt = step()
        torch.cuda.synchronize()
        launches = (ops.Context.get(device.index).launch_count - launches0) // 2
        if one_launch:
            ms = _time_call(step, 30)  # one launch per token: nothing for a graph to save
        else:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                nxt = step()
            ms = _time_call(graph.replay, 30)
        ops.Context.get(device.index).check()
        kv_bytes = shape.layers * 2 * shape.kv_heads * (ctx_len + 1) * shape.head_dim * 2
        gbs = (weight_bytes + kv_bytes) / (ms * 1e-3) / 1e9
        out.append({"workload": f"{shape.name}-{fmt}-greedy-token-ctx{ctx_len}", "ms_per_token": round(ms, 4),
                    "tokens_per_s": round(1e3 / ms, 1), "kernels_per_token": int(launches), "fused_projections": fused,
                    "weight_and_kv_gbs": round(gbs, 1), "hbm_frac_of_measured": round(gbs / peak_bw, 4),
                    "next_token": int(nxt[0])})
        if one_launch:
            del kernel
        else:
            del graph
        del caches
        torch.cuda.empty_cache()
    del model, layers, embed
    torch.cuda.empty_cache()
    return out


def moe_parity(x, y, idx, wts, logits_fn, w_router, router_bias, w_gate_up, w_down, top_k, tokens=None):
    """Checks one MoE layer's routing and output on the host.  Routing: the indices of every token must
    equal, bit for bit, the top-k (descending logit, lowest expert id among equals) of the fp32 router
    logits the library produced, and those logits must agree with a float64 product.  Output: sampled
    tokens against float64 expert FFNs (SiLU-multiply rounded to bf16 as stored, expert outputs rounded
    to bf16, weighted sum in ascending slot order).  x, y, idx, wts are this rank's tokens; the expert
    weights are the full [E, ...] tensors."""
    import numpy as np
    t = x.shape[0]
    logits = logits_fn().float().cpu().numpy()
    order = np.argsort(-logits, axis=1, kind="stable")[:, :top_k].astype(np.int32)
    idx_h = idx.cpu().numpy()
    exact = bool(np.array_equal(order, idx_h))
    par = Parity()
    ref_logits = host64(x) @ host64(w_router).T + (0 if router_bias is None else host64(router_bias)[None, :])
    par.add(logits, ref_logits)
    inter = w_gate_up.shape[1] // 2
    rows = sampled_rows(t) if tokens is None else tokens
    want = np.zeros((len(rows), x.shape[1]))
    wts_h = wts.float().cpu().numpy().astype(np.float64)
    for i, r in enumerate(rows):
        xr = host64(x[r])
        for slot in range(top_k):
            e = int(idx_h[r, slot])
            gu = host64(w_gate_up[e]) @ xr
            hid = bf16_round_np(act_np("silu", gu[:inter]) * gu[inter:])
            want[i] += wts_h[r, slot] * bf16_round_np(host64(w_down[e]) @ hid)
    par.add(host64(y[rows]), want)
    return par.result(f"router logits of {t} tokens and the layer output of {len(rows)} sampled tokens vs float64 on the host",
                      routing_indices_bit_exact=exact)


def measure_moe_profile_case(device, experts: int, tokens: int, iters: int):
    """A reduced MoE layer (Qwen3-30B-A3B expert shape, fewer experts and tokens) for profiler captures of
    the grouped expert GEMM: a few hundred MB of weights, a handful of launches."""
    import torch
    from izwi_b200 import moe, ops
    gen = torch.Generator(device=device).manual_seed(4)
    h, i, k = 2048, 768, 8
    rn = lambda *s, std=1.0: (torch.randn(*s, device=device, generator=gen) * std).to(torch.bfloat16)  # noqa: E731
    layer = moe.MoeLayer(rn(experts, h, std=h ** -0.5), rn(experts, std=0.5), rn(experts, 2 * i, h, std=0.02),
                         rn(experts, h, i, std=0.02), k)
    x = rn(tokens, h)
    ms = _time_call(lambda: layer.forward(x), iters, warmup=2)
    ops.Context.get(device.index).check()
    return {"workload": f"moe-layer-E{experts}-T{tokens}", "ms": round(ms, 4), "pairs": tokens * k,
            "weight_mb": round(experts * 3 * i * h * 2 / 1e6, 1)}


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
    ctx = ops.Context.get(device.index)
    for t in (1, 64, 4096):
        x = rn(t, h)
        state = {"i": 0}

        def step():
            layers[state["i"] % 3].forward(x)
            state["i"] += 1
        l0 = ctx.launch_count
        step()
        per_layer = ctx.launch_count - l0
        state["i"] = 0
        ms_eager = _time_call(step, 30)
        # a decode loop replays its launches from a CUDA graph: the three layers in one graph, time per layer
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for lay in layers:
                lay.forward(x)
        ms = _time_call(graph.replay, 30) / len(layers)
        del graph
        lay = layers[0]
        y, logits, idx, wts = lay.forward(x)
        touched = int(torch.unique(idx).numel())
        flops = 2.0 * t * k * 3 * i * h + 2.0 * t * e * h
        wbytes = touched * 3 * i * h * 2 + e * h * 2
        out.append({"workload": f"qwen3-30b-a3b-moe-layer-T{t}", "ms": round(ms, 4), "experts_touched": touched,
                    "tflops": round(flops / (ms * 1e-3) / 1e12, 2), "tensor_frac": round(flops / (ms * 1e-3) / 1e12 / peak_tf, 4),
                    "weight_gbs": round(wbytes / (ms * 1e-3) / 1e9, 1), "hbm_frac_of_measured": round(wbytes / (ms * 1e-3) / 1e9 / peak_bw, 4),
                    "kernels_per_layer": int(per_layer), "launch": "CUDA-graph replay of three layers", "ms_eager_launches": round(ms_eager, 4),
                    "parity": moe_parity(x, y, idx, wts, lambda: logits, lay.w_router, lay.router_bias, lay.w_gate_up,
                                         lay.w_down, k)})
    ctx.check()
    del layers
    torch.cuda.empty_cache()
    return out


# ----------------------------------------------------------------------------------------------
# sharded workloads: tensor-parallel Qwen3-8B, expert-parallel Qwen3-30B-A3B, batch-parallel encoders.
# Every rank draws the same full tensors from one seed and keeps its shard, so any rank can check its
# outputs against the unsharded weights.  world = 1 is the baseline point of the scaling curve.
# ----------------------------------------------------------------------------------------------
SHARDED = {
    # name: (kind, parameter)
    "qwen3-8b-tp-prefill-m2048": ("tp", 2048),
    "qwen3-8b-tp-decode-m1": ("tp", 1), "qwen3-8b-tp-decode-m8": ("tp", 8), "qwen3-8b-tp-decode-m32": ("tp", 32),
    "qwen3-30b-a3b-ep-t4096": ("ep", 4096), "qwen3-30b-a3b-ep-t64": ("ep", 64),
    "whisper-large-v3-b32": ("whisper-large-v3", 32), "fastconformer-b32": ("fastconformer", 32),
}
# the ones every default run reports under `sharded_cases`
SHARDED_DEFAULT = ["qwen3-8b-tp-prefill-m2048", "qwen3-8b-tp-decode-m1", "qwen3-8b-tp-decode-m32",
                   "qwen3-30b-a3b-ep-t4096", "qwen3-30b-a3b-ep-t64", "whisper-large-v3-b32", "fastconformer-b32"]
ENCODERS = {
    # name: (layers, d_model, ffn, frames per utterance, biases, activation, feed-forwards per layer)
    "whisper-large-v3": (32, 1280, 5120, 1500, True, "gelu_tanh", 1),
    "fastconformer": (24, 1024, 4096, 375, False, "silu", 2),
}


def _timed_case(step, steps, warmup, world, device_index, graph=False):
    """Warm-up, optional CUDA-graph capture of the step, `steps` timed calls (max over ranks)."""
    import torch
    from izwi_b200 import ops
    ctx = ops.Context.get(device_index)
    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    l0 = ctx.launch_count
    step()
    launches = ctx.launch_count - l0
    run = step
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step()
        run = g.replay
        for _ in range(3):
            run()
        torch.cuda.synchronize()
    ms, _, _ = time_steps(run, steps, world)
    ctx.check()
    return ms / steps, int(launches)


class TpStack:
    """The 36-layer Qwen3-8B linear stack, column/row split over `world` ranks."""

    def __init__(self, comm, world, rank, device, use_graph=True):
        import torch
        from izwi_b200 import parallel
        from izwi_b200 import workloads as wl
        self.comm, self.world, self.rank, self.device, self.use_graph = comm, world, rank, device, use_graph
        self.shape = shape = wl.QWEN3_8B
        gen = torch.Generator(device=device).manual_seed(3)
        rn = lambda *s, std=1.0: (torch.randn(*s, device=device, generator=gen) * std).to(torch.bfloat16)  # noqa: E731
        (_, n_qkv, h), (_, _, k_o), (_, n_gu, _), (_, _, k_d) = shape.projections
        self.layers, self.full0 = [], None
        for li in range(shape.layers):
            full = (rn(n_qkv, h, std=0.02), rn(h, k_o, std=0.02), rn(n_gu, h, std=0.02), rn(h, k_d, std=0.02))
            self.layers.append(parallel.TpDecoderLayer.from_full(comm, shape, *full, world, rank) if world > 1
                               else parallel.TpDecoderLayer(None, *full))
            if li == 0 and rank == 0:
                self.full0 = full          # the unsharded first layer, for the check
            del full

    def case(self, m, steps, warmup):
        import numpy as np
        import torch
        from izwi_b200 import parallel
        shape, world, rank = self.shape, self.world, self.rank
        (_, n_qkv, h), (_, _, k_o), _, _ = shape.projections
        gen = torch.Generator(device=self.device).manual_seed(300 + m)
        rn = lambda *s: torch.randn(*s, device=self.device, generator=gen).to(torch.bfloat16)  # noqa: E731
        x_a, x_o_full, x_m = rn(m, h), rn(m, k_o), rn(m, h)
        lo, hi = parallel.tp_row_split_cols(k_o, world, rank)
        x_o = x_o_full[:, lo:hi].contiguous()

        def step():
            for layer in self.layers:
                layer.forward(x_a, x_o, x_m)
            if self.comm is not None:
                self.comm.join()       # the sums run on a second stream: the step ends when they have
        if self.comm is not None:
            self.comm.reset_events()
        # a step is a fixed sequence of launches on two streams: captured once, replayed as a CUDA graph
        per_ms, launches = _timed_case(step, steps, warmup, world, self.device.index, graph=self.use_graph)
        flops = 2.0 * m * shape.layers * shape.weights_per_layer
        out = {"value": round(m / (per_ms * 1e-3), 2), "unit": "tokens/s", "ms_per_step": round(per_ms, 5), "n_gpus": world,
               "scaling": "strong", "launches_per_step": launches, "tflops_total": round(flops / (per_ms * 1e-3) / 1e12, 2),
               "weights_gbs_per_gpu": round(shape.layers * shape.weights_per_layer * 2 / world / (per_ms * 1e-3) / 1e9, 1),
               "collective": "none (one GPU)" if world == 1 else self.layers[0].collective_name(m),
               "parallelism": f"tp{world}: column-split QKV and gate/up, row-split O and down, 2 sums per layer"}
        qkv, o, down = self.layers[0].forward(x_a, x_o, x_m)      # every rank: the sums are collective
        if self.comm is not None:
            self.comm.join()
        torch.cuda.synchronize()
        if rank == 0:
            w_qkv, w_o, w_gu, w_d = self.full0
            rows = sampled_rows(m)
            mine = torch.from_numpy(parallel.tp_qkv_rows(shape.q_heads, shape.kv_heads, shape.head_dim, world, rank)).to(self.device)
            par = Parity()
            par.add(host64(qkv[rows]), linear_rows_ref(x_a, w_qkv[mine], None, rows))
            par.add(host64(o[rows]), linear_rows_ref(x_o_full, w_o, None, rows))
            hidden = bf16_round_np(linear_rows_ref(x_m, w_gu, None, rows, "swiglu"))
            par.add(host64(down[rows]), hidden @ host64(w_d).T)
            out["parity"] = par.result(f"layer 0, {len(rows)} sampled token rows: this rank's QKV columns, the summed O and "
                                       "down outputs vs float64 products of the unsharded weights on the host")
        return out


class EpStack:
    """Eight Qwen3-30B-A3B-shaped MoE layers, experts in contiguous blocks over `world` ranks."""
    H, I, E, K, LAYERS = 2048, 768, 128, 8, 8

    def __init__(self, comm, world, rank, device, max_tokens=4096, nccl=False):
        import torch
        from izwi_b200 import moe, parallel
        self.comm, self.world, self.rank, self.device, self.nccl = comm, world, rank, device, nccl
        gen = torch.Generator(device=device).manual_seed(4)
        rn = lambda *s, std=1.0: (torch.randn(*s, device=device, generator=gen) * std).to(torch.bfloat16)  # noqa: E731
        lo_e, hi_e = parallel.ep_expert_range(self.E, world, rank)
        self.layers, self.full0 = [], None
        for li in range(self.LAYERS):
            wr, br = rn(self.E, self.H, std=self.H ** -0.5), rn(self.E, std=0.5)
            wgu, wd = rn(self.E, 2 * self.I, self.H, std=0.02), rn(self.E, self.H, self.I, std=0.02)
            if world > 1:
                self.layers.append(parallel.EpMoeLayer(comm, wr, br, wgu[lo_e:hi_e].clone(), wd[lo_e:hi_e].clone(), self.E, self.K))
            else:
                self.layers.append(moe.MoeLayer(wr, br, wgu, wd, self.K))
            if li == 0 and rank == 0:
                self.full0 = (wr, br, wgu, wd)
            del wgu, wd
        if world > 1 and not nccl:
            # rows travel through NVLink peer memory with device-side counts (no host read per layer)
            comm.enable_peer_ep(self.E, self.H, (max_tokens + world - 1) // world, self.K)

    def case(self, t_total, steps, warmup):
        import torch
        from izwi_b200 import ops, parallel
        world, rank = self.world, self.rank
        gen = torch.Generator(device=self.device).manual_seed(400 + t_total)
        x_all = torch.randn(t_total, self.H, device=self.device, generator=gen).to(torch.bfloat16)
        lo_t, hi_t = parallel.split_range(t_total, world, rank)
        x = x_all[lo_t:hi_t].contiguous()

        def step():
            for layer in self.layers:
                layer.forward(x)
        # with the exchange over peer memory no step needs the host (counts stay on the device), so the
        # whole step replays from a CUDA graph; the NCCL path reads sizes on the host every layer
        per_ms, launches = _timed_case(step, steps, warmup, world, self.device.index, graph=not (world > 1 and self.nccl))
        flops = 2.0 * t_total * self.K * 3 * self.I * self.H * self.LAYERS
        out = {"value": round(t_total / (per_ms * 1e-3), 2), "unit": "tokens/s", "ms_per_step": round(per_ms, 5),
               "n_gpus": world, "scaling": "strong", "launches_per_step": launches, "layers": self.LAYERS,
               "tflops_total": round(flops / (per_ms * 1e-3) / 1e12, 2),
               "collective": "none (one GPU)" if world == 1 else (
                   "counts all-gather + izb_ep_alltoall over NCCL, sizes read by the host" if self.nccl
                   else "izb_ep_dispatch / izb_ep_return: rows stored into the owner's buffer over NVLink peer memory"),
               "parallelism": f"ep{world}: {self.E // world} experts per rank, tokens split, one exchange each way per layer"}
        res = self.layers[0].forward(x)                            # every rank: the exchange is collective
        torch.cuda.synchronize()
        if rank == 0 and hi_t > lo_t:
            wr, br, wgu, wd = self.full0
            y, idx, wts = (res[0], res[2], res[3]) if world == 1 else res
            logits = res[1] if world == 1 else self.layers[0].logits     # the logits the routing was made from
            out["parity"] = moe_parity(x, y, idx, wts, lambda: logits, wr, br,
                                       wgu, wd, self.K)
        return out


class EncStack:
    """QKV, O and feed-forward GEMMs of an ASR encoder, utterances split over ranks, weights replicated."""

    def __init__(self, name, world, rank, device):
        import torch
        self.name, self.world, self.rank, self.device = name, world, rank, device
        self.n_layers, self.d, self.ff, self.frames, has_bias, self.act, self.n_ffn = ENCODERS[name]
        gen = torch.Generator(device=device).manual_seed(5)
        rn = lambda *s, std=1.0: (torch.randn(*s, device=device, generator=gen) * std).to(torch.bfloat16)  # noqa: E731
        d, ff = self.d, self.ff
        self.layers = []
        for _ in range(self.n_layers):
            ws = {"qkv": rn(3 * d, d, std=0.02), "o": rn(d, d, std=0.02), "fc1": rn(ff, d, std=0.02), "fc2": rn(d, ff, std=0.02)}
            bs = {kk: (rn(v.shape[0], std=0.1) if has_bias else None) for kk, v in ws.items()}
            self.layers.append((ws, bs))

    def case(self, batch, steps, warmup):
        import torch
        from izwi_b200 import ops, parallel
        world, rank, d, ff = self.world, self.rank, self.d, self.ff
        lo_b, hi_b = parallel.batch_split(batch, world, rank)
        m = (hi_b - lo_b) * self.frames
        gen = torch.Generator(device=self.device).manual_seed(500 + batch)
        x_all = torch.randn(batch * self.frames, d, device=self.device, generator=gen).to(torch.bfloat16)
        x = x_all[lo_b * self.frames: hi_b * self.frames].contiguous() if m else x_all[:1]
        mk = lambda n: torch.empty(max(m, 1), n, device=self.device, dtype=torch.bfloat16)  # noqa: E731
        bufs = {"qkv": mk(3 * d), "o": mk(d), "ff": mk(ff), "d": mk(d)}

        def layer_forward(ws, bs):
            ops.linear(x, ws["qkv"], bias=bs["qkv"], out=bufs["qkv"])
            ops.linear(x, ws["o"], bias=bs["o"], out=bufs["o"])
            for _ in range(self.n_ffn):
                ops.linear(x, ws["fc1"], bias=bs["fc1"], out=bufs["ff"], epilogue=self.act)
                ops.linear(bufs["ff"], ws["fc2"], bias=bs["fc2"], out=bufs["d"])

        def step():
            if m:
                for ws, bs in self.layers:
                    layer_forward(ws, bs)
        # a pass is a fixed sequence of a hundred or more launches, short ones when the batch is split
        # eight ways: captured once, replayed as a CUDA graph
        per_ms, launches = _timed_case(step, steps, warmup, world, self.device.index, graph=m > 0)
        flops = 2.0 * batch * self.frames * self.n_layers * (4 * d * d + self.n_ffn * 2 * d * ff)
        out = {"value": round(batch / (per_ms * 1e-3), 2), "unit": "utterances/s", "ms_per_step": round(per_ms, 5),
               "n_gpus": world, "scaling": "strong", "launches_per_step": launches, "batch": batch, "frames": self.frames,
               "tflops_total": round(flops / (per_ms * 1e-3) / 1e12, 2), "collective": "none (independent utterances)",
               "launch": "CUDA graph replay of the whole pass",
               "parallelism": f"batch split over {world} ranks, weights replicated"}
        if rank == 0 and m:
            ws, bs = self.layers[0]
            layer_forward(ws, bs)
            torch.cuda.synchronize()
            rows = sampled_rows(m)
            par = Parity()
            par.add(host64(bufs["qkv"][rows]), linear_rows_ref(x, ws["qkv"], bs["qkv"], rows))
            par.add(host64(bufs["o"][rows]), linear_rows_ref(x, ws["o"], bs["o"], rows))
            hid = bf16_round_np(linear_rows_ref(x, ws["fc1"], bs["fc1"], rows, self.act))
            par.add(host64(bufs["ff"][rows]), hid)
            want = hid @ host64(ws["fc2"]).T + (0 if bs["fc2"] is None else host64(bs["fc2"])[None, :])
            par.add(host64(bufs["d"][rows]), want)
            out["parity"] = par.result(f"layer 0, {len(rows)} sampled frames: QKV, O, FFN1 + activation, FFN2 vs float64 on the host")
        return out


def run_sharded_cases(names, world, rank, device, comm, steps=None, warmup=3, nccl_ep=False, use_graph=True):
    """Runs the named sharded workloads in this process group, sharing the weights of one model between
    its cases.  Returns the list of result dicts (parity fields filled on rank 0)."""
    import torch
    out = []
    kinds = [SHARDED[n][0] for n in names]
    if "tp" in kinds:
        tp = TpStack(comm, world, rank, device, use_graph=use_graph)
        for n in names:
            if SHARDED[n][0] == "tp":
                m = SHARDED[n][1]
                out.append({"workload": n, **tp.case(m, steps or (10 if m > 32 else 20), warmup)})
        del tp
        torch.cuda.empty_cache()
    if "ep" in kinds:
        ep = EpStack(comm, world, rank, device, max_tokens=max(SHARDED[n][1] for n in names if SHARDED[n][0] == "ep"),
                     nccl=nccl_ep)
        for n in names:
            if SHARDED[n][0] == "ep":
                out.append({"workload": n, **ep.case(SHARDED[n][1], steps or 20, warmup)})
        del ep
        torch.cuda.empty_cache()
    for n in names:
        if SHARDED[n][0] in ENCODERS:
            enc = EncStack(SHARDED[n][0], world, rank, device)
            out.append({"workload": n, **enc.case(SHARDED[n][1], steps or 10, warmup)})
            del enc
            torch.cuda.empty_cache()
    order = {n: i for i, n in enumerate(names)}
    return sorted(out, key=lambda c: order[c["workload"]])


def make_comm(world, local):
    """The communicator of the sharded workloads: NCCL for set-up and fallback, sums through NVLink peer
    memory (one-shot up to 1 MB, two-shot up to 64 MB)."""
    if world == 1:
        return None
    from izwi_b200 import parallel
    comm = parallel.Comm(local)
    comm.enable_peer_allreduce(64 << 20)
    return comm


def headline_config(workload, fmt, m, layers, weight_bytes, world):
    return {"workload": workload, "weights": fmt, "tokens_per_step": m, "layers": layers, "projections_per_layer": 4,
            "weight_bytes": weight_bytes, "launch": "one grouped persistent launch per step",
            "l2": f"inputs larger than L2 ({weight_bytes / 1e6:.0f} MB streamed per step vs 126 MB)",
            "multi_gpu": "replicas only (the 0.6B decode stack does not shard)" if world > 1 else "single GPU"}


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
    block_ms, blocks, t0, t1 = time_blocks(group.launch, args.steps, world, args.min_ms)
    launches = (ctx.launch_count - launches0) // len(blocks)
    sampler.stop_flag.set()
    sampler.join(timeout=2)
    ctx.check()  # raises if any bounded device-side wait gave up

    per_ms = block_ms / args.steps
    tokens_per_s = world * m / (per_ms * 1e-3)
    achieved = stack.algorithmic_bytes / (per_ms * 1e-3) / 1e9

    # ---- end to end through the C ABI: host activations in, host results out, every step ----
    h_in = torch.empty_like(stack.acts_buf, device="cpu").pin_memory()
    h_in.copy_(stack.acts_buf)
    h_out = torch.empty_like(stack.outs_buf, device="cpu").pin_memory()
    host_group = wl.stack_group(stack, host_outs=h_out)  # the same problems, their y pointers in page-locked host memory

    def e2e_step():
        # one C-ABI call: host activations -> device, the launch (which stores every result straight into host
        # memory), and the wait for it: the caller reads the result before the next token
        host_group.launch_host(h_in, stack.acts_buf)

    e2e_steps = max(3, min(args.steps, 2000))
    for _ in range(3):
        e2e_step()
    e2e_block, e2e_blocks, _, _ = time_blocks(e2e_step, e2e_steps, world, args.min_ms / 2)
    e2e_tokens = world * m / (e2e_block / e2e_steps * 1e-3)
    ctx.check()
    e2e_match = bool(torch.equal(h_out, stack.outs_buf.cpu()))  # the host copy of the results against the device-resident run

    line = {
        "metric": METRIC, "value": round(tokens_per_s, 2), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(per_ms, 6),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": headline_config(args.workload, fmt, m, stack.shape.layers, stack.weight_bytes, world),
        "timing": {"what": f"median of {len(blocks)} blocks of exactly {args.steps} steps each (CUDA events, barrier and "
                           "synchronise around every block, max over ranks), repeated until the blocks add up to "
                           f"{args.min_ms:.0f} ms of device time",
                   "blocks": len(blocks), "block_ms_min": round(min(blocks), 5), "block_ms_median": round(block_ms, 5),
                   "block_ms_max": round(max(blocks), 5), "timed_ms_total": round(sum(blocks), 3)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "peak_kind": f"of {peak_kind}",
                     "frac_of_nominal_8000": round(achieved / 8000.0, 4),
                     "algorithmic_bytes_per_launch": stack.algorithmic_bytes,
                     "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(args.workload)},
        "e2e": {"value": round(e2e_tokens, 2), "unit": "tokens/s",
                "h2d_bytes_per_step": h_in.numel() * 2, "d2h_bytes_per_step": h_out.numel() * 2,
                "steps": e2e_steps, "blocks": len(e2e_blocks),
                "call": "izb_linear_group_launch_host: copy of the step's activations from page-locked host memory, the "
                        "launch, results stored by the kernel into page-locked host memory, stream wait",
                "results_match_device_run": e2e_match},
        "gpu_launches": int(launches),
        "clocks": sampler.summary(t0, t1),
    }

    if rank == 0 and not args.no_cpu_baseline:
        # parity of the timed path against the checker, on the spot, over every projection of the step
        cpu = CpuStack(stack)
        line["parity"] = cpu.parity().result(f"all {len(cpu.items)} projections of the step vs CPU port")
        if world == 1:
            n, dt = cpu.timed(args.cpu_seconds)
            line["cpu_baseline"] = {"value": round(n * m / dt, 3), "unit": "tokens/s", "cores": cpu.cores,
                                    "kind": "port",
                                    "sample": f"{n} full decode steps of the same stack (dequantise + fp32 dot, "
                                              f"OpenMP over weight rows), {dt:.1f} s"}
        del cpu
    del group, stack, h_in, h_out
    torch.cuda.empty_cache()
    if not args.no_sharded:
        # the configurations that do shard, at this world size, in the same process group
        comm = make_comm(world, local)
        line["sharded_cases"] = run_sharded_cases(SHARDED_DEFAULT, world, rank, device, comm)
        if comm is not None:
            comm.close()
    if rank == 0 and world == 1 and not args.no_cases:
        cases = []
        for wname in WORKLOADS:
            if wname == args.workload:
                continue
            cases.append(measure_case(wname, device, args.case_steps, 5, peak, check=not args.no_cpu_baseline))
        line["cases"] = cases
        line["gemm_cases"] = measure_gemm_cases(device)
        line["moe_cases"] = measure_moe_cases(device)
        line["attention_cases"] = measure_attention_cases(device)
        line["decode_token_cases"] = measure_decode_token_cases(device)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


def run_sharded(args):
    """One sharded workload on its own (`--workload <name> --gpus N` under torch.distributed.run)."""
    import torch
    from izwi_b200 import ops
    world, rank, local = dist_setup(args.gpus)
    device = torch.device("cuda", local)
    comm = make_comm(world, local)
    sampler = ClockSampler(local)
    sampler.start()
    t0 = time.perf_counter()
    case = run_sharded_cases([args.workload], world, rank, device, comm, steps=args.steps, warmup=args.warmup,
                             nccl_ep=args.nccl_ep, use_graph=not args.no_graph)[0]
    t1 = time.perf_counter()
    sampler.stop_flag.set()
    sampler.join(timeout=2)
    peak_tf, _ = load_tensor_peak()
    unit = case["unit"]
    line = {"metric": f"{args.workload}_{unit.split('/')[0]}_per_s", "value": case["value"], "unit": unit, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": case["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "l2": "weights larger than L2", "parallelism": case["parallelism"],
                       "collective": case["collective"]},
            "tflops_total": case["tflops_total"],
            "tensor_frac_per_gpu": round(case["tflops_total"] / world / peak_tf, 4),
            "gpu_launches": case["launches_per_step"] * args.steps, "parity": case.get("parity"),
            "clocks": sampler.summary(t0, t1)}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        comm.close()
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args):
    """The reference arm: the CPU restatement of the same stack on all the host cores this process may
    use (the reference's own Candle CPU path cannot be built without a Rust toolchain).  Under a
    multi-rank launch rank 0 alone runs it; the other ranks exit."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    dev = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    fmt, m = WORKLOADS[args.workload]
    stack = make_stack(args.workload, dev)
    cpu = CpuStack(stack)
    weight_bytes, layers = stack.weight_bytes, stack.shape.layers
    del stack
    warmup = max(3, min(args.warmup, 200))
    for _ in range(warmup):
        cpu.step()
    steps = max(1, min(args.steps, 50))  # each step is a full CPU decode step; bounded so the run ends in minutes
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu.step()
    dt = time.perf_counter() - t0
    v = round(steps * m / dt, 3)
    sample = f"{steps} full decode steps of the stack on {cpu.cores} host threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": round(dt / steps * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": headline_config(args.workload, fmt, m, layers, weight_bytes, args.gpus),
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
    ap.add_argument("--no-sharded", action="store_true", help="skip the sharded_cases block of the default run")
    ap.add_argument("--min-ms", type=float, default=500.0,
                    help="repeat the timed block of --steps steps until this much device time has been measured")
    ap.add_argument("--nccl-ep", action="store_true", help="expert-parallel workloads: exchange rows with NCCL instead of peer memory")
    ap.add_argument("--no-graph", action="store_true", help="sharded decode workloads: launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--attention-cases", action="store_true",
                    help="profiler captures: run only the decode-attention cases and exit")
    ap.add_argument("--decode-token-cases", action="store_true",
                    help="only the whole-greedy-token cases (eager steps, then a CUDA graph replayed)")
    ap.add_argument("--gemm-case", default=None,
                    help="profiler captures: run only this prefill / encoder GEMM shape (a name from gemm_cases) and exit")
    ap.add_argument("--moe-case", default=None,
                    help="profiler captures: run only a reduced MoE layer, given as EXPERTS,TOKENS (e.g. 16,512), and exit")
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
    if args.moe_case:
        import torch
        e, t = (int(v) for v in args.moe_case.split(","))
        print(json.dumps({"moe_case": measure_moe_profile_case(torch.device("cuda", 0), e, t, max(1, min(args.steps, 5)))}), flush=True)
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
