"""Seeded synthetic workloads shaped after the model families the hot path
serves.  No real weights, audio or prompts: every tensor is drawn from a seeded
generator with the layer dimensions and value distributions of the named model.

Weights are generated on the device (torch CUDA generator) so multi-gigabyte
stacks appear in seconds; anything a CPU checker needs is copied back.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .ops import BLOCK_SIZE, TYPE_SIZE


@dataclass(frozen=True)
class DecoderShape:
    name: str
    layers: int
    hidden: int
    q_heads: int
    kv_heads: int
    head_dim: int
    intermediate: int

    @property
    def projections(self) -> list[tuple[str, int, int]]:
        """(name, N = out, K = in) of the four projections of one layer."""
        qkv = (self.q_heads + 2 * self.kv_heads) * self.head_dim
        return [
            ("qkv", qkv, self.hidden),
            ("o", self.hidden, self.q_heads * self.head_dim),
            ("gate_up", 2 * self.intermediate, self.hidden),
            ("down", self.hidden, self.intermediate),
        ]

    @property
    def weights_per_layer(self) -> int:
        return sum(n * k for _, n, k in self.projections)


QWEN3_0_6B = DecoderShape("qwen3-0.6b", 28, 1024, 16, 8, 128, 3072)
QWEN3_8B = DecoderShape("qwen3-8b", 36, 4096, 32, 8, 128, 12288)


def weight_bytes(fmt: str, n: int, k: int) -> int:
    return n * k // BLOCK_SIZE[fmt] * TYPE_SIZE[fmt]


def make_bf16_weight(n: int, k: int, gen: torch.Generator, std: float = 0.02) -> torch.Tensor:
    return (torch.randn(n, k, device=gen.device, generator=gen, dtype=torch.float32) * std).to(torch.bfloat16)


def make_q8_0_weight(n: int, k: int, gen: torch.Generator, d_std: float = 0.002) -> torch.Tensor:
    """N rows of K/32 Q8_0 blocks: int8 codes uniform in [-127, 127], one fp16
    scale per block ~ |N(0, d_std)|.  Returned as raw bytes [N, K/32*34]."""
    nb = n * k // 32
    dev = gen.device
    d = (torch.randn(nb, device=dev, generator=gen) * d_std).abs().to(torch.float16)
    q = torch.randint(-127, 128, (nb, 32), device=dev, generator=gen, dtype=torch.int8)
    raw = torch.empty(nb, 34, device=dev, dtype=torch.uint8)
    raw[:, 0:2] = d.view(torch.uint8).reshape(nb, 2)
    raw[:, 2:] = q.view(torch.uint8)
    return raw.reshape(n, k // 32 * 34)


def make_q4_k_weight(n: int, k: int, gen: torch.Generator, d_std: float = 1e-4,
                     dmin_std: float = 7.5e-4) -> torch.Tensor:
    """N rows of K/256 Q4_K super-blocks built field by field: uniform 4-bit
    codes, uniform 6-bit sub-block scales and mins, fp16 d ~ |N(0, d_std)| and
    dmin ~ |N(0, dmin_std)|.  dmin_std = 7.5 * d_std centres the dequantised
    weights near zero (mean code 7.5) with a spread close to N(0, 0.02), so
    outputs stay O(1) like the dense stack's.  Raw bytes [N, K/256*144]."""
    nb = n * k // 256
    dev = gen.device
    raw = torch.empty(nb, 144, device=dev, dtype=torch.uint8)
    d = (torch.randn(nb, device=dev, generator=gen) * d_std).abs().to(torch.float16)
    dmin = (torch.randn(nb, device=dev, generator=gen) * dmin_std).abs().to(torch.float16)
    raw[:, 0:2] = d.view(torch.uint8).reshape(nb, 2)
    raw[:, 2:4] = dmin.view(torch.uint8).reshape(nb, 2)
    sc = torch.randint(0, 64, (nb, 8), device=dev, generator=gen, dtype=torch.uint8)
    mn = torch.randint(0, 64, (nb, 8), device=dev, generator=gen, dtype=torch.uint8)
    raw[:, 4:8] = (sc[:, 0:4] & 0x3F) | ((sc[:, 4:8] >> 4) << 6)
    raw[:, 8:12] = (mn[:, 0:4] & 0x3F) | ((mn[:, 4:8] >> 4) << 6)
    raw[:, 12:16] = (sc[:, 4:8] & 0x0F) | ((mn[:, 4:8] & 0x0F) << 4)
    raw[:, 16:] = torch.randint(0, 256, (nb, 128), device=dev, generator=gen, dtype=torch.uint8)
    return raw.reshape(n, k // 256 * 144)


def make_weight(fmt: str, n: int, k: int, gen: torch.Generator) -> torch.Tensor:
    if fmt == "bf16":
        return make_bf16_weight(n, k, gen)
    if fmt == "q8_0":
        return make_q8_0_weight(n, k, gen)
    if fmt == "q4_k":
        return make_q4_k_weight(n, k, gen)
    raise ValueError(fmt)


@dataclass
class LinearStack:
    """The linear stack of a decoder: four projections per layer, each with its
    own seeded activation matrix [M, K] (attention and norms are not part of
    this workload, so the projections of a step do not depend on one another)."""
    shape: DecoderShape
    fmt: str
    m: int
    weights: list  # [layer][proj] device tensors
    acts: list     # [layer][proj] bf16 [M, K], views into acts_buf
    outs: list     # [layer][proj] bf16 [M, N], views into outs_buf
    acts_buf: torch.Tensor = None  # all activations of a step, one contiguous buffer
    outs_buf: torch.Tensor = None  # all outputs of a step, one contiguous buffer

    @property
    def weight_bytes(self) -> int:
        return self.shape.layers * sum(weight_bytes(self.fmt, n, k) for _, n, k in self.shape.projections)

    @property
    def algorithmic_bytes(self) -> int:
        """Bytes one step must move: every weight once, activations in, outputs out."""
        io = sum(self.m * k * 2 + self.m * n * 2 for _, n, k in self.shape.projections)
        return self.weight_bytes + self.shape.layers * io

    @property
    def flops(self) -> int:
        return 2 * self.m * self.shape.layers * self.shape.weights_per_layer


def make_linear_stack(shape: DecoderShape, fmt: str, m: int, device: torch.device, weight_seed: int,
                      act_seed: int, layers: int | None = None) -> LinearStack:
    if layers is not None:
        shape = DecoderShape(shape.name, layers, shape.hidden, shape.q_heads, shape.kv_heads, shape.head_dim,
                             shape.intermediate)
    wgen = torch.Generator(device=device).manual_seed(weight_seed)
    agen = torch.Generator(device=device).manual_seed(act_seed)
    per_layer_in = sum(m * k for _, _, k in shape.projections)
    per_layer_out = sum(m * n for _, n, _ in shape.projections)
    acts_buf = torch.randn(shape.layers * per_layer_in, device=device, generator=agen,
                           dtype=torch.float32).to(torch.bfloat16)
    outs_buf = torch.zeros(shape.layers * per_layer_out, device=device, dtype=torch.bfloat16)
    weights, acts, outs = [], [], []
    ai = oi = 0
    for _ in range(shape.layers):
        wl, al, ol = [], [], []
        for _, n, k in shape.projections:
            wl.append(make_weight(fmt, n, k, wgen))
            al.append(acts_buf[ai: ai + m * k].view(m, k))
            ol.append(outs_buf[oi: oi + m * n].view(m, n))
            ai += m * k
            oi += m * n
        weights.append(wl)
        acts.append(al)
        outs.append(ol)
    return LinearStack(shape, fmt, m, weights, acts, outs, acts_buf, outs_buf)


def stack_group(stack: LinearStack, host_outs: torch.Tensor | None = None):
    """All projections of the stack as one grouped persistent launch.  `host_outs`: a page-locked host tensor shaped
    like `stack.outs_buf`; the launch then stores every result straight into it (no copy back afterwards)."""
    from . import ops
    import ctypes as C
    from . import _lib as L
    probs, scratch = [], []
    if host_outs is not None:
        assert host_outs.is_pinned() and host_outs.shape == stack.outs_buf.shape and host_outs.dtype == stack.outs_buf.dtype
    for wl, al, ol in zip(stack.weights, stack.acts, stack.outs):
        for (_, n, k), w, x, y in zip(stack.shape.projections, wl, al, ol):
            if host_outs is not None:
                at = (y.data_ptr() - stack.outs_buf.data_ptr()) // y.element_size()
                y = host_outs[at:at + y.numel()].view(y.shape)
            a = ops.linear_args(x, w, stack.fmt, n, k, y)
            need = L.lib().izb_linear_workspace_bytes_args(C.byref(a))
            if need:  # 3..16 tokens over block formats: room for the activations as the integer kernel reads them
                scratch.append(torch.empty(need, device=x.device, dtype=torch.uint8))
                a = ops.linear_args(x, w, stack.fmt, n, k, y, workspace=scratch[-1])
            probs.append(a)
    return ops.LinearGroup(probs, stack.acts_buf.device, keepalive=(stack, scratch, host_outs))
