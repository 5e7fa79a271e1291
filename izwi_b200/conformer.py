"""Host-side mirror of the convolution module of a Conformer encoder layer over the C ABI:
`ConformerConv` of crates/izwi-core/src/models/architectures/parakeet/asr/mod.rs:775-864.

    x [B, T, C] -> pointwise_conv1 (C -> 2C, 1x1, no bias) -> a * sigmoid(b)
               -> depthwise conv (kernel 9, same padding) with the batch norm folded in -> swish
               -> pointwise_conv2 (C -> C)

The pointwise convolutions are linear layers over the [B*T, C] rows (the first with the gated epilogue);
the depthwise convolution, folded bias and swish are one launch.  Activations never leave the
[B*T, C] layout, so the reference's transposes to [B, C, T] and back have no counterpart here.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L
from . import ops
from .ops import Context, _ptr, _stream


def fold_depthwise_conv1d_batch_norm(conv_weight: torch.Tensor, bn_weight, bn_bias, running_mean: torch.Tensor,
                                     running_var: torch.Tensor, eps: float):
    """`fold_depthwise_conv1d_batch_norm` (parakeet/asr/mod.rs:866-893): fp32 [C, 1, k] or [C, k] depthwise weight and the
    batch norm's statistics -> (folded weight bf16 [C, k], folded bias bf16 [C])."""
    w = conv_weight.reshape(conv_weight.shape[0], -1).float().contiguous()
    ch, k = w.shape
    f32 = lambda t: None if t is None else t.float().contiguous()  # noqa: E731
    g, b, m, v = f32(bn_weight), f32(bn_bias), f32(running_mean), f32(running_var)
    fw = torch.empty(ch, k, device=w.device, dtype=torch.bfloat16)
    fb = torch.empty(ch, device=w.device, dtype=torch.bfloat16)
    ctx = Context.get(w.device.index)
    L.check(L.lib().izb_fold_depthwise_conv1d_batch_norm(ctx.handle, _stream(), _ptr(w), _ptr(g), _ptr(b), _ptr(m), _ptr(v),
                                                         float(eps), ch, k, _ptr(fw), _ptr(fb)),
            "izb_fold_depthwise_conv1d_batch_norm")
    return fw, fb


def depthwise_conv1d_bias_swish(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, swish: bool = True) -> torch.Tensor:
    """x [B, T, C] bf16 (channels contiguous), weight [C, k] bf16, bias [C] bf16 -> [B, T, C]."""
    assert x.dtype == torch.bfloat16 and x.dim() == 3 and x.is_contiguous() and weight.dtype == torch.bfloat16 and weight.is_contiguous()
    b, t, ch = x.shape
    k = weight.shape[1]
    out = torch.empty_like(x)
    ctx = Context.get(x.device.index)
    L.check(L.lib().izb_depthwise_conv1d_bias_swish(ctx.handle, _stream(), _ptr(x), _ptr(weight), _ptr(bias), _ptr(out), b, t, ch, k,
                                                    (k - 1) // 2, ch, ch, 1 if swish else 0), "izb_depthwise_conv1d_bias_swish")
    return out


class ConformerConv:
    """Weights as the reference loads them: pointwise_conv1 [2C, C], the depthwise weight [C, k] with its batch
    norm (folded once, here), pointwise_conv2 [C, C]; all projections bf16, no biases."""

    def __init__(self, pointwise_conv1: torch.Tensor, depthwise_weight: torch.Tensor, bn_weight, bn_bias, running_mean,
                 running_var, bn_eps: float, pointwise_conv2: torch.Tensor):
        self.pointwise_conv1 = pointwise_conv1.contiguous()
        self.pointwise_conv2 = pointwise_conv2.contiguous()
        self.folded_depthwise_weight, self.folded_depthwise_bias = fold_depthwise_conv1d_batch_norm(
            depthwise_weight, bn_weight, bn_bias, running_mean, running_var, bn_eps)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, t, ch = x.shape
        gated = ops.linear(x.reshape(b * t, ch), self.pointwise_conv1, epilogue="glu")          # a * sigmoid(b)
        conv = depthwise_conv1d_bias_swish(gated.reshape(b, t, ch), self.folded_depthwise_weight, self.folded_depthwise_bias)
        return ops.linear(conv.reshape(b * t, ch), self.pointwise_conv2).reshape(b, t, ch)
