"""Host-side wrapper of the top-k mixture-of-experts entry points (izb_moe_*).  Torch tensors are
device buffers only; every step runs in libizwi_b200.so."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L
from .ops import EPILOGUE, Context, _ptr, _stream


def topk(logits: torch.Tensor, k: int):
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous()
    t, e = logits.shape
    idx = torch.empty(t, k, device=logits.device, dtype=torch.int32)
    wts = torch.empty(t, k, device=logits.device, dtype=torch.float32)
    ctx = Context.get(logits.device.index)
    L.check(L.lib().izb_moe_topk(ctx.handle, _stream(), _ptr(logits), t, e, k, _ptr(idx), _ptr(wts)), "izb_moe_topk")
    return idx, wts


def route(x: torch.Tensor, w_router: torch.Tensor, router_bias: torch.Tensor | None, k: int):
    """Router logits and expert choice in one launch: (logits [T, E] fp32, idx [T, k] int32, weights [T, k] fp32)."""
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    assert w_router.dtype == torch.bfloat16 and w_router.is_contiguous() and w_router.shape[1] == x.shape[1]
    t, (e, h) = x.shape[0], w_router.shape
    logits = torch.empty(t, e, device=x.device, dtype=torch.float32)
    idx = torch.empty(t, k, device=x.device, dtype=torch.int32)
    wts = torch.empty(t, k, device=x.device, dtype=torch.float32)
    ctx = Context.get(x.device.index)
    L.check(L.lib().izb_moe_route(ctx.handle, _stream(), _ptr(x), x.stride(0), _ptr(w_router), _ptr(router_bias), t, h, e, k,
                                  _ptr(logits), _ptr(idx), _ptr(wts)), "izb_moe_route")
    return logits, idx, wts


def permute(idx: torch.Tensor, n_experts: int):
    assert idx.dtype == torch.int32 and idx.is_contiguous()
    pairs = idx.numel()
    dev = idx.device
    offsets = torch.empty(n_experts + 1, device=dev, dtype=torch.int32)
    perm = torch.empty(pairs, device=dev, dtype=torch.int32)
    inv = torch.empty(pairs, device=dev, dtype=torch.int32)
    ctx = Context.get(dev.index)
    L.check(L.lib().izb_moe_permute(ctx.handle, _stream(), _ptr(idx), pairs, n_experts, _ptr(offsets), _ptr(perm),
                                    _ptr(inv)), "izb_moe_permute")
    return offsets, perm, inv


def gather(x: torch.Tensor, perm: torch.Tensor, k: int) -> torch.Tensor:
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    out = torch.empty(perm.numel(), x.shape[1], device=x.device, dtype=torch.bfloat16)
    ctx = Context.get(x.device.index)
    L.check(L.lib().izb_moe_gather(ctx.handle, _stream(), _ptr(x), x.stride(0), _ptr(perm), k, perm.numel(), x.shape[1],
                                   _ptr(out)), "izb_moe_gather")
    return out


def grouped_gemm(x_perm: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, epilogue: str | None = None,
                 out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    assert x_perm.dtype == torch.bfloat16 and x_perm.is_contiguous() and w.dtype == torch.bfloat16 and w.is_contiguous()
    e, n, k = w.shape
    rows = x_perm.shape[0]
    n_out = n // 2 if epilogue == "swiglu" else n
    y = torch.zeros(rows, n_out, device=x_perm.device, dtype=out_dtype)
    ctx = Context.get(x_perm.device.index)
    L.check(L.lib().izb_moe_grouped_gemm(ctx.handle, _stream(), _ptr(x_perm), _ptr(w), _ptr(offsets), _ptr(y),
                                         L.IZB_F32 if out_dtype == torch.float32 else L.IZB_BF16, rows, n, k, e,
                                         EPILOGUE[epilogue]), "izb_moe_grouped_gemm")
    return y


def combine(y_perm: torch.Tensor, inv: torch.Tensor, wts: torch.Tensor) -> torch.Tensor:
    t, k = wts.shape
    h = y_perm.shape[1]
    y = torch.empty(t, h, device=y_perm.device, dtype=torch.bfloat16)
    ctx = Context.get(y_perm.device.index)
    L.check(L.lib().izb_moe_combine(ctx.handle, _stream(), _ptr(y_perm), _ptr(inv), _ptr(wts), t, k, h, _ptr(y)),
            "izb_moe_combine")
    return y


class MoeLayer:
    """One MoE feed-forward layer: router [E, H] (+ bias), gate/up [E, 2I, H], down [E, H, I]."""

    def __init__(self, w_router, router_bias, w_gate_up, w_down, top_k: int):
        self.w_router, self.router_bias = w_router.contiguous(), router_bias
        self.w_gate_up, self.w_down = w_gate_up.contiguous(), w_down.contiguous()
        self.E, two_i, self.H = w_gate_up.shape
        self.I = two_i // 2
        self.top_k = top_k
        self._ws = None

    def forward(self, x: torch.Tensor):
        """Returns (y [T, H] bf16, logits [T, E] fp32, idx [T, k] int32, weights [T, k] fp32)."""
        assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()
        t = x.shape[0]
        lib = L.lib()
        need = lib.izb_moe_workspace_bytes(t, self.H, self.I, self.E, self.top_k)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, device=x.device, dtype=torch.uint8)
        y = torch.empty(t, self.H, device=x.device, dtype=torch.bfloat16)
        a = L.MoeArgs()
        a.x, a.w_router, a.router_bias = x.data_ptr(), self.w_router.data_ptr(), (
            0 if self.router_bias is None else self.router_bias.data_ptr())
        a.w_gate_up, a.w_down, a.y = self.w_gate_up.data_ptr(), self.w_down.data_ptr(), y.data_ptr()
        a.T, a.H, a.I, a.E, a.top_k = t, self.H, self.I, self.E, self.top_k
        a.workspace, a.workspace_bytes = self._ws.data_ptr(), self._ws.numel()
        ctx = Context.get(x.device.index)
        L.check(lib.izb_moe_forward(ctx.handle, _stream(), C.byref(a)), "izb_moe_forward")
        al = lambda v: (v + 255) // 256 * 256  # noqa: E731
        o_logits = 0
        o_idx = al(t * self.E * 4)
        o_wts = o_idx + al(t * self.top_k * 4)
        logits = self._ws[o_logits: o_logits + t * self.E * 4].view(torch.float32).view(t, self.E)
        idx = self._ws[o_idx: o_idx + t * self.top_k * 4].view(torch.int32).view(t, self.top_k)
        wts = self._ws[o_wts: o_wts + t * self.top_k * 4].view(torch.float32).view(t, self.top_k)
        return y, logits, idx, wts
