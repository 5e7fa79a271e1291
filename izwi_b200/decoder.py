"""One decode token through a Qwen3 decoder layer, assembled from the C-ABI entry points: the
host-side mirror of `Qwen3DecoderLayer::forward` / `Qwen3Attention::forward` for seq_len = 1
(crates/izwi-core/src/models/architectures/qwen3/core.rs:1863-1881, 1624-1732).

    normed = input_layernorm(x)                        izb_rms_norm (+ the previous layer's residual add)
    qkv    = qkv_proj(normed)                          izb_linear (fused QKV)
    q, k   = q_norm(q), k_norm(k); rope(q, k)          izb_rms_norm on head rows, izb_rope_pair
    cache  <- k, v                                     izb_kv_append
    attn   = softmax(q k^T / sqrt(d)) v                izb_decode_gqa_attention
    x      = x + o_proj(attn)                          izb_linear; the add is fused into the next norm
    normed = post_attention_layernorm(x)               izb_rms_norm with residual
    x      = x + down(silu(gate) * up)                 izb_linear, izb_silu_mul, izb_linear; add deferred likewise

For one or two tokens over block-quantised weights the norms, the silu-mul and both residual adds ride
inside the projections (`fused_linear`): six launches per layer instead of ten.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import ops


@dataclass
class Qwen3LayerWeights:
    fmt: str                      # "bf16" | "q8_0" | "q4_k": storage of the four projections
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    intermediate: int
    input_layernorm: torch.Tensor            # [hidden] bf16
    post_attention_layernorm: torch.Tensor   # [hidden] bf16
    q_norm: torch.Tensor | None              # [head_dim] bf16
    k_norm: torch.Tensor | None
    qkv: torch.Tensor             # rows: q heads, k heads, v heads (fused at load, core.rs:931-981)
    o: torch.Tensor
    gate_up: torch.Tensor         # rows: gate then up (core.rs:1132-1168)
    down: torch.Tensor
    eps: float = 1e-6


class KvCache:
    """Head-major cache of one layer: [batch, kv_heads, capacity, head_dim] for k and v."""

    def __init__(self, batch: int, kv_heads: int, capacity: int, head_dim: int, device):
        self.k = torch.zeros(batch, kv_heads, capacity, head_dim, device=device, dtype=torch.bfloat16)
        self.v = torch.zeros_like(self.k)
        self.capacity = capacity


class Qwen3DecoderLayer:
    def __init__(self, w: Qwen3LayerWeights, fused_qk: bool = True, fused_linear: bool = True):
        self.w = w
        self.fused_qk = fused_qk and w.head_dim in (64, 128)
        self.fused_linear = fused_linear
        self.fusion_max_tokens = ops.linear_fusion_max_tokens(w.fmt) if fused_linear else 0

    def forward(self, attn_in: torch.Tensor, residual: torch.Tensor | None, cos_half: torch.Tensor,
                sin_half: torch.Tensor, cache: KvCache, pos: int):
        """attn_in [batch, hidden]: the layer input, or the previous layer's MLP output when `residual`
        (the previous layer's pre-MLP stream) is given; returns (mlp_out, stream) so that the caller's
        next norm performs `stream + mlp_out`; with the projections fusing the adds, (stream, None).
        cos_half / sin_half [batch, head_dim / 2] for position `pos`."""
        w = self.w
        b = attn_in.shape[0]
        qd, kd = w.heads * w.head_dim, w.kv_heads * w.head_dim
        fuse = b <= self.fusion_max_tokens
        if residual is None and fuse:
            x = attn_in
            qkv = ops.linear(x, w.qkv, w.fmt, n=qd + 2 * kd, k=w.hidden, prologue="rms_norm",
                             norm_weight=w.input_layernorm, norm_eps=w.eps)
        else:
            if residual is None:
                x = attn_in
                normed = ops.rms_norm(x, w.input_layernorm, w.eps)
            else:
                normed, x = ops.rms_norm(attn_in, w.input_layernorm, w.eps, residual=residual, return_sum=True)
            qkv = ops.linear(normed, w.qkv, w.fmt, n=qd + 2 * kd, k=w.hidden)
        if self.fused_qk:
            # q/k norms, rotation and cache append in one launch, reading the fused QKV output in place
            q = ops.qk_norm_rope_append(qkv, w.q_norm, w.k_norm, w.eps, cos_half, sin_half, cache.k, cache.v, w.heads, pos)
        else:
            q = qkv[:, :qd].reshape(b, w.heads, w.head_dim)       # views of the fused output (narrow, core.rs:975-981)
            k = qkv[:, qd:qd + kd].reshape(b, w.kv_heads, w.head_dim)
            v = qkv[:, qd + kd:].reshape(b, w.kv_heads, w.head_dim)
            if w.q_norm is not None:
                q = ops.rms_norm(q, w.q_norm, w.eps)
                k = ops.rms_norm(k, w.k_norm, w.eps)
            else:
                q, k = q.contiguous(), k.contiguous()
            ops.rope_pair_(q, k, cos_half, sin_half)
            ops.kv_append_(k, v, cache.k, cache.v, pos)
        attn = ops.decode_gqa_attention(q, cache.k, cache.v, pos + 1)
        if fuse:
            x = ops.linear(attn.reshape(b, qd), w.o, w.fmt, n=w.hidden, k=qd, residual=x)
            gu = ops.linear(x, w.gate_up, w.fmt, n=2 * w.intermediate, k=w.hidden, prologue="rms_norm",
                            norm_weight=w.post_attention_layernorm, norm_eps=w.eps)
            return ops.linear(gu, w.down, w.fmt, n=w.hidden, k=w.intermediate, prologue="silu_mul", residual=x), None
        o = ops.linear(attn.reshape(b, qd), w.o, w.fmt, n=w.hidden, k=qd)
        normed2, x = ops.rms_norm(o, w.post_attention_layernorm, w.eps, residual=x, return_sum=True)
        gu = ops.linear(normed2, w.gate_up, w.fmt, n=2 * w.intermediate, k=w.hidden)
        act = ops.silu_mul(gu[:, :w.intermediate], gu[:, w.intermediate:])
        mlp_out = ops.linear(act, w.down, w.fmt, n=w.hidden, k=w.intermediate)
        return mlp_out, x


class Qwen3Decoder:
    """Embedding, decoder layers, final norm, lm_head and greedy choice for one token per sequence:
    the device side of `Qwen3Model::forward` + `argmax` for seq_len = 1
    (qwen3/core.rs:2099-2125, qwen3/chat.rs:574-601)."""

    def __init__(self, embed: torch.Tensor, layers: list, final_norm: torch.Tensor, lm_head: torch.Tensor, lm_head_fmt: str,
                 rope_theta: float = 1e6):
        self.embed, self.layers, self.final_norm = embed, layers, final_norm
        self.lm_head, self.lm_head_fmt = lm_head, lm_head_fmt
        w = layers[0].w
        self.w = w
        self.inv_freq = 1.0 / (rope_theta ** (torch.arange(0, w.head_dim, 2, device=embed.device, dtype=torch.float32)
                                              / w.head_dim))

    def rope_tables(self, pos: int, batch: int):
        ang = (pos * self.inv_freq)[None, :].expand(batch, -1)
        return ang.cos().to(torch.bfloat16).contiguous(), ang.sin().to(torch.bfloat16).contiguous()

    def step(self, tokens: torch.Tensor, caches: list, pos: int, cos_half=None, sin_half=None, return_logits: bool = False):
        """tokens [batch] int64 -> next tokens [batch] int32 (greedy); with return_logits also the fp32 logits."""
        if cos_half is None:
            cos_half, sin_half = self.rope_tables(pos, tokens.shape[0])
        out, stream = self.embed[tokens], None
        for layer, cache in zip(self.layers, caches):
            out, stream = layer.forward(out, stream, cos_half, sin_half, cache, pos)
        vocab = self.embed.shape[0]
        if stream is None and self.layers[0].fused_linear and out.shape[0] <= ops.linear_fusion_max_tokens(self.lm_head_fmt):
            logits = ops.linear(out, self.lm_head, self.lm_head_fmt, n=vocab, k=self.w.hidden, out_dtype=torch.float32,
                                prologue="rms_norm", norm_weight=self.final_norm, norm_eps=self.w.eps)
        else:
            hidden = ops.rms_norm(out, self.final_norm, self.w.eps, residual=stream)
            logits = ops.linear(hidden, self.lm_head, self.lm_head_fmt, n=vocab, k=self.w.hidden, out_dtype=torch.float32)
        nxt = ops.argmax_rows(logits)
        return (nxt, logits) if return_logits else nxt


class Qwen3TokenKernel:
    """The whole decode token of one sequence in one cooperative launch (izb_qwen3_decode_token): the same
    result as `Qwen3Decoder.step` for batch 1, without the ~200 launches.  Holds the device table of layer
    pointers and the workspace; `caches` are the `KvCache` objects of a batch of one."""

    def __init__(self, decoder: Qwen3Decoder, caches: list):
        import ctypes as C
        from . import _lib as L
        w = decoder.w
        dev = decoder.embed.device
        self.decoder, self.caches = decoder, caches
        rows = (L.Qwen3LayerPtrs * len(decoder.layers))()
        for i, (layer, cache) in enumerate(zip(decoder.layers, caches)):
            lw = layer.w
            assert cache.k.shape[0] == 1, "one sequence"
            rows[i] = L.Qwen3LayerPtrs(lw.input_layernorm.data_ptr(), lw.post_attention_layernorm.data_ptr(),
                                       0 if lw.q_norm is None else lw.q_norm.data_ptr(), 0 if lw.k_norm is None else lw.k_norm.data_ptr(),
                                       lw.qkv.data_ptr(), lw.o.data_ptr(), lw.gate_up.data_ptr(), lw.down.data_ptr(),
                                       cache.k.data_ptr(), cache.v.data_ptr())
        self.layer_table = rows  # host array of device pointers: the library copies it into the launch
        a = L.Qwen3DecodeArgs()
        a.wfmt, a.lm_head_fmt = ops.WFMT[w.fmt], ops.WFMT[decoder.lm_head_fmt]
        a.n_layers, a.hidden, a.heads, a.kv_heads, a.head_dim = len(decoder.layers), w.hidden, w.heads, w.kv_heads, w.head_dim
        a.intermediate, a.vocab = w.intermediate, decoder.embed.shape[0]
        a.kv_capacity, a.eps = caches[0].capacity, w.eps
        a.layers, a.embed, a.final_norm, a.lm_head = (C.cast(self.layer_table, C.c_void_p), decoder.embed.data_ptr(),
                                                      decoder.final_norm.data_ptr(), decoder.lm_head.data_ptr())
        self.ctx = ops.Context.get(dev.index)
        need = L.lib().izb_qwen3_decode_token_workspace_bytes(self.ctx.handle, C.byref(a))
        if need == 0:
            raise ValueError("this model is outside what izb_qwen3_decode_token takes")
        self.workspace = torch.zeros(need, device=dev, dtype=torch.uint8)
        a.workspace, a.workspace_bytes = self.workspace.data_ptr(), need
        self.args = a
        self.next_token = torch.zeros(1, device=dev, dtype=torch.int32)
        self.logits = torch.empty(a.vocab, device=dev, dtype=torch.float32)

    def step(self, token: torch.Tensor, pos: int, cos_half=None, sin_half=None, return_logits: bool = False):
        """token: int32 [1] on the device -> next token int32 [1] (a view of this object's buffer)."""
        import ctypes as C
        from . import _lib as L
        assert token.dtype == torch.int32 and token.numel() == 1 and token.is_cuda
        if cos_half is None:
            cos_half, sin_half = self.decoder.rope_tables(pos, 1)
        self.keep = (token, cos_half, sin_half)
        a = self.args
        a.pos, a.token, a.cos_half, a.sin_half = pos, token.data_ptr(), cos_half.data_ptr(), sin_half.data_ptr()
        a.logits = self.logits.data_ptr() if return_logits else None
        a.next_token = self.next_token.data_ptr()
        L.check(L.lib().izb_qwen3_decode_token(self.ctx.handle, ops._stream(), C.byref(a)), "izb_qwen3_decode_token")
        return (self.next_token, self.logits) if return_logits else self.next_token
