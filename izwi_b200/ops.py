"""Torch-tensor plumbing over the C ABI: tensors supply device pointers and the
current stream, nothing else.  Every function launches the CUDA kernels of
libizwi_b200.so; none has a PyTorch or CPU fallback."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L

WFMT = {"bf16": L.IZB_W_BF16, "q8_0": L.IZB_W_Q8_0, "q4_k": L.IZB_W_Q4_K, "q6_k": L.IZB_W_Q6_K}
BLOCK_SIZE = {"bf16": 1, "q8_0": 32, "q4_k": 256, "q6_k": 256}
TYPE_SIZE = {"bf16": 2, "q8_0": 34, "q4_k": 144, "q6_k": 210}


class Context:
    """One izb_ctx per device (see include/izwi_b200.h)."""

    _by_device: dict[int, "Context"] = {}

    def __init__(self, device: int = 0):
        handle = C.c_void_p()
        L.check(L.lib().izb_ctx_create(device, C.byref(handle)), "izb_ctx_create")
        self.handle = handle
        self.device = device

    @classmethod
    def get(cls, device: int | None = None) -> "Context":
        if device is None:
            device = torch.cuda.current_device()
        ctx = cls._by_device.get(device)
        if ctx is None:
            ctx = cls._by_device[device] = Context(device)
        return ctx

    def check(self) -> None:
        L.check(L.lib().izb_ctx_check(self.handle, _stream()), "izb_ctx_check")

    @property
    def launch_count(self) -> int:
        return int(L.lib().izb_ctx_launch_count(self.handle))


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def quantized_storage_bytes(rows: int, cols: int, fmt: str) -> int:
    out = C.c_size_t()
    L.check(L.lib().izb_quantized_storage_bytes(WFMT[fmt], rows, cols, C.byref(out)), "izb_quantized_storage_bytes")
    return out.value


def dequantize(raw: torch.Tensor, fmt: str, n_elems: int, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    assert raw.is_cuda and raw.dtype == torch.uint8 and raw.is_contiguous()
    out = torch.empty(n_elems, device=raw.device, dtype=dtype)
    code = L.IZB_F32 if dtype == torch.float32 else L.IZB_BF16
    ctx = Context.get(raw.device.index)
    L.check(L.lib().izb_dequantize(ctx.handle, _stream(), WFMT[fmt], _ptr(raw), n_elems, code, _ptr(out)),
            "izb_dequantize")
    return out


def dequantize_mlx_affine(packed: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor | None, out_dim: int, in_dim: int,
                          dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """MLX affine-packed weight ([out_dim, packed_in] uint8, or int32 / uint32 words) -> dense [out_dim, in_dim]:
    `load_weight` of models/shared/weights/mlx.rs on the device.  scales / biases fp32 [out_dim, groups] or
    [groups, out_dim]."""
    assert packed.is_cuda and packed.dim() == 2 and packed.is_contiguous() and packed.shape[0] == out_dim
    word_bits = 8 if packed.dtype == torch.uint8 else 32
    assert packed.dtype in (torch.uint8, torch.int32, torch.uint32)
    assert scales.dtype == torch.float32 and scales.dim() == 2 and scales.is_contiguous()
    transposed = scales.shape[0] != out_dim
    groups = scales.shape[0] if transposed else scales.shape[1]
    if transposed and scales.shape[1] != out_dim:
        raise ValueError("quantization scales shape mismatch")
    if biases is not None:
        assert biases.dtype == torch.float32 and biases.shape == scales.shape and biases.is_contiguous()
    out = torch.empty(out_dim, in_dim, device=packed.device, dtype=dtype)
    ctx = Context.get(packed.device.index)
    L.check(L.lib().izb_dequantize_mlx_affine(ctx.handle, _stream(), _ptr(packed), word_bits, packed.shape[1], _ptr(scales),
                                              None if biases is None else _ptr(biases), groups, 1 if transposed else 0, out_dim, in_dim,
                                              DTYPE[dtype], _ptr(out)), "izb_dequantize_mlx_affine")
    return out


EPILOGUE = {None: L.IZB_EPI_NONE, "none": L.IZB_EPI_NONE, "gelu": L.IZB_EPI_GELU, "silu": L.IZB_EPI_SILU,
            "swiglu": L.IZB_EPI_SWIGLU, "gelu_tanh": L.IZB_EPI_GELU_TANH, "glu": L.IZB_EPI_GLU}
PROLOGUE = {None: 0, "none": 0, "rms_norm": 1, "silu_mul": 2}  # izb_prologue
DTYPE = {torch.bfloat16: L.IZB_BF16, torch.float32: L.IZB_F32, torch.float16: L.IZB_F16}  # izb_dtype


def linear_args(x: torch.Tensor, w: torch.Tensor, fmt: str, n: int, k: int, y: torch.Tensor,
                bias: torch.Tensor | None = None, epilogue: str | None = None,
                workspace: torch.Tensor | None = None, prologue: str | None = None,
                norm_weight: torch.Tensor | None = None, norm_eps: float = 0.0,
                residual: torch.Tensor | None = None) -> L.LinearArgs:
    assert x.is_cuda and x.dtype in DTYPE and x.dim() == 2 and x.stride(1) == 1
    assert y.dim() == 2 and y.stride(1) == 1 and y.shape[0] == x.shape[0] and y.dtype in DTYPE
    a = L.LinearArgs()
    a.wfmt = WFMT[fmt]
    a.x_dtype, a.y_dtype = DTYPE[x.dtype], DTYPE[y.dtype]
    a.x, a.w, a.bias, a.y = x.data_ptr(), w.data_ptr(), (0 if bias is None else bias.data_ptr()), y.data_ptr()
    a.M, a.N, a.K = x.shape[0], n, k
    a.ldx, a.ldy = x.stride(0), y.stride(0)
    a.workspace = None if workspace is None else workspace.data_ptr()
    a.workspace_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    a.epilogue = EPILOGUE[epilogue]
    a.prologue = PROLOGUE[prologue]
    if prologue == "rms_norm":
        assert norm_weight is not None and norm_weight.dtype == torch.bfloat16 and norm_weight.shape == (k,)
        a.norm_weight, a.norm_eps = norm_weight.data_ptr(), float(norm_eps)
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.dim() == 2 and residual.stride(1) == 1
        assert residual.shape == y.shape
        a.residual, a.ld_residual = residual.data_ptr(), residual.stride(0)
    return a


def linear(x: torch.Tensor, w: torch.Tensor, fmt: str = "bf16", n: int | None = None, k: int | None = None,
           bias: torch.Tensor | None = None, out: torch.Tensor | None = None,
           out_dtype: torch.dtype = torch.bfloat16, epilogue: str | None = None,
           workspace: torch.Tensor | None | bool = True, prologue: str | None = None,
           norm_weight: torch.Tensor | None = None, norm_eps: float = 0.0,
           residual: torch.Tensor | None = None) -> torch.Tensor:
    """Y = epilogue(prologue(X) . W^T + bias) + residual.  `x` may have any number of leading dimensions
    (flattened to M like the reference's Linear); `w` is [N, K] bf16 or the raw
    GGML bytes of N rows of K values.  `workspace=True` lets this wrapper provide
    the scratch buffer the library asks for (it never allocates itself).
    `prologue` "rms_norm" (with `norm_weight`, `norm_eps`) or "silu_mul" (x is [.., 2K] = gate | up) is
    computed inside the kernel for at most `linear_fusion_max_tokens(fmt)` token rows and through the
    workspace otherwise; `residual` is added by the product's epilogue on every route.  fp32 / fp16 `x`
    is rounded to bf16 by one cast launch into the workspace; `out_dtype` may be bf16, fp32 or fp16."""
    if fmt == "bf16":
        n, k = w.shape
    assert n is not None and k is not None
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.shape[1] != (2 * k if prologue == "silu_mul" else k):
        raise ValueError(f"linear: input dim {x2.shape[1]} != weight in-dim {k}")
    n_out = n // 2 if epilogue in ("swiglu", "glu") else n
    y = out if out is not None else torch.empty(x2.shape[0], n_out, device=x.device, dtype=out_dtype)
    res2 = None if residual is None else residual.reshape(-1, n_out)
    if workspace is True:
        probe = linear_args(x2, w, fmt, n, k, y.reshape(-1, n_out), bias, epilogue, None, prologue, norm_weight, norm_eps, res2)
        need = L.lib().izb_linear_workspace_bytes_args(C.byref(probe))
        workspace = torch.empty(need, device=x.device, dtype=torch.uint8) if need else None
    elif workspace is False:
        workspace = None
    a = linear_args(x2, w, fmt, n, k, y.reshape(-1, n_out), bias, epilogue, workspace, prologue, norm_weight, norm_eps, res2)
    ctx = Context.get(x.device.index)
    L.check(L.lib().izb_linear(ctx.handle, _stream(), C.byref(a)), "izb_linear")
    return y.reshape(*lead, n_out)


def linear_fusion_max_tokens(fmt: str) -> int:
    """Most token rows for which `linear` takes a prologue or a residual with weights stored as `fmt`."""
    return int(L.lib().izb_linear_fusion_max_tokens(WFMT[fmt]))


def silu_mul(gate: torch.Tensor, up: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    assert gate.shape == up.shape and gate.dtype == torch.bfloat16 and up.dtype == torch.bfloat16
    g2, u2 = gate.reshape(-1, gate.shape[-1]), up.reshape(-1, up.shape[-1])
    assert g2.stride(1) == 1 and u2.stride(1) == 1
    o = out if out is not None else torch.empty(gate.shape, device=gate.device, dtype=torch.bfloat16)
    o2 = o.reshape(-1, o.shape[-1])
    ctx = Context.get(gate.device.index)
    L.check(L.lib().izb_silu_mul(ctx.handle, _stream(), _ptr(g2), _ptr(u2), _ptr(o2), g2.shape[0], g2.shape[1],
                                 g2.stride(0), u2.stride(0), o2.stride(0)), "izb_silu_mul")
    return o


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor | None = None,
             return_sum: bool = False):
    """`candle_nn::ops::rms_norm` behind `try_fused_rms_norm` (kernels/mod.rs:143-157), optionally after a
    residual add.  Rows are the leading dimensions flattened; returns out, or (out, x + residual)."""
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.shape == (x.shape[-1],)
    x2 = x.reshape(-1, x.shape[-1])
    assert x2.stride(1) == 1
    out = torch.empty(x.shape, device=x.device, dtype=torch.bfloat16)
    o2 = out.reshape(-1, out.shape[-1])
    r2 = s2 = None
    total = None
    if residual is not None:
        assert residual.shape == x.shape and residual.dtype == torch.bfloat16
        r2 = residual.reshape(-1, x.shape[-1])
        assert r2.stride(1) == 1
        if return_sum:
            total = torch.empty(x.shape, device=x.device, dtype=torch.bfloat16)
            s2 = total.reshape(-1, x.shape[-1])
    ctx = Context.get(x.device.index)
    L.check(L.lib().izb_rms_norm(ctx.handle, _stream(), _ptr(x2), _ptr(weight), None if r2 is None else _ptr(r2), _ptr(o2),
                                 None if s2 is None else _ptr(s2), x2.shape[0], x2.shape[1], x2.stride(0),
                                 0 if r2 is None else r2.stride(0), o2.stride(0), 0 if s2 is None else s2.stride(0),
                                 float(eps)), "izb_rms_norm")
    return (out, total) if return_sum else out


def argmax_rows(x: torch.Tensor, return_values: bool = False):
    """Greedy token choice over logits rows (`argmax`, qwen3/chat.rs:574-601) without the host copy."""
    assert x.dtype in (torch.bfloat16, torch.float32)
    x2 = x.reshape(-1, x.shape[-1])
    assert x2.stride(1) == 1
    idx = torch.empty(x2.shape[0], device=x.device, dtype=torch.int32)
    val = torch.empty(x2.shape[0], device=x.device, dtype=torch.float32) if return_values else None
    ctx = Context.get(x.device.index)
    L.check(L.lib().izb_argmax_rows(ctx.handle, _stream(), _ptr(x2), L.IZB_F32 if x.dtype == torch.float32 else L.IZB_BF16, x2.shape[0], x2.shape[1],
                                    x2.stride(0), _ptr(idx), None if val is None else _ptr(val)), "izb_argmax_rows")
    idx = idx.reshape(x.shape[:-1])
    return (idx, val.reshape(x.shape[:-1])) if return_values else idx


def sample_rows(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, uniform: torch.Tensor | None) -> torch.Tensor:
    """One token per logits row by temperature / top-k / top-p sampling on the device (`sample_from_logits`,
    lfm25_audio/sampling.rs:65-160); `uniform` holds one number in [0, 1) per row, drawn by the caller."""
    assert logits.dtype in (torch.bfloat16, torch.float32)
    x2 = logits.reshape(-1, logits.shape[-1])
    assert x2.stride(1) == 1
    if uniform is not None:
        assert uniform.dtype == torch.float32 and uniform.is_contiguous() and uniform.numel() == x2.shape[0]
    idx = torch.empty(x2.shape[0], device=logits.device, dtype=torch.int32)
    ctx = Context.get(logits.device.index)
    L.check(L.lib().izb_sample_rows(ctx.handle, _stream(), _ptr(x2), L.IZB_F32 if logits.dtype == torch.float32 else L.IZB_BF16,
                                    x2.shape[0], x2.shape[1], x2.stride(0), float(temperature), int(top_k), float(top_p),
                                    _ptr(uniform), _ptr(idx)), "izb_sample_rows")
    return idx.reshape(logits.shape[:-1])


def rope_pair_(q: torch.Tensor, k: torch.Tensor, cos_half: torch.Tensor, sin_half: torch.Tensor) -> None:
    """`apply_rotary_emb` on q and k (qwen3/core.rs:2402-2415), in place.  q [tokens, q_heads, d],
    k [tokens, k_heads, d], tables [tokens, d / 2]; all bf16."""
    assert q.dtype == k.dtype == cos_half.dtype == sin_half.dtype == torch.bfloat16
    tokens, qh, d = q.shape
    assert k.shape[0] == tokens and k.shape[2] == d and cos_half.shape == sin_half.shape == (tokens, d // 2)
    assert q.stride(2) == 1 and q.stride(1) == d and k.stride(2) == 1 and k.stride(1) == d
    assert cos_half.is_contiguous() and sin_half.is_contiguous()
    ctx = Context.get(q.device.index)
    L.check(L.lib().izb_rope_pair(ctx.handle, _stream(), _ptr(q), _ptr(k), _ptr(cos_half), _ptr(sin_half), tokens, qh,
                                  k.shape[1], d, q.stride(0), k.stride(0)), "izb_rope_pair")


def kv_append_(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos: int) -> None:
    """New token's k, v [batch, kv_heads, d] (views allowed: last two dims dense) into position `pos` of the caches."""
    b, kvh, d = k.shape
    assert v.shape == k.shape and k_cache.shape == v_cache.shape and k_cache.shape[:2] == (b, kvh) and k_cache.shape[3] == d
    assert k.stride(2) == 1 and k.stride(1) == d and v.stride(2) == 1 and v.stride(1) == d
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    ctx = Context.get(k.device.index)
    L.check(L.lib().izb_kv_append(ctx.handle, _stream(), _ptr(k), _ptr(v), _ptr(k_cache), _ptr(v_cache), b, kvh, d, pos,
                                  k_cache.shape[2], k.stride(0), v.stride(0)), "izb_kv_append")


def qk_norm_rope_append(qkv: torch.Tensor, q_norm: torch.Tensor | None, k_norm: torch.Tensor | None, eps: float,
                        cos_half: torch.Tensor, sin_half: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                        heads: int, pos: int) -> torch.Tensor:
    """q/k head norms, rotation and cache append of one decode token per sequence in one launch;
    qkv [batch, (heads + 2 kv_heads) * d] -> q [batch, heads, d]."""
    b = qkv.shape[0]
    kvh, cap, d = k_cache.shape[1], k_cache.shape[2], k_cache.shape[3]
    assert qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and qkv.shape[1] == (heads + 2 * kvh) * d
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and cos_half.is_contiguous() and sin_half.is_contiguous()
    q = torch.empty(b, heads, d, device=qkv.device, dtype=torch.bfloat16)
    ctx = Context.get(qkv.device.index)
    L.check(L.lib().izb_qk_norm_rope_append(ctx.handle, _stream(), _ptr(qkv), qkv.stride(0), _ptr(q_norm), _ptr(k_norm),
                                            float(eps), _ptr(cos_half), _ptr(sin_half), _ptr(q), q.stride(0), _ptr(k_cache),
                                            _ptr(v_cache), b, heads, kvh, d, pos, cap), "izb_qk_norm_rope_append")
    return q


def decode_gqa_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, kv_len: int,
                         scale: float | None = None, out: torch.Tensor | None = None,
                         workspace: torch.Tensor | None = None) -> torch.Tensor:
    """`dense_decode_attention` (qwen3/core.rs:2189-2225): q [batch, heads, d], caches
    [batch, kv_heads, capacity, d] (head-major), the first kv_len positions valid."""
    assert q.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16
    b, h, d = q.shape
    assert k_cache.shape == v_cache.shape and k_cache.shape[0] == b and k_cache.shape[3] == d
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and q.stride(2) == 1 and q.stride(1) == d
    kvh, cap = k_cache.shape[1], k_cache.shape[2]
    if out is None:
        out = torch.empty(b, h, d, device=q.device, dtype=torch.bfloat16)
    ctx = Context.get(q.device.index)
    need = L.lib().izb_decode_gqa_attention_workspace_bytes(ctx.handle, b, h, kvh, d, kv_len)
    ws = workspace if workspace is not None and workspace.numel() * workspace.element_size() >= need else (
        torch.empty(need, device=q.device, dtype=torch.uint8) if need else None)
    L.check(L.lib().izb_decode_gqa_attention(ctx.handle, _stream(), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), b, h,
                                             kvh, d, kv_len, cap, q.stride(0), out.stride(0),
                                             float(d ** -0.5 if scale is None else scale), _ptr(ws), need),
            "izb_decode_gqa_attention")
    return out


def embed_rows(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """Embedding lookup (`embed_tokens`, qwen3/core.rs:2099-2103): table [vocab, hidden] bf16, ids int32 [tokens]."""
    assert table.dtype == torch.bfloat16 and table.is_contiguous() and ids.dtype == torch.int32 and ids.is_contiguous()
    out = torch.empty(ids.numel(), table.shape[1], device=table.device, dtype=torch.bfloat16)
    ctx = Context.get(table.device.index)
    L.check(L.lib().izb_embed_rows(ctx.handle, _stream(), _ptr(table), table.shape[0], table.shape[1], _ptr(ids), ids.numel(),
                                   _ptr(out), out.stride(0)), "izb_embed_rows")
    return out


def qk_norm_rope_append_seq(qkv: torch.Tensor, q_norm: torch.Tensor | None, k_norm: torch.Tensor | None, eps: float,
                            cos_half: torch.Tensor, sin_half: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                            heads: int, q_len: int, pos0: int) -> torch.Tensor:
    """q/k head norms, rotation and cache append for q_len consecutive tokens per sequence:
    qkv [batch * q_len, (heads + 2 kv_heads) * d], tables [q_len, d / 2] -> q [batch * q_len, heads, d]."""
    rows = qkv.shape[0]
    b = rows // q_len
    kvh, cap, d = k_cache.shape[1], k_cache.shape[2], k_cache.shape[3]
    assert qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and qkv.shape[1] == (heads + 2 * kvh) * d and b * q_len == rows
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and cos_half.is_contiguous() and sin_half.is_contiguous()
    assert cos_half.shape == sin_half.shape == (q_len, d // 2)
    q = torch.empty(rows, heads, d, device=qkv.device, dtype=torch.bfloat16)
    ctx = Context.get(qkv.device.index)
    L.check(L.lib().izb_qk_norm_rope_append_seq(ctx.handle, _stream(), _ptr(qkv), qkv.stride(0), _ptr(q_norm), _ptr(k_norm),
                                                float(eps), _ptr(cos_half), _ptr(sin_half), _ptr(q), q.stride(0), _ptr(k_cache),
                                                _ptr(v_cache), b, q_len, heads, kvh, d, pos0, cap), "izb_qk_norm_rope_append_seq")
    return q


def prefill_gqa_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, q_len: int, pos0: int,
                          scale: float | None = None) -> torch.Tensor:
    """Causal attention of q_len new tokens per sequence (already appended at pos0 ..) over the cache:
    q [batch * q_len, heads, d] -> out of the same shape."""
    assert q.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16
    rows, h, d = q.shape
    b = rows // q_len
    assert k_cache.shape == v_cache.shape and k_cache.shape[0] == b and k_cache.shape[3] == d
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and q.stride(2) == 1 and q.stride(1) == d
    out = torch.empty(rows, h, d, device=q.device, dtype=torch.bfloat16)
    ctx = Context.get(q.device.index)
    L.check(L.lib().izb_prefill_gqa_attention(ctx.handle, _stream(), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), b, q_len, h,
                                              k_cache.shape[1], d, pos0, k_cache.shape[2], q.stride(0), out.stride(0),
                                              float(d ** -0.5 if scale is None else scale)), "izb_prefill_gqa_attention")
    return out


class LinearGroup:
    """A set of independent small-M linear layers run by one persistent launch
    (izb_linear_group_*).  Keeps the tensors alive and owns the device copy of
    the plan."""

    def __init__(self, problems: list[L.LinearArgs], device: torch.device, keepalive=None):
        self.n = len(problems)
        self.ctx = Context.get(device.index)
        arr = (L.LinearArgs * self.n)(*problems)
        nbytes = L.lib().izb_linear_group_plan_bytes(self.n)
        self.host_plan = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
        L.check(L.lib().izb_linear_group_plan(self.ctx.handle, arr, self.n, C.c_void_p(self.host_plan.data_ptr()),
                                              nbytes), "izb_linear_group_plan")
        self.dev_plan = self.host_plan.to(device)
        self.keepalive = keepalive

    def launch(self) -> None:
        L.check(L.lib().izb_linear_group_launch(self.ctx.handle, _stream(), C.c_void_p(self.host_plan.data_ptr()),
                                                C.c_void_p(self.dev_plan.data_ptr())), "izb_linear_group_launch")

    def launch_host(self, host_in: torch.Tensor, dev_in: torch.Tensor, dev_out: torch.Tensor | None = None,
                    host_out: torch.Tensor | None = None) -> None:
        """One step for a caller with host tensors (izb_linear_group_launch_host): `host_in` -> `dev_in` (the buffer
        the problems' x pointers lie in), the launch, `dev_out` -> `host_out`; returns when the results are in host
        memory.  Without `dev_out` / `host_out` nothing is copied back: for a group whose y pointers already lie in
        page-locked host memory."""
        assert not host_in.is_cuda and dev_in.is_cuda and host_in.is_contiguous() and dev_in.is_contiguous()
        assert host_in.dtype == dev_in.dtype and host_in.numel() <= dev_in.numel()
        # The copy goes out first, through torch, and the C call below gets no input bytes: what ctypes spends on the
        # ten arguments then overlaps the copy instead of standing in front of it (6 us of a 110 us step).  A C or
        # Rust caller passes host_in / in_bytes and has neither cost.
        dev_in.view(-1)[:host_in.numel()].copy_(host_in.view(-1), non_blocking=True)
        in_bytes = 0
        out_bytes, p_dev_out, p_host_out = 0, None, None
        if host_out is not None:
            assert dev_out is not None and dev_out.is_cuda and not host_out.is_cuda and dev_out.is_contiguous() and host_out.is_contiguous()
            out_bytes = host_out.numel() * host_out.element_size()
            assert out_bytes <= dev_out.numel() * dev_out.element_size()
            p_dev_out, p_host_out = C.c_void_p(dev_out.data_ptr()), C.c_void_p(host_out.data_ptr())
        L.check(L.lib().izb_linear_group_launch_host(self.ctx.handle, _stream(), C.c_void_p(self.host_plan.data_ptr()),
                                                     C.c_void_p(self.dev_plan.data_ptr()), None, None, in_bytes, p_dev_out, p_host_out,
                                                     out_bytes),
                "izb_linear_group_launch_host")
