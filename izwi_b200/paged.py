"""Host-side mirror of the reference's paged KV cache over the C ABI
(crates/izwi-core/src/models/shared/attention/paged.rs): `KvCacheQuantization`, pages appended with
`append_to_pages`, `materialize_pages`, `paged_decode_attention`.  The pool, the page table and the
sequence lengths are device buffers; nothing here computes on the host."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L
from .ops import Context, _ptr, _stream

DEFAULT_KV_PAGE_SIZE = 64                     # paged.rs:10
QUANT = {"none": 0, "int8": 1, "q4_0": 2}


def kv_quantization_from_dtype_hint(dtype: str) -> str:
    """`KvCacheQuantization::from_dtype_hint` (paged.rs:25-36)."""
    d = dtype.strip().lower()
    if d in ("int8", "i8", "q8", "q8_0"):
        return "int8"
    if d in ("q4_0", "q4"):
        return "q4_0"
    return "none"


class PagedKvCache:
    """The K and V pages of `batch` sequences for one layer: every sequence owns `max_pages` pool pages
    (a fixed page table; a serving engine would hand pages out on demand)."""

    def __init__(self, batch: int, kv_heads: int, head_dim: int, max_tokens: int, device, quantization: str = "none",
                 page_size: int = DEFAULT_KV_PAGE_SIZE):
        if page_size <= 0:
            raise ValueError("KV page size must be greater than zero")          # append_to_pages, paged.rs:352-356
        self.batch, self.kv_heads, self.head_dim, self.page_size = batch, kv_heads, head_dim, page_size
        self.quantization = quantization
        q = QUANT[quantization]
        self.max_pages = (max_tokens + page_size - 1) // page_size
        n_pages = batch * self.max_pages
        lib = L.lib()
        nbytes, nscales = lib.izb_kv_page_bytes(q, page_size, kv_heads, head_dim), lib.izb_kv_page_scales(q, page_size, kv_heads, head_dim)
        self.k_values = torch.zeros(n_pages * nbytes, device=device, dtype=torch.uint8)
        self.v_values = torch.zeros(n_pages * nbytes, device=device, dtype=torch.uint8)
        self.k_scales = torch.ones(max(n_pages * nscales, 1), device=device, dtype=torch.float32)
        self.v_scales = torch.ones(max(n_pages * nscales, 1), device=device, dtype=torch.float32)
        self.page_table = torch.arange(n_pages, device=device, dtype=torch.int32).reshape(batch, self.max_pages).contiguous()
        self.seq_lens = torch.zeros(batch, device=device, dtype=torch.int32)
        self.max_tokens = self.max_pages * page_size
        self._desc = L.KvPages(self.k_values.data_ptr(), self.v_values.data_ptr(), self.k_scales.data_ptr() if nscales else None,
                               self.v_scales.data_ptr() if nscales else None, self.page_table.data_ptr(), q, page_size, kv_heads,
                               head_dim, self.max_pages)

    def append(self, k: torch.Tensor, v: torch.Tensor) -> None:
        """k, v [batch, n_new, kv_heads, head_dim] bf16 (the reference's `[batch, seq, heads, dim]`)."""
        b, n_new = k.shape[0], k.shape[1]
        assert k.shape == v.shape == (b, n_new, self.kv_heads, self.head_dim) and b == self.batch
        assert k.dtype == v.dtype == torch.bfloat16 and k.is_contiguous() and v.is_contiguous()
        ctx = Context.get(k.device.index)
        row = self.kv_heads * self.head_dim
        L.check(L.lib().izb_kv_pages_append(ctx.handle, _stream(), C.byref(self._desc), _ptr(k), _ptr(v), b, n_new, row, row,
                                            _ptr(self.seq_lens)), "izb_kv_pages_append")
        self.seq_lens += n_new            # on the device, after the append in stream order

    def materialize(self, which: str, max_len: int) -> torch.Tensor:
        """Dense [batch, max_len, kv_heads, head_dim] bf16 copy of the cached keys ("k") or values ("v")."""
        out = torch.zeros(self.batch, max_len, self.kv_heads, self.head_dim, device=self.k_values.device, dtype=torch.bfloat16)
        ctx = Context.get(out.device.index)
        row = self.kv_heads * self.head_dim
        L.check(L.lib().izb_kv_pages_materialize(ctx.handle, _stream(), C.byref(self._desc), 0 if which == "k" else 1, self.batch,
                                                 _ptr(self.seq_lens), _ptr(out), row, max_len * row), "izb_kv_pages_materialize")
        return out

    def decode_attention(self, q: torch.Tensor, scale: float | None = None) -> torch.Tensor:
        """`paged_decode_attention` (paged.rs:578-628): q [batch, heads, head_dim] -> same shape."""
        assert q.dtype == torch.bfloat16 and q.dim() == 3 and q.stride(2) == 1 and q.stride(1) == self.head_dim
        b, h, d = q.shape
        if h % self.kv_heads != 0:
            raise ValueError(f"Paged decode attention received invalid head layout: num_heads={h}, num_kv_heads={self.kv_heads}")
        out = torch.empty(b, h, d, device=q.device, dtype=torch.bfloat16)
        ctx = Context.get(q.device.index)
        need = L.lib().izb_paged_decode_gqa_attention_workspace_bytes(ctx.handle, b, h, self.kv_heads, d, self.max_tokens)
        ws = torch.empty(need, device=q.device, dtype=torch.uint8) if need else None
        L.check(L.lib().izb_paged_decode_gqa_attention(ctx.handle, _stream(), _ptr(q), C.byref(self._desc), _ptr(self.seq_lens),
                                                       _ptr(out), b, h, self.max_tokens, q.stride(0), out.stride(0),
                                                       float(d ** -0.5 if scale is None else scale), _ptr(ws), need),
                "izb_paged_decode_gqa_attention")
        return out
