"""Host-side mirror of the reference's projection types over the C ABI.

Same names, argument meaning and error behaviour as
crates/izwi-core/src/models/architectures/qwen3/core.rs, so the parity tests
read like the reference's own unit tests:

  Qwen3Projection                 core.rs:671-728, forward :791-832
  Qwen3FusedQkvProjection         core.rs:931-981
  Qwen3FusedGateUpProjection      core.rs:1132-1168
  packed_qmatmul_from_qtensors    core.rs:846-885
  Qwen3Mlp                        core.rs:1786-1798

Tensors are torch CUDA tensors used purely as device buffers; all arithmetic
happens in libizwi_b200.so.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import ops


class InferenceError(RuntimeError):
    """Counterpart of izwi_core::Error::InferenceError."""


@dataclass(frozen=True)
class Qwen3ProjectionDiagnostics:
    dense_projection_count: int = 0
    dense_bias_projection_count: int = 0
    quantized_projection_count: int = 0

    def add(self, other: "Qwen3ProjectionDiagnostics") -> "Qwen3ProjectionDiagnostics":
        return Qwen3ProjectionDiagnostics(
            self.dense_projection_count + other.dense_projection_count,
            self.dense_bias_projection_count + other.dense_bias_projection_count,
            self.quantized_projection_count + other.quantized_projection_count)


@dataclass
class QTensor:
    """Raw GGML block bytes of a [rows, cols] matrix on the device."""
    data: torch.Tensor  # uint8, contiguous
    rows: int
    cols: int
    dtype: str          # "q8_0" | "q4_k"

    def dequantize(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        return ops.dequantize(self.data.reshape(-1), self.dtype, self.rows * self.cols, dtype).reshape(self.rows, self.cols)


def quantized_storage_bytes(rows: int, cols: int, dtype: str) -> int:
    try:
        return ops.quantized_storage_bytes(rows, cols, dtype)
    except Exception as exc:
        raise InferenceError(
            f"Qwen3 quantized projection element count {rows * cols} is not divisible by block size "
            f"{ops.BLOCK_SIZE[dtype]}") from exc


def packed_qmatmul_from_qtensors(tensors: list[QTensor]) -> "Qwen3Projection":
    """Row-wise concatenation of raw GGML bytes into one quantized projection."""
    if not tensors:
        raise InferenceError("Cannot pack empty Qwen3 quantized projection group")
    dtype, cols = tensors[0].dtype, tensors[0].cols
    total_rows = 0
    for t in tensors:
        if t.cols != cols:
            raise InferenceError(f"Qwen3 quantized projection group input mismatch: expected {cols}, got {t.cols}")
        if t.dtype != dtype:
            raise InferenceError(f"Qwen3 quantized projection group dtype mismatch: expected {dtype}, got {t.dtype}")
        total_rows += t.rows
    raw = torch.cat([t.data.reshape(-1) for t in tensors])
    expected = quantized_storage_bytes(total_rows, cols, dtype)
    if raw.numel() != expected:
        raise InferenceError(f"Qwen3 packed quantized projection has {raw.numel()} bytes, expected {expected}")
    return Qwen3Projection.quantized(QTensor(raw, total_rows, cols, dtype))


class Qwen3Projection:
    """Dense (bf16 weight, optional bias) or Quantized (GGML blocks) linear layer."""

    def __init__(self, kind: str, weight, bias: torch.Tensor | None = None):
        self.kind = kind
        self.weight = weight
        self.bias = bias

    @classmethod
    def dense(cls, weight: torch.Tensor, bias: torch.Tensor | None = None) -> "Qwen3Projection":
        if weight.dim() != 2:
            raise InferenceError("dense projection weight must be [out, in]")
        if bias is not None and bias.shape != (weight.shape[0],):
            raise InferenceError("dense projection bias must be [out]")
        w = weight.to(torch.bfloat16).contiguous()
        b = None if bias is None else bias.to(torch.bfloat16).contiguous()
        return cls("dense", w, b)

    @classmethod
    def tied_dense(cls, weight: torch.Tensor) -> "Qwen3Projection":
        return cls.dense(weight, None)

    @classmethod
    def quantized(cls, qtensor: QTensor) -> "Qwen3Projection":
        quantized_storage_bytes(qtensor.rows, qtensor.cols, qtensor.dtype)
        return cls("quantized", qtensor)

    @property
    def out_dim(self) -> int:
        return self.weight.shape[0] if self.kind == "dense" else self.weight.rows

    @property
    def in_dim(self) -> int:
        return self.weight.shape[1] if self.kind == "dense" else self.weight.cols

    def diagnostics(self) -> Qwen3ProjectionDiagnostics:
        if self.kind == "dense":
            return Qwen3ProjectionDiagnostics(1, int(self.bias is not None), 0)
        return Qwen3ProjectionDiagnostics(0, 0, 1)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from . import use_b200_kernels
        if not use_b200_kernels():
            # the gate next to IZWI_FUSED_KERNELS (kernels/mod.rs:46-57): off means the caller's own
            # (Candle) path; this mirror has none to fall back to and says so
            raise InferenceError("IZWI_B200_KERNELS is off: the B200 projection kernels are disabled")
        if not x.is_cuda:
            raise InferenceError("projection input must be a CUDA tensor")
        xb = x.to(torch.bfloat16)
        if not xb.is_contiguous():
            xb = xb.contiguous()
        if self.kind == "dense":
            y = ops.linear(xb, self.weight, "bf16", bias=self.bias)
        else:
            q = self.weight
            y = ops.linear(xb, q.data, q.dtype, n=q.rows, k=q.cols)
        return y if x.dtype == torch.bfloat16 else y.to(x.dtype)

    def logits_for_tokens(self, hidden: torch.Tensor, token_ids: list[int]) -> list[tuple[int, float]]:
        """Logits of selected output rows (core.rs:747-763): the full projection, then a gather."""
        if not token_ids:
            return []
        full = self.forward(hidden).to(torch.float32).reshape(-1)
        return [(int(t), float(full[t])) for t in token_ids]


def _concat_biases(name: str, projs: list[Qwen3Projection]):
    have = [p.bias is not None for p in projs]
    if not any(have):
        return None
    if not all(have):
        raise InferenceError(f"{name} cannot fuse projections with mixed bias presence")
    return torch.cat([p.bias for p in projs], dim=0)


class Qwen3FusedQkvProjection:
    def __init__(self, q_proj: Qwen3Projection, k_proj: Qwen3Projection, v_proj: Qwen3Projection):
        in_dim = q_proj.in_dim
        if k_proj.in_dim != in_dim or v_proj.in_dim != in_dim:
            raise InferenceError("Qwen3 fused QKV projection input dimensions do not match")
        self.q_out, self.k_out, self.v_out = q_proj.out_dim, k_proj.out_dim, v_proj.out_dim
        weight = torch.cat([q_proj.weight, k_proj.weight, v_proj.weight], dim=0)
        bias = _concat_biases("Qwen3 fused QKV projection", [q_proj, k_proj, v_proj])
        self.bias_count = sum(int(p.bias is not None) for p in (q_proj, k_proj, v_proj))
        self.fused = Qwen3Projection.dense(weight, bias)

    def forward(self, x: torch.Tensor):
        qkv = self.fused.forward(x)
        return (qkv[..., : self.q_out], qkv[..., self.q_out: self.q_out + self.k_out],
                qkv[..., self.q_out + self.k_out:])

    def diagnostics(self) -> Qwen3ProjectionDiagnostics:
        return Qwen3ProjectionDiagnostics(3, self.bias_count, 0)


class Qwen3FusedGateUpProjection:
    def __init__(self, gate_proj: Qwen3Projection, up_proj: Qwen3Projection):
        if up_proj.out_dim != gate_proj.out_dim or up_proj.in_dim != gate_proj.in_dim:
            raise InferenceError("Qwen3 fused MLP projection dimensions do not match")
        self.intermediate_size = gate_proj.out_dim
        weight = torch.cat([gate_proj.weight, up_proj.weight], dim=0)
        bias = _concat_biases("Qwen3 fused MLP projection", [gate_proj, up_proj])
        self.bias_count = sum(int(p.bias is not None) for p in (gate_proj, up_proj))
        self.fused = Qwen3Projection.dense(weight, bias)

    def forward(self, x: torch.Tensor):
        gu = self.fused.forward(x)
        return gu[..., : self.intermediate_size], gu[..., self.intermediate_size:]

    def diagnostics(self) -> Qwen3ProjectionDiagnostics:
        return Qwen3ProjectionDiagnostics(2, self.bias_count, 0)


class Qwen3FusedQuantizedProjection:
    """Fused quantized QKV / gate-up: byte-packed rows, one matmul, narrow."""

    def __init__(self, parts: list[QTensor]):
        self.fused = packed_qmatmul_from_qtensors(parts)
        self.splits = [p.rows for p in parts]

    def forward(self, x: torch.Tensor):
        y = self.fused.forward(x)
        return tuple(torch.split(y, self.splits, dim=-1))

    def diagnostics(self) -> Qwen3ProjectionDiagnostics:
        return Qwen3ProjectionDiagnostics(0, 0, len(self.splits))


class Qwen3Mlp:
    """down( silu(gate) * up ) with the fused gate/up projection and the fused SiLU-multiply."""

    def __init__(self, gate_up_proj, down_proj: Qwen3Projection):
        self.gate_up_proj = gate_up_proj
        self.down_proj = down_proj

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        gate, up = self.gate_up_proj.forward(x)
        hidden = ops.silu_mul(gate, up)
        return self.down_proj.forward(hidden)
