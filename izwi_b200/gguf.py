"""GGUF weight source over the C ABI (`izb_gguf_*`): the host-side mirror of the reference's
`GgufLoader` (crates/izwi-core/src/models/shared/weights/gguf.rs:36-143).  Same method names and
meaning; errors carry the reference's message texts.  Quantised tensors are uploaded as the raw
GGML block bytes the kernels multiply in place (`load_qtensor`); `load_tensor` dequantises on the
GPU (bit-exact with GGML) and casts."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from pathlib import Path

from . import _lib as L

GGML_TYPE_NAMES = {0: "F32", 1: "F16", 2: "Q4_0", 3: "Q4_1", 6: "Q5_0", 7: "Q5_1", 8: "Q8_0", 9: "Q8_1", 10: "Q2_K",
                   11: "Q3_K", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K", 15: "Q8_K", 24: "I8", 25: "I16", 26: "I32",
                   27: "I64", 28: "F64", 30: "BF16"}
WFMT_NAMES = {L.IZB_W_BF16: "bf16", L.IZB_W_Q8_0: "q8_0", L.IZB_W_Q4_K: "q4_k", L.IZB_W_Q6_K: "q6_k"}


class ModelLoadError(RuntimeError):
    """`Error::ModelLoadError` of the reference (error.rs)."""


@dataclass
class GgufModelInfo:
    """`GgufModelInfo` (gguf.rs:20-33)."""
    path: Path
    architecture: str | None
    parameter_count: int | None
    quantization: str | None
    metadata: dict = field(default_factory=dict)


@dataclass
class TensorInfo:
    name: str
    ggml_type: int
    dtype: str                 # GGML type name, e.g. "Q4_K"
    wfmt: str | None           # format name the kernels accept for these bytes ("q8_0", ...), else None
    shape: tuple               # outermost first
    rows: int
    cols: int
    nbytes: int
    _data: int = 0             # host address inside the mapping


@dataclass
class QTensor:
    """Raw GGML bytes of one tensor on the device (Candle's `QTensor`)."""
    data: "object"             # torch.uint8 tensor
    dtype: str                 # "q8_0" | "q4_k" | "q6_k" | "bf16" | GGML type name for other types
    shape: tuple
    rows: int
    cols: int


class GgufLoader:
    def __init__(self, path: Path, handle: C.c_void_p):
        self.path = Path(path)
        self._h = handle
        self._lib = L.lib()
        self._infos: dict[str, TensorInfo] = {}
        t = L.GgufTensor()
        for i in range(self._lib.izb_gguf_tensor_count(self._h)):
            rc = self._lib.izb_gguf_tensor_at(self._h, i, C.byref(t))
            if rc != 0:
                raise ModelLoadError(f"Failed to parse GGUF file: tensor {i}: status {rc}")
            info = self._to_info(t)
            self._infos[info.name] = info

    @staticmethod
    def _to_info(t: L.GgufTensor) -> TensorInfo:
        return TensorInfo(name=t.name.decode(), ggml_type=t.ggml_type,
                          dtype=GGML_TYPE_NAMES.get(t.ggml_type, str(t.ggml_type)),
                          wfmt=WFMT_NAMES.get(t.wfmt), shape=tuple(int(t.dims[d]) for d in range(t.n_dims)),
                          rows=int(t.rows), cols=int(t.cols), nbytes=int(t.bytes), _data=int(t.data or 0))

    # ---- construction -------------------------------------------------------------------------
    @classmethod
    def from_path(cls, path) -> "GgufLoader":
        """`GgufLoader::from_path` (gguf.rs:45-68)."""
        h = C.c_void_p()
        p = Path(path)
        if not p.is_file():
            raise ModelLoadError(f"Failed to open GGUF file: {p}")
        rc = L.lib().izb_gguf_open(str(p).encode(), C.byref(h))
        if rc != 0:
            raise ModelLoadError(f"Failed to parse GGUF file: {L.lib().izb_status_string(rc).decode()}")
        return cls(p, h)

    def close(self):
        if self._h:
            self._lib.izb_gguf_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- metadata -----------------------------------------------------------------------------
    def metadata_keys(self) -> list:
        return [self._lib.izb_gguf_meta_key(self._h, i).decode() for i in range(self._lib.izb_gguf_meta_count(self._h))]

    def get_metadata_string(self, key: str):
        p, n = C.c_void_p(), C.c_size_t()
        if self._lib.izb_gguf_meta_str(self._h, key.encode(), C.byref(p), C.byref(n)) != 0:
            return None
        return C.string_at(p.value, n.value).decode("utf-8", "replace")

    def get_metadata_u64(self, key: str):
        v = C.c_uint64()
        return int(v.value) if self._lib.izb_gguf_meta_u64(self._h, key.encode(), C.byref(v)) == 0 else None

    def get_metadata_f64(self, key: str):
        v = C.c_double()
        return float(v.value) if self._lib.izb_gguf_meta_f64(self._h, key.encode(), C.byref(v)) == 0 else None

    def detect_quantization_from_tensors(self):
        """The most common quantised tensor type, as the reference reports it when the file carries
        no `general.quantization_type` (gguf.rs: `detect_quantization_from_tensors`)."""
        counts: dict[str, int] = {}
        for t in self._infos.values():
            if t.dtype not in ("F32", "F16", "BF16", "F64", "I8", "I16", "I32", "I64"):
                counts[t.dtype] = counts.get(t.dtype, 0) + 1
        return max(counts, key=counts.get) if counts else None

    def get_model_info(self) -> GgufModelInfo:
        """`GgufLoader::get_model_info` (gguf.rs:71-98)."""
        arch = self.get_metadata_string("general.architecture") or self.get_metadata_string("general.name")
        quant = self.get_metadata_string("general.quantization_type") or self.detect_quantization_from_tensors()
        meta = {}
        for k in self.metadata_keys():
            s = self.get_metadata_string(k)
            if s is None:
                u = self.get_metadata_u64(k)
                s = str(u) if u is not None else None
            if s is None:
                f = self.get_metadata_f64(k)
                s = repr(f) if f is not None else None
            if s is not None:
                meta[k] = s
        return GgufModelInfo(self.path, arch, self.get_metadata_u64("general.parameter_count"), quant, meta)

    # ---- tensors ------------------------------------------------------------------------------
    def tensor_names(self) -> list:
        return list(self._infos)

    def has_tensor(self, name: str) -> bool:
        """`GgufLoader::has_tensor` (gguf.rs:101-103)."""
        return name in self._infos

    def tensor_shape(self, name: str):
        """`GgufLoader::tensor_shape` (gguf.rs:106-111)."""
        t = self._infos.get(name)
        return None if t is None else list(t.shape)

    def tensor_info(self, name: str) -> TensorInfo:
        if name not in self._infos:
            raise ModelLoadError(f"Failed to load tensor '{name}' from GGUF: tensor not found")
        return self._infos[name]

    def tensor_bytes(self, name: str) -> bytes:
        """The tensor's bytes as they sit in the file (host copy)."""
        t = self.tensor_info(name)
        return C.string_at(t._data, t.nbytes)

    def load_qtensor(self, name: str, device) -> QTensor:
        """`GgufLoader::load_qtensor` (gguf.rs:117-125): the raw block bytes on the device."""
        import torch
        info = self.tensor_info(name)
        t = L.GgufTensor()
        if self._lib.izb_gguf_find(self._h, name.encode(), C.byref(t)) != 0:
            raise ModelLoadError(f"Failed to load tensor '{name}' from GGUF: tensor not found")
        dst = torch.empty(max(info.nbytes, 1), dtype=torch.uint8, device=device)[: info.nbytes]
        stream = torch.cuda.current_stream(dst.device).cuda_stream
        with torch.cuda.device(dst.device):
            rc = self._lib.izb_gguf_upload(self._h, C.byref(t), dst.data_ptr(), info.nbytes, stream)
        if rc != 0:
            raise ModelLoadError(f"Failed to load tensor '{name}' from GGUF: status {rc}")
        return QTensor(dst, info.wfmt or info.dtype, info.shape, info.rows, info.cols)

    def load_tensor(self, name: str, dtype, device):
        """`GgufLoader::load_tensor` (gguf.rs:128-143): dequantise when necessary, then cast."""
        import torch

        from . import ops
        q = self.load_qtensor(name, device)
        if q.dtype in ("q8_0", "q4_k", "q6_k"):
            out = ops.dequantize(q.data, q.dtype, q.rows * q.cols, torch.float32)
        elif q.dtype == "bf16":
            out = q.data.view(torch.bfloat16)
        elif q.dtype == "F32":
            out = q.data.view(torch.float32)
        elif q.dtype == "F16":
            out = q.data.view(torch.float16)
        else:
            raise ModelLoadError(f"Failed to dequantize tensor '{name}': unsupported GGML type {q.dtype}")
        return out.reshape(q.shape).to(dtype)
