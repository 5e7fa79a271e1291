"""CPU oracle for the izwi-core matrix-multiplication hot path.

TEST INFRASTRUCTURE ONLY.  This module restates, in NumPy, the arithmetic that
izwi-core delegates to Candle for its Linear / QMatMul call sites, so that the
CUDA kernels can be checked against it.  Nothing in the shipped package may
import it: only the test-suite, the smoke check and the CPU-baseline leg of the
benchmark do, and only as the checker.

The reference's arithmetic lives in un-vendored crates (candle-core /
candle-nn / candle-transformers 0.10.2, CPU GEMM crate `gemm` 0.18.2 / 0.19.0,
`half` 2.7.1), whose sources are not available, so each function follows the
reference *call site* it stands in for and the published GGML block formats.

Pinning:
  * Linear / fused-projection / packed-Q8_0 behaviour is pinned by the
    reference's own unit tests, restated as fixtures in tests/golden/
    (crates/izwi-core/src/models/architectures/qwen3/core.rs:2481-2684,
    3100-3142).
  * Q8_0 / Q4_K block dequantisation is pinned bit-exactly against
    gguf-py 0.19.0 (`gguf.quants.dequantize`), the GGML project's own Python
    restatement of ggml-quants.c; vectors committed in tests/golden/.
  * PARITY UNPINNED for: bf16 GEMM numerics, QMatMul-vs-dense numerics
    (Candle's CPU QMatMul quantises activations per block; see
    `qmatmul_q8_activations`), and everything MoE / tensor-parallel /
    expert-parallel (the reference has no such code; the rules below are this
    project's own specification).
"""
from __future__ import annotations

import numpy as np

# ----------------------------------------------------------------------------
# dtype helpers
# ----------------------------------------------------------------------------

def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round fp32 to the nearest bf16 (ties to even) and return it as fp32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    nan = np.isnan(x)
    out = rounded.astype(np.uint32).view(np.float32).copy()
    out[nan] = np.nan
    return out.reshape(x.shape)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit pattern (uint16), round to nearest even."""
    return (bf16_round(x).view(np.uint32) >> 16).astype(np.uint16)


def bf16_from_bits(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ----------------------------------------------------------------------------
# Linear and the fused projections
# ----------------------------------------------------------------------------

def linear(x: np.ndarray, w: np.ndarray, b: np.ndarray | None = None) -> np.ndarray:
    """`Linear::forward`: Y = X . W^T (+ b), W stored [out, in].

    Call sites: qwen3/core.rs:794 (Qwen3Projection::Dense), :975 (fused QKV),
    :1163 (fused gate/up).  Leading dimensions of X are flattened to M and
    restored afterwards, the rule the reference restates itself in
    granite_speech/asr/runtime.rs:1754-1768.  fp32 with fp64 accumulation so
    the oracle is not the noisy side of a comparison.
    """
    x = np.asarray(x, dtype=np.float32)
    w = np.asarray(w, dtype=np.float32)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.shape[1] != w.shape[1]:
        raise ValueError(f"linear: input dim {x2.shape[1]} != weight in-dim {w.shape[1]}")
    y = (x2.astype(np.float64) @ w.astype(np.float64).T)
    if b is not None:
        y = y + np.asarray(b, dtype=np.float64)
    return y.astype(np.float32).reshape(*lead, w.shape[0])


def concat_biases(name: str, biases: list) -> np.ndarray | None:
    """`concat_linear_biases` (qwen3/core.rs:911-929): all-or-none."""
    present = [b is not None for b in biases]
    if not any(present):
        return None
    if not all(present):
        raise ValueError(f"{name} cannot fuse projections with mixed bias presence")
    return np.concatenate([np.asarray(b, dtype=np.float32) for b in biases], axis=0)


def fused_qkv(x, wq, wk, wv, bq=None, bk=None, bv=None):
    """`Qwen3FusedQkvProjection::{new,forward}` (qwen3/core.rs:931-981).

    W = cat(Wq, Wk, Wv) along the output rows, one matmul, then the last
    dimension is narrowed into q | k | v.
    """
    wq, wk, wv = (np.asarray(t, dtype=np.float32) for t in (wq, wk, wv))
    if wk.shape[1] != wq.shape[1] or wv.shape[1] != wq.shape[1]:
        raise ValueError("Qwen3 fused QKV projection input dimensions do not match")
    w = np.concatenate([wq, wk, wv], axis=0)
    b = concat_biases("Qwen3 fused QKV projection", [bq, bk, bv])
    y = linear(x, w, b)
    q_out, k_out = wq.shape[0], wk.shape[0]
    return y[..., :q_out], y[..., q_out:q_out + k_out], y[..., q_out + k_out:]


def fused_gate_up(x, wg, wu, bg=None, bu=None):
    """`Qwen3FusedGateUpProjection::{new,forward}` (qwen3/core.rs:1132-1168)."""
    wg, wu = np.asarray(wg, dtype=np.float32), np.asarray(wu, dtype=np.float32)
    if wu.shape[0] != wg.shape[0] or wu.shape[1] != wg.shape[1]:
        raise ValueError("Qwen3 fused MLP projection dimensions do not match")
    w = np.concatenate([wg, wu], axis=0)
    b = concat_biases("Qwen3 fused MLP projection", [bg, bu])
    y = linear(x, w, b)
    inter = wg.shape[0]
    return y[..., :inter], y[..., inter:]


def silu_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """`try_fused_silu_mul` (kernels/mod.rs:94-108 -> kernels/cuda.rs:51-62).

    silu(g) * u with silu(x) = x / (1 + exp(-x)), the formula of the
    reference's own fused kernel (kernels/metal.rs:39-40); fp32 math.
    """
    g = np.asarray(gate, dtype=np.float32)
    u = np.asarray(up, dtype=np.float32)
    if g.shape != u.shape:
        raise ValueError("silu_mul: gate/up shape mismatch")
    with np.errstate(over="ignore"):
        return (g / (np.float32(1.0) + np.exp(-g))) * u


def gelu_tanh(x: np.ndarray) -> np.ndarray:
    """tanh-form GELU, 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))): what the reference writes out
    wherever it spells GELU itself (audio/codec.rs:135-137, voxtral/realtime/audio.rs:73-88) and, by
    its separate use of `gelu_erf()` elsewhere, what `Tensor::gelu()` after Whisper's fc1 stands for
    (whisper/model.rs:311-317).  Candle's source is absent, so that mapping is inferred."""
    x = np.asarray(x, dtype=np.float64)
    return (0.5 * x * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (x + 0.044715 * x ** 3)))).astype(np.float32)


def gelu_erf(x: np.ndarray) -> np.ndarray:
    """Exact (erf) GELU: the reference's `gelu_erf()` call sites (granite_speech/asr/runtime.rs:1639,
    qwen3/tts/speech_tokenizer.rs:670)."""
    from math import sqrt
    from scipy.special import erf
    x = np.asarray(x, dtype=np.float64)
    return (0.5 * x * (1.0 + erf(x / sqrt(2.0)))).astype(np.float32)


def mlp_forward(x, w_gate_up, w_down, inter, round_bf16=False):
    """`Qwen3Mlp::forward` (qwen3/core.rs:1786-1798): down(silu(gate) * up)."""
    gu = linear(x, w_gate_up)
    if round_bf16:
        gu = bf16_round(gu)
    h = silu_mul(gu[..., :inter], gu[..., inter:])
    if round_bf16:
        h = bf16_round(h)
    return linear(h, w_down)


# ----------------------------------------------------------------------------
# GGML block formats (Q8_0, Q4_K)
# ----------------------------------------------------------------------------

Q8_0, Q4_K, Q6_K = "q8_0", "q4_k", "q6_k"
BLOCK_SIZE = {Q8_0: 32, Q4_K: 256, Q6_K: 256}
TYPE_SIZE = {Q8_0: 34, Q4_K: 144, Q6_K: 210}


def quantized_storage_bytes(rows: int, cols: int, fmt: str) -> int:
    """`quantized_storage_bytes` (qwen3/core.rs:891-909)."""
    elems = rows * cols
    if elems % BLOCK_SIZE[fmt] != 0:
        raise ValueError(
            f"Qwen3 quantized projection element count {elems} is not divisible by block size {BLOCK_SIZE[fmt]}")
    return elems // BLOCK_SIZE[fmt] * TYPE_SIZE[fmt]


def pack_quantized_rows(tensors: list) -> tuple:
    """`packed_qmatmul_from_qtensors` (qwen3/core.rs:846-885).

    `tensors` is a list of (raw_bytes, rows, cols, fmt); the raw GGML bytes are
    concatenated row-wise.  Returns (raw, total_rows, cols, fmt).
    """
    if not tensors:
        raise ValueError("Cannot pack empty Qwen3 quantized projection group")
    raw0, total_rows, cols, fmt = tensors[0]
    parts = [np.asarray(raw0, dtype=np.uint8).ravel()]
    for raw, r, c, f in tensors[1:]:
        if c != cols:
            raise ValueError(f"Qwen3 quantized projection group input mismatch: expected {cols}, got {c}")
        if f != fmt:
            raise ValueError(f"Qwen3 quantized projection group dtype mismatch: expected {fmt}, got {f}")
        parts.append(np.asarray(raw, dtype=np.uint8).ravel())
        total_rows += r
    out = np.concatenate(parts)
    expected = quantized_storage_bytes(total_rows, cols, fmt)
    if out.size != expected:
        raise ValueError(f"Qwen3 packed quantized projection has {out.size} bytes, expected {expected}")
    return out, total_rows, cols, fmt


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """GGML Q8_0 quantisation of an fp32 array (last dim % 32 == 0).

    Per 32-value block: d = max|x| / 127, q = round-half-away(x / d) as int8,
    stored as fp16 d followed by 32 int8.  This is what `QTensor::quantize(..,
    GgmlDType::Q8_0)` does in the reference's packed-QMatMul test
    (qwen3/core.rs:3112-3113).
    """
    x = np.asarray(x, dtype=np.float32)
    blocks = x.reshape(-1, 32)
    d = np.abs(blocks).max(axis=1, keepdims=True) / np.float32(127.0)
    with np.errstate(divide="ignore"):
        inv = np.where(d == 0, np.float32(0), np.float32(1.0) / d).astype(np.float32)
    v = blocks * inv
    q = (np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))).astype(np.int8)
    out = np.empty((blocks.shape[0], 34), dtype=np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def dequantize_mlx_affine(packed: np.ndarray, scales: np.ndarray, biases, out_dim: int, in_dim: int) -> np.ndarray:
    """MLX affine-packed weights -> dense fp32 [out_dim, in_dim] (models/shared/weights/mlx.rs:50-236).
    `packed` is uint32 or uint8 [out_dim, packed_in]; pack = in_dim / packed_in values sit in one word,
    bits = word_bits / pack each, value pi of a word at bit pi * bits.  `scales` / `biases` are
    [out_dim, groups] or [groups, out_dim] (transposed back, mlx.rs:66-74); biases may be None (zeros).
    value = q * scale + bias in fp32, the product and the sum rounded separately."""
    packed = np.asarray(packed)
    if packed.dtype not in (np.uint32, np.uint8) or packed.ndim != 2:
        raise ValueError("packed weight must be a 2-D uint32 or uint8 array")
    word_bits = 32 if packed.dtype == np.uint32 else 8
    if packed.shape[0] != out_dim:
        raise ValueError(f"quantized weight rows mismatch: expected out_dim={out_dim}, packed_rows={packed.shape[0]}")
    packed_in = packed.shape[1]
    if packed_in == 0 or in_dim == 0:
        raise ValueError("invalid packed shape for quantized weight")
    if in_dim % packed_in != 0:
        raise ValueError(f"incompatible input dim: expected_in={in_dim}, packed_in={packed_in}")
    pack = in_dim // packed_in
    if word_bits % pack != 0:
        raise ValueError(f"invalid quant packing factor: word_bits={word_bits}, pack_factor={pack}")
    bits = word_bits // pack
    if bits == 0 or bits > 8:
        raise ValueError(f"unsupported quantization bit-width inferred from packing: {bits}")
    scales = np.asarray(scales, dtype=np.float32)
    if scales.ndim != 2 or scales.size == 0:
        raise ValueError("empty quantization scales")
    biases = None if biases is None else np.asarray(biases, dtype=np.float32)
    if scales.shape[0] == out_dim:
        groups = scales.shape[1]
    elif scales.shape[1] == out_dim:
        groups = scales.shape[0]
        scales = scales.T
        biases = None if biases is None else biases.T
    else:
        raise ValueError(f"quantization scales shape mismatch: expected out_dim={out_dim}, got {scales.shape}")
    if groups == 0 or in_dim % groups != 0:
        raise ValueError(f"invalid quantization groups: in_dim={in_dim}, groups={groups}")
    if biases is None:
        biases = np.zeros((out_dim, groups), dtype=np.float32)
    elif biases.shape != (out_dim, groups):
        raise ValueError(f"quantization biases shape mismatch: expected ({out_dim},{groups})")
    group_size = in_dim // groups
    mask = np.uint32((1 << bits) - 1)
    words = packed.astype(np.uint32)
    shifts = (np.arange(pack, dtype=np.uint32) * np.uint32(bits))[None, None, :]
    q = ((words[:, :, None] >> shifts) & mask).reshape(out_dim, in_dim).astype(np.float32)
    g = np.arange(in_dim) // group_size
    prod = (q * scales[:, g]).astype(np.float32)
    return (prod + biases[:, g]).astype(np.float32)


def dequantize_q8_0(raw: np.ndarray) -> np.ndarray:
    """Q8_0: 34-byte blocks of (fp16 d, 32 x int8 q); value = d * q in fp32."""
    blocks = np.asarray(raw, dtype=np.uint8).reshape(-1, 34)
    d = blocks[:, :2].copy().view(np.float16).astype(np.float32)
    q = blocks[:, 2:].copy().view(np.int8).astype(np.float32)
    return (d * q).reshape(-1)


def q4_k_scale_min(scales: np.ndarray) -> tuple:
    """Unpack the 12 scale bytes of a Q4_K super-block into 8 six-bit scales
    and 8 six-bit mins.  Bytes 0-3 hold the low 6 bits of scales 0-3 (top two
    bits: high bits of scales 4-7), bytes 4-7 the same for mins, bytes 8-11
    the low nibbles of scales 4-7 (low half) and of mins 4-7 (high half)."""
    s = np.asarray(scales, dtype=np.uint8).reshape(-1, 12)
    a, b, c = s[:, 0:4], s[:, 4:8], s[:, 8:12]
    sc = np.concatenate([a & 0x3F, (c & 0x0F) | ((a >> 2) & 0x30)], axis=1)
    mn = np.concatenate([b & 0x3F, (c >> 4) | ((b >> 2) & 0x30)], axis=1)
    return sc, mn


def dequantize_q4_k(raw: np.ndarray) -> np.ndarray:
    """Q4_K: 144-byte super-blocks of 256 values: fp16 d, fp16 dmin, 12 bytes
    of 6-bit sub-block scales/mins, 128 bytes of 4-bit codes.  Codes are laid
    out in four 32-byte groups; in group j the low nibbles are sub-block 2j and
    the high nibbles sub-block 2j+1.  value = (d*sc)*q - (dmin*m), each product
    and the difference rounded to fp32 separately (no fused multiply-add)."""
    blocks = np.asarray(raw, dtype=np.uint8).reshape(-1, 144)
    d = blocks[:, 0:2].copy().view(np.float16).astype(np.float32)
    dmin = blocks[:, 2:4].copy().view(np.float16).astype(np.float32)
    sc, mn = q4_k_scale_min(blocks[:, 4:16])
    dsc = (d * sc.astype(np.float32))            # [nb, 8]
    dm = (dmin * mn.astype(np.float32))          # [nb, 8]
    qs = blocks[:, 16:].reshape(-1, 4, 32)
    lo = (qs & 0x0F).astype(np.float32)
    hi = (qs >> 4).astype(np.float32)
    q = np.stack([lo, hi], axis=2).reshape(-1, 8, 32)   # sub-block order 0..7
    y = dsc[:, :, None] * q
    y = y - dm[:, :, None]
    return y.astype(np.float32).reshape(-1)


def dequantize_q6_k(raw: np.ndarray) -> np.ndarray:
    """Q6_K (the format of some tensors inside Q4_K_M files): 210-byte super-blocks of 256 values:
    128 bytes of low nibbles `ql`, 64 bytes of 2-bit high parts `qh`, 16 int8 scales (one per 16
    values), fp16 d.  In each half of 128 values, value l + 32 g (l < 32, g < 4) takes its low
    nibble from ql[l + 32 (g & 1)] (low nibble for g < 2, high nibble otherwise), its high two
    bits from bits 2g..2g+1 of qh[l], and scale index l / 16 + 2 g; code = that 6-bit number - 32.
    value = (d * scale) * code, the two products rounded to fp32 separately."""
    blocks = np.asarray(raw, dtype=np.uint8).reshape(-1, 210)
    nb = blocks.shape[0]
    ql = blocks[:, 0:128].reshape(nb, 2, 2, 32)          # [block, half, g & 1, l]
    qh = blocks[:, 128:192].reshape(nb, 2, 32)           # [block, half, l]
    sc = blocks[:, 192:208].copy().view(np.int8).astype(np.float32).reshape(nb, 2, 8)
    d = blocks[:, 208:210].copy().view(np.float16).astype(np.float32)  # [nb, 1]
    out = np.empty((nb, 2, 4, 32), dtype=np.float32)
    for g in range(4):
        nib = (ql[:, :, g & 1, :] & 0x0F) if g < 2 else (ql[:, :, g & 1, :] >> 4)
        hi = (qh >> (2 * g)) & 3
        q = (nib | (hi << 4)).astype(np.int16) - 32
        scale = sc[:, :, 2 * g:2 * g + 2]                  # [nb, 2, 2]: l / 16 selects
        dsc = (d[:, :, None] * scale).astype(np.float32)  # [nb, 2, 2]
        dsc_l = np.repeat(dsc, 16, axis=2)                 # [nb, 2, 32]
        out[:, :, g, :] = dsc_l * q.astype(np.float32)
    return out.reshape(-1)


def dequantize(raw: np.ndarray, fmt: str) -> np.ndarray:
    if fmt == Q8_0:
        return dequantize_q8_0(raw)
    if fmt == Q4_K:
        return dequantize_q4_k(raw)
    if fmt == Q6_K:
        return dequantize_q6_k(raw)
    raise ValueError(f"unknown format {fmt}")


def make_q6_k_blocks(rng: np.random.Generator, n_blocks: int, d_scale=2e-4) -> np.ndarray:
    """Synthetic Q6_K super-blocks built field by field: uniform 6-bit codes, int8 scales uniform
    in [-128, 127], fp16 d ~ |N(0, scale)|."""
    out = np.empty((n_blocks, 210), dtype=np.uint8)
    out[:, 0:192] = rng.integers(0, 256, (n_blocks, 192), dtype=np.uint8)
    out[:, 192:208] = rng.integers(-128, 128, (n_blocks, 16), dtype=np.int8).view(np.uint8)
    d = np.abs(rng.normal(0.0, d_scale, n_blocks)).astype(np.float16)
    out[:, 208:210] = d.view(np.uint8).reshape(-1, 2)
    return out.reshape(-1)


def make_q4_k_blocks(rng: np.random.Generator, n_blocks: int, d_scale=0.002, dmin_scale=0.002) -> np.ndarray:
    """Synthetic Q4_K super-blocks built field by field (never from raw random
    bytes, which would put NaN/Inf into the fp16 fields): uniform 4-bit codes,
    uniform 6-bit scales and mins, fp16 d and dmin ~ |N(0, scale)|."""
    out = np.empty((n_blocks, 144), dtype=np.uint8)
    d = np.abs(rng.normal(0.0, d_scale, n_blocks)).astype(np.float16)
    dmin = np.abs(rng.normal(0.0, dmin_scale, n_blocks)).astype(np.float16)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = dmin.view(np.uint8).reshape(-1, 2)
    sc = rng.integers(0, 64, (n_blocks, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, (n_blocks, 8), dtype=np.uint8)
    out[:, 4:8] = (sc[:, 0:4] & 0x3F) | ((sc[:, 4:8] >> 4) << 6)
    out[:, 8:12] = (mn[:, 0:4] & 0x3F) | ((mn[:, 4:8] >> 4) << 6)
    out[:, 12:16] = (sc[:, 4:8] & 0x0F) | ((mn[:, 4:8] & 0x0F) << 4)
    out[:, 16:] = rng.integers(0, 256, (n_blocks, 128), dtype=np.uint8)
    return out.reshape(-1)


def make_q8_0_blocks(rng: np.random.Generator, n_blocks: int, d_scale=0.002) -> np.ndarray:
    """Synthetic Q8_0 blocks: int8 uniform in [-127, 127], fp16 d ~ |N(0, scale)|."""
    out = np.empty((n_blocks, 34), dtype=np.uint8)
    d = np.abs(rng.normal(0.0, d_scale, n_blocks)).astype(np.float16)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:] = rng.integers(-127, 128, (n_blocks, 32), dtype=np.int8).view(np.uint8)
    return out.reshape(-1)


def qmatmul(x: np.ndarray, raw: np.ndarray, n: int, k: int, fmt: str) -> np.ndarray:
    """`QMatMul::forward` (call site qwen3/core.rs:812) stated as the exact
    product dequant(W) . X in fp32 (fp64 accumulate): the primary target."""
    w = dequantize(raw, fmt).reshape(n, k)
    return linear(x, w)


def qmatmul_q8_activations(x: np.ndarray, raw: np.ndarray, n: int, k: int) -> np.ndarray:
    """Q8_0 x Q8_0 emulation of the GGML CPU convention: activations are
    themselves quantised to Q8_0 per 32-value block and the block dot products
    are integer.  Used only to *report* the gap between that convention and the
    exact product above, and for the packed-vs-separate structural test."""
    x = np.asarray(x, dtype=np.float32)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, k)
    xq = quantize_q8_0(x2).reshape(x2.shape[0], k // 32, 34)
    xd = xq[:, :, :2].copy().view(np.float16).astype(np.float32)[..., 0]
    xi = xq[:, :, 2:].copy().view(np.int8).astype(np.int32)
    wb = np.asarray(raw, dtype=np.uint8).reshape(n, k // 32, 34)
    wd = wb[:, :, :2].copy().view(np.float16).astype(np.float32)[..., 0]
    wi = wb[:, :, 2:].copy().view(np.int8).astype(np.int32)
    isum = np.einsum("mbk,nbk->mnb", xi, wi).astype(np.float32)
    y = (isum * xd[:, None, :] * wd[None, :, :]).sum(axis=2, dtype=np.float32)
    return y.reshape(*lead, n)


# ----------------------------------------------------------------------------
# Mixture-of-experts path.  The reference has no MoE code; the rules below are
# this project's specification (softmax -> top-k -> renormalise; ties go to
# the lowest expert id; stable (expert, token) order; fixed combine order).
# ----------------------------------------------------------------------------

def moe_router_logits(x, w_router, bias=None):
    """logits[T, E] = X . Wr^T + bias, fp32."""
    return linear(x, w_router, bias)


def moe_topk(logits: np.ndarray, k: int) -> tuple:
    """Top-k experts per token by logit, descending; equal logits resolve to
    the lowest expert id.  Weights are the softmax over all experts
    renormalised over the selected k, which equals a softmax over the k
    selected logits; computed as exp(l - l_max) / sum in fp32."""
    logits = np.asarray(logits, dtype=np.float32)
    t, e = logits.shape
    order = np.lexsort((np.broadcast_to(np.arange(e), (t, e)), -logits.astype(np.float64)), axis=1)
    idx = order[:, :k].astype(np.int32)
    sel = np.take_along_axis(logits, idx, axis=1)
    ex = np.exp(sel - sel[:, :1])
    w = ex / ex.sum(axis=1, keepdims=True, dtype=np.float32)
    return idx, w.astype(np.float32)


def moe_permute(idx: np.ndarray, n_experts: int) -> tuple:
    """Stable sort of the (token, slot) pairs by expert.

    Returns (offsets[E+1], perm[T*k]) where perm[p] = t*k + slot is the pair
    that lands in permuted row p; inside one expert the pairs keep ascending
    (token, slot) order."""
    flat = np.asarray(idx, dtype=np.int64).reshape(-1)
    perm = np.argsort(flat, kind="stable").astype(np.int32)
    counts = np.bincount(flat, minlength=n_experts)
    offsets = np.zeros(n_experts + 1, dtype=np.int32)
    offsets[1:] = np.cumsum(counts)
    return offsets, perm


def moe_expert_ffn(xe, wg, wu, wd, round_bf16=True):
    """One expert: down( silu(x.Wg^T) * (x.Wu^T) ); intermediate rounded to
    bf16 where the GPU path stores bf16."""
    g = linear(xe, wg)
    u = linear(xe, wu)
    if round_bf16:
        g, u = bf16_round(g), bf16_round(u)
    h = silu_mul(g, u)
    if round_bf16:
        h = bf16_round(h)
    return linear(h, wd)


def moe_forward(x, w_router, router_bias, wg, wu, wd, k, round_bf16=True, logits=None):
    """Whole MoE FFN layer.  wg/wu: [E, I, H], wd: [E, H, I].

    Y[t] = sum over slots in ascending slot order of w[t,slot] * FFN_e(x[t]),
    accumulated in fp32."""
    x = np.asarray(x, dtype=np.float32)
    t, h = x.shape
    e = wg.shape[0]
    if logits is None:
        logits = moe_router_logits(x, w_router, router_bias)
    idx, wts = moe_topk(logits, k)
    offsets, perm = moe_permute(idx, e)
    xp = x[perm // k]
    yp = np.zeros((t * k, wd.shape[1]), dtype=np.float32)
    for ex in range(e):
        lo, hi = offsets[ex], offsets[ex + 1]
        if hi > lo:
            yp[lo:hi] = moe_expert_ffn(xp[lo:hi], wg[ex], wu[ex], wd[ex], round_bf16)
    if round_bf16:
        yp = bf16_round(yp)
    inv = np.empty(t * k, dtype=np.int64)
    inv[perm] = np.arange(t * k)
    y = np.zeros((t, wd.shape[1]), dtype=np.float32)
    for slot in range(k):
        y += wts[:, slot:slot + 1] * yp[inv[np.arange(t) * k + slot]]
    return y, dict(logits=logits, idx=idx, weights=wts, offsets=offsets, perm=perm)


# ----------------------------------------------------------------------------
# accuracy gates
# ----------------------------------------------------------------------------

def rel_err_and_cosine(got: np.ndarray, want: np.ndarray) -> tuple:
    """Max |got-want| relative to max|want| of the same row, and the cosine of
    the flattened tensors: the two gates stated for bf16 matmul outputs
    (max relative error <= 2e-2, cosine >= 0.9999)."""
    g = np.asarray(got, dtype=np.float64).reshape(-1, got.shape[-1])
    w = np.asarray(want, dtype=np.float64).reshape(-1, want.shape[-1])
    denom = np.abs(w).max(axis=1, keepdims=True)
    denom = np.where(denom == 0, 1.0, denom)
    rel = float((np.abs(g - w) / denom).max()) if g.size else 0.0
    gn, wn = np.linalg.norm(g), np.linalg.norm(w)
    cos = float((g * w).sum() / (gn * wn)) if gn > 0 and wn > 0 else 1.0
    return rel, cos


# ---------------------------------------------------------------------------
# glue around the projections of a decode step
# ---------------------------------------------------------------------------
def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float, residual: np.ndarray | None = None):
    """`candle_nn::ops::rms_norm` as called by `try_fused_rms_norm` (kernels/cuda.rs:78-84) and by
    `RmsNorm::forward` for the q/k norms (qwen3/core.rs:1446-1463): x * rsqrt(mean(x^2) + eps) *
    weight over the last dimension, fp32 arithmetic on bf16 inputs, one rounding to bf16.  With a
    residual the sum is first rounded to bf16, as the reference's bf16 tensor add does.
    Returns (out, h) with h the (rounded) input of the normalisation."""
    h = np.asarray(x, dtype=np.float32)
    if residual is not None:
        h = bf16_round(h + np.asarray(residual, dtype=np.float32))
    ms = (h.astype(np.float64) ** 2).mean(axis=-1, keepdims=True)
    scale = (1.0 / np.sqrt(ms + eps)).astype(np.float32)
    out = bf16_round(h * scale * np.asarray(weight, dtype=np.float32))
    return out, h


def argmax_rows(x: np.ndarray):
    """Greedy choice over logits rows (`argmax`, qwen3/chat.rs:574-601): lowest index among equal
    maxima; NaN is never selected (a row of only NaN gives index 0)."""
    x = np.asarray(x, dtype=np.float32)
    clean = np.where(np.isnan(x), -np.inf, x)
    return clean.argmax(axis=-1).astype(np.int32), clean.max(axis=-1)


def rope_pair(x: np.ndarray, cos_half: np.ndarray, sin_half: np.ndarray) -> np.ndarray:
    """`apply_rotary_emb` (qwen3/core.rs:2402-2415) on x [tokens, heads, d] with tables
    [tokens, d / 2]: first half x1 cos - x2 sin, second half x1 sin + x2 cos; fp32, one rounding."""
    x = np.asarray(x, dtype=np.float32)
    half = x.shape[-1] // 2
    c = np.asarray(cos_half, dtype=np.float32)[:, None, :]
    s = np.asarray(sin_half, dtype=np.float32)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return bf16_round(np.concatenate([x1 * c - x2 * s, x1 * s + x2 * c], axis=-1))


def decode_gqa_attention(q: np.ndarray, k_cache: np.ndarray, v_cache: np.ndarray, kv_len: int, scale: float) -> np.ndarray:
    """`dense_decode_attention` (qwen3/core.rs:2189-2225): q [batch, heads, d] against head-major
    caches [batch, kv_heads, capacity, d]; softmax(q k^T * scale) v per head in fp64, query head h
    reading KV head h // (heads // kv_heads) (`repeat_kv`).  Returns fp32 (not rounded)."""
    q = np.asarray(q, dtype=np.float64)
    b, h, d = q.shape
    kvh = k_cache.shape[1]
    g = h // kvh
    out = np.empty((b, h, d), dtype=np.float64)
    for bi in range(b):
        for hi in range(h):
            k = np.asarray(k_cache[bi, hi // g, :kv_len], dtype=np.float64)
            v = np.asarray(v_cache[bi, hi // g, :kv_len], dtype=np.float64)
            s = k @ q[bi, hi] * scale
            p = np.exp(s - s.max())
            out[bi, hi] = (p / p.sum()) @ v
    return out.astype(np.float32)


# ----------------------------------------------------------------------------
# Conformer convolution module (parakeet/asr/mod.rs:775-893)
# ----------------------------------------------------------------------------

def glu(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """`x_a.broadcast_mul(&ops::sigmoid(&x_b))` behind pointwise_conv1 (parakeet/asr/mod.rs:832-834)."""
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return (a / (1.0 + np.exp(-b))).astype(np.float32)


def fold_depthwise_conv1d_batch_norm(conv_weight, bn_weight, bn_bias, running_mean, running_var, eps):
    """`fold_depthwise_conv1d_batch_norm` (parakeet/asr/mod.rs:866-893): conv_weight [C, k] fp32."""
    std = np.sqrt(np.asarray(running_var, dtype=np.float32) + np.float32(eps))
    scale = (np.asarray(bn_weight, dtype=np.float32) / std) if bn_weight is not None else (np.float32(1.0) / std)
    if bn_bias is not None:
        folded_bias = np.asarray(bn_bias, dtype=np.float32) - scale * np.asarray(running_mean, dtype=np.float32)
    else:
        folded_bias = -(scale * np.asarray(running_mean, dtype=np.float32))
    return (np.asarray(conv_weight, dtype=np.float32) * scale[:, None]).astype(np.float32), folded_bias.astype(np.float32)


def depthwise_conv1d_bias_swish(x: np.ndarray, weight: np.ndarray, bias, swish: bool = True) -> np.ndarray:
    """Depthwise "same" convolution over time, folded bias, swish (`swish`, parakeet/asr/mod.rs:1215-1217):
    x [B, T, C], weight [C, k], zero padding (k - 1) / 2 on both ends of every utterance."""
    x = np.asarray(x, dtype=np.float64)
    w = np.asarray(weight, dtype=np.float64)
    b, t, c = x.shape
    k = w.shape[1]
    pad = (k - 1) // 2
    xp = np.zeros((b, t + 2 * pad, c))
    xp[:, pad:pad + t] = x
    out = np.zeros((b, t, c))
    for j in range(k):
        out += xp[:, j:j + t] * w[None, None, :, j]
    if bias is not None:
        out += np.asarray(bias, dtype=np.float64)[None, None, :]
    if swish:
        out = out / (1.0 + np.exp(-out))
    return out.astype(np.float32)


# ----------------------------------------------------------------------------
# token sampling (lfm25_audio/sampling.rs:65-160, qwen3/tts/mod.rs:2293-2440)
# ----------------------------------------------------------------------------

def sample_from_logits(logits: np.ndarray, temperature: float, top_k: int, top_p: float, u: float):
    """`sample_from_logits` restated: returns (token, margin) where margin is the distance of `u` from the
    nearest boundary of the cumulative distribution it was compared with (a draw that close to a boundary
    may legitimately fall either way under a different summation order).  float64 arithmetic."""
    logits = np.asarray(logits, dtype=np.float32)
    finite = np.isfinite(logits)
    if temperature <= 1e-5 or not finite.any():
        masked = np.where(finite, logits, -np.inf)
        return int(np.argmax(masked)), 1.0
    values = logits.astype(np.float32) * np.float32(1.0 / max(temperature, 1e-5))   # the kernel multiplies by 1 / T
    cand = np.nonzero(finite)[0]
    ordered = False
    if 0 < top_k < len(cand):
        order = np.argsort(-values[cand].astype(np.float64), kind="stable")
        cand = cand[order][:top_k]
        ordered = True
    v = values[cand].astype(np.float64)
    probs = np.exp(v - v.max())
    probs /= probs.sum()
    if top_p < 1.0:
        order = np.argsort(-probs, kind="stable")
        cand, probs = cand[order], probs[order]
        cum = np.cumsum(probs)
        keep = int(np.searchsorted(cum, max(top_p, 1e-6), side="left")) + 1
        keep = max(1, min(keep, len(cand)))
        cand, probs = cand[:keep], probs[:keep]
        probs = probs / probs.sum()
        ordered = True
    cum = np.cumsum(probs)
    pos = int(np.searchsorted(cum, u, side="left"))
    pos = min(pos, len(cand) - 1)
    edges = np.concatenate([[0.0], cum])
    margin = float(np.abs(edges - u).min())
    return int(cand[pos]), margin


# ----------------------------------------------------------------------------
# paged KV cache (models/shared/attention/paged.rs)
# ----------------------------------------------------------------------------

def _round_half_away(x: np.ndarray) -> np.ndarray:
    """f32::round: halves away from zero."""
    return np.sign(x) * np.floor(np.abs(x) + 0.5)


def kv_quantize_int8(page: np.ndarray):
    """`quantize_tensor_int8` (paged.rs:158-184) for a bf16 page: every product is rounded to bf16, as
    the reference computes in the cache dtype.  Returns (u8 values, f32 scale)."""
    x = bf16_round(np.asarray(page, dtype=np.float32))
    max_abs = np.float32(np.abs(x).max()) if x.size else np.float32(0)
    scale = np.float32(max(np.float32(max_abs / np.float32(127.0)), np.float32(1e-8))) if max_abs > 0 else np.float32(1.0)
    inv = bf16_round(np.array([np.float32(1.0) / scale], dtype=np.float32))[0]
    y = bf16_round(x * inv)
    y = _round_half_away(np.clip(y, -127.0, 127.0))
    return (y + 128.0).astype(np.uint8), scale


def kv_dequantize_int8(values: np.ndarray, scale) -> np.ndarray:
    """`dequantize_tensor_int8` (paged.rs:186-198): bf16 result."""
    dense = values.astype(np.float32) - np.float32(128.0)
    if abs(float(scale) - 1.0) < np.finfo(np.float32).eps:
        return dense
    return bf16_round(dense * bf16_round(np.array([scale], dtype=np.float32))[0])


def kv_quantize_q4_0(page: np.ndarray):
    """`quantize_tensor_q4_0` (paged.rs:204-268): flat blocks of 32, scale = max|x| / 7 (1 if zero), codes
    clamp(round(x / scale), -7, 7) + 8, two per byte (low nibble first).  Returns (packed u8, f32 scales)."""
    x = bf16_round(np.asarray(page, dtype=np.float32)).reshape(-1)
    assert x.size % 32 == 0
    blocks = x.reshape(-1, 32)
    max_abs = np.abs(blocks).max(axis=1).astype(np.float32)
    scales = np.where(max_abs > 0, max_abs / np.float32(7.0), np.float32(1.0)).astype(np.float32)
    inv = (np.float32(1.0) / scales).astype(np.float32)
    q = np.clip(_round_half_away((blocks * inv[:, None]).astype(np.float32)), -7, 7).astype(np.int32) + 8
    packed = (q[:, 0::2] & 0x0F) | ((q[:, 1::2] & 0x0F) << 4)
    return packed.astype(np.uint8).reshape(-1), scales


def kv_dequantize_q4_0(packed: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """`dequantize_tensor_q4_0` (paged.rs:270-343), then the cast to the cache dtype (bf16)."""
    b = packed.reshape(-1, 16)
    q = np.empty((b.shape[0], 32), dtype=np.float32)
    q[:, 0::2] = (b & 0x0F).astype(np.float32)
    q[:, 1::2] = (b >> 4).astype(np.float32)
    return bf16_round(((q - np.float32(8.0)) * scales[:, None].astype(np.float32)).reshape(-1))


class KvPages:
    """One sequence's pages of K or V: `append_to_pages` (paged.rs:345-388) and `materialize_pages`
    (:390-405).  Pages hold [page_seq, kv_heads, head_dim] values (batch 1)."""

    def __init__(self, page_size: int, quantization: str):
        if page_size <= 0:
            raise ValueError("KV page size must be greater than zero")
        self.page_size, self.quantization, self.pages = page_size, quantization, []

    def _from_dense(self, t: np.ndarray):
        t = bf16_round(np.asarray(t, dtype=np.float32))
        if self.quantization == "none":
            return ("dense", t)
        if self.quantization == "int8":
            v, s = kv_quantize_int8(t)
            return ("int8", v, s, t.shape)
        v, s = kv_quantize_q4_0(t)
        return ("q4_0", v, s, t.shape)

    @staticmethod
    def _to_dense(page) -> np.ndarray:
        if page[0] == "dense":
            return page[1]
        if page[0] == "int8":
            return kv_dequantize_int8(page[1], page[2]).reshape(page[3])
        return kv_dequantize_q4_0(page[1], page[2]).reshape(page[3])

    def append(self, rows: np.ndarray) -> None:
        """rows [seq, kv_heads, head_dim]: the last page is filled first (and rebuilt), then new pages pushed."""
        cursor, n = 0, rows.shape[0]
        while cursor < n:
            if self.pages and self._to_dense(self.pages[-1]).shape[0] < self.page_size:
                last = self._to_dense(self.pages[-1])
                take = min(self.page_size - last.shape[0], n - cursor)
                self.pages[-1] = self._from_dense(np.concatenate([last, rows[cursor:cursor + take]], axis=0))
            else:
                take = min(self.page_size, n - cursor)
                self.pages.append(self._from_dense(rows[cursor:cursor + take]))
            cursor += take

    def materialize(self) -> np.ndarray:
        return np.concatenate([self._to_dense(p) for p in self.pages], axis=0)


def paged_decode_attention(q: np.ndarray, k_pages: KvPages, v_pages: KvPages, scale: float) -> np.ndarray:
    """`paged_decode_attention` (paged.rs:486-628) for one sequence: q [heads, d]; a running maximum, sum
    and output over the pages, query head h reading KV head h // (heads // kv_heads).  float64."""
    h, d = q.shape
    run_max = np.full(h, -np.inf)
    run_sum = np.zeros(h)
    run_out = np.zeros((h, d))
    for kp, vp in zip(k_pages.pages, v_pages.pages):
        k, v = KvPages._to_dense(kp).astype(np.float64), KvPages._to_dense(vp).astype(np.float64)
        rep = h // k.shape[1]
        for head in range(h):
            s = (k[:, head // rep] @ q[head].astype(np.float64)) * scale
            m = s.max()
            e = np.exp(s - m)
            new_max = max(run_max[head], m)
            cs, ps = np.exp(run_max[head] - new_max), np.exp(m - new_max)
            run_sum[head] = run_sum[head] * cs + e.sum() * ps
            run_out[head] = run_out[head] * cs + (e @ v[:, head // rep]) * ps
            run_max[head] = new_max
    return (run_out / run_sum[:, None]).astype(np.float32)
