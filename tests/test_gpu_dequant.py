"""Block dequantisation on the GPU: bit-exact against the gguf-py golden vectors
and the oracle, through izb_dequantize."""
import numpy as np
import pytest
import torch

import izwi_oracle as o
from gpu_util import to_np

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k", "q6_k"])
def test_golden_vectors_bit_exact(cuda, golden_dir, fmt):
    from izwi_b200 import ops
    vec = np.load(golden_dir / "ggml_dequant.npz")
    raw = torch.from_numpy(vec[f"{fmt}_raw"]).to(cuda)
    want = vec[f"{fmt}_f32"]
    got = ops.dequantize(raw, fmt, want.size, torch.float32)
    assert np.array_equal(to_np(got).view(np.uint32), want.view(np.uint32))
    got16 = ops.dequantize(raw, fmt, want.size, torch.bfloat16)
    assert np.array_equal(to_np(got16).view(np.uint32), o.bf16_round(want).view(np.uint32))


@pytest.mark.parametrize("fmt,n_blocks", [("q8_0", 1), ("q8_0", 4099), ("q4_k", 1), ("q4_k", 2053), ("q6_k", 1), ("q6_k", 1031)])
def test_seeded_blocks_bit_exact(cuda, fmt, n_blocks):
    from izwi_b200 import ops
    rng = np.random.default_rng(n_blocks)
    raw = {"q8_0": o.make_q8_0_blocks, "q4_k": o.make_q4_k_blocks, "q6_k": o.make_q6_k_blocks}[fmt](rng, n_blocks)
    want = o.dequantize(raw, fmt)
    got = ops.dequantize(torch.from_numpy(raw).to(cuda), fmt, want.size)
    assert np.array_equal(to_np(got).view(np.uint32), want.view(np.uint32))


def test_empty_and_bad_arguments(cuda):
    from izwi_b200 import IzbError, ops
    empty = torch.empty(0, dtype=torch.uint8, device=cuda)
    assert ops.dequantize(empty, "q8_0", 0).numel() == 0
    raw = torch.zeros(34, dtype=torch.uint8, device=cuda)
    with pytest.raises(IzbError) as e:
        ops.dequantize(raw, "q8_0", 33)
    assert e.value.status == -1
    with pytest.raises(IzbError) as e:
        ops.dequantize(raw, "bf16", 32)
    assert e.value.status == -2


def test_full_size_round_trip_property(cuda):
    """At full projection size: quantise -> dequantise on the GPU reproduces the
    oracle's value for every element and stays within half a code step of the
    source (plus the fp16 rounding of the block scale, at most 127 * 2^-11 of a step)."""
    from izwi_b200 import ops
    rng = np.random.default_rng(11)
    w = rng.normal(0, 0.02, (4096, 1024)).astype(np.float32)
    raw = o.quantize_q8_0(w)
    got = to_np(ops.dequantize(torch.from_numpy(raw).to(cuda), "q8_0", w.size)).reshape(w.shape)
    assert np.array_equal(got.view(np.uint32), o.dequantize_q8_0(raw).reshape(w.shape).view(np.uint32))
    step = np.abs(w.reshape(-1, 32)).max(axis=1, keepdims=True) / 127
    assert (np.abs(got - w).reshape(-1, 32) <= (0.5 + 127 * 2.0 ** -11) * step * 1.01 + 1e-9).all()


@pytest.mark.parametrize("word,bits,group", [("u32", 4, 64), ("u32", 8, 32), ("u32", 2, 128), ("u8", 8, 64), ("u8", 4, 32), ("u32", 4, 8)])
@pytest.mark.parametrize("transposed,with_bias", [(False, True), (True, True), (False, False)])
def test_mlx_affine_bit_exact(cuda, word, bits, group, transposed, with_bias):
    """MLX affine-packed weights expanded on the device: fp32 output equal bit for bit to the restatement of the
    reference's host loops, bf16 / fp16 output equal to its rounding (`to_dtype`)."""
    from izwi_b200 import ops
    rng = np.random.default_rng(bits * 100 + group)
    out_dim, in_dim = 37, 512
    word_bits = 32 if word == "u32" else 8
    pack = word_bits // bits
    if word == "u32":
        packed = rng.integers(0, 2 ** 32, (out_dim, in_dim // pack), dtype=np.uint32)
        pd = torch.from_numpy(packed.view(np.int32)).to(cuda)
    else:
        packed = rng.integers(0, 256, (out_dim, in_dim // pack), dtype=np.uint8)
        pd = torch.from_numpy(packed).to(cuda)
    groups = in_dim // group
    sc = rng.normal(0, 0.05, (out_dim, groups)).astype(np.float32)
    bi = rng.normal(0, 1, (out_dim, groups)).astype(np.float32) if with_bias else None
    want = o.dequantize_mlx_affine(packed, sc, bi, out_dim, in_dim)
    lay = (lambda a: np.ascontiguousarray(a.T)) if transposed else (lambda a: a)  # noqa: E731
    sd = torch.from_numpy(lay(sc)).to(cuda)
    bd = None if bi is None else torch.from_numpy(lay(bi)).to(cuda)
    got = ops.dequantize_mlx_affine(pd, sd, bd, out_dim, in_dim, dtype=torch.float32)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    got16 = ops.dequantize_mlx_affine(pd, sd, bd, out_dim, in_dim, dtype=torch.bfloat16)
    assert torch.equal(got16.cpu(), torch.from_numpy(want).to(torch.bfloat16))
    goth = ops.dequantize_mlx_affine(pd, sd, bd, out_dim, in_dim, dtype=torch.float16)
    assert torch.equal(goth.cpu(), torch.from_numpy(want).to(torch.float16))
    ops.Context.get(0).check()


def test_mlx_affine_refuses_what_the_reference_refuses(cuda):
    import ctypes as C
    from izwi_b200 import _lib as L
    from izwi_b200 import ops
    ctx = ops.Context.get(0)
    p = torch.zeros(4, 16, device=cuda, dtype=torch.int32)
    s = torch.ones(4, 2, device=cuda)
    out = torch.empty(4, 128, device=cuda)
    call = lambda word_bits, packed_in, groups, in_dim: L.lib().izb_dequantize_mlx_affine(  # noqa: E731
        ctx.handle, ops._stream(), p.data_ptr(), word_bits, packed_in, s.data_ptr(), None, groups, 0, 4, in_dim, L.IZB_F32, out.data_ptr())
    assert call(32, 16, 2, 128) == L.IZB_OK
    assert call(16, 16, 2, 128) == L.IZB_ERR_BAD_ARG   # words of 8 or 32 bits
    assert call(32, 16, 2, 120) == L.IZB_ERR_BAD_ARG   # in_dim not a multiple of packed_in
    assert call(32, 16, 2, 48) == L.IZB_ERR_BAD_ARG    # three values per word: 32 % 3
    assert call(32, 16, 3, 128) == L.IZB_ERR_BAD_ARG   # in_dim not a multiple of groups
    assert call(32, 2, 2, 128) == L.IZB_ERR_BAD_ARG    # 64 values per 32-bit word
