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
