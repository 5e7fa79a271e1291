"""GGUF file -> device -> kernels: tensors written by gguf-py are uploaded as raw block bytes and
multiplied in place; `load_tensor` dequantises bit-exactly."""
import numpy as np
import pytest
import torch

import izwi_oracle as o
from gpu_util import assert_matmul_close, bf16_np, to_np

pytestmark = pytest.mark.gpu
gguf = pytest.importorskip("gguf")


def test_load_and_multiply_from_file(cuda, tmp_path):
    from izwi_b200 import ops
    from izwi_b200.gguf import GgufLoader
    rng = np.random.default_rng(8)
    n, k = 192, 1024
    raws = {"blk.0.attn_q.weight": ("q4_k", o.make_q4_k_blocks(rng, n * k // 256, 1e-4, 7.5e-4), gguf.GGMLQuantizationType.Q4_K),
            "blk.0.attn_output.weight": ("q8_0", o.make_q8_0_blocks(rng, n * k // 32), gguf.GGMLQuantizationType.Q8_0),
            "blk.0.ffn_down.weight": ("q6_k", o.make_q6_k_blocks(rng, n * k // 256), gguf.GGMLQuantizationType.Q6_K)}
    norm = rng.normal(1, 0.1, k).astype(np.float32)
    path = tmp_path / "m.gguf"
    w = gguf.GGUFWriter(str(path), "qwen3")
    for name, (_, raw, qt) in raws.items():
        w.add_tensor(name, raw.reshape(n, -1), raw_dtype=qt)
    w.add_tensor("blk.0.attn_norm.weight", norm)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()

    g = GgufLoader.from_path(path)
    x = bf16_np(rng.normal(0, 1, (2, k)))
    xd = torch.from_numpy(x).to(cuda).to(torch.bfloat16)
    for name, (fmt, raw, _) in raws.items():
        q = g.load_qtensor(name, cuda)
        assert q.dtype == fmt and (q.rows, q.cols) == (n, k)
        assert np.array_equal(q.data.cpu().numpy(), raw)
        want_w = o.dequantize(raw, fmt).reshape(n, k)
        got = ops.linear(xd, q.data, fmt, n=n, k=k)
        ops.Context.get(0).check()
        assert_matmul_close(got, o.linear(x, want_w), name)
        deq = g.load_tensor(name, torch.float32, cuda)
        assert deq.shape == (n, k)
        assert np.array_equal(to_np(deq).view(np.uint32), want_w.view(np.uint32))
    assert np.array_equal(to_np(g.load_tensor("blk.0.attn_norm.weight", torch.float32, cuda)), norm)
    assert g.load_tensor("blk.0.attn_norm.weight", torch.bfloat16, cuda).dtype == torch.bfloat16
