"""The tcgen05/TMEM GEMM (M > 32) through izb_linear: prefill and encoder shapes, fused
epilogues, block-quantised weights through the dequantise-to-workspace route.  Same gates as the
decode tests: max relative error <= 2e-2, cosine >= 0.9999 against the fp32 oracle on
bf16-rounded inputs."""
import numpy as np
import pytest
import torch

import izwi_oracle as o
from gpu_util import assert_matmul_close, bf16_np, make_weight_np, to_np, upload_weight

pytestmark = pytest.mark.gpu


def run_gemm(cuda, m, n, k, seed, fmt="bf16", bias=False, epilogue=None, out_dtype=torch.bfloat16, x_std=1.0):
    from izwi_b200 import ops
    rng = np.random.default_rng(seed)
    raw, wf = make_weight_np(fmt, n, k, rng)
    x = bf16_np(rng.normal(0, x_std, (m, k)))
    b = bf16_np(rng.normal(0, 0.5, n)) if bias else None
    pre = o.linear(x, wf, b)
    if epilogue == "gelu":
        want = o.gelu_erf(pre)
    elif epilogue == "gelu_tanh":
        want = o.gelu_tanh(pre)
    elif epilogue == "silu":
        want = o.silu_mul(pre, np.ones_like(pre))
    elif epilogue == "swiglu":
        want = o.silu_mul(pre[:, : n // 2], pre[:, n // 2:])
    else:
        want = pre
    xd = torch.from_numpy(x).to(cuda).to(torch.bfloat16)
    bd = None if b is None else torch.from_numpy(b).to(cuda).to(torch.bfloat16)
    got = ops.linear(xd, upload_weight(fmt, raw, cuda), fmt, n=n, k=k, bias=bd, out_dtype=out_dtype, epilogue=epilogue)
    ops.Context.get(0).check()
    return assert_matmul_close(got, want, f"gemm {fmt} M={m} N={n} K={k} epi={epilogue}")


def test_single_tile(cuda):
    run_gemm(cuda, 128, 256, 64, seed=1)


@pytest.mark.parametrize("m,n,k", [(33, 64, 64), (64, 64, 128), (129, 200, 72), (375, 1024, 1024), (300, 520, 1096),
                                   (1500, 1280, 1280), (2048, 1024, 3072), (257, 4096, 1024)])
def test_shapes(cuda, m, n, k):
    run_gemm(cuda, m, n, k, seed=m + n)


def test_every_accumulator_width(cuda):
    # many tiles -> 256 wide, fewer -> 128, few -> 64
    run_gemm(cuda, 4096, 2048, 256, seed=3)
    run_gemm(cuda, 1024, 1024, 256, seed=4)
    run_gemm(cuda, 128, 1024, 256, seed=5)


def test_long_k_wraps_the_ring_many_times(cuda):
    run_gemm(cuda, 200, 384, 12288, seed=6)


def test_bias_and_f32_output(cuda):
    run_gemm(cuda, 260, 1280, 640, seed=7, bias=True)
    run_gemm(cuda, 100, 330, 512, seed=8, bias=True, out_dtype=torch.float32)


@pytest.mark.parametrize("epilogue", ["gelu", "gelu_tanh", "silu", "swiglu"])
def test_fused_epilogues(cuda, epilogue):
    run_gemm(cuda, 375, 2048, 1024, seed=9, bias=(epilogue != "swiglu"), epilogue=epilogue, x_std=1.0)
    run_gemm(cuda, 70, 6144, 1024, seed=10, epilogue=epilogue)
    run_gemm(cuda, 4, 512, 256, seed=11, epilogue=epilogue)  # small M with an epilogue still takes the GEMM


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k"])
def test_quantized_prefill_through_workspace(cuda, fmt):
    run_gemm(cuda, 300, 1024, 2048, seed=12, fmt=fmt)
    run_gemm(cuda, 128, 6144, 1024, seed=13, fmt=fmt, epilogue="swiglu")


def test_quantized_without_workspace_falls_back_to_streaming(cuda):
    from izwi_b200 import ops
    rng = np.random.default_rng(14)
    n, k, m = 256, 512, 130
    raw, wf = make_weight_np("q8_0", n, k, rng)
    x = bf16_np(rng.normal(0, 1, (m, k)))
    got = ops.linear(torch.from_numpy(x).to(cuda).to(torch.bfloat16), upload_weight("q8_0", raw, cuda), "q8_0", n=n, k=k,
                     workspace=False)
    assert_matmul_close(got, o.linear(x, wf), "no workspace")


def test_repeated_launches_are_deterministic(cuda):
    from izwi_b200 import ops
    gen = torch.Generator(device=cuda).manual_seed(1)
    x = torch.randn(512, 1024, device=cuda, generator=gen).to(torch.bfloat16)
    w = (torch.randn(1536, 1024, device=cuda, generator=gen) * 0.02).to(torch.bfloat16)
    first = ops.linear(x, w)
    for _ in range(5):
        assert torch.equal(ops.linear(x, w), first)
    ops.Context.get(0).check()


def test_full_size_prefill_properties(cuda):
    """Qwen3-8B prefill gate/up (M = 2048, N = 24576, K = 4096): linearity in X and agreement with
    the streaming kernel on sampled token rows; no CPU product at this size."""
    from izwi_b200 import ops
    gen = torch.Generator(device=cuda).manual_seed(3)
    m, n, k = 2048, 24576, 4096
    w = (torch.randn(n, k, device=cuda, generator=gen) * 0.02).to(torch.bfloat16)
    x = torch.randn(m, k, device=cuda, generator=gen).to(torch.bfloat16)
    y = ops.linear(x, w, out_dtype=torch.float32)
    y2 = ops.linear((x.float() * 2).to(torch.bfloat16), w, out_dtype=torch.float32)
    assert torch.allclose(y2, 2 * y, rtol=1e-5, atol=1e-4)
    rows = torch.tensor([0, 1, 127, 128, 1000, 2047], device=cuda)
    ys = ops.linear(x[rows].contiguous(), w, out_dtype=torch.float32)   # M = 6 -> streaming kernel
    assert torch.allclose(y[rows], ys, rtol=2e-3, atol=2e-3)
    ops.Context.get(0).check()


def _rows_f64(x, w, rows, bias=None):
    """float64 product of sampled activation rows with the whole weight, on the host."""
    v = x[rows].double().cpu().numpy() @ w.double().cpu().numpy().T
    return v if bias is None else v + bias.double().cpu().numpy()[None, :]


@pytest.mark.parametrize("name,m,n,k,epilogue,bias", [
    ("qwen3-8b prefill qkv", 2048, 6144, 4096, None, False),
    ("qwen3-8b prefill gate/up + SwiGLU", 2048, 24576, 4096, "swiglu", False),
    ("qwen3-8b prefill down", 2048, 4096, 12288, None, False),
    ("whisper b32 fc1 + bias + GELU", 48000, 5120, 1280, "gelu_tanh", True),
    ("whisper b32 fc2 + bias", 48000, 1280, 5120, None, True),
    ("fastconformer b32 ffn1 + SiLU", 12000, 4096, 1024, "silu", False),
])
def test_full_size_against_float64_on_sampled_rows(cuda, name, m, n, k, epilogue, bias):
    """The prefill and encoder GEMMs at the full sizes of the configurations, checked against a float64
    product of the same bf16 inputs on sampled token rows (first, last, tile edges, middle)."""
    from izwi_b200 import ops
    gen = torch.Generator(device=cuda).manual_seed(m + n)
    w = (torch.randn(n, k, device=cuda, generator=gen) * 0.02).to(torch.bfloat16)
    x = torch.randn(m, k, device=cuda, generator=gen).to(torch.bfloat16)
    b = (torch.randn(n, device=cuda, generator=gen) * 0.1).to(torch.bfloat16) if bias else None
    y = ops.linear(x, w, bias=b, epilogue=epilogue)
    ops.Context.get(0).check()
    rows = sorted({0, 1, 127, 128, m // 2, m - 129, m - 1})
    pre = _rows_f64(x, w, rows, b).astype(np.float32)
    if epilogue == "swiglu":
        want = o.silu_mul(pre[:, : n // 2], pre[:, n // 2:])
    elif epilogue == "gelu_tanh":
        want = o.gelu_tanh(pre)
    elif epilogue == "silu":
        want = o.silu_mul(pre, np.ones_like(pre))
    else:
        want = pre
    assert_matmul_close(y[rows], want, name)
