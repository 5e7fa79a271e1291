"""Linear layers on the GPU through the C ABI, checked against the oracle on the
same seeded inputs.  Gates: max relative error <= 2e-2 (relative to the row's
max |y|) and cosine >= 0.9999, the tolerance stated for bf16 matmul outputs
accumulated in fp32."""
import numpy as np
import pytest
import torch

import izwi_oracle as o
from gpu_util import assert_matmul_close, bf16_np, make_weight_np, to_np, upload_weight

pytestmark = pytest.mark.gpu

QWEN06 = [(4096, 1024), (1024, 2048), (6144, 1024), (1024, 3072)]


def run_linear(cuda, fmt, m, n, k, seed, bias=False, out_dtype=torch.bfloat16):
    from izwi_b200 import ops
    rng = np.random.default_rng(seed)
    raw, wf = make_weight_np(fmt, n, k, rng)
    x = bf16_np(rng.normal(0, 1, (m, k)))
    b = bf16_np(rng.normal(0, 0.5, n)) if bias else None
    want = o.linear(x, wf, b)
    xd = torch.from_numpy(x).to(cuda).to(torch.bfloat16)
    bd = None if b is None else torch.from_numpy(b).to(cuda).to(torch.bfloat16)
    got = ops.linear(xd, upload_weight(fmt, raw, cuda), fmt, n=n, k=k, bias=bd, out_dtype=out_dtype)
    ops.Context.get(0).check()
    return assert_matmul_close(got, want, f"{fmt} M={m} N={n} K={k}")


@pytest.mark.parametrize("fmt", ["bf16", "q8_0", "q4_k"])
@pytest.mark.parametrize("m", [1, 4, 16, 64])
def test_qwen3_0_6b_projection_shapes(cuda, fmt, m):
    for i, (n, k) in enumerate(QWEN06):
        run_linear(cuda, fmt, m, n, k, seed=100 + i)


@pytest.mark.parametrize("fmt", ["bf16", "q8_0", "q4_k"])
@pytest.mark.parametrize("m,n,k", [(1, 1, 256), (3, 17, 256), (7, 16, 512), (8, 130, 768), (9, 1000, 256),
                                   (33, 64, 1280), (2, 48, 5120), (5, 257, 2304)])
def test_ragged_shapes(cuda, fmt, m, n, k):
    run_linear(cuda, fmt, m, n, k, seed=m * 1000 + n)


@pytest.mark.parametrize("rt,ks", [(1, 1), (1, 2), (1, 4), (2, 1), (2, 2), (2, 4), (4, 2), (4, 4)])
@pytest.mark.parametrize("fmt", ["bf16", "q8_0", "q4_k"])
def test_every_tile_configuration(cuda, fmt, rt, ks, monkeypatch):
    """Each (row tiles per warp, k-split) variant of the streaming kernel, forced in turn,
    for every token-group count it is compiled for."""
    monkeypatch.setenv("IZB_SKINNY_RT", str(rt))
    monkeypatch.setenv("IZB_SKINNY_KS", str(ks))
    monkeypatch.setenv("IZB_SKINNY_IMMA_MAX_M", "0")  # keep 3..16 tokens on the kernel under test
    for m in (2, 12, 20, 40):
        if rt * ((m + 7) // 8 if m <= 16 else (4 if m <= 32 else 8)) > 8:
            continue
        run_linear(cuda, fmt, m, 336, 1536, seed=rt * 10 + ks + m)


def test_q8_0_large_activations_stay_exact(cuda):
    """The Q8_0 path lifts bf16 activations to fp16; that is exact up to |x| = 65504."""
    from izwi_b200 import ops
    rng = np.random.default_rng(12)
    n, k, m = 128, 512, 3
    raw, wf = make_weight_np("q8_0", n, k, rng)
    x = bf16_np(rng.normal(0, 1, (m, k)) * np.array([[1.0], [900.0], [2.0e4]]))
    assert np.abs(x).max() < 65504
    got = ops.linear(torch.from_numpy(x).to(cuda).to(torch.bfloat16), upload_weight("q8_0", raw, cuda), "q8_0", n=n, k=k,
                     out_dtype=torch.float32)
    want = o.linear(x, wf)
    assert np.abs(to_np(got) - want).max() <= 1e-4 * np.abs(want).max()


def test_small_k_chunks_and_two_stages(cuda, monkeypatch):
    """Many k-chunks per tile and the shallowest ring: exercises barrier phase wrap-around."""
    monkeypatch.setenv("IZB_SKINNY_STAGE_KB", "4")
    monkeypatch.setenv("IZB_SKINNY_STAGES", "2")
    for fmt in ("bf16", "q8_0", "q4_k"):
        run_linear(cuda, fmt, 5, 200, 4096, seed=77)


def test_bias_and_f32_output(cuda):
    run_linear(cuda, "bf16", 3, 1280, 1280, seed=5, bias=True)
    run_linear(cuda, "bf16", 6, 640, 1024, seed=6, bias=True, out_dtype=torch.float32)
    run_linear(cuda, "q8_0", 2, 512, 1024, seed=7, out_dtype=torch.float32)


def test_m_above_64_is_chunked(cuda):
    run_linear(cuda, "bf16", 150, 384, 512, seed=8)
    run_linear(cuda, "q4_k", 70, 256, 512, seed=9)


def test_strided_rows_and_leading_dims(cuda):
    from izwi_b200 import ops
    rng = np.random.default_rng(3)
    n, k = 96, 256
    raw, wf = make_weight_np("bf16", n, k, rng)
    w = upload_weight("bf16", raw, cuda)
    x = bf16_np(rng.normal(0, 1, (2, 3, k)))
    xd = torch.from_numpy(x).to(cuda).to(torch.bfloat16)
    got = ops.linear(xd, w)
    assert got.shape == (2, 3, n)
    assert_matmul_close(got, o.linear(x, wf), "3-D input")
    big = torch.zeros(5, 2 * k, device=cuda, dtype=torch.bfloat16)
    big[:, :k] = xd.reshape(6, k)[:5]
    ybig = torch.zeros(5, 3 * n, device=cuda, dtype=torch.bfloat16)
    ops.linear(big[:, :k], w, out=ybig[:, n:2 * n])
    assert_matmul_close(ybig[:, n:2 * n], o.linear(x.reshape(6, k)[:5], wf), "strided")
    assert float(ybig[:, :n].abs().max()) == 0.0 and float(ybig[:, 2 * n:].abs().max()) == 0.0


def test_linearity_property_full_size(cuda):
    """Full-size gate/up projection of the 8B shape: W(a+b) = Wa + Wb and scaling,
    within bf16 output rounding; no CPU product needed at this size."""
    from izwi_b200 import ops
    gen = torch.Generator(device=cuda).manual_seed(3)
    n, k = 24576, 4096
    w = (torch.randn(n, k, device=cuda, generator=gen) * 0.02).to(torch.bfloat16)
    a = torch.randn(1, k, device=cuda, generator=gen).to(torch.bfloat16)
    ya = ops.linear(a, w, out_dtype=torch.float32)
    y2 = ops.linear((a.float() * 2).to(torch.bfloat16), w, out_dtype=torch.float32)
    assert torch.allclose(y2, 2 * ya, rtol=1e-5, atol=1e-5)
    rows = torch.randint(0, n, (64,), device=cuda, generator=gen)
    want = (w[rows].double() @ a.double().T).squeeze(1)
    assert torch.allclose(ya[0, rows].double(), want, rtol=1e-3, atol=1e-3)


def test_rejects_bad_arguments(cuda):
    from izwi_b200 import IzbError, ops
    w = torch.zeros(64, 256, device=cuda, dtype=torch.bfloat16)
    x = torch.zeros(2, 256, device=cuda, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        ops.linear(torch.zeros(2, 128, device=cuda, dtype=torch.bfloat16), w)
    with pytest.raises(IzbError) as e:      # bf16 rows must be a multiple of 8 values (16 bytes)
        ops.linear(torch.zeros(2, 44, device=cuda, dtype=torch.bfloat16),
                   torch.zeros(8, 44, device=cuda, dtype=torch.bfloat16))
    assert e.value.status == -2
    with pytest.raises(IzbError) as e:      # a Q8_0 row that is not a whole number of 32-value blocks
        ops.linear(torch.zeros(2, 48, device=cuda, dtype=torch.bfloat16),
                   torch.zeros(2 * 48 // 32 * 34, device=cuda, dtype=torch.uint8), "q8_0", n=2, k=48)
    assert e.value.status == -1
    with pytest.raises(IzbError) as e:      # misaligned weight pointer
        ops.linear(x, torch.zeros(64 * 256 + 8, device=cuda, dtype=torch.bfloat16)[1:64 * 256 + 1].reshape(64, 256))
    assert e.value.status == -1
    assert ops.linear(torch.zeros(0, 256, device=cuda, dtype=torch.bfloat16), w).shape == (0, 64)
    ops.Context.get(0).check()


# ---- one and two tokens over Q8_0 / Q4_K: the integer dot-product kernel ----
# Activations travel as 16-bit block fixed point (exponent of each 32-value block's maximum), the
# dot products are exact integers, so with fp32 output the result sits far inside the bf16 gates.

@pytest.mark.parametrize("fmt", ["q8_0", "q4_k"])
@pytest.mark.parametrize("m", [1, 2])
def test_integer_dot_kernel_is_tight_in_fp32(cuda, fmt, m):
    from izwi_b200 import ops
    rng = np.random.default_rng(500 + m)
    n, k = 192, 2048
    raw, wf = make_weight_np(fmt, n, k, rng)
    x = bf16_np(rng.normal(0, 1, (m, k)))
    got = ops.linear(torch.from_numpy(x).to(cuda).to(torch.bfloat16), upload_weight(fmt, raw, cuda), fmt, n=n, k=k,
                     out_dtype=torch.float32)
    ops.Context.get(0).check()
    want = o.linear(x, wf)
    assert np.abs(to_np(got) - want).max() <= 2e-4 * np.abs(want).max()


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k"])
def test_integer_dot_kernel_outliers_zeros_and_tiny_blocks(cuda, fmt):
    """Blocks whose maximum dwarfs the other values (those lose low bits: absolute error at most
    2^-15 of the block maximum), all-zero blocks, blocks of very small magnitude, a zero token."""
    from izwi_b200 import ops
    rng = np.random.default_rng(77)
    n, k = 130, 1024
    raw, wf = make_weight_np(fmt, n, k, rng)
    x = rng.normal(0, 1, (2, k)).astype(np.float32)
    x[0, 5] = 3000.0            # outlier inside block 0
    x[0, 300] = -4.0e4          # a second, larger one
    x[0, 64:96] = 0.0           # an all-zero block
    x[0, 128:160] *= 1e-30      # a block far below every other
    x[1, :] = 0.0               # a token of zeros
    x = bf16_np(x)
    got = ops.linear(torch.from_numpy(x).to(cuda).to(torch.bfloat16), upload_weight(fmt, raw, cuda), fmt, n=n, k=k,
                     out_dtype=torch.float32)
    ops.Context.get(0).check()
    g = to_np(got)
    want = o.linear(x, wf)
    assert np.isfinite(g).all()
    assert np.all(g[1] == 0.0)
    # per-block error bound: 32 values * 2^-15 * block max * max |w|, summed over the blocks
    blk_max = np.abs(x[0]).reshape(-1, 32).max(axis=1)
    bound = (32 * 2.0 ** -15 * blk_max).sum() * np.abs(wf).max() + 1e-5 * np.abs(want[0]).max()
    assert np.abs(g[0] - want[0]).max() <= bound
    assert_matmul_close(got, want, f"{fmt} outliers")


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k"])
def test_integer_dot_kernel_matches_tensor_core_path(cuda, fmt, monkeypatch):
    """The same call through the mma.sync consumers (integer kernel switched off) agrees within the gates."""
    from izwi_b200 import ops
    rng = np.random.default_rng(91)
    n, k = 320, 1536
    raw, wf = make_weight_np(fmt, n, k, rng)
    x = bf16_np(rng.normal(0, 1, (2, k)))
    xd, wd = torch.from_numpy(x).to(cuda).to(torch.bfloat16), upload_weight(fmt, raw, cuda)
    a = ops.linear(xd, wd, fmt, n=n, k=k, out_dtype=torch.float32)
    monkeypatch.setenv("IZB_SKINNY_GEMV_MAX_M", "0")
    b = ops.linear(xd, wd, fmt, n=n, k=k, out_dtype=torch.float32)
    ops.Context.get(0).check()
    want = o.linear(x, wf)
    assert_matmul_close(a, want, "integer kernel")
    assert_matmul_close(b, want, "tensor-core consumers")
    assert np.abs(to_np(a) - to_np(b)).max() <= 2e-2 * np.abs(want).max()


def test_integer_dot_kernel_non_finite_activation_poisons_only_its_token(cuda):
    from izwi_b200 import ops
    rng = np.random.default_rng(5)
    n, k = 64, 512
    raw, wf = make_weight_np("q8_0", n, k, rng)
    x = bf16_np(rng.normal(0, 1, (2, k)))
    x[0, 40] = np.inf
    got = to_np(ops.linear(torch.from_numpy(x).to(cuda).to(torch.bfloat16), upload_weight("q8_0", raw, cuda), "q8_0",
                           n=n, k=k, out_dtype=torch.float32))
    ops.Context.get(0).check()
    assert not np.isfinite(got[0]).any()
    assert np.isfinite(got[1]).all()
    assert np.abs(got[1] - o.linear(x[1:2], wf)[0]).max() <= 2e-4 * np.abs(got[1]).max()


# ---- Q6_K (tensors of Q4_K_M files): dequantised into the workspace, multiplied by the bf16 kernels ----

@pytest.mark.parametrize("m", [1, 7, 40, 300])
def test_q6_k_linear_through_workspace(cuda, m):
    from izwi_b200 import ops
    rng = np.random.default_rng(600 + m)
    n, k = 136, 1024
    raw = o.make_q6_k_blocks(rng, n * k // 256)
    wf = o.dequantize(raw, "q6_k").reshape(n, k)
    x = bf16_np(rng.normal(0, 1, (m, k)))
    got = ops.linear(torch.from_numpy(x).to(cuda).to(torch.bfloat16), torch.from_numpy(raw).to(cuda), "q6_k", n=n, k=k)
    ops.Context.get(0).check()
    assert_matmul_close(got, o.linear(x, wf), f"q6_k M={m}")


def test_q6_k_linear_needs_the_workspace(cuda):
    from izwi_b200 import IzbError, ops
    raw = torch.zeros(4 * 210, dtype=torch.uint8, device=cuda)
    x = torch.zeros(1, 1024, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(IzbError) as e:
        ops.linear(x, raw, "q6_k", n=1, k=1024, workspace=False)
    assert e.value.status == -1


# ---- row widths the streaming kernels do not walk, and the workspace query that goes with them ----

def test_bf16_width_off_the_streaming_grid_takes_the_gemm(cuda):
    run_linear(cuda, "bf16", 2, 8, 40, seed=700)        # K = 40: not a multiple of 64, still a multiple of 8
    run_linear(cuda, "bf16", 5, 200, 328, seed=701)


@pytest.mark.parametrize("m", [1, 9, 70])
def test_q8_0_width_of_384_goes_through_the_workspace(cuda, m):
    """An encoder width such as 384 is whole Q8_0 blocks but not whole 256-value boxes: the reference's
    QMatMul takes it, so izb_linear does too, on the GEMM, with the workspace its query asks for."""
    from izwi_b200 import IzbError, _lib as L, ops
    n, k = 96, 384
    assert L.lib().izb_linear_workspace_bytes_ex(L.IZB_W_Q8_0, m, n, k, L.IZB_EPI_NONE) == n * k * 2
    run_linear(cuda, "q8_0", m, n, k, seed=710 + m)
    raw = torch.zeros(n * k // 32 * 34, device=cuda, dtype=torch.uint8)
    with pytest.raises(IzbError) as e:      # ... and says so when the caller brings none
        ops.linear(torch.zeros(m, k, device=cuda, dtype=torch.bfloat16), raw, "q8_0", n=n, k=k, workspace=False)
    assert e.value.status == -2


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k"])
@pytest.mark.parametrize("m", [3, 64, 200])
def test_workspace_query_then_call_with_a_fused_epilogue(cuda, fmt, m):
    """What a C or Rust caller does: ask izb_linear_workspace_bytes_ex with the epilogue of the call,
    allocate that much, pass it.  Straight through the C ABI, no Python-side sizing."""
    import ctypes as C

    from izwi_b200 import _lib as L
    from izwi_b200 import ops
    rng = np.random.default_rng(720 + m)
    n, k = 512, 1024
    raw, wf = make_weight_np(fmt, n, k, rng)
    x = bf16_np(rng.normal(0, 1, (m, k)))
    lib, ctx = L.lib(), ops.Context.get(0)
    assert lib.izb_linear_workspace_bytes(ops.WFMT[fmt], m, n, k) == (n * k * 2 if m > 64 else 0)
    need = lib.izb_linear_workspace_bytes_ex(ops.WFMT[fmt], m, n, k, L.IZB_EPI_SWIGLU)
    assert need == n * k * 2
    ws = torch.empty(need, device=cuda, dtype=torch.uint8)
    xd, wd = torch.from_numpy(x).to(cuda).to(torch.bfloat16), upload_weight(fmt, raw, cuda)
    y = torch.empty(m, n // 2, device=cuda, dtype=torch.bfloat16)
    a = ops.linear_args(xd, wd, fmt, n, k, y, epilogue="swiglu", workspace=ws)
    assert lib.izb_linear(ctx.handle, None, C.byref(a)) == L.IZB_OK
    ctx.check()
    pre = o.linear(x, wf)
    assert_matmul_close(y, o.silu_mul(pre[:, : n // 2], pre[:, n // 2:]), f"{fmt} M={m} swiglu through a queried workspace")
    a.workspace, a.workspace_bytes = None, 0
    assert lib.izb_linear(ctx.handle, None, C.byref(a)) == L.IZB_ERR_BAD_ARG   # the documented answer without it


@pytest.mark.parametrize("x_dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("y_dtype", [torch.float16, torch.float32, torch.bfloat16])
@pytest.mark.parametrize("fmt,m", [("bf16", 1), ("bf16", 24), ("bf16", 300), ("q8_0", 2), ("q8_0", 40), ("q8_0", 200),
                                   ("q4_k", 1), ("q4_k", 12), ("q6_k", 5)])
def test_f32_and_f16_activations_and_outputs(cuda, fmt, m, x_dtype, y_dtype):
    """The dtypes the reference's CUDA policy hands these call sites: fp32 / fp16 activations are rounded to
    bf16 once (the oracle rounds the same way) and the output is stored in the asked-for type, on every route:
    one- and two-token integer kernel, streaming kernels, dequantise-then-GEMM."""
    from izwi_b200 import ops
    n, k = 328, 768
    rng = np.random.default_rng(m * 7 + len(fmt))
    raw, wf = make_weight_np(fmt, n, k, rng)
    x_host = rng.normal(0, 1, (m, k)).astype(np.float16 if x_dtype == torch.float16 else np.float32)
    b = bf16_np(rng.normal(0, 0.5, n))
    want = o.linear(bf16_np(x_host.astype(np.float32)), wf, b)
    xd = torch.from_numpy(x_host).to(cuda)
    padded = torch.zeros(m, k + 8, device=cuda, dtype=x_dtype)  # a row stride wider than K
    padded[:, :k] = xd
    for src in (xd, padded[:, :k]):
        got = ops.linear(src, upload_weight(fmt, raw, cuda), fmt, n=n, k=k, bias=torch.from_numpy(b).to(cuda).to(torch.bfloat16),
                         out_dtype=y_dtype)
        ops.Context.get(0).check()
        assert got.dtype == y_dtype
        assert_matmul_close(got, want, f"{fmt} M={m} x={x_dtype} y={y_dtype}")


def test_f16_output_with_epilogue_and_residual(cuda):
    from izwi_b200 import ops
    rng = np.random.default_rng(5)
    m, n, k = 150, 512, 640
    raw, wf = make_weight_np("bf16", n, k, rng)
    x = bf16_np(rng.normal(0, 1, (m, k)))
    res = bf16_np(rng.normal(0, 1, (m, n)))
    want = o.linear(x, wf, None) + res
    got = ops.linear(torch.from_numpy(x).to(cuda).to(torch.bfloat16), upload_weight("bf16", raw, cuda), "bf16",
                     residual=torch.from_numpy(res).to(cuda).to(torch.bfloat16), out_dtype=torch.float16)
    assert_matmul_close(got, want, "f16 out + residual")
    want = o.gelu_erf(o.linear(x, wf, None))
    got = ops.linear(torch.from_numpy(x).to(cuda).to(torch.bfloat16), upload_weight("bf16", raw, cuda), "bf16", epilogue="gelu",
                     out_dtype=torch.float16)
    assert_matmul_close(got, want, "f16 out + gelu")


def test_typed_activations_refuse_a_prologue_and_a_missing_workspace(cuda):
    from izwi_b200 import _lib as L
    from izwi_b200 import ops
    import ctypes as C
    x = torch.randn(3, 512, device=cuda, dtype=torch.float32)
    w = torch.randn(64, 512, device=cuda, dtype=torch.bfloat16)
    y = torch.empty(3, 64, device=cuda, dtype=torch.bfloat16)
    ctx = ops.Context.get(0)
    a = ops.linear_args(x, w, "bf16", 64, 512, y)
    assert L.lib().izb_linear_workspace_bytes_args(C.byref(a)) >= 3 * 512 * 2
    assert L.lib().izb_linear(ctx.handle, ops._stream(), C.byref(a)) == L.IZB_ERR_BAD_ARG
    ws = torch.empty(8192, device=cuda, dtype=torch.uint8)
    nw = torch.ones(512, device=cuda, dtype=torch.bfloat16)
    a = ops.linear_args(x, w, "bf16", 64, 512, y, workspace=ws, prologue="rms_norm", norm_weight=nw, norm_eps=1e-6)
    assert L.lib().izb_linear(ctx.handle, ops._stream(), C.byref(a)) == L.IZB_ERR_UNSUPPORTED


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k"])
@pytest.mark.parametrize("m", [3, 5, 8, 9, 13, 16])
def test_integer_tensor_core_kernel_every_variant(cuda, fmt, m, monkeypatch):
    """The int8 mma.sync kernel for 3..16 tokens, both formats and both token-group counts, whatever the
    defaults currently route to it; residual and bias ride in its epilogue; ragged N and M."""
    from izwi_b200 import ops
    monkeypatch.setenv("IZB_SKINNY_IMMA_MAX_M", "16")
    monkeypatch.setenv("IZB_SKINNY_IMMA_Q4_K", "1")
    for i, (n, k) in enumerate([(4096, 1024), (1000, 2048), (130, 768), (17, 256), (1024, 3072)]):
        rng = np.random.default_rng(m * 100 + i)
        raw, wf = make_weight_np(fmt, n, k, rng)
        x = bf16_np(rng.normal(0, 1, (m, k)))
        b = bf16_np(rng.normal(0, 0.5, n))
        res = bf16_np(rng.normal(0, 1, (m, n)))
        want = o.linear(x, wf, b) + res
        before = ops.Context.get(0).launch_count
        got = ops.linear(torch.from_numpy(x).to(cuda).to(torch.bfloat16), upload_weight(fmt, raw, cuda), fmt, n=n, k=k,
                         bias=torch.from_numpy(b).to(cuda).to(torch.bfloat16),
                         residual=torch.from_numpy(res).to(cuda).to(torch.bfloat16), out_dtype=torch.float32)
        assert ops.Context.get(0).launch_count - before == 2  # activation conversion + product
        ops.Context.get(0).check()
        rel, cos = assert_matmul_close(got, want, f"imma {fmt} M={m} N={n} K={k}")
        assert rel < 5e-3 and cos > 0.999997  # 16-bit fixed-point activations: no visible loss against the bf16 product


def test_integer_kernel_needs_its_workspace_and_says_so(cuda):
    """Without room for the converted activations the call still runs (on the floating-point consumers);
    the workspace query names the bytes that switch the faster kernel on."""
    import ctypes as C
    from izwi_b200 import _lib as L
    from izwi_b200 import ops
    rng = np.random.default_rng(3)
    m, n, k = 4, 512, 1024
    raw, wf = make_weight_np("q8_0", n, k, rng)
    x = bf16_np(rng.normal(0, 1, (m, k)))
    xd, wd = torch.from_numpy(x).to(cuda).to(torch.bfloat16), upload_weight("q8_0", raw, cuda)
    y = torch.empty(m, n, device=cuda, dtype=torch.bfloat16)
    a = ops.linear_args(xd, wd, "q8_0", n, k, y)
    assert L.lib().izb_linear_workspace_bytes_args(C.byref(a)) == k // 32 * 72 * 16
    ctx = ops.Context.get(0)
    before = ctx.launch_count
    got = ops.linear(xd, wd, "q8_0", n=n, k=k, workspace=False)
    assert ctx.launch_count - before == 1
    assert_matmul_close(got, o.linear(x, wf, None), "no workspace")
