"""izb_linear_quantized_static: the prefill linear layer over block-quantised weights for callers
that cannot supply a workspace or tolerate a device allocation (a host runtime whose own pool owns
all device memory; an audio thread that must not stall in cudaMalloc).  It keeps the dequantised
weights in a fixed array inside the library instead.

Checked through the C ABI against the ordinary entry point (izb_linear with a caller workspace) on
two calls in a row with different weights: the second call proves that what the first left in the
shared array does not leak into later results.  Collected last on purpose, so a run that stops at
the first failure has already executed every other test; it also passes alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import izwi_oracle as o
from gpu_util import MAX_REL_ERR, MIN_COSINE, bf16_np, make_weight_np, to_np, upload_weight

pytestmark = pytest.mark.gpu


def call_static(ctx, fmt, x, w, y, m, n, k, epilogue=0, bias=None):
    from izwi_b200 import _lib as L
    from izwi_b200 import ops
    return L.lib().izb_linear_quantized_static(
        ctx.handle, C.c_void_p(torch.cuda.current_stream().cuda_stream), ops.WFMT[fmt], C.c_void_p(x.data_ptr()),
        C.c_void_p(w.data_ptr()), C.c_void_p(0 if bias is None else bias.data_ptr()), C.c_void_p(y.data_ptr()),
        L.IZB_BF16, m, n, k, epilogue)


def set_up_once(ctx, cuda):
    """The documented one-off: the first call on a device looks up the array's address, and that is
    also when the CUDA runtime (which loads a library's device code on first use) makes the array
    resident, so the device's free memory drops by the array's size once, here, and never again."""
    x = torch.zeros(65, 256, device=cuda, dtype=torch.bfloat16)
    w = torch.zeros(8 * 256 // 32 * 34, device=cuda, dtype=torch.uint8)
    y = torch.empty(65, 8, device=cuda, dtype=torch.bfloat16)
    assert call_static(ctx, "q8_0", x, w, y, 65, 8, 256) == 0
    ctx.check()


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k"])
def test_matches_workspace_entry_point_twice_in_a_row(cuda, fmt):
    from izwi_b200 import ops
    ctx = ops.Context.get(0)
    rng = np.random.default_rng(99)
    set_up_once(ctx, cuda)
    for call, (m, n, k) in enumerate([(200, 1024, 2048), (96, 3072, 1024)]):
        raw, wf = make_weight_np(fmt, n, k, rng)
        x = bf16_np(rng.normal(0, 1, (m, k)))
        xd = torch.from_numpy(x).to(cuda).to(torch.bfloat16)
        wd = upload_weight(fmt, raw, cuda)
        want = ops.linear(xd, wd, fmt, n=n, k=k)                  # existing entry point, caller workspace
        got = torch.full((m, n), float("nan"), device=cuda, dtype=torch.bfloat16)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()            # the driver's figure: sees any cudaMalloc, not only torch's
        assert call_static(ctx, fmt, xd, wd, got, m, n, k) == 0
        ctx.check()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, "the call changed the device's free memory"
        rel, cos = o.rel_err_and_cosine(to_np(got), to_np(want))
        assert rel <= MAX_REL_ERR and cos >= MIN_COSINE, (call, rel, cos)
        assert torch.equal(got, want), f"call {call}: same kernels, same inputs, so the same bits"
        rel, cos = o.rel_err_and_cosine(to_np(got), o.linear(x, wf))
        assert rel <= MAX_REL_ERR and cos >= MIN_COSINE, (call, rel, cos)


def test_rejects_sizes_beyond_the_fixed_array(cuda):
    from izwi_b200 import _lib as L
    from izwi_b200 import ops
    ctx = ops.Context.get(0)
    limit = L.lib().izb_static_scratch_bytes()
    assert limit == 16 * 1024 * 1024
    n, k = 4096, 4096                                              # 32 MiB of bf16: twice the array
    assert n * k * 2 > limit
    x = torch.zeros(65, k, device=cuda, dtype=torch.bfloat16)
    w = torch.zeros(n * k // 32 * 34, device=cuda, dtype=torch.uint8)
    y = torch.full((65, n), 7.0, device=cuda, dtype=torch.bfloat16)
    assert call_static(ctx, "q8_0", x, w, y, 65, n, k) == L.IZB_ERR_SCRATCH_TOO_SMALL
    assert b"scratch" in L.lib().izb_status_string(L.IZB_ERR_SCRATCH_TOO_SMALL)
    torch.cuda.synchronize()
    assert float(y.min()) == 7.0                                   # nothing was launched
    assert call_static(ctx, "bf16", x, w, y, 65, 64, 256) == L.IZB_ERR_BAD_ARG


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k"])
@pytest.mark.parametrize("m", [5, 64, 130])
def test_bias_epilogue_and_small_batches(cuda, fmt, m):
    """Bias and a fused SwiGLU through the static entry point, for token counts on both sides of the 64
    at which izb_linear would switch kernels: same bits as izb_linear with a caller workspace, and
    within the matmul gates of the oracle."""
    from izwi_b200 import _lib as L
    from izwi_b200 import ops
    ctx = ops.Context.get(0)
    rng = np.random.default_rng(300 + m)
    n, k = 1024, 512
    raw, wf = make_weight_np(fmt, n, k, rng)
    x = bf16_np(rng.normal(0, 1, (m, k)))
    b = bf16_np(rng.normal(0, 0.5, n))
    xd = torch.from_numpy(x).to(cuda).to(torch.bfloat16)
    bd = torch.from_numpy(b).to(cuda).to(torch.bfloat16)
    wd = upload_weight(fmt, raw, cuda)
    want = ops.linear(xd, wd, fmt, n=n, k=k, bias=bd, epilogue="swiglu")
    got = torch.full((m, n // 2), float("nan"), device=cuda, dtype=torch.bfloat16)
    set_up_once(ctx, cuda)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    assert call_static(ctx, fmt, xd, wd, got, m, n, k, epilogue=L.IZB_EPI_SWIGLU, bias=bd) == 0
    ctx.check()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.equal(got, want)
    pre = o.linear(x, wf, b)
    rel, cos = o.rel_err_and_cosine(to_np(got), o.silu_mul(pre[:, : n // 2], pre[:, n // 2:]))
    assert rel <= MAX_REL_ERR and cos >= MIN_COSINE, (fmt, m, rel, cos)


def test_rejects_rows_that_are_not_whole_blocks(cuda):
    from izwi_b200 import _lib as L
    from izwi_b200 import ops
    ctx = ops.Context.get(0)
    x = torch.zeros(70, 48, device=cuda, dtype=torch.bfloat16)
    w = torch.zeros(2 * 48 // 32 * 34, device=cuda, dtype=torch.uint8)
    y = torch.zeros(70, 2, device=cuda, dtype=torch.bfloat16)
    assert call_static(ctx, "q8_0", x, w, y, 70, 2, 48) == L.IZB_ERR_BAD_ARG
