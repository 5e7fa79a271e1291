"""RMS normalisation and arg-max on the GPU through the C ABI against the oracle."""
import numpy as np
import pytest
import torch

import izwi_oracle as o
from gpu_util import bf16_np, to_np

pytestmark = pytest.mark.gpu


def _one_ulp_close(got, want):
    """bf16 outputs computed in fp32: at most one bf16 step apart (the sum of squares is fp32 on
    the GPU, fp64 in the oracle), and equal for nearly every element."""
    g, w = got.astype(np.float32), want.astype(np.float32)
    step = np.maximum(np.abs(w), 1e-30) * 2.0 ** -7
    assert (np.abs(g - w) <= step).all()
    assert (g == w).mean() > 0.98


@pytest.mark.parametrize("rows,cols", [(1, 1024), (7, 4096), (33, 128), (8 * 16, 128), (3, 5120), (2, 1000), (5, 513)])
def test_rms_norm_matches_oracle(cuda, rows, cols):
    from izwi_b200 import ops
    rng = np.random.default_rng(rows * 7 + cols)
    x = bf16_np(rng.normal(0, 2, (rows, cols)))
    w = bf16_np(rng.normal(1, 0.2, cols))
    xd, wd = torch.from_numpy(x).to(cuda).to(torch.bfloat16), torch.from_numpy(w).to(cuda).to(torch.bfloat16)
    got = to_np(ops.rms_norm(xd, wd, 1e-6))
    ops.Context.get(0).check()
    want, _ = o.rms_norm(x, w, 1e-6)
    _one_ulp_close(got, want)


def test_rms_norm_with_residual_and_views(cuda):
    from izwi_b200 import ops
    rng = np.random.default_rng(5)
    rows, cols = 6, 2048
    big = torch.from_numpy(bf16_np(rng.normal(0, 1, (rows, 3 * cols)))).to(cuda).to(torch.bfloat16)
    x = big[:, cols:2 * cols]                      # a strided view: rows 3 * cols apart
    r = torch.from_numpy(bf16_np(rng.normal(0, 1, (rows, cols)))).to(cuda).to(torch.bfloat16)
    w = torch.from_numpy(bf16_np(rng.normal(1, 0.1, cols))).to(cuda).to(torch.bfloat16)
    out, total = ops.rms_norm(x, w, 1e-5, residual=r, return_sum=True)
    want, h = o.rms_norm(to_np(x), to_np(w), 1e-5, residual=to_np(r))
    assert np.array_equal(to_np(total), h)         # the rounded sum is bit-exact
    _one_ulp_close(to_np(out), want)
    # q/k norm form: [tokens, heads, head_dim] flattened to rows of head_dim
    q = torch.from_numpy(bf16_np(rng.normal(0, 1, (4, 16, 128)))).to(cuda).to(torch.bfloat16)
    wq = torch.from_numpy(bf16_np(rng.normal(1, 0.1, 128))).to(cuda).to(torch.bfloat16)
    got = ops.rms_norm(q, wq, 1e-6)
    assert got.shape == q.shape
    _one_ulp_close(to_np(got), o.rms_norm(to_np(q), to_np(wq), 1e-6)[0])


def test_rms_norm_bad_arguments(cuda):
    from izwi_b200 import IzbError, _lib, ops
    ctx = ops.Context.get(0)
    x = torch.zeros(2, 64, dtype=torch.bfloat16, device=cuda)
    w = torch.ones(64, dtype=torch.bfloat16, device=cuda)
    L = _lib.lib()
    assert L.izb_rms_norm(ctx.handle, None, x.data_ptr(), w.data_ptr(), None, x.data_ptr(), None, 2, 64, 32, 0, 64, 0, 1e-6) == -1
    assert L.izb_rms_norm(ctx.handle, None, x.data_ptr(), w.data_ptr(), None, x.data_ptr(), x.data_ptr(), 2, 64, 64, 0, 64, 64, 1e-6) == -1
    assert L.izb_rms_norm(ctx.handle, None, x.data_ptr(), w.data_ptr(), None, x.data_ptr(), None, 0, 64, 64, 0, 64, 0, 1e-6) == 0
    assert IzbError is not None


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_argmax_rows(cuda, dtype):
    from izwi_b200 import ops
    rng = np.random.default_rng(9)
    x = rng.normal(0, 3, (5, 151936)).astype(np.float32)
    x[1, 100] = x[1, 70000] = 50.0        # equal maxima: lowest index wins
    x[2, :] = -1.0                          # all equal: index 0
    x[3, 151935] = 99.0                     # last element
    x[4, 17] = np.nan
    x[4, 5] = 60.0
    xd = torch.from_numpy(x).to(cuda).to(dtype)
    idx, val = ops.argmax_rows(xd, return_values=True)
    ops.Context.get(0).check()
    want_i, want_v = o.argmax_rows(to_np(xd))
    assert np.array_equal(idx.cpu().numpy(), want_i)
    assert np.array_equal(val.cpu().numpy(), want_v)
    assert list(want_i[1:4]) == [100, 0, 151935] and want_i[4] == 5
    nan_row = torch.full((1, 40), float("nan"), device=cuda, dtype=dtype)
    i2, v2 = ops.argmax_rows(nan_row, return_values=True)
    assert int(i2[0]) == 0 and float(v2[0]) == float("-inf")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_argmax_long_rows_split_across_ctas(cuda, dtype):
    """Rows of a vocabulary's length take several CTAs each: ties across the CTA boundaries, -inf and
    NaN rows, and back-to-back calls (the per-row scratch must come back clean)."""
    from izwi_b200 import ops
    rng = np.random.default_rng(19)
    cols = 151936
    for rows in (1, 2, 7):
        x = rng.normal(0, 3, (rows, cols)).astype(np.float32)
        x[0, [8440, 8441, 75968, cols - 1]] = 40.0   # equal maxima in different CTAs' ranges
        if rows > 1:
            x[1, :] = -np.inf
            x[1, 90000] = -1e30
        if rows > 2:
            x[2, :] = np.nan
            x[3, :] = -np.inf
            x[4, :] = np.nan
            x[4, cols - 1] = -np.inf
            x[5, :] = -0.0
            x[5, 131072] = 0.0                        # +0 == -0: the lowest index still wins
        xd = torch.from_numpy(x).to(cuda).to(dtype)
        for _ in range(3):
            idx, val = ops.argmax_rows(xd, return_values=True)
        ops.Context.get(0).check()
        want_i, want_v = o.argmax_rows(to_np(xd))
        assert np.array_equal(idx.cpu().numpy(), want_i), (rows, idx.cpu().numpy(), want_i)
        assert np.array_equal(val.cpu().numpy(), want_v)
        assert want_i[0] == 8440


def test_lm_head_greedy_token(cuda):
    """lm_head GEMV over Q8_0 weights followed by the on-device arg-max equals the oracle's choice."""
    from izwi_b200 import ops
    rng = np.random.default_rng(10)
    n, k = 4096, 1024
    raw = o.make_q8_0_blocks(rng, n * k // 32)
    wf = o.dequantize(raw, "q8_0").reshape(n, k)
    x = bf16_np(rng.normal(0, 1, (1, k)))
    logits = ops.linear(torch.from_numpy(x).to(cuda).to(torch.bfloat16), torch.from_numpy(raw).to(cuda), "q8_0", n=n, k=k,
                        out_dtype=torch.float32)
    tok = int(ops.argmax_rows(logits)[0])
    want = o.linear(x, wf)[0]
    assert want[tok] >= np.sort(want)[-1] - 1e-3 * np.abs(want).max()
