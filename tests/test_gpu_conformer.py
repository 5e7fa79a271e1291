"""The Conformer convolution module (parakeet/asr/mod.rs:775-893) on the GPU against the oracle: batch-norm folding,
the gated pointwise convolution (a linear layer with the GLU epilogue), the depthwise convolution with folded
bias and swish, and the whole module at the FastConformer shape (d_model 1024, kernel 9, 375 frames)."""
import numpy as np
import pytest
import torch

import izwi_oracle as o
from gpu_util import assert_matmul_close, bf16_np, to_np

pytestmark = pytest.mark.gpu


def _dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda).to(torch.bfloat16)


def test_fold_batch_norm(cuda):
    from izwi_b200 import conformer
    rng = np.random.default_rng(1)
    c, k = 256, 9
    w = rng.normal(0, 0.3, (c, 1, k)).astype(np.float32)
    gamma, beta = rng.normal(1, 0.2, c).astype(np.float32), rng.normal(0, 0.2, c).astype(np.float32)
    mean, var = rng.normal(0, 0.5, c).astype(np.float32), rng.uniform(0.2, 2.0, c).astype(np.float32)
    t = lambda a: torch.from_numpy(a).to(cuda)  # noqa: E731
    for g, b in ((gamma, beta), (None, None)):
        fw, fb = conformer.fold_depthwise_conv1d_batch_norm(t(w), None if g is None else t(g), None if b is None else t(b), t(mean),
                                                            t(var), 1e-5)
        want_w, want_b = o.fold_depthwise_conv1d_batch_norm(w.reshape(c, k), g, b, mean, var, 1e-5)
        # fp32 arithmetic, one rounding to bf16: within one bf16 step of the oracle's fp32 value
        assert np.abs(to_np(fw) - want_w).max() <= 2.0 ** -8 * np.abs(want_w).max()
        assert np.abs(to_np(fb) - want_b).max() <= 2.0 ** -8 * max(np.abs(want_b).max(), 1e-3)


@pytest.mark.parametrize("b,t,c,k", [(1, 375, 1024, 9), (3, 50, 256, 9), (2, 1, 64, 9), (1, 7, 8, 31), (4, 130, 512, 3), (1, 5, 16, 1)])
def test_depthwise_conv_bias_swish(cuda, b, t, c, k):
    from izwi_b200 import conformer, ops
    rng = np.random.default_rng(t + c)
    x = bf16_np(rng.normal(0, 1, (b, t, c)))
    w = bf16_np(rng.normal(0, 0.3, (c, k)))
    bias = bf16_np(rng.normal(0, 0.3, c))
    for swish, bb in ((True, bias), (False, None)):
        got = conformer.depthwise_conv1d_bias_swish(_dev(x, cuda), _dev(w, cuda), None if bb is None else _dev(bb, cuda), swish=swish)
        ops.Context.get(0).check()
        want = o.depthwise_conv1d_bias_swish(x, w, bb, swish=swish)
        assert_matmul_close(got.reshape(b * t, c), want.reshape(b * t, c), f"depthwise conv B={b} T={t} C={c} k={k} swish={swish}")


@pytest.mark.parametrize("m,c", [(375, 1024), (70, 256), (3000, 1024)])
def test_gated_pointwise_conv_is_a_linear_layer_with_glu(cuda, m, c):
    from izwi_b200 import ops
    rng = np.random.default_rng(m)
    x = bf16_np(rng.normal(0, 1, (m, c)))
    w = bf16_np(rng.normal(0, 0.03, (2 * c, c)))
    got = ops.linear(_dev(x, cuda), _dev(w, cuda), epilogue="glu")
    ops.Context.get(0).check()
    pre = o.linear(x, w)
    assert_matmul_close(got, o.glu(pre[:, :c], pre[:, c:]), f"pointwise_conv1 + GLU M={m} C={c}")


def test_whole_module_at_the_fastconformer_shape(cuda):
    from izwi_b200 import conformer, ops
    rng = np.random.default_rng(9)
    b, t, c, k = 2, 375, 1024, 9
    x = bf16_np(rng.normal(0, 1, (b, t, c)))
    w1 = bf16_np(rng.normal(0, 0.03, (2 * c, c)))
    w2 = bf16_np(rng.normal(0, 0.03, (c, c)))
    dw = rng.normal(0, 0.3, (c, k)).astype(np.float32)
    gamma, beta = rng.normal(1, 0.1, c).astype(np.float32), rng.normal(0, 0.1, c).astype(np.float32)
    mean, var = rng.normal(0, 0.2, c).astype(np.float32), rng.uniform(0.5, 1.5, c).astype(np.float32)
    f = lambda a: torch.from_numpy(a).to(cuda)  # noqa: E731
    mod = conformer.ConformerConv(_dev(w1, cuda), f(dw), f(gamma), f(beta), f(mean), f(var), 1e-5, _dev(w2, cuda))
    got = mod.forward(_dev(x, cuda))
    ops.Context.get(0).check()
    # the oracle's composition, each stored tensor rounded to bf16 as the reference's tensors are
    fw, fb = o.fold_depthwise_conv1d_batch_norm(dw, gamma, beta, mean, var, 1e-5)
    pre = o.linear(x.reshape(b * t, c), w1)
    gated = bf16_np(o.glu(pre[:, :c], pre[:, c:])).reshape(b, t, c)
    conv = bf16_np(o.depthwise_conv1d_bias_swish(gated, bf16_np(fw), bf16_np(fb)))
    want = o.linear(conv.reshape(b * t, c), w2)
    assert_matmul_close(got.reshape(b * t, c), want, "ConformerConv")
