"""The grouped persistent launch (izb_linear_group_*): many independent small-M
linear layers in one kernel, checked problem by problem against the oracle and
against the single-problem entry point."""
import numpy as np
import pytest
import torch

import izwi_oracle as o
from gpu_util import assert_matmul_close, bf16_np, make_weight_np, upload_weight

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt", ["bf16", "q8_0", "q4_k"])
@pytest.mark.parametrize("m", [1, 16])
def test_group_of_mixed_shapes(cuda, fmt, m):
    from izwi_b200 import ops
    rng = np.random.default_rng(40 + m)
    shapes = [(4096, 1024), (1024, 2048), (6144, 1024), (1024, 3072), (24, 256), (200, 512)] * 2
    probs, keep, wants = [], [], []
    for i, (n, k) in enumerate(shapes):
        raw, wf = make_weight_np(fmt, n, k, rng)
        mi = m if i % 3 else max(1, m // 2)            # ragged M inside one group
        x = bf16_np(rng.normal(0, 1, (mi, k)))
        xd = torch.from_numpy(x).to(cuda).to(torch.bfloat16)
        wd = upload_weight(fmt, raw, cuda)
        yd = torch.full((mi, n), float("nan"), device=cuda, dtype=torch.bfloat16)
        probs.append(ops.linear_args(xd, wd, fmt, n, k, yd))
        keep.append((xd, wd, yd))
        wants.append(o.linear(x, wf))
    group = ops.LinearGroup(probs, cuda, keepalive=keep)
    for _ in range(2):                                   # the plan is reusable
        group.launch()
    group.ctx.check()
    for (xd, wd, yd), want, (n, k) in zip(keep, wants, shapes):
        assert_matmul_close(yd, want, f"group {fmt} N={n} K={k}")
        # the single-problem launch may pick another row tile / k split, so the fp32 sums can be
        # ordered differently: agreement to bf16 rounding, not bit for bit
        single = ops.linear(xd, wd, fmt, n=n, k=k)
        assert_matmul_close(single, yd.float().cpu().numpy(), "single vs grouped")


def test_group_plan_rejects_mixed_formats_and_large_m(cuda):
    from izwi_b200 import IzbError, ops
    x = torch.zeros(2, 256, device=cuda, dtype=torch.bfloat16)
    w = torch.zeros(8, 256, device=cuda, dtype=torch.bfloat16)
    q = torch.zeros(8 * 272, device=cuda, dtype=torch.uint8)
    y = torch.zeros(2, 8, device=cuda, dtype=torch.bfloat16)
    with pytest.raises(IzbError) as e:
        ops.LinearGroup([ops.linear_args(x, w, "bf16", 8, 256, y), ops.linear_args(x, q, "q8_0", 8, 256, y)], cuda)
    assert e.value.status == -1
    xl = torch.zeros(65, 256, device=cuda, dtype=torch.bfloat16)
    yl = torch.zeros(65, 8, device=cuda, dtype=torch.bfloat16)
    with pytest.raises(IzbError) as e:
        ops.LinearGroup([ops.linear_args(xl, w, "bf16", 8, 256, yl)], cuda)
    assert e.value.status == -2


def test_group_step_with_host_buffers(cuda):
    """izb_linear_group_launch_host: activations from page-locked host memory, results back in host memory when the
    call returns; every step sees that step's inputs."""
    from izwi_b200 import ops
    rng = np.random.default_rng(61)
    shapes = [(1024, 512), (512, 1024), (768, 512)]
    acts = torch.zeros(sum(k for _, k in shapes), device=cuda, dtype=torch.bfloat16)
    outs = torch.zeros(sum(n for n, _ in shapes), device=cuda, dtype=torch.bfloat16)
    probs, keep, weights = [], [], []
    xo = yo = 0
    for n, k in shapes:
        raw, wf = make_weight_np("q8_0", n, k, rng)
        wd = upload_weight("q8_0", raw, cuda)
        probs.append(ops.linear_args(acts[xo:xo + k].view(1, k), wd, "q8_0", n, k, outs[yo:yo + n].view(1, n)))
        keep.append(wd)
        weights.append(wf)
        xo, yo = xo + k, yo + n
    group = ops.LinearGroup(probs, cuda, keepalive=keep)
    h_in = torch.empty(acts.shape, dtype=torch.bfloat16).pin_memory()
    h_out = torch.empty(outs.shape, dtype=torch.bfloat16).pin_memory()
    for step in range(3):
        x = bf16_np(rng.normal(0, 1, acts.shape[0]))
        h_in.copy_(torch.from_numpy(x).to(torch.bfloat16))
        h_out.fill_(float("nan"))
        group.launch_host(h_in, acts, outs, h_out)  # no synchronisation here: the call returns with the results
        got = h_out.float().numpy()
        xo = yo = 0
        for (n, k), wf in zip(shapes, weights):
            assert_matmul_close(torch.from_numpy(got[yo:yo + n][None, :]), o.linear(x[None, xo:xo + k], wf), f"host step {step} N={n}")
            xo, yo = xo + k, yo + n
    group.ctx.check()
    # the same problems with their y pointers in page-locked host memory: the kernel stores there, nothing is copied back
    direct = torch.empty(outs.shape, dtype=torch.bfloat16).pin_memory()
    probs2, yo = [], 0
    for (n, k), p_dev in zip(shapes, probs):
        a2 = ops.linear_args(acts[:k].view(1, k), keep[0], "q8_0", n, k, direct[yo:yo + n].view(1, n))
        a2.x, a2.w = p_dev.x, p_dev.w
        probs2.append(a2)
        yo += n
    group2 = ops.LinearGroup(probs2, cuda, keepalive=keep)
    direct.fill_(float("nan"))
    group2.launch_host(h_in, acts)
    assert torch.equal(direct, h_out)
    import ctypes as C
    from izwi_b200 import _lib as L
    # the whole step in the C call, as a C or Rust caller makes it: copy in, launch, copy out, wait
    acts.zero_()
    copied = torch.empty(outs.shape, dtype=torch.bfloat16).pin_memory()
    copied.fill_(float("nan"))
    st = L.lib().izb_linear_group_launch_host(group.ctx.handle, C.c_void_p(torch.cuda.current_stream().cuda_stream),
                                              C.c_void_p(group.host_plan.data_ptr()), C.c_void_p(group.dev_plan.data_ptr()),
                                              C.c_void_p(h_in.data_ptr()), C.c_void_p(acts.data_ptr()), h_in.numel() * 2,
                                              C.c_void_p(outs.data_ptr()), C.c_void_p(copied.data_ptr()), copied.numel() * 2)
    assert st == 0
    assert torch.equal(copied, h_out)
    st = L.lib().izb_linear_group_launch_host(group.ctx.handle, None, C.c_void_p(group.host_plan.data_ptr()), C.c_void_p(group.dev_plan.data_ptr()),
                                              None, C.c_void_p(acts.data_ptr()), 16, C.c_void_p(outs.data_ptr()), C.c_void_p(h_out.data_ptr()), 16)
    assert st == L.IZB_ERR_BAD_ARG
