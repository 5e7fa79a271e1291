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
