"""Failure detection without a GPU fault: a wait that nothing satisfies gives up after its limit,
the kernel returns normally, the host reads IZB_ERR_TIMEOUT exactly once, and the context keeps
working.  The wait is the bounded mbarrier wait every pipeline kernel of the library uses."""
import time

import numpy as np
import pytest
import torch

import izwi_oracle as o
from gpu_util import assert_matmul_close, bf16_np

pytestmark = pytest.mark.gpu


def test_wait_runs_out_and_context_stays_usable(cuda):
    from izwi_b200 import IzbError, _lib, ops
    ctx = ops.Context.get(0)
    ctx.check()                                   # clean to begin with
    t0 = time.time()
    _lib.check(_lib.lib().izb_ctx_selftest_wait_timeout(ctx.handle, None), "selftest")
    with pytest.raises(IzbError) as e:
        ctx.check()                               # synchronises: the kernel has given up by now
    waited = time.time() - t0
    assert e.value.status == _lib.IZB_ERR_TIMEOUT
    assert "bounded device-side wait gave up" in str(e.value)
    assert 0.3 < waited < 10.0, waited            # the limit is about a second of SM clocks, not forever
    ctx.check()                                   # reported once, then cleared
    # the context and the device are fine: a normal call still gives the right answer
    rng = np.random.default_rng(1)
    raw = o.make_q8_0_blocks(rng, 64 * 512 // 32)
    x = bf16_np(rng.normal(0, 1, (1, 512)))
    got = ops.linear(torch.from_numpy(x).to(cuda).to(torch.bfloat16), torch.from_numpy(raw).to(cuda), "q8_0", n=64, k=512)
    ctx.check()
    assert_matmul_close(got, o.linear(x, o.dequantize(raw, "q8_0").reshape(64, 512)), "after a time-out")
