"""Decode-step fusions of the one- and two-token block-format kernel: RmsNorm or silu(gate) * up in
front of the product, a residual row added behind it.  Each is checked twice: against the oracle's
composition of the separate steps (which rounds the intermediate to bf16, as the reference's
tensors do) at the gates stated for bf16 matmul outputs, and against the same composition without
that rounding at a tighter bound, since the fused kernel skips it."""
import numpy as np
import pytest
import torch

import izwi_oracle as o
from gpu_util import assert_matmul_close, bf16_np, make_weight_np, to_np, upload_weight

pytestmark = pytest.mark.gpu

SHAPES = [(4096, 1024), (1024, 3072), (130, 768), (1, 256), (200, 5120)]
EPS = 1e-6


def dev_bf16(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda).to(torch.bfloat16)


def tight_close(got, xin, wf, what, extra=None):
    """Against the composition without the intermediate rounding: one rounding of the output (2^-8 of
    the value covers bf16) plus 2e-4 of sum |x| |w|, the magnitude the fixed-point error scales with."""
    want = o.linear(xin, wf)
    mag = np.abs(xin) @ np.abs(wf).T
    if extra is not None:
        want = want + extra
        mag = mag + np.abs(extra)
    err = np.abs(to_np(got) - want)
    tol = 2.0 ** -8 * np.abs(want) + 2e-4 * mag
    assert (err <= tol).all(), f"{what}: worst excess {(err / tol).max():.2f}x of the bound"


def norm_unrounded(x, g):
    ms = (x.astype(np.float64) ** 2).mean(axis=-1, keepdims=True)
    return (x * (1.0 / np.sqrt(ms + EPS)).astype(np.float32) * g).astype(np.float32)


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k"])
@pytest.mark.parametrize("m", [1, 2])
def test_rms_norm_prologue(cuda, fmt, m):
    from izwi_b200 import ops
    for i, (n, k) in enumerate(SHAPES):
        rng = np.random.default_rng(500 + 10 * i + m)
        raw, wf = make_weight_np(fmt, n, k, rng)
        x = bf16_np(rng.normal(0, 3.0, (m, k)))
        g = bf16_np(rng.normal(1.0, 0.3, k))
        normed, _ = o.rms_norm(x, g, EPS)
        got = ops.linear(dev_bf16(x, cuda), upload_weight(fmt, raw, cuda), fmt, n=n, k=k, prologue="rms_norm",
                         norm_weight=dev_bf16(g, cuda), norm_eps=EPS)
        ops.Context.get(0).check()
        assert_matmul_close(got, o.linear(normed, wf), f"rms_norm + {fmt} M={m} N={n} K={k}")
        tight_close(got, norm_unrounded(x, g), wf, f"rms_norm + {fmt} M={m} N={n} K={k} (unrounded)")


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k"])
@pytest.mark.parametrize("m", [1, 2])
def test_silu_mul_prologue(cuda, fmt, m):
    from izwi_b200 import ops
    for i, (n, k) in enumerate(SHAPES):
        rng = np.random.default_rng(600 + 10 * i + m)
        raw, wf = make_weight_np(fmt, n, k, rng)
        gu = bf16_np(rng.normal(0, 2.0, (m, 2 * k)))
        act = o.silu_mul(gu[:, :k], gu[:, k:])
        got = ops.linear(dev_bf16(gu, cuda), upload_weight(fmt, raw, cuda), fmt, n=n, k=k, prologue="silu_mul")
        ops.Context.get(0).check()
        assert_matmul_close(got, o.linear(bf16_np(act), wf), f"silu_mul + {fmt} M={m} N={n} K={k}")
        tight_close(got, act, wf, f"silu_mul + {fmt} M={m} N={n} K={k} (unrounded)")


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k"])
@pytest.mark.parametrize("m", [1, 2])
def test_residual_bias_and_everything_at_once(cuda, fmt, m):
    from izwi_b200 import ops
    n, k = 1024, 2048
    rng = np.random.default_rng(700 + m)
    raw, wf = make_weight_np(fmt, n, k, rng)
    wd = upload_weight(fmt, raw, cuda)
    x = bf16_np(rng.normal(0, 1.0, (m, k)))
    res = bf16_np(rng.normal(0, 1.0, (m, n)))
    b = bf16_np(rng.normal(0, 0.5, n))
    g = bf16_np(rng.normal(1.0, 0.3, k))
    # a residual alone, in a strided buffer
    res_wide = torch.zeros(m, n + 64, device=cuda, dtype=torch.bfloat16)
    res_wide[:, :n] = dev_bf16(res, cuda)
    got = ops.linear(dev_bf16(x, cuda), wd, fmt, n=n, k=k, residual=res_wide[:, :n], out_dtype=torch.float32)
    ops.Context.get(0).check()
    want = o.linear(x, wf) + res
    assert np.abs(to_np(got) - want).max() <= 2e-4 * np.abs(want).max()
    # the reference's order: the projection output is a bf16 tensor before the add
    assert_matmul_close(got, bf16_np(o.linear(x, wf)) + res, "residual after a rounded projection")
    # norm, bias and residual together, bf16 output
    got = ops.linear(dev_bf16(x, cuda), wd, fmt, n=n, k=k, bias=dev_bf16(b, cuda), prologue="rms_norm",
                     norm_weight=dev_bf16(g, cuda), norm_eps=EPS, residual=dev_bf16(res, cuda))
    ops.Context.get(0).check()
    tight_close(got, norm_unrounded(x, g), wf, "norm + bias + residual", extra=res + b)
    # silu_mul and residual: the down projection of a decode step
    gu = bf16_np(rng.normal(0, 2.0, (m, 2 * k)))
    got = ops.linear(dev_bf16(gu, cuda), wd, fmt, n=n, k=k, prologue="silu_mul", residual=dev_bf16(res, cuda))
    ops.Context.get(0).check()
    tight_close(got, o.silu_mul(gu[:, :k], gu[:, k:]), wf, "silu_mul + residual", extra=res)


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k"])
def test_group_mixes_fused_and_plain_problems(cuda, fmt):
    """One persistent launch over problems with and without a prologue / residual, ragged M."""
    from izwi_b200 import ops
    rng = np.random.default_rng(800)
    specs = [("rms_norm", 2, 2048, 1024, False), (None, 1, 1024, 1024, True), ("silu_mul", 2, 1024, 3072, True),
             (None, 2, 520, 512, False), ("rms_norm", 1, 64, 256, True)]
    probs, keep, wants = [], [], []
    for pro, m, n, k, with_res in specs:
        raw, wf = make_weight_np(fmt, n, k, rng)
        x = bf16_np(rng.normal(0, 1.5, (m, 2 * k if pro == "silu_mul" else k)))
        g = bf16_np(rng.normal(1.0, 0.3, k))
        res = bf16_np(rng.normal(0, 1.0, (m, n)))
        xin = norm_unrounded(x, g) if pro == "rms_norm" else o.silu_mul(x[:, :k], x[:, k:]) if pro == "silu_mul" else x
        wants.append((xin, wf, res if with_res else None))
        xd, wd, gd, rd = dev_bf16(x, cuda), upload_weight(fmt, raw, cuda), dev_bf16(g, cuda), dev_bf16(res, cuda)
        yd = torch.full((m, n), float("nan"), device=cuda, dtype=torch.bfloat16)
        probs.append(ops.linear_args(xd, wd, fmt, n, k, yd, prologue=pro, norm_weight=gd if pro == "rms_norm" else None,
                                     norm_eps=EPS, residual=rd if with_res else None))
        keep.append((xd, wd, gd, rd, yd))
    group = ops.LinearGroup(probs, cuda, keepalive=keep)
    for _ in range(2):
        group.launch()
    group.ctx.check()
    for (_, _, _, _, yd), (xin, wf, res), spec in zip(keep, wants, specs):
        tight_close(yd, xin, wf, f"group {fmt} {spec}", extra=res)


def test_edge_values(cuda):
    """A zero row (rsqrt(eps) stays finite), activations and norm weights whose mantissas are all ones,
    and a non-finite activation poisoning only its own token."""
    from izwi_b200 import ops
    rng = np.random.default_rng(900)
    n, k = 256, 1024
    raw, wf = make_weight_np("q8_0", n, k, rng)
    wd = upload_weight("q8_0", raw, cuda)
    g = bf16_np(np.full(k, 1.9921875))   # bf16 mantissa all ones
    x = np.zeros((2, k), dtype=np.float32)
    x[1] = bf16_np(np.full(k, 255.0))
    got = ops.linear(dev_bf16(x, cuda), wd, "q8_0", n=n, k=k, prologue="rms_norm", norm_weight=dev_bf16(g, cuda),
                     norm_eps=EPS, out_dtype=torch.float32)
    ops.Context.get(0).check()
    want = o.linear(norm_unrounded(x, g), wf)
    assert np.all(to_np(got)[0] == 0.0)
    assert np.abs(to_np(got)[1] - want[1]).max() <= 2e-4 * np.abs(want[1]).max()
    gu = bf16_np(rng.normal(0, 2.0, (2, 2 * k)))
    gu[0, 5] = np.inf
    got = to_np(ops.linear(dev_bf16(gu, cuda), wd, "q8_0", n=n, k=k, prologue="silu_mul", out_dtype=torch.float32))
    ops.Context.get(0).check()
    assert not np.isfinite(got[0]).any()
    want = o.linear(o.silu_mul(gu[1:, :k], gu[1:, k:]), wf)
    assert np.abs(got[1] - want[0]).max() <= 2e-4 * np.abs(want).max()


def test_where_the_prologue_is_computed(cuda):
    from izwi_b200 import IzbError, ops
    assert ops.linear_fusion_max_tokens("q8_0") == 2 and ops.linear_fusion_max_tokens("q4_k") == 2
    assert ops.linear_fusion_max_tokens("bf16") == 0
    k, n = 256, 8
    g = torch.ones(k, device=cuda, dtype=torch.bfloat16)
    q = torch.zeros(n * k // 32 * 34, device=cuda, dtype=torch.uint8)
    # outside the in-kernel case the prologue goes through the workspace: without one the call is refused ...
    x = torch.zeros(3, k, device=cuda, dtype=torch.bfloat16)
    with pytest.raises(IzbError) as e:
        ops.linear(x, q, "q8_0", n=n, k=k, prologue="rms_norm", norm_weight=g, norm_eps=EPS, workspace=False)
    assert e.value.status == -1
    # ... and a group wider than two tokens declines a prologue at plan time (the grouped launch has no workspace)
    x = torch.zeros(4, k, device=cuda, dtype=torch.bfloat16)
    y = torch.zeros(4, n, device=cuda, dtype=torch.bfloat16)
    with pytest.raises(IzbError) as e:
        ops.LinearGroup([ops.linear_args(x, q, "q8_0", n, k, y, prologue="rms_norm", norm_weight=g, norm_eps=EPS)], cuda)
    assert e.value.status == -2


@pytest.mark.parametrize("fmt,m", [("bf16", 1), ("bf16", 5), ("bf16", 32), ("bf16", 40), ("bf16", 300), ("q8_0", 3),
                                   ("q8_0", 16), ("q8_0", 40), ("q8_0", 64), ("q8_0", 70), ("q8_0", 300), ("q4_k", 5),
                                   ("q4_k", 24), ("q4_k", 200), ("q6_k", 1), ("q6_k", 90)])
def test_prologue_and_residual_on_every_route(cuda, fmt, m):
    """The decoder layer's glue for every weight format and token count: the same call as for one token.
    Where the kernel has no prologue stage the library stores the normalised rows (bf16) and multiplies
    them, so the result must match the oracle's composition with its bf16 intermediate; the residual is
    added by whichever kernel runs the product."""
    from izwi_b200 import ops
    n, k = 768, 1024
    rng = np.random.default_rng(900 + m)
    if fmt == "q6_k":
        raw = o.make_q6_k_blocks(rng, n * k // 256)
        wf = o.dequantize(raw, "q6_k").reshape(n, k)
        wd = torch.from_numpy(raw).to(cuda)
    else:
        raw, wf = make_weight_np(fmt, n, k, rng)
        wd = upload_weight(fmt, raw, cuda)
    x = bf16_np(rng.normal(0, 2.0, (m, k)))
    g = bf16_np(rng.normal(1.0, 0.3, k))
    res = bf16_np(rng.normal(0, 1.0, (m, n)))
    normed, _ = o.rms_norm(x, g, EPS)
    got = ops.linear(dev_bf16(x, cuda), wd, fmt, n=n, k=k, prologue="rms_norm", norm_weight=dev_bf16(g, cuda), norm_eps=EPS,
                     residual=dev_bf16(res, cuda))
    ops.Context.get(0).check()
    assert_matmul_close(got, o.linear(normed, wf) + res, f"rms_norm + {fmt} + residual M={m}")
    gu = bf16_np(rng.normal(0, 2.0, (m, 2 * k)))
    act = bf16_np(o.silu_mul(gu[:, :k], gu[:, k:]))
    got = ops.linear(dev_bf16(gu, cuda), wd, fmt, n=n, k=k, prologue="silu_mul", residual=dev_bf16(res, cuda))
    ops.Context.get(0).check()
    assert_matmul_close(got, o.linear(act, wf) + res, f"silu_mul + {fmt} + residual M={m}")
    # residual alone, fp32 output
    got = ops.linear(dev_bf16(x, cuda), wd, fmt, n=n, k=k, residual=dev_bf16(res, cuda), out_dtype=torch.float32)
    ops.Context.get(0).check()
    assert_matmul_close(got, o.linear(x, wf) + res, f"{fmt} + residual M={m} fp32 out")


def test_residual_behind_a_fused_epilogue_and_ragged_width(cuda):
    """GEMM route: residual after SwiGLU (half as many columns) and on a width that is not a multiple of 8."""
    from izwi_b200 import ops
    rng = np.random.default_rng(950)
    m, n, k = 150, 520, 512
    raw, wf = make_weight_np("bf16", n, k, rng)
    x = bf16_np(rng.normal(0, 1.0, (m, k)))
    pre = o.linear(x, wf)
    res = bf16_np(rng.normal(0, 1.0, (m, n // 2)))
    got = ops.linear(dev_bf16(x, cuda), upload_weight("bf16", raw, cuda), epilogue="swiglu", residual=dev_bf16(res, cuda))
    assert_matmul_close(got, o.silu_mul(pre[:, : n // 2], pre[:, n // 2:]) + res, "swiglu + residual")
    n2 = 515
    raw2, wf2 = make_weight_np("bf16", n2, k, rng)
    res2 = bf16_np(rng.normal(0, 1.0, (m, n2)))
    got = ops.linear(dev_bf16(x, cuda), upload_weight("bf16", raw2, cuda), residual=dev_bf16(res2, cuda))
    ops.Context.get(0).check()
    assert_matmul_close(got, o.linear(x, wf2) + res2, "ragged width + residual")


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k"])
def test_k_split_over_a_cluster_matches_the_single_cta_walk(cuda, fmt, monkeypatch):
    """A lone small projection splits the k chunks of each row tile over a cluster of CTAs; the sums must
    agree with the unsplit kernel to fp32 reordering, for every cluster size and with all fusions on."""
    from izwi_b200 import ops
    rng = np.random.default_rng(950)
    for m, n, k in ((1, 1024, 3072), (2, 1024, 2048), (1, 70, 4096), (2, 4096, 1024), (1, 64, 768)):
        raw, wf = make_weight_np(fmt, n, k, rng)
        wd = upload_weight(fmt, raw, cuda)
        x = dev_bf16(bf16_np(rng.normal(0, 1.5, (m, k))), cuda)
        gu = dev_bf16(bf16_np(rng.normal(0, 1.5, (m, 2 * k))), cuda)
        g = dev_bf16(bf16_np(rng.normal(1.0, 0.3, k)), cuda)
        res = dev_bf16(bf16_np(rng.normal(0, 1.0, (m, n))), cuda)

        def run_all():
            return [ops.linear(x, wd, fmt, n=n, k=k, out_dtype=torch.float32),
                    ops.linear(x, wd, fmt, n=n, k=k, out_dtype=torch.float32, prologue="rms_norm", norm_weight=g, norm_eps=EPS,
                               residual=res),
                    ops.linear(gu, wd, fmt, n=n, k=k, out_dtype=torch.float32, prologue="silu_mul", residual=res)]
        monkeypatch.setenv("IZB_SKINNY_GEMV_KSPLIT", "1")
        base = run_all()
        for cap in (2, 4, 8):
            monkeypatch.setenv("IZB_SKINNY_GEMV_KSPLIT", str(cap))
            for got, want in zip(run_all(), base):
                ops.Context.get(0).check()
                scale = float(want.abs().max())
                assert float((got - want).abs().max()) <= 1e-5 * scale, (fmt, m, n, k, cap)
    ops.Context.get(0).check()
