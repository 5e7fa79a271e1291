"""The reference's own projection unit tests (qwen3/core.rs:2481-2684, 3100-3142),
restated against the CUDA path through the host-side mirror of its types."""
import json

import numpy as np
import pytest
import torch

import izwi_oracle as o
from gpu_util import assert_matmul_close, bf16_np, to_np

pytestmark = pytest.mark.gpu


def pad_k(a, k=64):
    """The kernels need in-dim % 64 == 0; zero columns do not change the product."""
    a = np.asarray(a, dtype=np.float32)
    out = np.zeros(a.shape[:-1] + (k,), np.float32)
    out[..., : a.shape[-1]] = a
    return out


@pytest.fixture(scope="module")
def cases(golden_dir):
    return json.loads((golden_dir / "reference_cases.json").read_text())


def dev(a, cuda):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(cuda)


def test_dense_projection_loads_optional_bias(cuda, cases):
    from izwi_b200.projection import Qwen3Projection, Qwen3ProjectionDiagnostics
    c = cases["dense_projection_with_bias"]
    proj = Qwen3Projection.dense(dev(pad_k(c["weight"]), cuda), dev(c["bias"], cuda))
    assert proj.diagnostics() == Qwen3ProjectionDiagnostics(1, 1, 0)
    out = proj.forward(dev(pad_k(c["input"]), cuda))
    assert to_np(out).tolist() == c["expected"]


def test_dense_projection_keeps_no_bias_path(cuda, cases):
    from izwi_b200.projection import Qwen3Projection, Qwen3ProjectionDiagnostics
    c = cases["dense_projection_no_bias"]
    proj = Qwen3Projection.dense(dev(pad_k(c["weight"]), cuda))
    assert proj.diagnostics() == Qwen3ProjectionDiagnostics(1, 0, 0)
    assert to_np(proj.forward(dev(pad_k(c["input"]), cuda))).tolist() == c["expected"]


def test_selected_logits_match_full_projection(cuda, cases):
    from izwi_b200.projection import Qwen3Projection
    c = cases["selected_logits"]
    proj = Qwen3Projection.dense(dev(pad_k(c["weight"]), cuda), dev(c["bias"], cuda))
    hidden = dev(pad_k(c["hidden"]), cuda)
    sel = proj.logits_for_tokens(hidden, c["token_ids"])
    full = to_np(proj.forward(hidden))[0]
    assert [t for t, _ in sel] == c["token_ids"]
    for tok, val in sel:
        assert abs(val - full[tok]) < c["tol"]
    assert proj.logits_for_tokens(hidden, []) == []


def test_fused_qkv_matches_separate_dense_projections(cuda, cases):
    from izwi_b200.projection import Qwen3FusedQkvProjection, Qwen3Projection
    c = cases["fused_qkv"]
    q, k, v = (Qwen3Projection.dense(dev(pad_k(c[n]), cuda)) for n in ("q", "k", "v"))
    fused = Qwen3FusedQkvProjection(q, k, v)
    x = dev(pad_k(c["input"]), cuda)
    fq, fk, fv = fused.forward(x)
    # fused == separate holds exactly: same kernel, same per-row arithmetic
    for got, proj in ((fq, q), (fk, k), (fv, v)):
        assert got.shape == (1, 2, proj.out_dim)
        assert torch.equal(got, proj.forward(x))
    # and both sit within bf16 rounding of the fp32 oracle
    want = o.fused_qkv(bf16_np(pad_k(c["input"])), *(bf16_np(pad_k(c[n])) for n in ("q", "k", "v")))
    for got, w in zip((fq, fk, fv), want):
        assert np.abs(to_np(got) - w).max() <= 2e-2
    assert fused.diagnostics().dense_projection_count == 3


def test_fused_gate_up_matches_separate_dense_projections(cuda, cases):
    from izwi_b200.projection import Qwen3FusedGateUpProjection, Qwen3Projection
    c = cases["fused_gate_up"]
    gate = Qwen3Projection.dense(dev(pad_k(c["gate"]), cuda), dev(c["gate_bias"], cuda))
    up = Qwen3Projection.dense(dev(pad_k(c["up"]), cuda), dev(c["up_bias"], cuda))
    fused = Qwen3FusedGateUpProjection(gate, up)
    x = dev(pad_k(c["input"]), cuda)
    g, u = fused.forward(x)
    assert torch.equal(g, gate.forward(x)) and torch.equal(u, up.forward(x))
    assert fused.diagnostics().dense_bias_projection_count == 2


def test_fused_projection_errors(cuda):
    from izwi_b200.projection import (InferenceError, Qwen3FusedGateUpProjection, Qwen3FusedQkvProjection,
                                      Qwen3Projection)
    a = Qwen3Projection.dense(torch.zeros(2, 64, device=cuda), torch.zeros(2, device=cuda))
    b = Qwen3Projection.dense(torch.zeros(2, 64, device=cuda))
    c = Qwen3Projection.dense(torch.zeros(2, 128, device=cuda))
    with pytest.raises(InferenceError, match="mixed bias"):
        Qwen3FusedGateUpProjection(a, b)
    with pytest.raises(InferenceError, match="do not match"):
        Qwen3FusedQkvProjection(b, c, b)
    with pytest.raises(InferenceError, match="CUDA"):
        b.forward(torch.zeros(1, 64))


def test_packed_qmatmul_matches_separate_q8_0(cuda):
    """packed_qmatmul_matches_separate_q8_0_on_cpu with the rows tiled out to K = 256
    (the kernels' minimum aligned run of Q8_0 blocks)."""
    from izwi_b200.projection import QTensor, Qwen3Projection, packed_qmatmul_from_qtensors
    idx = np.arange(64 * 8, dtype=np.float32)
    w1 = (((idx % 64) - 31.0) / 8.0).reshape(2, 256)
    w2 = ((15.0 - (idx[:256] % 32)) / 7.0).reshape(1, 256)
    x = (((idx[:256] % 32) + 1.0) / 16.0).reshape(1, 256)
    q1, q2 = o.quantize_q8_0(w1), o.quantize_q8_0(w2)
    t1 = QTensor(torch.from_numpy(q1).to(cuda), 2, 256, "q8_0")
    t2 = QTensor(torch.from_numpy(q2).to(cuda), 1, 256, "q8_0")
    packed = packed_qmatmul_from_qtensors([t1, t2])
    xd = dev(x, cuda)
    out = packed.forward(xd)
    sep = torch.cat([Qwen3Projection.quantized(t1).forward(xd), Qwen3Projection.quantized(t2).forward(xd)], dim=1)
    assert torch.equal(out, sep)
    raw, n, k, f = o.pack_quantized_rows([(q1, 2, 256, o.Q8_0), (q2, 1, 256, o.Q8_0)])
    assert_matmul_close(out, o.qmatmul(bf16_np(x), raw, n, k, f), "packed q8_0")
    assert packed.diagnostics().quantized_projection_count == 1


def test_packed_qmatmul_errors(cuda):
    from izwi_b200.projection import InferenceError, QTensor, packed_qmatmul_from_qtensors
    z = torch.zeros(272, dtype=torch.uint8, device=cuda)
    with pytest.raises(InferenceError, match="empty"):
        packed_qmatmul_from_qtensors([])
    with pytest.raises(InferenceError, match="input mismatch"):
        packed_qmatmul_from_qtensors([QTensor(z, 1, 256, "q8_0"), QTensor(torch.cat([z, z]), 1, 512, "q8_0")])
    with pytest.raises(InferenceError, match="dtype mismatch"):
        packed_qmatmul_from_qtensors([QTensor(z, 1, 256, "q8_0"), QTensor(z[:144], 1, 256, "q4_k")])
    with pytest.raises(InferenceError, match="bytes, expected"):
        packed_qmatmul_from_qtensors([QTensor(z[:200], 1, 256, "q8_0")])


@pytest.mark.parametrize("fmt", ["bf16", "q4_k"])
def test_mlp_forward_matches_oracle(cuda, fmt):
    """Qwen3Mlp::forward: fused gate/up -> silu*up -> down on the 0.6B shape."""
    from izwi_b200.projection import (QTensor, Qwen3FusedGateUpProjection, Qwen3FusedQuantizedProjection, Qwen3Mlp,
                                      Qwen3Projection)
    from gpu_util import make_weight_np, upload_weight
    rng = np.random.default_rng(21)
    hidden, inter, m = 1024, 3072, 4
    x = bf16_np(rng.normal(0, 1, (m, hidden)))
    rg, wg = make_weight_np(fmt, inter, hidden, rng)
    ru, wu = make_weight_np(fmt, inter, hidden, rng)
    rd, wd = make_weight_np(fmt, hidden, inter, rng)
    if fmt == "bf16":
        gu = Qwen3FusedGateUpProjection(Qwen3Projection.dense(upload_weight(fmt, rg, cuda)),
                                        Qwen3Projection.dense(upload_weight(fmt, ru, cuda)))
        down = Qwen3Projection.dense(upload_weight(fmt, rd, cuda))
    else:
        gu = Qwen3FusedQuantizedProjection([QTensor(upload_weight(fmt, rg, cuda), inter, hidden, fmt),
                                            QTensor(upload_weight(fmt, ru, cuda), inter, hidden, fmt)])
        down = Qwen3Projection.quantized(QTensor(upload_weight(fmt, rd, cuda), hidden, inter, fmt))
    got = Qwen3Mlp(gu, down).forward(torch.from_numpy(x).to(cuda).to(torch.bfloat16))
    want = o.mlp_forward(x, np.concatenate([wg, wu]), wd, inter, round_bf16=True)
    assert_matmul_close(got, want, f"mlp {fmt}")


def test_silu_mul_matches_oracle(cuda):
    from izwi_b200 import ops
    rng = np.random.default_rng(2)
    for shape in ((1, 3072), (5, 12288), (3, 7), (2, 3, 768)):
        g = bf16_np(rng.normal(0, 2, shape))
        u = bf16_np(rng.normal(0, 1, shape))
        got = ops.silu_mul(torch.from_numpy(g).to(cuda).to(torch.bfloat16), torch.from_numpy(u).to(cuda).to(torch.bfloat16))
        want = o.silu_mul(g, u)
        assert got.shape == shape
        # one bf16 rounding of an fp32 result computed with a fast exp
        assert np.abs(to_np(got) - want).max() <= np.abs(want).max() * 2 ** -8 + 1e-6
