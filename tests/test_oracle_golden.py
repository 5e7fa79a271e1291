"""The oracle against the golden fixtures: gguf-py dequantisation vectors and the
reference's own unit-test cases (qwen3/core.rs:2481-2684, 3100-3142)."""
import ctypes
import json
import subprocess

import numpy as np
import pytest

import izwi_oracle as o


@pytest.fixture(scope="module")
def vec(golden_dir):
    return np.load(golden_dir / "ggml_dequant.npz")


@pytest.fixture(scope="module")
def cases(golden_dir):
    return json.loads((golden_dir / "reference_cases.json").read_text())


@pytest.fixture(scope="module")
def oracle_c():
    from conftest import ROOT
    subprocess.run(["make", "-C", str(ROOT / "oracle")], check=True, capture_output=True)
    return ctypes.CDLL(str(ROOT / "oracle" / "liboracle_c.so"))


def test_q8_0_dequant_bit_exact(vec):
    got = o.dequantize_q8_0(vec["q8_0_raw"])
    assert np.array_equal(got.view(np.uint32), vec["q8_0_f32"].view(np.uint32))


def test_q4_k_dequant_bit_exact(vec):
    got = o.dequantize_q4_k(vec["q4_k_raw"])
    assert np.array_equal(got.view(np.uint32), vec["q4_k_f32"].view(np.uint32))


def test_q6_k_dequant_bit_exact(vec):
    got = o.dequantize_q6_k(vec["q6_k_raw"])
    assert np.array_equal(got.view(np.uint32), vec["q6_k_f32"].view(np.uint32))


def test_q6_k_storage_bytes():
    assert o.quantized_storage_bytes(4, 512, "q6_k") == 8 * 210
    with pytest.raises(Exception):
        o.quantized_storage_bytes(1, 100, "q6_k")


def test_q8_0_quantize_matches_ggml(vec):
    assert np.array_equal(o.quantize_q8_0(vec["quant_in"]), vec["quant_q8_0"])


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k"])
def test_c_port_dequant_bit_exact(vec, oracle_c, fmt):
    raw = np.ascontiguousarray(vec[f"{fmt}_raw"])
    n = raw.size // o.TYPE_SIZE[fmt] * o.BLOCK_SIZE[fmt]
    out = np.empty(n, np.float32)
    getattr(oracle_c, f"orc_dequantize_{fmt}")(raw.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(n),
                                                out.ctypes.data_as(ctypes.c_void_p))
    assert np.array_equal(out.view(np.uint32), vec[f"{fmt}_f32"].view(np.uint32))


@pytest.mark.parametrize("fmt,code", [("q8_0", 0), ("q4_k", 1)])
def test_c_port_qlinear_matches_numpy(oracle_c, fmt, code):
    rng = np.random.default_rng(5)
    n, k, m = 96, 512, 3
    mk = o.make_q8_0_blocks if fmt == "q8_0" else o.make_q4_k_blocks
    raw = mk(rng, n * k // o.BLOCK_SIZE[fmt])
    x = rng.normal(size=(m, k)).astype(np.float32)
    y = np.empty((m, n), np.float32)
    rc = oracle_c.orc_qlinear_f32(code, x.ctypes.data_as(ctypes.c_void_p), raw.ctypes.data_as(ctypes.c_void_p),
                                  y.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(m), ctypes.c_int64(n),
                                  ctypes.c_int64(k))
    assert rc == 0
    rel, cos = o.rel_err_and_cosine(y, o.qmatmul(x, raw, n, k, fmt))
    assert rel < 1e-5 and cos > 0.999999


def test_dense_projection_known_answers(cases):
    for name in ("dense_projection_with_bias", "dense_projection_no_bias"):
        c = cases[name]
        got = o.linear(np.array(c["input"]), np.array(c["weight"]), None if c["bias"] is None else np.array(c["bias"]))
        assert got.tolist() == c["expected"]


def test_selected_logits_match_full(cases):
    c = cases["selected_logits"]
    full = o.linear(np.array(c["hidden"]), np.array(c["weight"]), np.array(c["bias"]))[0]
    w = np.array(c["weight"], dtype=np.float32)
    b = np.array(c["bias"], dtype=np.float32)
    for tok in c["token_ids"]:
        sel = o.linear(np.array(c["hidden"]), w[tok:tok + 1], b[tok:tok + 1])[0, 0]
        assert abs(sel - full[tok]) < c["tol"]


def test_fused_qkv_matches_separate(cases):
    c = cases["fused_qkv"]
    x = np.array(c["input"], dtype=np.float32)
    q, k, v = o.fused_qkv(x, c["q"], c["k"], c["v"])
    for got, w in ((q, c["q"]), (k, c["k"]), (v, c["v"])):
        want = o.linear(x, np.array(w))
        assert got.shape == want.shape == (1, 2, len(w))
        assert np.abs(got - want).max() <= c["tol"]


def test_fused_gate_up_matches_separate(cases):
    c = cases["fused_gate_up"]
    x = np.array(c["input"], dtype=np.float32)
    g, u = o.fused_gate_up(x, c["gate"], c["up"], np.array(c["gate_bias"]), np.array(c["up_bias"]))
    assert np.abs(g - o.linear(x, np.array(c["gate"]), np.array(c["gate_bias"]))).max() <= c["tol"]
    assert np.abs(u - o.linear(x, np.array(c["up"]), np.array(c["up_bias"]))).max() <= c["tol"]


def test_fused_rejects_mixed_bias_and_dim_mismatch():
    x = np.zeros((1, 3), np.float32)
    w = np.zeros((2, 3), np.float32)
    with pytest.raises(ValueError, match="mixed bias"):
        o.fused_gate_up(x, w, w, np.zeros(2), None)
    with pytest.raises(ValueError, match="do not match"):
        o.fused_qkv(x, w, np.zeros((2, 4), np.float32), w)


def test_packed_q8_0_matches_separate(cases):
    """packed_qmatmul_matches_separate_q8_0_on_cpu (qwen3/core.rs:3100-3142)."""
    idx = np.arange(64, dtype=np.float32)
    w1 = ((idx - 31.0) / 8.0).reshape(2, 32)
    w2 = ((15.0 - idx[:32]) / 7.0).reshape(1, 32)
    x = ((idx[:32] + 1.0) / 16.0).reshape(1, 32)
    q1, q2 = o.quantize_q8_0(w1), o.quantize_q8_0(w2)
    raw, n, k, fmt = o.pack_quantized_rows([(q1, 2, 32, o.Q8_0), (q2, 1, 32, o.Q8_0)])
    assert (n, k) == (3, 32) and raw.size == o.quantized_storage_bytes(3, 32, o.Q8_0)
    for mm in (o.qmatmul, lambda x_, r_, n_, k_, f_=None: o.qmatmul_q8_activations(x_, r_, n_, k_)):
        packed = mm(x, raw, 3, 32, o.Q8_0)
        sep = np.concatenate([mm(x, q1, 2, 32, o.Q8_0), mm(x, q2, 1, 32, o.Q8_0)], axis=1)
        assert np.abs(packed - sep).max() <= cases["packed_q8_0"]["tol"]
    # the two conventions (exact product vs 8-bit activations) agree to quantisation noise
    rel, cos = o.rel_err_and_cosine(o.qmatmul_q8_activations(x, raw, 3, 32), o.qmatmul(x, raw, 3, 32, o.Q8_0))
    assert rel < 2e-2 and cos > 0.9999


def test_pack_rejects_mismatches():
    q = o.quantize_q8_0(np.ones((1, 32), np.float32))
    with pytest.raises(ValueError, match="empty"):
        o.pack_quantized_rows([])
    with pytest.raises(ValueError, match="input mismatch"):
        o.pack_quantized_rows([(q, 1, 32, o.Q8_0), (np.concatenate([q, q]), 1, 64, o.Q8_0)])
    with pytest.raises(ValueError, match="dtype mismatch"):
        o.pack_quantized_rows([(q, 1, 32, o.Q8_0), (q, 1, 32, o.Q4_K)])
    with pytest.raises(ValueError, match="not divisible"):
        o.quantized_storage_bytes(3, 100, o.Q4_K)


def test_silu_mul_formula():
    g = np.array([-3.0, -0.5, 0.0, 0.5, 3.0], np.float32)
    u = np.array([2.0, -1.0, 5.0, 1.5, -0.25], np.float32)
    want = g.astype(np.float64) / (1 + np.exp(-g.astype(np.float64))) * u
    assert np.abs(o.silu_mul(g, u) - want).max() < 1e-6


def test_bf16_round_ties_to_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.4e38], np.float32)
    r = o.bf16_round(x)
    assert r[0] == 1.0 and r[1] == 1.0 and r[2] == np.float32(1.015625)
    assert np.array_equal(o.bf16_from_bits(o.bf16_bits(x)), r)


def test_moe_topk_ties_and_weights():
    lg = np.zeros((2, 8), np.float32)
    lg[0, [5, 2, 7]] = 3.0
    lg[1] = np.arange(8)
    idx, w = o.moe_topk(lg, 4)
    assert idx[0].tolist() == [2, 5, 7, 0] and idx[1].tolist() == [7, 6, 5, 4]
    assert np.allclose(w.sum(axis=1), 1.0, atol=1e-6)
    full = np.exp(lg - lg.max(1, keepdims=True))
    full /= full.sum(1, keepdims=True)
    sel = np.take_along_axis(full, idx.astype(np.int64), 1)
    assert np.allclose(w, sel / sel.sum(1, keepdims=True), atol=1e-6)


def test_moe_permute_stable():
    idx = np.array([[3, 1], [1, 0], [3, 0]], np.int32)
    off, perm = o.moe_permute(idx, 4)
    assert off.tolist() == [0, 2, 4, 4, 6]
    assert perm.tolist() == [3, 5, 1, 2, 0, 4]


def test_rms_norm_known_answer_and_residual():
    out, h = o.rms_norm(np.array([[3.0, 4.0]], dtype=np.float32), np.array([1.0, 2.0], dtype=np.float32), 0.0)
    assert np.allclose(out, [[3 / np.sqrt(12.5), 8 / np.sqrt(12.5)]], rtol=2 ** -8)
    out2, h2 = o.rms_norm(np.array([[1.0, 1.0]], dtype=np.float32), np.ones(2, dtype=np.float32), 0.0,
                          residual=np.array([[2.0, 3.0]], dtype=np.float32))
    assert np.array_equal(h2, [[3.0, 4.0]]) and np.allclose(out2, [[3 / np.sqrt(12.5), 4 / np.sqrt(12.5)]], rtol=2 ** -8)


def test_argmax_rows_ties_and_nan():
    idx, val = o.argmax_rows(np.array([[1.0, 5.0, 5.0, np.nan], [np.nan, np.nan, np.nan, np.nan]]))
    assert list(idx) == [1, 0] and val[0] == 5.0 and val[1] == -np.inf


# The known-answer tests of the reference's MLX-affine loader (models/shared/weights/mlx.rs:420-486), read as text.
MLX_KNOWN = [
    (np.array([[0x76543210]], dtype=np.uint32), [[0.1, 0.2]], [[-1.0, 0.5]], 1, 8,
     [-1.0 + 0.0 * 0.1, -1.0 + 1.0 * 0.1, -1.0 + 2.0 * 0.1, -1.0 + 3.0 * 0.1, 0.5 + 4.0 * 0.2, 0.5 + 5.0 * 0.2, 0.5 + 6.0 * 0.2, 0.5 + 7.0 * 0.2]),
    (np.array([[1, 2, 3, 4]], dtype=np.uint8), [[0.5, 2.0]], [[0.0, -1.0]], 1, 4, [0.5, 1.0, 5.0, 7.0]),
    (np.array([[0x76543210]], dtype=np.uint32), [[0.1, 0.2]], None, 1, 8,
     [0.0 * 0.1, 1.0 * 0.1, 2.0 * 0.1, 3.0 * 0.1, 4.0 * 0.2, 5.0 * 0.2, 6.0 * 0.2, 7.0 * 0.2]),
    (np.array([[1, 2, 3, 4]], dtype=np.uint8), [[0.5, 2.0]], None, 1, 4, [0.5, 1.0, 6.0, 8.0]),
]


@pytest.mark.parametrize("case", range(len(MLX_KNOWN)))
def test_mlx_affine_known_answers(case):
    import izwi_oracle as o
    packed, scales, biases, out_dim, in_dim, want = MLX_KNOWN[case]
    got = o.dequantize_mlx_affine(packed, np.array(scales, dtype=np.float32), None if biases is None else np.array(biases, dtype=np.float32),
                                  out_dim, in_dim)
    assert got.shape == (out_dim, in_dim) and got.dtype == np.float32
    assert np.abs(got.reshape(-1) - np.array(want, dtype=np.float64)).max() < 1e-6  # the reference's own tolerance


def test_mlx_affine_transposed_params_and_shape_rules():
    import izwi_oracle as o
    rng = np.random.default_rng(0)
    out_dim, in_dim, groups = 6, 128, 4
    packed = rng.integers(0, 2 ** 32, (out_dim, in_dim // 8), dtype=np.uint32)
    sc, bi = rng.normal(0, 0.1, (out_dim, groups)).astype(np.float32), rng.normal(0, 1, (out_dim, groups)).astype(np.float32)
    a = o.dequantize_mlx_affine(packed, sc, bi, out_dim, in_dim)
    b = o.dequantize_mlx_affine(packed, np.ascontiguousarray(sc.T), np.ascontiguousarray(bi.T), out_dim, in_dim)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    # element by element, as the reference's loops compute it
    for r, c in ((0, 0), (3, 37), (5, 127)):
        q = (int(packed[r, c // 8]) >> ((c % 8) * 4)) & 15
        assert a[r, c] == np.float32(np.float32(q) * sc[r, c // 32]) + bi[r, c // 32]
    for bad in (lambda: o.dequantize_mlx_affine(packed, sc, bi, out_dim + 1, in_dim),                # rows mismatch
                lambda: o.dequantize_mlx_affine(packed, sc, bi, out_dim, in_dim + 8),                # in_dim % packed_in
                lambda: o.dequantize_mlx_affine(packed, sc, bi, out_dim, 16 * 3),                    # word_bits % pack
                lambda: o.dequantize_mlx_affine(packed, sc[:, :3], bi[:, :3], out_dim, in_dim),      # in_dim % groups
                lambda: o.dequantize_mlx_affine(packed, sc, bi[:, :2], out_dim, in_dim)):            # biases shape
        with pytest.raises(ValueError):
            bad()
