"""RoPE and single-query GQA attention on the GPU through the C ABI against the oracle.
Gates for the attention output (bf16, fp32 accumulation, `__expf`): max abs error <= 2e-2 of the
largest |out| and cosine >= 0.9999, the matmul gates of this project."""
import numpy as np
import pytest
import torch

import izwi_oracle as o
from gpu_util import assert_matmul_close, bf16_np, to_np

pytestmark = pytest.mark.gpu


def _dev(a, cuda):
    return torch.from_numpy(a).to(cuda).to(torch.bfloat16)


@pytest.mark.parametrize("tokens,qh,kh,d", [(1, 16, 8, 128), (5, 32, 8, 128), (3, 4, 4, 64), (64, 8, 2, 128)])
def test_rope_pair(cuda, tokens, qh, kh, d):
    from izwi_b200 import ops
    rng = np.random.default_rng(tokens + d)
    q, k = bf16_np(rng.normal(0, 1, (tokens, qh, d))), bf16_np(rng.normal(0, 1, (tokens, kh, d)))
    ang = rng.uniform(0, 6.28, (tokens, d // 2))
    c, s = bf16_np(np.cos(ang)), bf16_np(np.sin(ang))
    qd, kd = _dev(q, cuda), _dev(k, cuda)
    ops.rope_pair_(qd, kd, _dev(c, cuda), _dev(s, cuda))
    ops.Context.get(0).check()
    for got, x in ((qd, q), (kd, k)):
        want = o.rope_pair(x, c, s)
        g = to_np(got)
        assert (np.abs(g - want) <= np.maximum(np.abs(want), 2.0 ** -6) * 2.0 ** -7).all()
        assert (g == want).mean() > 0.97


@pytest.mark.parametrize("b,h,kvh,d,kv_len,cap", [
    (1, 16, 8, 128, 1, 8), (1, 16, 8, 128, 127, 128), (1, 16, 8, 128, 129, 256), (2, 32, 8, 128, 1000, 1024),
    (1, 32, 4, 128, 4096, 4096), (3, 8, 8, 64, 333, 400), (1, 12, 4, 128, 700, 700), (4, 16, 2, 64, 2049, 4096)])
def test_decode_gqa_attention(cuda, b, h, kvh, d, kv_len, cap):
    from izwi_b200 import ops
    rng = np.random.default_rng(kv_len + h)
    q = bf16_np(rng.normal(0, 1, (b, h, d)))
    k = bf16_np(rng.normal(0, 1, (b, kvh, cap, d)))
    v = bf16_np(rng.normal(0, 1, (b, kvh, cap, d)))
    k[:, :, kv_len:] = 1e30  # positions past kv_len must never be read into the result
    v[:, :, kv_len:] = 1e30
    got = ops.decode_gqa_attention(_dev(q, cuda), _dev(k, cuda), _dev(v, cuda), kv_len)
    ops.Context.get(0).check()
    want = o.decode_gqa_attention(q, k, v, kv_len, d ** -0.5)
    assert_matmul_close(got.reshape(b * h, d), want.reshape(b * h, d), f"attention kv_len={kv_len}")


def test_decode_gqa_attention_peaked_scores_and_arguments(cuda):
    """One position dominates (large logit): the running-max rescaling must not lose it."""
    from izwi_b200 import IzbError, ops
    rng = np.random.default_rng(2)
    b, h, kvh, d, kv_len = 1, 8, 2, 128, 900
    q = bf16_np(rng.normal(0, 1, (b, h, d)))
    k = bf16_np(rng.normal(0, 1, (b, kvh, kv_len, d)))
    v = bf16_np(rng.normal(0, 1, (b, kvh, kv_len, d)))
    k[0, :, 777] = bf16_np(q[0, ::4] * 6.0)  # aligned with query heads 0 and 4: scores near 6 |q|^2 / sqrt(d)
    got = ops.decode_gqa_attention(_dev(q, cuda), _dev(k, cuda), _dev(v, cuda), kv_len)
    want = o.decode_gqa_attention(q, k, v, kv_len, d ** -0.5)
    assert_matmul_close(got.reshape(h, d), want.reshape(h, d), "peaked")
    with pytest.raises(IzbError) as e:
        ops.decode_gqa_attention(_dev(q, cuda), _dev(k, cuda), _dev(v, cuda), kv_len + 1)  # beyond the capacity
    assert e.value.status == -1
    q96 = torch.zeros(1, 8, 96, dtype=torch.bfloat16, device=cuda)
    kv96 = torch.zeros(1, 2, 16, 96, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(IzbError) as e:
        ops.decode_gqa_attention(q96, kv96, kv96, 16)
    assert e.value.status == -2


@pytest.mark.parametrize("b,h,kvh,d,with_norm", [(1, 16, 8, 128, True), (3, 8, 4, 64, True), (2, 32, 8, 128, False)])
def test_fused_qk_norm_rope_append(cuda, b, h, kvh, d, with_norm):
    """One launch against the composition norm -> rotation -> append of the oracle.  The fused kernel
    rounds once where the composition rounds after the norm and after the rotation: at most two bf16
    steps apart, equal for most elements."""
    from izwi_b200 import ops
    rng = np.random.default_rng(b * 10 + d)
    qkv = bf16_np(rng.normal(0, 1, (b, (h + 2 * kvh) * d)))
    qn, kn = bf16_np(rng.normal(1, 0.1, d)), bf16_np(rng.normal(1, 0.1, d))
    ang = rng.uniform(0, 6.28, (b, d // 2))
    c, s = bf16_np(np.cos(ang)), bf16_np(np.sin(ang))
    cap, pos = 9, 5
    kc = torch.zeros(b, kvh, cap, d, device=cuda, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    q = ops.qk_norm_rope_append(_dev(qkv, cuda), _dev(qn, cuda) if with_norm else None, _dev(kn, cuda) if with_norm else None,
                                1e-6, _dev(c, cuda), _dev(s, cuda), kc, vc, h, pos)
    ops.Context.get(0).check()
    q_in = qkv[:, :h * d].reshape(b, h, d)
    k_in = qkv[:, h * d:(h + kvh) * d].reshape(b, kvh, d)
    v_in = qkv[:, (h + kvh) * d:].reshape(b, kvh, d)
    def single_rounding(x, w):
        """The fused arithmetic restated: norm and rotation in fp32, one rounding at the end."""
        y = x.astype(np.float32)
        if with_norm:
            ms = (y.astype(np.float64) ** 2).mean(axis=-1, keepdims=True)
            y = y * (1.0 / np.sqrt(ms + 1e-6)).astype(np.float32) * w
        half = d // 2
        cc, ss = c[:, None, :], s[:, None, :]
        return y, o.bf16_round(np.concatenate([y[..., :half] * cc - y[..., half:] * ss,
                                               y[..., :half] * ss + y[..., half:] * cc], axis=-1))

    for got, x, w in ((to_np(q), q_in, qn), (to_np(kc[:, :, pos]), k_in, kn)):
        y, want1 = single_rounding(x, w)
        mag = np.abs(y).max(axis=-1, keepdims=True)                     # the rotation can cancel: bound by the inputs
        assert (np.abs(got - want1) <= mag * 2.0 ** -8).all()
        assert (got == want1).mean() > 0.97
        # against the reference's sequence (norm rounded to bf16, then rotated and rounded again)
        xn = o.rms_norm(x, w, 1e-6)[0] if with_norm else x
        want2 = o.rope_pair(xn, c, s)
        assert (np.abs(got - want2) <= mag * 2.0 ** -6).all()
    assert np.array_equal(to_np(vc[:, :, pos]), v_in)
    untouched = torch.cat([kc[:, :, :pos], kc[:, :, pos + 1:]], dim=2)
    assert float(untouched.abs().max()) == 0.0


def test_unaligned_query_is_refused_before_any_launch(cuda):
    """q is read with 16-byte loads: a base that is not 16-byte aligned, or a token stride that is not a
    multiple of 8 elements, must come back as IZB_ERR_BAD_ARG from the host-side checks (nothing runs)."""
    import ctypes as C

    from izwi_b200 import _lib as L
    from izwi_b200 import ops
    ctx = ops.Context.get(0)
    b, h, kvh, d, cap = 2, 8, 4, 64, 32
    kc = torch.zeros(b, kvh, cap, d, device=cuda, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    qbuf = torch.zeros(b * (h * d + 8) + 8, device=cuda, dtype=torch.bfloat16)
    out = torch.full((b, h, d), 3.0, device=cuda, dtype=torch.bfloat16)
    launches = ctx.launch_count

    def call(q_ptr, ld_q):
        return L.lib().izb_decode_gqa_attention(ctx.handle, None, C.c_void_p(q_ptr), C.c_void_p(kc.data_ptr()),
                                                C.c_void_p(vc.data_ptr()), C.c_void_p(out.data_ptr()), b, h, kvh, d, 16, cap,
                                                ld_q, h * d, 0.125, None, 0)
    assert call(qbuf.data_ptr() + 2, h * d) == L.IZB_ERR_BAD_ARG       # base 2 bytes off
    assert call(qbuf.data_ptr(), h * d + 4) == L.IZB_ERR_BAD_ARG       # rows 8 bytes off
    assert ctx.launch_count == launches
    torch.cuda.synchronize()
    assert float(out.min()) == 3.0
    assert call(qbuf.data_ptr(), h * d + 8) == L.IZB_OK                # an aligned, padded layout is fine
    ctx.check()


# ---- a prompt's tokens: embedding rows, q/k norm + rotation + append for a run of tokens, causal attention ----

def test_embed_rows_and_out_of_range_id(cuda):
    from izwi_b200 import IzbError, _lib, ops
    rng = np.random.default_rng(5)
    table = bf16_np(rng.normal(0, 1, (50, 64)))
    ids = np.array([0, 49, 7, 7, 13], dtype=np.int32)
    got = ops.embed_rows(_dev(table, cuda), torch.from_numpy(ids).to(cuda))
    ops.Context.get(0).check()
    assert np.array_equal(to_np(got), table[ids])
    bad = ops.embed_rows(_dev(table, cuda), torch.tensor([3, 50, -1], dtype=torch.int32, device=cuda))
    with pytest.raises(IzbError) as e:
        ops.Context.get(0).check()
    assert e.value.status == _lib.IZB_ERR_BAD_ARG          # reported after the fact, as a bad argument
    assert np.array_equal(to_np(bad)[0], table[3]) and not to_np(bad)[1:].any()
    ops.Context.get(0).check()


@pytest.mark.parametrize("b,q_len,h,kvh,d,pos0,cap", [(1, 1, 16, 8, 128, 0, 8), (1, 7, 16, 8, 128, 0, 16),
                                                     (2, 33, 8, 2, 64, 5, 64), (1, 70, 4, 4, 128, 0, 128),
                                                     (1, 3, 32, 8, 128, 250, 256)])
def test_prompt_tokens_norm_rope_append_and_causal_attention(cuda, b, q_len, h, kvh, d, pos0, cap):
    """qk_norm_rope_append_seq + prefill_gqa_attention against the oracle's per-token composition: head
    norms, rotation by the token's position, cache append, then each new token attends to everything up
    to and including itself.  Earlier positions of the cache hold random keys and values."""
    from izwi_b200 import ops
    rng = np.random.default_rng(q_len * 100 + h)
    eps = 1e-6
    qkv = bf16_np(rng.normal(0, 1, (b * q_len, (h + 2 * kvh) * d)))
    qn, kn = bf16_np(rng.normal(1, 0.1, d)), bf16_np(rng.normal(1, 0.1, d))
    kc, vc = bf16_np(rng.normal(0, 1, (b, kvh, cap, d))), bf16_np(rng.normal(0, 1, (b, kvh, cap, d)))
    inv = 1.0 / (10000.0 ** (np.arange(0, d, 2) / d))
    ang = (pos0 + np.arange(q_len))[:, None] * inv[None, :]
    cos, sin = bf16_np(np.cos(ang)), bf16_np(np.sin(ang))
    kcd, vcd = _dev(kc, cuda), _dev(vc, cuda)
    q = ops.qk_norm_rope_append_seq(_dev(qkv, cuda), _dev(qn, cuda), _dev(kn, cuda), eps, _dev(cos, cuda), _dev(sin, cuda), kcd, vcd,
                                    h, q_len, pos0)
    out = ops.prefill_gqa_attention(q, kcd, vcd, q_len, pos0)
    ops.Context.get(0).check()
    # oracle: token by token
    want_q = np.zeros((b * q_len, h, d), dtype=np.float32)
    want = np.zeros((b * q_len, h, d), dtype=np.float32)
    for bi in range(b):
        for i in range(q_len):
            row = qkv[bi * q_len + i]
            qh = row[: h * d].reshape(1, h, d)
            kh = row[h * d: (h + kvh) * d].reshape(1, kvh, d)
            vh = row[(h + kvh) * d:].reshape(kvh, d)
            qh, _ = o.rms_norm(qh, qn, eps)
            kh, _ = o.rms_norm(kh, kn, eps)
            qh = o.rope_pair(qh, cos[i:i + 1], sin[i:i + 1])
            kh = o.rope_pair(kh, cos[i:i + 1], sin[i:i + 1])
            kc[bi, :, pos0 + i], vc[bi, :, pos0 + i] = kh[0], vh
            want_q[bi * q_len + i] = qh[0]
            want[bi * q_len + i] = o.decode_gqa_attention(qh, kc[bi:bi + 1], vc[bi:bi + 1], pos0 + i + 1, d ** -0.5)[0]
    # the fused kernel rounds once where the composition rounds after the norm and after the rotation
    assert np.abs(to_np(q) - want_q).max() <= 3e-2 * np.abs(want_q).max()
    assert np.abs(to_np(kcd)[:, :, pos0:pos0 + q_len] - kc[:, :, pos0:pos0 + q_len]).max() <= 3e-2 * np.abs(kc).max()
    assert np.array_equal(to_np(vcd), vc)
    assert_matmul_close(out.reshape(b * q_len, h * d), want.reshape(b * q_len, h * d), f"causal attention q_len={q_len}")
