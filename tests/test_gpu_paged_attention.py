"""The paged KV cache (models/shared/attention/paged.rs) on the GPU against the oracle's restatement: page
bytes and scales bit for bit after prompt-sized and token-by-token appends (Int8 pages are rebuilt with a
new scale whenever they grow, Q4_0 blocks re-quantised from their bf16 contents, as the reference does),
the dense copy, and single-token attention over the pages.  Also the reference's own test bounds: a
quantised page stays within 0.08 (Int8) / 0.16 (Q4_0) of the dense values for N(0, 1) inputs
(paged.rs tests `test_quantized_materialize_close_to_dense`, `test_q4_0_quantized_materialize_close_to_dense`)."""
import numpy as np
import pytest
import torch

import izwi_oracle as o
from gpu_util import assert_matmul_close, bf16_np, to_np

pytestmark = pytest.mark.gpu


def _dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda).to(torch.bfloat16)


def _build(cuda, quant, batch, kvh, d, page, chunks, rng):
    """Appends the same chunks on the GPU and in the oracle; returns (cache, [per-sequence (k_pages, v_pages)])."""
    from izwi_b200 import paged
    total = sum(chunks)
    cache = paged.PagedKvCache(batch, kvh, d, total + page, cuda, quant, page)
    ref = [(o.KvPages(page, quant), o.KvPages(page, quant)) for _ in range(batch)]
    for n in chunks:
        k, v = bf16_np(rng.normal(0, 1, (batch, n, kvh, d))), bf16_np(rng.normal(0, 1, (batch, n, kvh, d)))
        cache.append(_dev(k, cuda), _dev(v, cuda))
        for b in range(batch):
            ref[b][0].append(k[b])
            ref[b][1].append(v[b])
    return cache, ref


@pytest.mark.parametrize("quant", ["none", "int8", "q4_0"])
@pytest.mark.parametrize("batch,kvh,d,page,chunks", [(1, 8, 128, 64, [70, 1, 1, 1]), (2, 2, 64, 4, [10, 3]), (1, 4, 128, 16, [1] * 20),
                                                     (3, 8, 64, 64, [5, 64, 1]), (1, 2, 64, 5, [17])])
def test_appends_give_the_reference_pages_bit_for_bit(cuda, quant, batch, kvh, d, page, chunks):
    from izwi_b200 import ops
    rng = np.random.default_rng(len(chunks) * 10 + page)
    cache, ref = _build(cuda, quant, batch, kvh, d, page, chunks, rng)
    ops.Context.get(0).check()
    total = sum(chunks)
    assert cache.seq_lens.cpu().tolist() == [total] * batch
    for which, sel in (("k", 0), ("v", 1)):
        dense = to_np(cache.materialize(which, total))
        for b in range(batch):
            want = ref[b][sel].materialize()
            assert len(ref[b][sel].pages) == (total + page - 1) // page          # append_to_pages respects the page size
            assert np.array_equal(dense[b], want), (quant, which, b, float(np.abs(dense[b] - want).max()))
    # the stored bytes and scales of the first sequence's last page
    if quant != "none":
        row = kvh * d
        nbytes = page * row if quant == "int8" else page * row // 2
        last = (total - 1) // page
        held = total - last * page
        pool_page = int(cache.page_table[0, last])
        kind, vals, scales, _ = ref[0][0].pages[-1]
        got_vals = cache.k_values[pool_page * nbytes: pool_page * nbytes + vals.size].cpu().numpy()
        assert np.array_equal(got_vals, vals.reshape(-1))
        if quant == "int8":
            assert np.float32(cache.k_scales[pool_page].item()) == np.float32(scales)
        else:
            per = page * row // 32
            assert np.array_equal(cache.k_scales[pool_page * per: pool_page * per + held * row // 32].cpu().numpy(), scales)


@pytest.mark.parametrize("quant,bound", [("int8", 0.08), ("q4_0", 0.16)])
def test_quantised_pages_stay_close_to_dense(cuda, quant, bound):
    rng = np.random.default_rng(4)
    from izwi_b200 import paged
    k = bf16_np(rng.normal(0, 1, (1, 17, 2, 64)) * 0.25)
    cache = paged.PagedKvCache(1, 2, 64, 32, cuda, quant, 5)
    cache.append(_dev(k, cuda), _dev(k, cuda))
    assert np.abs(to_np(cache.materialize("k", 17)) - k).max() < bound


@pytest.mark.parametrize("quant", ["none", "int8", "q4_0"])
@pytest.mark.parametrize("batch,h,kvh,d,page,total", [(1, 16, 8, 128, 64, 300), (2, 8, 2, 64, 16, 45), (1, 32, 8, 128, 64, 4100),
                                                      (4, 4, 4, 64, 64, 1), (1, 12, 4, 128, 7, 100)])
def test_paged_decode_attention(cuda, quant, batch, h, kvh, d, page, total):
    from izwi_b200 import ops
    rng = np.random.default_rng(total + h)
    cache, ref = _build(cuda, quant, batch, kvh, d, page, [total], rng)
    q = bf16_np(rng.normal(0, 1, (batch, h, d)))
    got = cache.decode_attention(_dev(q, cuda))
    ops.Context.get(0).check()
    want = np.stack([o.paged_decode_attention(q[b], ref[b][0], ref[b][1], d ** -0.5) for b in range(batch)])
    assert_matmul_close(got.reshape(batch, h * d), want.reshape(batch, h * d), f"paged attention {quant} len={total}")


def test_page_table_too_short_is_reported(cuda):
    from izwi_b200 import IzbError, _lib, ops, paged
    cache = paged.PagedKvCache(1, 2, 64, 8, cuda, "int8", 4)             # two pages
    k = torch.zeros(1, 9, 2, 64, device=cuda, dtype=torch.bfloat16)     # needs three
    cache.append(k, k)
    with pytest.raises(IzbError) as e:
        ops.Context.get(0).check()
    assert e.value.status == _lib.IZB_ERR_BAD_ARG
    ops.Context.get(0).check()


def test_dtype_hints():
    from izwi_b200 import paged
    assert paged.kv_quantization_from_dtype_hint(" INT8 ") == "int8" and paged.kv_quantization_from_dtype_hint("q8") == "int8"
    assert paged.kv_quantization_from_dtype_hint("q4") == "q4_0" and paged.kv_quantization_from_dtype_hint("bf16") == "none"
