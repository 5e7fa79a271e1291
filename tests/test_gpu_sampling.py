"""izb_sample_rows against the oracle's restatement of the reference's host-side sampler: greedy, pure
temperature (index order), top-k, top-p and both, on fp32 and bf16 logits (bf16 logits tie often, which
exercises the equal-value groups), rows with non-finite entries, and the frequencies of many draws."""
import numpy as np
import pytest
import torch

import izwi_oracle as o
from gpu_util import bf16_np

pytestmark = pytest.mark.gpu

CASES = [(0.0, 0, 1.0), (1.0, 0, 1.0), (0.7, 50, 1.0), (0.9, 0, 0.9), (1.3, 40, 0.8), (0.5, 1, 1.0), (1.0, 5, 0.3),
         (2.0, 0, 0.999), (1.0, 100000, 0.5)]


def _check(cuda, logits_np, dtype, temperature, top_k, top_p, us):
    from izwi_b200 import ops
    rows = len(us)
    lg = torch.from_numpy(np.repeat(logits_np[None, :], rows, axis=0)).to(cuda).to(dtype)
    u = torch.from_numpy(np.asarray(us, dtype=np.float32)).to(cuda)
    got = ops.sample_rows(lg, temperature, top_k, top_p, u).cpu().numpy()
    ops.Context.get(0).check()
    held = lg[0].float().cpu().numpy()                       # what the kernel saw (bf16-rounded where bf16)
    bad = 0
    for r, uu in enumerate(us):
        want, margin = o.sample_from_logits(held, temperature, top_k, top_p, float(np.float32(uu)))
        if got[r] != want:
            # a draw within 1e-5 of a boundary of the cumulative distribution may fall either way; an equal-valued
            # neighbour in a tie group is the same outcome under another summation order only at such a boundary
            assert margin < 1e-5, (temperature, top_k, top_p, uu, int(got[r]), want, margin)
            bad += 1
    assert bad <= max(1, rows // 20)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("temperature,top_k,top_p", CASES)
def test_draws_match_the_oracle(cuda, dtype, temperature, top_k, top_p):
    rng = np.random.default_rng(int(temperature * 10) + top_k)
    for vocab, spread in ((1000, 3.0), (151936, 4.0), (37, 1.0)):
        logits = (rng.normal(0, spread, vocab)).astype(np.float32)
        us = np.concatenate([[0.0, 0.5, 0.999999], rng.uniform(0, 1, 29)])
        _check(cuda, logits, dtype, temperature, top_k, top_p, us)


def test_non_finite_logits_are_never_drawn(cuda):
    rng = np.random.default_rng(3)
    logits = rng.normal(0, 2, 5000).astype(np.float32)
    logits[::7] = -np.inf
    logits[5] = np.nan
    logits[11] = np.inf
    for temperature, top_k, top_p in ((1.0, 0, 1.0), (0.8, 20, 0.9), (0.0, 0, 1.0)):
        _check(cuda, logits, torch.float32, temperature, top_k, top_p, rng.uniform(0, 1, 40))


def test_frequencies_follow_the_distribution(cuda):
    from izwi_b200 import ops
    rng = np.random.default_rng(8)
    logits = np.array([2.0, 1.0, 0.0, -1.0, -30.0, 1.0], dtype=np.float32)
    n = 20000
    lg = torch.from_numpy(np.repeat(logits[None, :], n, axis=0)).to(cuda)
    u = torch.from_numpy(rng.uniform(0, 1, n).astype(np.float32)).to(cuda)
    got = ops.sample_rows(lg, 1.0, 0, 1.0, u).cpu().numpy()
    p = np.exp(logits - logits.max())
    p /= p.sum()
    freq = np.bincount(got, minlength=len(logits)) / n
    assert np.abs(freq - p).max() < 0.015
    top2 = ops.sample_rows(lg, 1.0, 2, 1.0, u).cpu().numpy()
    assert set(np.unique(top2)) <= {0, 1}            # of the two equal logits the lower index is the one kept
    ops.Context.get(0).check()
