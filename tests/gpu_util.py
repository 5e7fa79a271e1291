"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

import izwi_oracle as o

# The gates stated for bf16 matmul outputs accumulated in fp32.
MAX_REL_ERR = 2e-2
MIN_COSINE = 0.9999


def to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().to(torch.float32).cpu().numpy()


def bf16_np(x: np.ndarray) -> np.ndarray:
    return o.bf16_round(np.asarray(x, dtype=np.float32))


def assert_matmul_close(got: torch.Tensor, want: np.ndarray, what: str = ""):
    g = to_np(got)
    assert g.shape == want.shape, (what, g.shape, want.shape)
    assert np.isfinite(g).all(), f"{what}: non-finite output"
    rel, cos = o.rel_err_and_cosine(g, want)
    assert rel <= MAX_REL_ERR and cos >= MIN_COSINE, f"{what}: max rel err {rel:.3e}, cosine {cos:.6f}"
    return rel, cos


def make_weight_np(fmt: str, n: int, k: int, rng: np.random.Generator):
    """Returns (device-ready raw ndarray, fp32 dequantised [n, k])."""
    if fmt == "bf16":
        w = bf16_np(rng.normal(0, 0.02, (n, k)))
        return w, w
    if fmt == "q8_0":
        raw = o.make_q8_0_blocks(rng, n * k // 32)
    elif fmt == "q6_k":
        raw = o.make_q6_k_blocks(rng, n * k // 256)
    else:
        raw = o.make_q4_k_blocks(rng, n * k // 256, d_scale=1e-4, dmin_scale=7.5e-4)
    return raw, o.dequantize(raw, fmt).reshape(n, k)


def upload_weight(fmt: str, raw: np.ndarray, device) -> torch.Tensor:
    if fmt == "bf16":
        return torch.from_numpy(raw).to(device).to(torch.bfloat16)
    return torch.from_numpy(raw).to(device)
