"""Generates the committed golden fixtures.

Run from the repository root:  python tests/golden/make_golden.py

  ggml_dequant.npz   seeded Q8_0 / Q4_K / Q6_K blocks together with the fp32 values that
                     gguf-py 0.19.0 (`gguf.quants.dequantize`, the GGML project's own
                     Python statement of ggml-quants.c) produces for them, plus Q8_0
                     quantisation of a seeded fp32 matrix.
  reference_cases.json  the literal inputs / expected outputs of the reference's unit
                     tests for this path (crates/izwi-core/src/models/architectures/
                     qwen3/core.rs:2481-2511, 2514-2545, 2569-2595, 2598-2684,
                     3100-3142), transcribed as data.
"""
import json
import sys
from pathlib import Path

import numpy as np
from gguf import GGMLQuantizationType as T
from gguf import quants

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent / "oracle"))
import izwi_oracle as o  # noqa: E402


def main():
    rng = np.random.default_rng(20240607)
    q8 = o.make_q8_0_blocks(rng, 48)
    q4 = o.make_q4_k_blocks(rng, 24, d_scale=1e-4, dmin_scale=7.5e-4)
    # edge blocks: zero scale, extreme codes, extreme 6-bit scales
    q8e = q8[: 34 * 4].copy().reshape(4, 34)
    q8e[0, 0:2] = 0
    q8e[1, 2:] = np.int8(-127).view(np.uint8)
    q8e[2, 2:] = 127
    q8e[3, 0:2] = np.array([0x7BFF], dtype=np.uint16).view(np.uint8)  # largest finite fp16
    q4e = q4[: 144 * 3].copy().reshape(3, 144)
    q4e[0, 4:16] = 0xFF
    q4e[1, 16:] = 0xFF
    q4e[2, 0:4] = 0
    q8 = np.concatenate([q8, q8e.reshape(-1)])
    q4 = np.concatenate([q4, q4e.reshape(-1)])
    f = rng.normal(0, 0.05, (6, 96)).astype(np.float32)
    f[0, :32] = 0
    # drawn after everything above so that the earlier vectors keep their values
    q6 = o.make_q6_k_blocks(rng, 20)
    q6e = q6[: 210 * 3].copy().reshape(3, 210)
    q6e[0, 0:192] = 0xFF                                   # largest codes (+31)
    q6e[1, 0:192] = 0x00                                   # smallest codes (-32)
    q6e[1, 192:208] = np.int8(-128).view(np.uint8)         # extreme scales
    q6e[2, 208:210] = 0                                    # zero super-block scale
    q6 = np.concatenate([q6, q6e.reshape(-1)])
    np.savez_compressed(
        HERE / "ggml_dequant.npz",
        q8_0_raw=q8,
        q8_0_f32=quants.dequantize(q8.reshape(1, -1), T.Q8_0).reshape(-1),
        q4_k_raw=q4,
        q4_k_f32=quants.dequantize(q4.reshape(1, -1), T.Q4_K).reshape(-1),
        q6_k_raw=q6,
        q6_k_f32=quants.dequantize(q6.reshape(1, -1), T.Q6_K).reshape(-1),
        quant_in=f,
        quant_q8_0=quants.quantize(f, T.Q8_0).reshape(-1),
    )
    cases = {
        "dense_projection_with_bias": {
            "weight": [[1.0, 2.0], [3.0, 4.0]], "bias": [0.5, -1.0], "input": [[2.0, 3.0]],
            "expected": [[8.5, 17.0]]},
        "dense_projection_no_bias": {
            "weight": [[1.0, 2.0], [3.0, 4.0]], "bias": None, "input": [[2.0, 3.0]],
            "expected": [[8.0, 18.0]]},
        "selected_logits": {
            "weight": [[1.0, 0.0, 0.5], [-1.0, 0.25, 2.0], [-0.5, 1.5, 0.75], [-0.25, 1.25, 0.5]],
            "bias": [0.1, -0.2, 0.3, 0.4], "hidden": [[0.5, -1.0, 2.0]], "token_ids": [3, 1], "tol": 1e-6},
        "fused_qkv": {
            "q": [[0.1, 0.2, 0.3], [-0.4, 0.5, 0.6], [0.7, -0.8, 0.9], [1.0, -1.1, 1.2]],
            "k": [[0.3, -0.2, 0.1], [0.6, 0.4, -0.5]],
            "v": [[-0.7, 0.8, 0.9], [0.2, -0.1, 0.4]],
            "input": [[[1.0, -2.0, 0.5], [0.25, 1.5, -0.75]]], "tol": 1e-5},
        "fused_gate_up": {
            "gate": [[0.1, -0.2, 0.3], [0.4, 0.5, -0.6], [-0.7, 0.8, 0.9]], "gate_bias": [0.1, -0.2, 0.3],
            "up": [[-0.3, 0.2, 0.1], [0.6, -0.4, 0.5], [0.7, 0.9, -0.8]], "up_bias": [0.2, 0.4, -0.6],
            "input": [[[1.0, -2.0, 0.5], [0.25, 1.5, -0.75]]], "tol": 1e-5},
        "packed_q8_0": {
            "w1": {"rows": 2, "cols": 32, "formula": "(idx - 31) / 8"},
            "w2": {"rows": 1, "cols": 32, "formula": "(15 - idx) / 7"},
            "x": {"rows": 1, "cols": 32, "formula": "(idx + 1) / 16"}, "tol": 1e-5},
    }
    (HERE / "reference_cases.json").write_text(json.dumps(cases, indent=1) + "\n")
    print("wrote", HERE / "ggml_dequant.npz", HERE / "reference_cases.json")


if __name__ == "__main__":
    main()
