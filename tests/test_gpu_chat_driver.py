"""The compiled host driver (izwi_b200/host/izwi_chat.hpp: GgufLoader, Qwen3Model::forward,
Qwen3ChatModel::start_decode / decode_step) on a small Qwen3-shaped model written to a GGUF file with
gguf-py: the prompt through the prefill path (GEMM + causal attention) and through the one-token
path must give the logits the Python mirror of the decode step gives (itself checked against the
oracle in test_gpu_decode_step.py), and the greedy continuation must follow those logits."""
import subprocess

import numpy as np
import pytest
import torch

import izwi_oracle as o
from gpu_util import bf16_np

gguf = pytest.importorskip("gguf")
pytestmark = pytest.mark.gpu

HID, HEADS, KVH, D, INTER, LAYERS, VOCAB, EPS, THETA = 256, 4, 2, 64, 512, 2, 512, 1e-6, 1e6
# the same model with heads of 128: the shape the one-launch token (izb_qwen3_decode_token) takes
WIDE_HEADS, WIDE_KVH, WIDE_D = 2, 1, 128


@pytest.fixture(scope="module")
def selftest():
    from izwi_b200 import build
    build.build()
    return build.build_host_selftest()


def _q8(rng, n, k, scale):
    raw = o.make_q8_0_blocks(rng, n * k // 32, d_scale=scale)
    return raw.reshape(n, -1)


def _write_model(tmp_path_factory, HEADS, KVH, D):
    rng = np.random.default_rng(77)
    path = tmp_path_factory.mktemp("chat") / f"tiny-qwen3-q8_0-d{D}.gguf"
    t = {"token_embd.weight": bf16_np(rng.normal(0, 0.5, (VOCAB, HID))),
         "output_norm.weight": rng.normal(1, 0.1, HID).astype(np.float32),
         "output.weight": _q8(rng, VOCAB, HID, 6e-4)}
    for i in range(LAYERS):
        p = f"blk.{i}."
        t[p + "attn_norm.weight"] = rng.normal(1, 0.1, HID).astype(np.float32)
        t[p + "ffn_norm.weight"] = rng.normal(1, 0.1, HID).astype(np.float32)
        t[p + "attn_q_norm.weight"] = rng.normal(1, 0.1, D).astype(np.float32)
        t[p + "attn_k_norm.weight"] = rng.normal(1, 0.1, D).astype(np.float32)
        t[p + "attn_q.weight"] = _q8(rng, HEADS * D, HID, 6e-4)
        t[p + "attn_k.weight"] = _q8(rng, KVH * D, HID, 6e-4)
        t[p + "attn_v.weight"] = _q8(rng, KVH * D, HID, 6e-4)
        t[p + "attn_output.weight"] = _q8(rng, HID, HEADS * D, 6e-4)
        t[p + "ffn_gate.weight"] = _q8(rng, INTER, HID, 6e-4)
        t[p + "ffn_up.weight"] = _q8(rng, INTER, HID, 6e-4)
        t[p + "ffn_down.weight"] = _q8(rng, HID, INTER, 4e-4)
    w = gguf.GGUFWriter(str(path), "qwen3")
    w.add_uint32("qwen3.block_count", LAYERS)
    w.add_uint32("qwen3.embedding_length", HID)
    w.add_uint32("qwen3.attention.head_count", HEADS)
    w.add_uint32("qwen3.attention.head_count_kv", KVH)
    w.add_uint32("qwen3.attention.key_length", D)
    w.add_uint32("qwen3.feed_forward_length", INTER)
    w.add_float32("qwen3.attention.layer_norm_rms_epsilon", EPS)
    w.add_float32("qwen3.rope.freq_base", THETA)
    for name, data in t.items():
        if data.dtype == np.uint8:
            w.add_tensor(name, data, raw_dtype=gguf.GGMLQuantizationType.Q8_0)
        elif name == "token_embd.weight":
            w.add_tensor(name, (data.view(np.uint32) >> 16).astype(np.uint16).view(np.uint8).reshape(VOCAB, HID * 2),
                         raw_dtype=gguf.GGMLQuantizationType.BF16)
        else:
            w.add_tensor(name, data)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return path, t


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    return _write_model(tmp_path_factory, HEADS, KVH, D)


@pytest.fixture(scope="module")
def wide_model(tmp_path_factory):
    return _write_model(tmp_path_factory, WIDE_HEADS, WIDE_KVH, WIDE_D)


def _python_mirror(t, cuda, HEADS=HEADS, KVH=KVH, D=D):
    from izwi_b200 import decoder
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)  # noqa: E731
    bf = lambda a: dev(a.astype(np.float32)).to(torch.bfloat16)  # noqa: E731
    layers = []
    for i in range(LAYERS):
        p = f"blk.{i}."
        qkv = np.concatenate([t[p + "attn_q.weight"], t[p + "attn_k.weight"], t[p + "attn_v.weight"]], axis=0)
        gu = np.concatenate([t[p + "ffn_gate.weight"], t[p + "ffn_up.weight"]], axis=0)
        layers.append(decoder.Qwen3DecoderLayer(decoder.Qwen3LayerWeights(
            "q8_0", HID, HEADS, KVH, D, INTER, bf(t[p + "attn_norm.weight"]), bf(t[p + "ffn_norm.weight"]),
            bf(t[p + "attn_q_norm.weight"]), bf(t[p + "attn_k_norm.weight"]), dev(qkv), dev(t[p + "attn_output.weight"]), dev(gu),
            dev(t[p + "ffn_down.weight"]), EPS)))
    return decoder.Qwen3Decoder(bf(t["token_embd.weight"]), layers, bf(t["output_norm.weight"]), dev(t["output.weight"]), "q8_0",
                                rope_theta=THETA)


def _run(selftest, path, tmp_path, mode, prompt, max_new, env=None, with_launches=False):
    import os
    out = tmp_path / f"logits_{mode}.bin"
    proc = subprocess.run([str(selftest), "chat", str(path), str(max_new), str(out), mode, *map(str, prompt)],
                          capture_output=True, text=True, timeout=300, env=None if env is None else {**os.environ, **env})
    assert proc.returncode == 0 and "chat: ok" in proc.stdout, proc.stdout + proc.stderr
    line = [ln for ln in proc.stdout.splitlines() if ln.startswith("generated:")][0]
    tokens = [int(v) for v in line.split()[1:]]
    positions = int([ln for ln in proc.stdout.splitlines() if ln.startswith("positions:")][0].split()[1])
    if with_launches:
        launches = int([ln for ln in proc.stdout.splitlines() if ln.startswith("launches:")][0].split()[1])
        return np.fromfile(out, dtype=np.float32), tokens, positions, launches
    return np.fromfile(out, dtype=np.float32), tokens, positions


@pytest.mark.parametrize("prompt_len", [1, 2, 7, 70])
def test_prefill_then_greedy_decode_follows_the_decode_step_mirror(cuda, selftest, model, tmp_path, prompt_len):
    from izwi_b200 import decoder, ops
    path, t = model
    rng = np.random.default_rng(prompt_len)
    prompt = [int(v) for v in rng.integers(1, VOCAB, prompt_len)]
    max_new = 6
    logits_p, tokens_p, pos_p = _run(selftest, path, tmp_path, "prefill", prompt, max_new)
    logits_d, tokens_d, pos_d = _run(selftest, path, tmp_path, "decode", prompt, max_new)
    # the Python mirror, token by token; then forced along the C++ driver's own choices
    mirror = _python_mirror(t, cuda)
    caches = [decoder.KvCache(1, KVH, 256, D, cuda) for _ in range(LAYERS)]
    for pos, tok in enumerate(prompt):
        _, logits = mirror.step(torch.tensor([tok], device=cuda), caches, pos, return_logits=True)
    want = logits[0].float().cpu().numpy()
    ops.Context.get(0).check()
    for got, what in ((logits_p, "prefill"), (logits_d, "token by token")):
        rel, cos = o.rel_err_and_cosine(got[None, :], want[None, :])
        assert rel <= 3e-2 and cos >= 0.9995, (what, prompt_len, rel, cos)
    # greedy continuation: every token the driver chose must be (one of) the best under the mirror's logits
    assert len(tokens_p) <= max_new and pos_p == prompt_len + len(tokens_p)   # every kept token was fed back once
    spread = float(want.max() - want.min())
    pos = prompt_len
    for tok in tokens_p:
        assert want[tok] >= want.max() - 2e-2 * spread, ("driver token is not a maximum of the mirror's logits", tok)
        _, logits = mirror.step(torch.tensor([tok], device=cuda), caches, pos, return_logits=True)
        want = logits[0].float().cpu().numpy()
        pos += 1
    if tokens_d and tokens_p:
        assert tokens_d[0] == tokens_p[0] or abs(logits_d[tokens_d[0]] - logits_d[tokens_p[0]]) <= 2e-2 * spread


def test_single_tokens_go_through_the_one_launch_kernel(cuda, selftest, wide_model, tmp_path):
    """A model the one-launch token takes (Q8_0 everywhere, head_dim 128): every single-token forward of the
    driver is one launch, and logits and greedy tokens agree with the composed step (the same driver with
    IZWI_B200_TOKEN_KERNEL=0) and with the Python mirror."""
    from izwi_b200 import decoder, ops
    path, t = wide_model
    prompt, max_new = [11, 403, 77, 250, 9], 6
    on = _run(selftest, path, tmp_path, "decode", prompt, max_new, with_launches=True)
    off = _run(selftest, path, tmp_path, "decode", prompt, max_new, env={"IZWI_B200_TOKEN_KERNEL": "0"}, with_launches=True)
    # 4 forced prompt steps + up to 6 generated tokens: one launch each (+ the arg-max per generated token and the
    # first token's composed... the first prompt token goes through start_decode's forward of one token as well)
    steps = len(prompt) + len(on[1])
    assert on[3] <= 2 * steps + 2, on[3]
    assert off[3] >= 8 * steps, off[3]
    rel, cos = o.rel_err_and_cosine(on[0][None, :], off[0][None, :])
    assert rel <= 3e-2 and cos >= 0.9995, (rel, cos)
    mirror = _python_mirror(t, cuda, WIDE_HEADS, WIDE_KVH, WIDE_D)
    caches = [decoder.KvCache(1, WIDE_KVH, 256, WIDE_D, cuda) for _ in range(LAYERS)]
    for pos, tok in enumerate(prompt):
        _, logits = mirror.step(torch.tensor([tok], device=cuda), caches, pos, return_logits=True)
    want = logits[0].float().cpu().numpy()
    ops.Context.get(0).check()
    rel, cos = o.rel_err_and_cosine(on[0][None, :], want[None, :])
    assert rel <= 3e-2 and cos >= 0.9995, (rel, cos)
    spread = float(want.max() - want.min())
    pos = len(prompt)
    for tok in on[1]:
        assert want[tok] >= want.max() - 2e-2 * spread, ("driver token is not a maximum of the mirror's logits", tok)
        _, logits = mirror.step(torch.tensor([tok], device=cuda), caches, pos, return_logits=True)
        want = logits[0].float().cpu().numpy()
        pos += 1
