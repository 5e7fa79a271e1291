"""GGUF reader (C ABI `izb_gguf_*` and the `GgufLoader` mirror) against files written by gguf-py,
the GGML project's own writer: header, metadata, tensor directory, raw bytes; malformed files are
rejected with a status, never read out of bounds."""
import ctypes as C
import struct

import numpy as np
import pytest

import izwi_oracle as o

gguf = pytest.importorskip("gguf")


@pytest.fixture(scope="module")
def sample(tmp_path_factory):
    """A small file in the llama.cpp naming scheme with the tensor types a Q4_K_M model mixes."""
    path = tmp_path_factory.mktemp("gguf") / "tiny-q4_k_m.gguf"
    rng = np.random.default_rng(3)
    tensors = {
        "token_embd.weight": (o.make_q6_k_blocks(rng, 8 * 512 // 256).reshape(8, -1), gguf.GGMLQuantizationType.Q6_K, (8, 512)),
        "blk.0.attn_q.weight": (o.make_q4_k_blocks(rng, 16 * 512 // 256).reshape(16, -1), gguf.GGMLQuantizationType.Q4_K, (16, 512)),
        "blk.0.ffn_down.weight": (o.make_q8_0_blocks(rng, 4 * 64 // 32).reshape(4, -1), gguf.GGMLQuantizationType.Q8_0, (4, 64)),
        "blk.0.attn_norm.weight": (rng.normal(1, 0.1, 512).astype(np.float32), None, (512,)),
        "blk.0.attn_k.bias": (rng.normal(0, 0.1, 16).astype(np.float16), None, (16,)),
    }
    w = gguf.GGUFWriter(str(path), "qwen3")
    w.add_name("tiny")
    w.add_uint32("qwen3.block_count", 1)
    w.add_uint64("general.parameter_count", 12345678901)
    w.add_float32("qwen3.attention.layer_norm_rms_epsilon", 1e-6)
    w.add_bool("tiny.flag", True)
    w.add_int32("tiny.negative", -7)
    w.add_array("tokenizer.ggml.tokens", ["a", "bc", "def"])
    w.add_array("tiny.ints", [1, 2, 3, 4])
    for name, (data, qtype, _) in tensors.items():
        w.add_tensor(name, data, raw_dtype=qtype)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return path, tensors


def test_directory_metadata_and_bytes(sample):
    from izwi_b200.gguf import GgufLoader
    path, tensors = sample
    g = GgufLoader.from_path(path)
    assert set(g.tensor_names()) == set(tensors)
    for name, (data, qtype, shape) in tensors.items():
        info = g.tensor_info(name)
        assert info.shape == tuple(shape) and g.tensor_shape(name) == list(shape)
        assert info.nbytes == data.nbytes
        assert g.tensor_bytes(name) == data.tobytes()
        assert g.has_tensor(name)
    assert g.tensor_info("token_embd.weight").wfmt == "q6_k" and g.tensor_info("token_embd.weight").dtype == "Q6_K"
    assert g.tensor_info("blk.0.attn_q.weight").wfmt == "q4_k"
    assert g.tensor_info("blk.0.ffn_down.weight").wfmt == "q8_0"
    assert g.tensor_info("blk.0.attn_norm.weight").wfmt is None and g.tensor_info("blk.0.attn_norm.weight").dtype == "F32"
    assert (g.tensor_info("blk.0.attn_q.weight").rows, g.tensor_info("blk.0.attn_q.weight").cols) == (16, 512)
    assert not g.has_tensor("blk.1.attn_q.weight") and g.tensor_shape("nope") is None
    # metadata
    assert g.get_metadata_string("general.architecture") == "qwen3"
    assert g.get_metadata_u64("qwen3.block_count") == 1
    assert g.get_metadata_u64("general.parameter_count") == 12345678901
    assert abs(g.get_metadata_f64("qwen3.attention.layer_norm_rms_epsilon") - 1e-6) < 1e-12
    assert g.get_metadata_u64("tiny.flag") == 1
    assert g.get_metadata_u64("tiny.negative") == 2 ** 64 - 7
    assert g.get_metadata_f64("tiny.negative") == -7.0
    assert g.get_metadata_string("qwen3.block_count") is None          # wrong type
    assert g.get_metadata_u64("tokenizer.ggml.tokens") is None         # arrays are skipped, not scalars
    assert g.get_metadata_string("missing.key") is None
    info = g.get_model_info()
    assert info.architecture == "qwen3" and info.parameter_count == 12345678901
    assert info.quantization in ("Q4_K", "Q6_K", "Q8_0")               # no quantization_type key: detected from tensors
    assert info.metadata["general.name"] == "tiny"
    # dequantising the bytes the reader hands out reproduces the oracle's values
    raw = np.frombuffer(g.tensor_bytes("token_embd.weight"), dtype=np.uint8)
    assert np.array_equal(o.dequantize(raw, "q6_k"), o.dequantize(tensors["token_embd.weight"][0].reshape(-1), "q6_k"))
    g.close()


def _open_status(path):
    from izwi_b200 import _lib
    h = C.c_void_p()
    rc = _lib.lib().izb_gguf_open(str(path).encode(), C.byref(h))
    if rc == 0:
        _lib.lib().izb_gguf_close(h)
    return rc


def test_malformed_files_are_rejected(sample, tmp_path):
    from izwi_b200.gguf import GgufLoader, ModelLoadError
    path, _ = sample
    good = path.read_bytes()
    assert _open_status(path) == 0
    cases = {
        "missing": None,
        "short": good[:20],
        "bad_magic": b"GGML" + good[4:],
        "version_9": good[:4] + struct.pack("<I", 9) + good[8:],
        "huge_tensor_count": good[:8] + struct.pack("<Q", 2 ** 60) + good[16:],
        "huge_kv_count": good[:16] + struct.pack("<Q", 2 ** 60) + good[24:],
        "truncated_directory": good[:200],
        "truncated_data": good[:-64],
        "string_length_past_end": good[:24] + struct.pack("<Q", 2 ** 40) + good[32:],
    }
    for name, blob in cases.items():
        p = tmp_path / f"{name}.gguf"
        if blob is not None:
            p.write_bytes(blob)
        rc = _open_status(p)
        assert rc in (-1, -2), (name, rc)
        with pytest.raises(ModelLoadError):
            GgufLoader.from_path(p)
    # every single-byte truncation of the header + directory region fails cleanly or parses a valid prefix
    for cut in range(24, min(len(good), 1400), 37):
        p = tmp_path / "cut.gguf"
        p.write_bytes(good[:cut])
        assert _open_status(p) in (0, -1, -2)


def test_missing_tensor_message(sample):
    from izwi_b200.gguf import GgufLoader, ModelLoadError
    g = GgufLoader.from_path(sample[0])
    with pytest.raises(ModelLoadError, match="Failed to load tensor 'output.weight' from GGUF"):
        g.tensor_info("output.weight")
