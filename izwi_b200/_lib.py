"""ctypes binding of the C ABI declared in include/izwi_b200.h.

There is no fallback: if the shared library is missing the import of any
compute wrapper raises, so a box without the CUDA build fails loudly.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libizwi_b200.so"

IZB_OK = 0
IZB_ERR_BAD_ARG = -1
IZB_ERR_UNSUPPORTED = -2
IZB_ERR_LAUNCH = -3
IZB_ERR_TIMEOUT = -4
IZB_ERR_NO_DEVICE = -5
IZB_ERR_SCRATCH_TOO_SMALL = -6

IZB_BF16, IZB_F32, IZB_F16 = 0, 1, 2
IZB_W_BF16, IZB_W_Q8_0, IZB_W_Q4_K, IZB_W_Q6_K = 0, 1, 2, 3
IZB_EPI_NONE, IZB_EPI_GELU, IZB_EPI_SILU, IZB_EPI_SWIGLU, IZB_EPI_GELU_TANH, IZB_EPI_GLU = 0, 1, 2, 3, 4, 5


class LinearArgs(C.Structure):
    _fields_ = [
        ("wfmt", C.c_int32), ("y_dtype", C.c_int32),
        ("x", C.c_void_p), ("w", C.c_void_p), ("bias", C.c_void_p), ("y", C.c_void_p),
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("ldx", C.c_int64), ("ldy", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("epilogue", C.c_int32), ("prologue", C.c_int32),
        ("norm_weight", C.c_void_p), ("residual", C.c_void_p), ("ld_residual", C.c_int64),
        ("norm_eps", C.c_float), ("x_dtype", C.c_int32),
    ]


class KvPages(C.Structure):
    """Mirror of izb_kv_pages."""
    _fields_ = [("k_values", C.c_void_p), ("v_values", C.c_void_p), ("k_scales", C.c_void_p), ("v_scales", C.c_void_p),
                ("page_table", C.c_void_p), ("quantization", C.c_int32), ("page_size", C.c_int32), ("kv_heads", C.c_int32),
                ("head_dim", C.c_int32), ("max_pages_per_seq", C.c_int64)]


class Qwen3LayerPtrs(C.Structure):
    """Mirror of izb_qwen3_layer_ptrs."""
    _fields_ = [("input_norm", C.c_void_p), ("post_norm", C.c_void_p), ("q_norm", C.c_void_p), ("k_norm", C.c_void_p),
                ("qkv", C.c_void_p), ("o", C.c_void_p), ("gate_up", C.c_void_p), ("down", C.c_void_p),
                ("k_cache", C.c_void_p), ("v_cache", C.c_void_p)]


class Qwen3DecodeArgs(C.Structure):
    """Mirror of izb_qwen3_decode_args."""
    _fields_ = [("wfmt", C.c_int32), ("lm_head_fmt", C.c_int32),
                ("n_layers", C.c_int32), ("hidden", C.c_int32), ("heads", C.c_int32), ("kv_heads", C.c_int32),
                ("head_dim", C.c_int32), ("intermediate", C.c_int32), ("vocab", C.c_int32), ("pos", C.c_int32),
                ("kv_capacity", C.c_int64), ("eps", C.c_float), ("reserved_", C.c_int32),
                ("layers", C.c_void_p), ("embed", C.c_void_p), ("final_norm", C.c_void_p), ("lm_head", C.c_void_p),
                ("token", C.c_void_p), ("cos_half", C.c_void_p), ("sin_half", C.c_void_p), ("logits", C.c_void_p),
                ("next_token", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


class MoeArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("w_router", C.c_void_p), ("router_bias", C.c_void_p), ("w_gate_up", C.c_void_p),
        ("w_down", C.c_void_p), ("y", C.c_void_p),
        ("T", C.c_int64), ("H", C.c_int64), ("I", C.c_int64), ("E", C.c_int64),
        ("top_k", C.c_int32), ("reserved_", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


_SIGNATURES = {
    "izb_version": (C.c_int32, []),
    "izb_kernels_enabled": (C.c_int32, []),
    "izb_status_string": (C.c_char_p, [C.c_int32]),
    "izb_ctx_create": (C.c_int32, [C.c_int32, C.POINTER(C.c_void_p)]),
    "izb_ctx_destroy": (C.c_int32, [C.c_void_p]),
    "izb_ctx_check": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "izb_ctx_launch_count": (C.c_int64, [C.c_void_p]),
    "izb_ctx_selftest_wait_timeout": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "izb_quantized_storage_bytes": (C.c_int32, [C.c_int32, C.c_int64, C.c_int64, C.POINTER(C.c_size_t)]),
    "izb_dequantize": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p]),
    "izb_linear_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int64, C.c_int64, C.c_int64]),
    "izb_linear_workspace_bytes_ex": (C.c_size_t, [C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_int32]),
    "izb_linear_workspace_bytes_args": (C.c_size_t, [C.POINTER(LinearArgs)]),
    "izb_linear": (C.c_int32, [C.c_void_p, C.c_void_p, C.POINTER(LinearArgs)]),
    "izb_linear_fusion_max_tokens": (C.c_int32, [C.c_int32]),
    "izb_linear_bf16": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_int64, C.c_int64, C.c_int64]),
    "izb_linear_q8_0": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_int64, C.c_int64, C.c_int64]),
    "izb_linear_q4_k": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_int64, C.c_int64, C.c_int64]),
    "izb_linear_group_plan_bytes": (C.c_size_t, [C.c_int32]),
    "izb_linear_group_plan": (C.c_int32, [C.c_void_p, C.POINTER(LinearArgs), C.c_int32, C.c_void_p, C.c_size_t]),
    "izb_linear_group_launch": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "izb_linear_group_launch_host": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                                                 C.c_void_p, C.c_void_p, C.c_size_t]),
    "izb_static_scratch_bytes": (C.c_size_t, []),
    "izb_linear_quantized_static": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
                                                C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_int32]),
    "izb_moe_route": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                  C.c_int64, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "izb_moe_topk": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p]),
    "izb_moe_permute": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p,
                                    C.c_void_p]),
    "izb_moe_gather": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.c_int64,
                                   C.c_int64, C.c_void_p]),
    "izb_moe_grouped_gemm": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int32]),
    "izb_moe_combine": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32,
                                    C.c_int64, C.c_void_p]),
    "izb_moe_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int32]),
    "izb_moe_forward": (C.c_int32, [C.c_void_p, C.c_void_p, C.POINTER(MoeArgs)]),
    "izb_comm_unique_id": (C.c_int32, [C.c_void_p]),
    "izb_comm_init": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.POINTER(C.c_void_p)]),
    "izb_comm_destroy": (C.c_int32, [C.c_void_p]),
    "izb_tp_allreduce": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32]),
    "izb_comm_allgather": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64]),
    "izb_ep_alltoall": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_int64), C.c_void_p,
                                    C.POINTER(C.c_int64), C.c_int64]),
    "izb_ar_create": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_size_t, C.POINTER(C.c_void_p)]),
    "izb_ar_local_handle": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "izb_ar_connect": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "izb_ar_max_bytes": (C.c_size_t, [C.c_void_p]),
    "izb_ar_allreduce": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32]),
    "izb_ar_operand": (C.c_void_p, [C.c_void_p, C.c_int32]),
    "izb_ar_result": (C.c_void_p, [C.c_void_p, C.c_int32]),
    "izb_ar_allreduce_region": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int32]),
    "izb_ar_destroy": (C.c_int32, [C.c_void_p]),
    "izb_silu_mul": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64]),
    "izb_ep_create": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int32,
                                  C.POINTER(C.c_void_p)]),
    "izb_ep_local_handle": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "izb_ep_connect": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "izb_ep_recv_capacity_rows": (C.c_int64, [C.c_void_p]),
    "izb_ep_recv_rows": (C.c_void_p, [C.c_void_p]),
    "izb_ep_recv_offsets": (C.c_void_p, [C.c_void_p]),
    "izb_ep_returned_rows": (C.c_void_p, [C.c_void_p]),
    "izb_ep_dispatch": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64]),
    "izb_ep_return": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "izb_ep_destroy": (C.c_int32, [C.c_void_p]),
    "izb_rms_norm": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_float]),
    "izb_argmax_rows": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int64,
                                    C.c_void_p, C.c_void_p]),
    "izb_sample_rows": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_float,
                                    C.c_int32, C.c_float, C.c_void_p, C.c_void_p]),
    "izb_rope_pair": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                  C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int64]),
    "izb_kv_append": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                  C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_int64]),
    "izb_qk_norm_rope_append": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_float,
                                            C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64,
                                            C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int64]),
    "izb_decode_gqa_attention_workspace_bytes": (C.c_size_t, [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32,
                                                             C.c_int64]),
    "izb_decode_gqa_attention": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                             C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.c_int64,
                                             C.c_int64, C.c_float, C.c_void_p, C.c_size_t]),
    "izb_kv_page_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "izb_kv_page_scales": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "izb_kv_pages_append": (C.c_int32, [C.c_void_p, C.c_void_p, C.POINTER(KvPages), C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                        C.c_int64, C.c_int64, C.c_void_p]),
    "izb_kv_pages_materialize": (C.c_int32, [C.c_void_p, C.c_void_p, C.POINTER(KvPages), C.c_int32, C.c_int64, C.c_void_p,
                                             C.c_void_p, C.c_int64, C.c_int64]),
    "izb_paged_decode_gqa_attention_workspace_bytes": (C.c_size_t, [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32,
                                                                   C.c_int64]),
    "izb_paged_decode_gqa_attention": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(KvPages), C.c_void_p, C.c_void_p,
                                                   C.c_int64, C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_float, C.c_void_p,
                                                   C.c_size_t]),
    "izb_embed_rows": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p,
                                   C.c_int64]),
    "izb_qk_norm_rope_append_seq": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_float,
                                                C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64,
                                                C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int64]),
    "izb_prefill_gqa_attention": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                              C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.c_int64,
                                              C.c_int64, C.c_float]),
    "izb_fold_depthwise_conv1d_batch_norm": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                         C.c_void_p, C.c_float, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p]),
    "izb_depthwise_conv1d_bias_swish": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                    C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_int64, C.c_int64,
                                                    C.c_int32]),
    "izb_dequantize_mlx_affine": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_void_p, C.c_void_p,
                                              C.c_int64, C.c_int32, C.c_int64, C.c_int64, C.c_int32, C.c_void_p]),
    "izb_qwen3_decode_token_workspace_bytes": (C.c_size_t, [C.c_void_p, C.POINTER(Qwen3DecodeArgs)]),
    "izb_qwen3_decode_token": (C.c_int32, [C.c_void_p, C.c_void_p, C.POINTER(Qwen3DecodeArgs)]),
    "izb_gguf_open": (C.c_int32, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "izb_gguf_close": (C.c_int32, [C.c_void_p]),
    "izb_gguf_version": (C.c_int32, [C.c_void_p]),
    "izb_gguf_tensor_count": (C.c_int64, [C.c_void_p]),
    "izb_gguf_tensor_at": (C.c_int32, [C.c_void_p, C.c_int64, C.c_void_p]),
    "izb_gguf_find": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_void_p]),
    "izb_gguf_meta_count": (C.c_int64, [C.c_void_p]),
    "izb_gguf_meta_key": (C.c_char_p, [C.c_void_p, C.c_int64]),
    "izb_gguf_meta_u64": (C.c_int32, [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint64)]),
    "izb_gguf_meta_f64": (C.c_int32, [C.c_void_p, C.c_char_p, C.POINTER(C.c_double)]),
    "izb_gguf_meta_str": (C.c_int32, [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p), C.POINTER(C.c_size_t)]),
    "izb_gguf_upload": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
}


class GgufTensor(C.Structure):
    """Mirror of izb_gguf_tensor."""
    _fields_ = [("name", C.c_char_p), ("ggml_type", C.c_int32), ("wfmt", C.c_int32), ("n_dims", C.c_int32),
                ("reserved_", C.c_int32), ("dims", C.c_int64 * 4), ("rows", C.c_int64), ("cols", C.c_int64),
                ("data", C.c_void_p), ("bytes", C.c_size_t)]

_lib = None


def exported_symbols() -> list[str]:
    return sorted(_SIGNATURES)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m izwi_b200.build` "
                "(there is no CPU or PyTorch fallback for these ops)")
        handle = C.CDLL(str(LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


class IzbError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().izb_status_string(status).decode()
        super().__init__(f"{where}: {msg} ({status})")


def check(status: int, where: str) -> None:
    if status != IZB_OK:
        raise IzbError(status, where)
