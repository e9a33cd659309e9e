"""ctypes binding of the C ABI declared in include/et_b200.h.

The shared library is built in-tree by ``effective_transformer_b200.build``.
There is no CPU fallback: if the library is missing, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libet_b200.so")

ET_OK, ET_INVALID_ARGUMENT, ET_CUDA_ERROR, ET_WORKSPACE_TOO_SMALL, ET_DEVICE_TIMEOUT, ET_NOT_READY = range(6)
ET_FP32, ET_FP16 = 0, 1
NOALLOC_MAX_BATCH = 16384   # ET_NOALLOC_MAX_BATCH in include/et_b200.h
STATUS_NAMES = {0: "ET_OK", 1: "ET_INVALID_ARGUMENT", 2: "ET_CUDA_ERROR", 3: "ET_WORKSPACE_TOO_SMALL",
                4: "ET_DEVICE_TIMEOUT", 5: "ET_NOT_READY"}

PROF_NAMES = ["padding_offsets", "remove_padding", "gemm_qkv", "attention", "gemm_attn_out", "layernorm",
              "gemm_ffn1", "gemm_ffn2", "restore_padding", "embedding", "pooler"]

vp, ip, i32, i64 = C.c_void_p, C.POINTER(C.c_int), C.c_int, C.c_longlong


class Config(C.Structure):
    _fields_ = [("dtype", i32), ("num_layers", i32), ("head_num", i32), ("size_per_head", i32),
                ("ffn_dim", i32), ("max_batch_size", i32), ("max_seq_len", i32),
                ("layernorm_eps", C.c_float), ("device", i32)]


class TransformerParam(C.Structure):
    _fields_ = [("batch_size", i32), ("from_seq_len", i32), ("to_seq_len", i32), ("head_num", i32),
                ("size_per_head", i32)]


class EncoderParam(C.Structure):
    _fields_ = [(n, vp) for n in (
        "from_tensor", "to_tensor", "attr_kernel_Q", "attr_kernel_K", "attr_kernel_V", "attr_bias_Q",
        "attr_bias_K", "attr_bias_V", "attr_mask", "attr_output_kernel", "attr_output_bias",
        "attr_output_layernorm_gamma", "attr_output_layernorm_beta", "inter_kernel", "inter_bias",
        "output_kernel", "output_bias", "output_layernorm_gamma", "output_layernorm_beta",
        "batch_idx", "word_idx", "valid_word_num", "transformer_out", "stream")]


class InputParam(C.Structure):
    _fields_ = [("from_tensor", vp), ("mask", vp), ("valid_word_num", vp), ("batch_idx", vp),
                ("word_idx", vp), ("batch_size", i32), ("from_seq_len", i32), ("head_num", i32),
                ("size_per_head", i32), ("to_tensor", vp), ("stream", vp)]


class OutputParam(C.Structure):
    _fields_ = [("from_tensor", vp), ("valid_word_num", vp), ("batch_idx", vp), ("word_idx", vp),
                ("batch_size", i32), ("from_seq_len", i32), ("head_num", i32), ("size_per_head", i32),
                ("to_tensor", vp), ("stream", vp)]


# name -> (restype, argtypes); every symbol declared in include/et_b200.h
SIGNATURES = {
    "et_create": (i32, [C.POINTER(Config), C.POINTER(vp)]),
    "et_destroy": (i32, [vp]),
    "et_last_error": (C.c_char_p, [vp]),
    "et_set_layer_weights": (i32, [vp, i32, C.POINTER(vp), i32]),
    "et_workspace_bytes": (i32, [vp, i32, i32, C.POINTER(C.c_size_t)]),
    "et_input": (i32, [vp, C.POINTER(InputParam)]),
    "et_layer": (i32, [vp, i32, C.POINTER(EncoderParam), C.POINTER(TransformerParam)]),
    "et_output": (i32, [vp, C.POINTER(OutputParam)]),
    "et_forward": (i32, [vp, vp, vp, vp, i32, i32, vp]),
    "et_forward_host": (i32, [vp, vp, vp, vp, i32, i32, ip]),
    "et_set_embedding_weights": (i32, [vp, vp, i32, vp, i32, vp, i32, vp, vp, C.c_float, i32]),
    "et_set_pooler_weights": (i32, [vp, vp, vp, i32]),
    "et_forward_ids": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, vp]),
    "et_forward_ids_host": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, ip]),
    "et_pooler": (i32, [vp, vp, vp, vp, i32, i32, vp]),
    "et_last_packed_output": (i32, [vp, C.POINTER(vp), C.POINTER(vp)]),
    "et_graph_capture": (i32, [vp, vp, vp, vp, i32, i32]),
    "et_graph_capture_ids": (i32, [vp, vp, vp, vp, vp, vp, i32, i32]),
    "et_graph_launch": (i32, [vp, vp]),
    "et_graph_release": (i32, [vp]),
    "et_device_status": (i32, [vp, vp, ip]),
    "et_last_padding_info": (i32, [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(vp)]),
    "et_set_profiling": (i32, [vp, i32]),
    "et_get_profile": (i32, [vp, C.POINTER(C.c_double), C.POINTER(C.c_longlong), i32]),
    "et_copy_to_host": (i32, [vp, vp, C.c_size_t, vp]),
    "et_set_debug_simt": (i32, [vp, i32]),
    "et_set_fused_layernorm": (i32, [vp, i32]),
    "et_set_deferred_layernorm": (i32, [vp, i32]),
    "et_host_chunk_shares": (i32, [vp, ip, ip, ip]),
    "et_selftest_wait_timeout": (i32, [vp, vp]),
    "et_workspace_allocated_bytes": (i32, [vp, C.POINTER(C.c_size_t)]),
    "et_gemm_fused": (i32, [vp, vp, vp, vp, vp, vp, C.c_float, vp, vp, vp, i32, i32, i32, i32, vp, vp]),
    "et_fold_layernorm": (i32, [vp, vp, vp, vp, vp, vp, vp, i32, i32, vp]),
    "et_gemm_deferred_norm": (i32, [vp, vp, vp, vp, vp, vp, vp, C.c_float, vp, vp, vp, vp, i32, i32, i32, i32, vp, vp]),
    "et_padding_offsets": (i32, [vp, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp]),
    "et_padding_offsets_noalloc": (i32, [vp, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp]),
    "et_remove_padding": (i32, [i32, vp, vp, vp, vp, vp, i32, i32, i32, vp]),
    "et_restore_padding": (i32, [i32, vp, vp, vp, vp, vp, i32, i32, i32, vp]),
    "et_add_qkv_bias_transpose": (i32, [i32, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp]),
    "et_add_bias_gelu": (i32, [i32, vp, vp, vp, i32, i32, vp]),
    "et_add_bias_input_layernorm": (i32, [i32, vp, vp, vp, vp, vp, vp, i32, i32, C.c_float, vp]),
    "et_embedding_layernorm": (i32, [i32, vp, vp, vp, vp, vp, vp, i32, vp, i32, vp, vp, vp, C.c_float, vp,
                                     i32, i32, i32, vp]),
    "et_gather_first_tokens": (i32, [i32, vp, vp, vp, i32, i32, i32, vp]),
    "et_attention": (i32, [i32, vp, vp, vp, i64, i64, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp]),
    "et_attention_cross": (i32, [i32, vp, i64, vp, vp, i64, i64, vp, vp, vp, i32, i32, i32, i32, i32, vp]),
    "et_attention_general_mask": (i32, [i32, vp, vp, vp, i64, i64, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32,
                                        vp]),
    "et_set_general_mask": (i32, [vp, i32]),
    "et_forward_general_mask": (i32, [vp, vp, vp, vp, vp, i32, i32, vp]),
    "et_attention_plan_ints": (C.c_size_t, [i32, i32]),
    "et_attention_plan": (i32, [vp, i32, i32, vp, vp]),
    "et_attention_tiles": (i32, [vp, vp, vp, i64, i64, vp, vp, i32, i32, i32, i32, i32, vp, vp]),
    "et_attention_tiles_general_mask": (i32, [vp, vp, vp, i64, i64, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp]),
    "et_gemm": (i32, [i32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp]),
    "et_pack_weight": (i32, [i32, vp, vp, i32, i32, vp]),
    "et_split_tf32": (i32, [vp, vp, vp, vp, i32, i32, vp]),
    "et_gemm_fp32_tensor": (i32, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, vp]),
}

_lib: Optional[C.CDLL] = None


def load() -> C.CDLL:
    """Loads libet_b200.so and attaches the prototypes.  Raises if the library
    has not been built: the product has no other execution path."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "libet_b200.so is missing: build it with `python -m effective_transformer_b200.build` "
            "(there is no CPU or PyTorch fallback for this path)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class EtError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(code, code)}: {message}")
        self.code = code


def check(code: int, handle=None) -> None:
    if code != ET_OK:
        msg = load().et_last_error(handle)
        raise EtError(code, msg.decode() if msg else "")
