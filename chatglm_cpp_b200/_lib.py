"""ctypes binding of libcglm_attn.so, the C ABI declared in include/cglm_attn.h.

There is no fallback: if the CUDA library has not been built, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libcglm_attn.so")

OK, ERR_INVALID_ARG, ERR_CUDA, ERR_WORKSPACE, ERR_UNSUPPORTED, ERR_TIMEOUT, ERR_NO_DEVICE = 0, -1, -2, -3, -4, -5, -6
ROPE_GPTJ, ROPE_NEOX, ROPE_CHATGLM, ROPE_CHATGLM2, ROPE_DISABLED = 0, 2, 4, 8, 10000
MASK_CAUSAL, MASK_CHATGLM = 0, 1
SEQ_NO_APPEND, SEQ_PARTIAL, SEQ_USE_KV_LOCAL, SEQ_N_PAST_DEVICE, SEQ_CACHE_SETTLED = 1, 2, 4, 8, 16
SEQ_QKV_F16, SEQ_OUT_F16, SEQ_Q_ROPED = 32, 64, 128
HOST_INTERLEAVED_QKV, HOST_F16 = 1, 2


class AttnDesc(C.Structure):
    _fields_ = [("n_head", C.c_int), ("n_kv_head", C.c_int), ("head_dim", C.c_int), ("max_len", C.c_int),
                ("n_virtual", C.c_int), ("rope_type", C.c_int), ("rope_theta", C.c_float), ("mask_type", C.c_int)]


class AttnSeq(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
                ("q_tok_stride", C.c_longlong), ("q_head_stride", C.c_longlong),
                ("kv_tok_stride", C.c_longlong), ("kv_head_stride", C.c_longlong),
                ("slot", C.c_int), ("qlen", C.c_int), ("n_past", C.c_int), ("n_ctx", C.c_int),
                ("position_ids", C.c_void_p), ("out", C.c_void_p), ("q_roped", C.c_void_p),
                ("k_roped", C.c_void_p), ("kv_local", C.c_int), ("flags", C.c_int), ("partial", C.c_void_p),
                ("n_past_dev", C.c_void_p)]


class ModelConfig(C.Structure):
    """cglm_model_config of include/cglm_model_file.h."""
    _fields_ = [("model_type", C.c_int), ("version", C.c_int), ("dtype", C.c_int), ("vocab_size", C.c_int),
                ("hidden_size", C.c_int), ("num_attention_heads", C.c_int), ("num_key_value_heads", C.c_int),
                ("num_hidden_layers", C.c_int), ("intermediate_size", C.c_int), ("norm_eps", C.c_float),
                ("num_virtual_tokens", C.c_int), ("rope_theta", C.c_float), ("max_length", C.c_int),
                ("bos_token_id", C.c_int), ("eos_token_id", C.c_int), ("pad_token_id", C.c_int), ("sep_token_id", C.c_int),
                ("hidden_act", C.c_int), ("use_qkv_bias", C.c_int), ("use_dense_bias", C.c_int),
                ("interleaved_qkv", C.c_int), ("tie_word_embeddings", C.c_int), ("rope_type", C.c_int),
                ("attn_mask_type", C.c_int)]


class TensorInfo(C.Structure):
    """cglm_tensor_info of include/cglm_model_file.h."""
    _fields_ = [("name", C.c_char_p), ("ndim", C.c_int), ("ne", C.c_longlong * 4), ("dtype", C.c_int),
                ("data", C.c_void_p), ("nbytes", C.c_size_t), ("offset", C.c_size_t)]


# every symbol include/cglm_attn.h and include/cglm_model_file.h declare: name -> (restype, argtypes)
SYMBOLS = {
    "cglm_kv_arena_create": (C.c_int, [C.POINTER(AttnDesc), C.c_int, C.POINTER(C.c_void_p)]),
    "cglm_kv_arena_adopt": (C.c_int, [C.POINTER(AttnDesc), C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)]),
    "cglm_kv_angle_table_bytes": (C.c_size_t, [C.POINTER(AttnDesc)]),
    "cglm_kv_arena_destroy": (C.c_int, [C.c_void_p]),
    "cglm_kv_arena_k_cache": (C.c_void_p, [C.c_void_p, C.c_int]),
    "cglm_kv_arena_v_cache": (C.c_void_p, [C.c_void_p, C.c_int]),
    "cglm_kv_arena_n_slots": (C.c_int, [C.c_void_p]),
    "cglm_kv_arena_pitch": (C.c_int, [C.c_void_p]),
    "cglm_kv_arena_desc": (C.POINTER(AttnDesc), [C.c_void_p]),
    "cglm_kv_slot_bytes": (C.c_size_t, [C.POINTER(AttnDesc)]),
    "cglm_kv_slot_copy": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "cglm_attn_workspace_bytes": (C.c_size_t, [C.POINTER(AttnDesc), C.c_int, C.c_int]),
    "cglm_attn_workspace_init": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p]),
    "cglm_attn_workspace_status": (C.c_int, [C.c_void_p, C.c_void_p]),
    "cglm_attn_forward": (C.c_int, [C.c_void_p, C.POINTER(AttnSeq), C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]),
    "cglm_qkv_linear_forward": (C.c_int, [C.c_void_p, C.POINTER(AttnSeq), C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
                                          C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "cglm_linear_forward": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                                      C.c_void_p, C.c_size_t, C.c_void_p]),
    "cglm_linear_workspace_bytes": (C.c_size_t, []),
    "cglm_linear_kernel_plan": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int)]),
    "cglm_convert_f32_to_f16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "cglm_seq_advance": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "cglm_attn_forward_host": (C.c_int, [C.c_void_p, C.POINTER(AttnSeq), C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                         C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "cglm_attn_host_drain": (C.c_int, [C.c_void_p, C.c_void_p]),
    "cglm_attn_decode_static": (C.c_int, [C.c_void_p, C.POINTER(AttnSeq), C.c_int, C.c_int, C.c_void_p]),
    "cglm_attn_splitkv_combine": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "cglm_attn_splitkv_xchg_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "cglm_xchg_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "cglm_xchg_free": (C.c_int, [C.c_void_p]),
    "cglm_xchg_read": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "cglm_xchg_export": (C.c_int, [C.c_void_p, C.c_char_p]),
    "cglm_xchg_import": (C.c_int, [C.c_char_p, C.c_int, C.POINTER(C.c_void_p)]),
    "cglm_attn_splitkv_step": (C.c_int, [C.c_void_p, C.POINTER(AttnSeq), C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_void_p,
                                         C.c_int, C.c_uint, C.c_void_p, C.c_size_t, C.c_void_p]),
    "cglm_kv_load_prefix": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "cglm_synth_fill_f16": (C.c_int, [C.c_void_p, C.c_longlong, C.c_ulonglong, C.c_ulonglong, C.c_longlong, C.c_void_p, C.c_void_p]),
    "cglm_synth_fill_f32": (C.c_int, [C.c_void_p, C.c_longlong, C.c_ulonglong, C.c_ulonglong, C.c_longlong, C.c_void_p, C.c_void_p]),
    "cglm_status_string": (C.c_char_p, [C.c_int]),
    "cglm_last_error_string": (C.c_char_p, []),
    "cglm_launch_count": (C.c_ulonglong, []),
    # include/cglm_model_file.h
    "cglm_model_file_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "cglm_model_file_open_memory": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "cglm_model_file_close": (C.c_int, [C.c_void_p]),
    "cglm_model_file_config": (C.c_int, [C.c_void_p, C.POINTER(ModelConfig)]),
    "cglm_model_file_tokenizer": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_size_t)]),
    "cglm_model_file_n_tensors": (C.c_int, [C.c_void_p]),
    "cglm_model_file_tensor": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(TensorInfo)]),
    "cglm_model_file_find": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(TensorInfo)]),
    "cglm_model_file_attn_desc": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(AttnDesc)]),
    "cglm_model_file_attn_weight_name": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_char_p, C.c_size_t]),
    "cglm_model_file_load_prefix": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "cglm_model_file_load_attn_weight": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]),
}

_lib = None


def lib():
    """The loaded library with argtypes set.  Raises if the CUDA library is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m chatglm_cpp_b200.build` "
                "(this package has no CPU or PyTorch fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


class CglmError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().cglm_status_string(status).decode()
        detail = lib().cglm_last_error_string().decode()
        super().__init__(f"{where}: {msg}" + (f" ({detail})" if detail and status == ERR_CUDA else ""))


def check(status: int, where: str) -> None:
    if status != OK:
        raise CglmError(status, where)
