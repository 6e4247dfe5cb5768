"""ctypes binding of the CPU oracle (``attn_oracle.c``) -- test infrastructure only.

The oracle restates BasicAttention::forward (chatglm.cpp:620-721) and its RoPE helpers
(chatglm.cpp:523-618) on the CPU.  Tests, the smoke check and the bench's CPU-baseline leg use it
as the checker; nothing in the shipped package imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle_attn.so")

ROPE_GPTJ, ROPE_NEOX, ROPE_CHATGLM, ROPE_CHATGLM2, ROPE_DISABLED = 0, 2, 4, 8, 10000
MASK_CAUSAL, MASK_CHATGLM = 0, 1


class Numerics(C.Structure):
    _fields_ = [("round_q_f16", C.c_int), ("round_p_f16", C.c_int), ("softmax_double", C.c_int),
                ("theta_powf", C.c_int)]


class Cfg(C.Structure):
    _fields_ = [("n_head", C.c_int), ("n_kv_head", C.c_int), ("head_dim", C.c_int), ("max_len", C.c_int),
                ("n_virtual", C.c_int), ("rope_type", C.c_int), ("rope_theta", C.c_float),
                ("mask_type", C.c_int), ("num", Numerics)]


def build(force: bool = False) -> str:
    """Compile the oracle with its Makefile if the shared library is missing or stale."""
    src = os.path.join(_HERE, "attn_oracle.c")
    hdr = os.path.join(_HERE, "attn_oracle.h")
    stale = (not os.path.exists(_LIB_PATH)
             or os.path.getmtime(_LIB_PATH) < max(os.path.getmtime(src), os.path.getmtime(hdr)))
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle_attn.so"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        fp, ip, u16p = C.POINTER(C.c_float), C.POINTER(C.c_int), C.POINTER(C.c_uint16)
        _lib.oracle_numerics_ggml.restype = Numerics
        _lib.oracle_numerics_f32.restype = Numerics
        _lib.oracle_f32_to_f16.restype = C.c_uint16
        _lib.oracle_f32_to_f16.argtypes = [C.c_float]
        _lib.oracle_f16_to_f32.restype = C.c_float
        _lib.oracle_f16_to_f32.argtypes = [C.c_uint16]
        _lib.oracle_position_ids_glm2.argtypes = [C.c_int, C.c_int, ip]
        _lib.oracle_position_ids_glm.argtypes = [C.c_int, C.c_int, C.c_int, ip]
        _lib.oracle_attention_mask_glm.argtypes = [C.c_int, C.c_int, fp]
        _lib.oracle_apply_rotary_emb.argtypes = [C.POINTER(Cfg), fp, C.c_long, C.c_long, C.c_int, C.c_int, ip]
        _lib.oracle_attn_forward.restype = C.c_int
        _lib.oracle_attn_forward.argtypes = [C.POINTER(Cfg), fp, C.c_long, C.c_long, fp, fp, C.c_long, C.c_long,
                                             u16p, u16p, ip, fp, C.c_int, C.c_int, fp, fp, fp]
        _lib.oracle_load_prefix_cache.argtypes = [C.POINTER(Cfg), u16p, u16p, u16p]
        _lib.oracle_attn_partial.restype = C.c_int
        _lib.oracle_attn_partial.argtypes = [C.POINTER(Cfg), fp, u16p, u16p, C.c_int, C.c_int, fp, fp, fp]
        _lib.oracle_attn_combine.argtypes = [C.c_int, C.c_int, C.c_int, fp, fp, fp, fp]
        _lib.oracle_attn_decode_batch.restype = C.c_int
        _lib.oracle_attn_decode_batch.argtypes = [C.POINTER(Cfg), C.c_int, C.POINTER(fp), C.POINTER(fp),
                                                  C.POINTER(fp), C.c_long, C.c_long, C.POINTER(u16p),
                                                  C.POINTER(u16p), ip, ip, C.POINTER(fp), C.c_int]
        _lib.oracle_linear.argtypes = [fp, C.c_int, C.c_int, C.c_void_p, C.c_int, fp, C.c_int, C.c_int, fp]
        _lib.oracle_synth_fill_f16.argtypes = [u16p, C.c_longlong, C.c_ulonglong, C.c_ulonglong, C.c_longlong, u16p]
        _lib.oracle_synth_fill_f32.argtypes = [fp, C.c_longlong, C.c_ulonglong, C.c_ulonglong, C.c_longlong, fp]
    return _lib


def linear(x: np.ndarray, weight: np.ndarray, bias: np.ndarray | None = None, round_x_f16: bool = False) -> np.ndarray:
    """Linear::forward (chatglm.cpp:418-426).  x [n_tok, in] f32; weight [out, in] f32 or f16; bias [out] or None."""
    x = np.ascontiguousarray(np.atleast_2d(x), np.float32)
    w_f16 = weight.dtype == np.float16
    weight = np.ascontiguousarray(weight)
    out_f, in_f = weight.shape
    assert x.shape[1] == in_f
    y = np.zeros((x.shape[0], out_f), np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    lib().oracle_linear(_fp(x), x.shape[0], in_f, weight.ctypes.data_as(C.c_void_p), int(w_f16),
                        _fp(b) if b is not None else None, out_f, int(round_x_f16), _fp(y))
    return y


def synth_table():
    """The 65536-point N(0,1) quantile table (f32, and the same values rounded to f16) the synthetic data draws from."""
    from scipy.special import ndtri
    t32 = ndtri((np.arange(65536, dtype=np.float64) + 0.5) / 65536.0).astype(np.float32)
    return t32, t32.astype(np.float16).view(np.uint16)


def synth_fill(n: int, seed: int, tensor_id: int, first: int, table: np.ndarray) -> np.ndarray:
    """Elements [first, first + n) of synthetic tensor `tensor_id`: the host twin of cglm_synth_fill_f16 / _f32."""
    table = np.ascontiguousarray(table)
    if table.dtype == np.uint16:
        out = np.empty(n, np.uint16)
        lib().oracle_synth_fill_f16(_u16p(out), n, seed, tensor_id, first, _u16p(table))
    else:
        out = np.empty(n, np.float32)
        lib().oracle_synth_fill_f32(_fp(out), n, seed, tensor_id, first, _fp(table))
    return out


def _fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float)) if a is not None else None


def _ip(a):
    return a.ctypes.data_as(C.POINTER(C.c_int)) if a is not None else None


def _u16p(a):
    return a.ctypes.data_as(C.POINTER(C.c_uint16))


def make_cfg(n_head, n_kv_head, head_dim, max_len, n_virtual=0, rope_type=ROPE_CHATGLM2, rope_theta=10000.0,
             mask_type=MASK_CAUSAL, numerics="ggml") -> Cfg:
    """``max_len`` is the cache capacity in tokens, i.e. max_length + n_virtual (chatglm.h:452-455)."""
    num = lib().oracle_numerics_ggml() if numerics == "ggml" else lib().oracle_numerics_f32()
    return Cfg(n_head, n_kv_head, head_dim, max_len, n_virtual, rope_type, rope_theta, mask_type, num)


def new_caches(cfg: Cfg):
    """Zeroed k_cache [G][M][D] and v_cache [G][D][M] as uint16 views of f16 storage."""
    k = np.zeros((cfg.n_kv_head, cfg.max_len, cfg.head_dim), np.uint16)
    v = np.zeros((cfg.n_kv_head, cfg.head_dim, cfg.max_len), np.uint16)
    return k, v


def position_ids(cfg: Cfg, qlen: int, n_past: int, n_ctx: int | None = None) -> np.ndarray:
    """Position ids as the model's set_graph_inputs makes them (chatglm.cpp:1142-1153, 1319-1327)."""
    if cfg.rope_type == ROPE_CHATGLM:
        ids = np.zeros(2 * qlen, np.int32)
        lib().oracle_position_ids_glm(qlen, n_past, n_ctx if n_ctx is not None else qlen, _ip(ids))
    else:
        ids = np.zeros(qlen, np.int32)
        lib().oracle_position_ids_glm2(qlen, n_past, _ip(ids))
    return ids


def attention_mask_glm(qlen: int, kvlen: int) -> np.ndarray:
    m = np.zeros((qlen, kvlen), np.float32)
    lib().oracle_attention_mask_glm(qlen, kvlen, _fp(m))
    return m


def apply_rotary_emb(cfg: Cfg, x: np.ndarray, ids: np.ndarray) -> np.ndarray:
    """x: [qlen, n_heads, D] f32 -> roped copy."""
    x = np.ascontiguousarray(x, np.float32).copy()
    qlen, nh, d = x.shape
    ids = np.ascontiguousarray(ids, np.int32)
    lib().oracle_apply_rotary_emb(C.byref(cfg), _fp(x), nh * d, d, nh, qlen, _ip(ids))
    return x


def split_qkv(cfg: Cfg, qkv: np.ndarray, interleaved: bool):
    """Views of a fused qkv activation [qlen, (H+2G)*D] (chatglm.cpp:636-653).

    Returns (q, k, v, q_tok_stride, q_head_stride, kv_tok_stride, kv_head_stride) with strides in elements.
    """
    H, G, D = cfg.n_head, cfg.n_kv_head, cfg.head_dim
    qkv = np.ascontiguousarray(qkv, np.float32)
    row = qkv.shape[1]
    flat = qkv.reshape(-1)
    if interleaved:
        assert H == G
        return flat[0:], flat[D:], flat[2 * D:], row, 3 * D, row, 3 * D
    return flat[0:], flat[H * D:], flat[(H + G) * D:], row, D, row, D


def attn_forward(cfg: Cfg, qkv: np.ndarray, interleaved: bool, k_cache: np.ndarray, v_cache: np.ndarray,
                 n_past: int, n_ctx: int | None = None, ids: np.ndarray | None = None, want_roped: bool = False):
    """Run the oracle on a fused qkv activation; caches are updated in place.

    Returns context_layer [qlen, H*D] (and the roped q [qlen,H,D] / k [qlen,G,D] when asked).
    """
    H, G, D = cfg.n_head, cfg.n_kv_head, cfg.head_dim
    qkv = np.ascontiguousarray(qkv, np.float32)
    qlen = qkv.shape[0]
    q, k, v, qts, qhs, kts, khs = split_qkv(cfg, qkv, interleaved)
    if ids is None:
        ids = position_ids(cfg, qlen, n_past, n_ctx)
    ids = np.ascontiguousarray(ids, np.int32)
    mask = None
    if n_past == 0 and cfg.mask_type == MASK_CHATGLM:
        mask = attention_mask_glm(qlen, cfg.n_virtual + qlen)
    out = np.zeros((qlen, H * D), np.float32)
    qr = np.zeros((qlen, H, D), np.float32) if want_roped else None
    kr = np.zeros((qlen, G, D), np.float32) if want_roped else None
    rc = lib().oracle_attn_forward(C.byref(cfg), _fp(q), qts, qhs, _fp(k), _fp(v), kts, khs, _u16p(k_cache),
                                   _u16p(v_cache), _ip(ids), _fp(mask), qlen, n_past, _fp(out), _fp(qr), _fp(kr))
    if rc != 0:
        raise ValueError("oracle_attn_forward: bad arguments")
    return (out, qr, kr) if want_roped else out


def load_prefix_cache(cfg: Cfg, past_kv: np.ndarray, k_cache: np.ndarray, v_cache: np.ndarray) -> None:
    """past_kv: f16 bits [2][G][V][D] for one layer (chatglm.h:580-615)."""
    past_kv = np.ascontiguousarray(past_kv.view(np.uint16))
    lib().oracle_load_prefix_cache(C.byref(cfg), _u16p(past_kv), _u16p(k_cache), _u16p(v_cache))


def attn_partial(cfg: Cfg, q_roped: np.ndarray, k_cache, v_cache, kv_begin: int, kv_end: int):
    H, D = cfg.n_head, cfg.head_dim
    q_roped = np.ascontiguousarray(q_roped, np.float32)
    acc = np.zeros((H, D), np.float32)
    m = np.zeros(H, np.float32)
    l = np.zeros(H, np.float32)
    rc = lib().oracle_attn_partial(C.byref(cfg), _fp(q_roped), _u16p(k_cache), _u16p(v_cache), kv_begin, kv_end,
                                   _fp(acc), _fp(m), _fp(l))
    if rc != 0:
        raise ValueError("oracle_attn_partial: bad range")
    return acc, m, l


def attn_combine(acc: np.ndarray, m: np.ndarray, l: np.ndarray) -> np.ndarray:
    n, H, D = acc.shape
    acc = np.ascontiguousarray(acc, np.float32)
    m = np.ascontiguousarray(m, np.float32)
    l = np.ascontiguousarray(l, np.float32)
    out = np.zeros((H, D), np.float32)
    lib().oracle_attn_combine(H, D, n, _fp(acc), _fp(m), _fp(l), _fp(out))
    return out


def attn_decode_batch(cfg: Cfg, q, k, v, q_head_stride, kv_head_stride, k_caches, v_caches, n_past, n_ctx=None,
                      n_threads: int = 0):
    """Batched one-token decode over independent sequences (lists of arrays), OpenMP-parallel."""
    n = len(q)
    H, D = cfg.n_head, cfg.head_dim
    fp, u16p = C.POINTER(C.c_float), C.POINTER(C.c_uint16)
    outs = [np.zeros(H * D, np.float32) for _ in range(n)]
    qa = (fp * n)(*[_fp(a) for a in q])
    ka = (fp * n)(*[_fp(a) for a in k])
    va = (fp * n)(*[_fp(a) for a in v])
    kc = (u16p * n)(*[_u16p(a) for a in k_caches])
    vc = (u16p * n)(*[_u16p(a) for a in v_caches])
    oa = (fp * n)(*[_fp(a) for a in outs])
    npast = np.ascontiguousarray(n_past, np.int32)
    nctx = np.ascontiguousarray(n_ctx, np.int32) if n_ctx is not None else None
    rc = lib().oracle_attn_decode_batch(C.byref(cfg), n, qa, ka, va, q_head_stride, kv_head_stride, kc, vc,
                                        _ip(npast), _ip(nctx), oa, n_threads)
    if rc != 0:
        raise ValueError("oracle_attn_decode_batch: bad arguments")
    return outs
