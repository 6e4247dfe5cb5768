"""Writer of synthetic model files in the container format of li-plus/chatglm.cpp, for the reader's tests.

Follows the converter byte for byte where the reader cares (chatglm_cpp/convert.py:133-209 dump_tensor /
dump_state_dict, :199-209 BaseConverter.convert, :225-258 and :299-333 dump_config, :212-222 prefix cache layout)
with random weights of a small shape instead of a Hugging Face checkpoint, and a dummy tokenizer blob.
"""
from __future__ import annotations

import io
import struct

import numpy as np

GGML_MEM_ALIGN = 16
F32, F16, Q4_0, Q8_0 = 0, 1, 2, 8
CHATGLM, CHATGLM2, CHATGLM3, CHATGLM4 = 1, 2, 3, 4


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """Blocks of 32: f16 scale + 32 int8 (the layout only; the reader never dequantises)."""
    b = x.reshape(-1, 32).astype(np.float32)
    scale = np.abs(b).max(axis=1, keepdims=True) / 127.0
    scale[scale == 0] = 1.0
    q = np.clip(np.round(b / scale), -128, 127).astype(np.int8)
    return np.concatenate([scale.astype(np.float16).view(np.int8), q], axis=1)


def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    """Blocks of 32: f16 scale + 16 bytes of nibbles."""
    b = x.reshape(-1, 32).astype(np.float32)
    idx = np.abs(b).argmax(axis=1)
    scale = b[np.arange(b.shape[0]), idx][:, None] / -8.0
    scale[scale == 0] = 1.0
    q = np.clip(np.round(b / scale + 8), 0, 15).astype(np.uint8)
    packed = (q[:, :16] | (q[:, 16:] << 4)).view(np.int8)
    return np.concatenate([scale.astype(np.float16).view(np.int8), packed], axis=1)


def dump_tensor(f, name: str, tensor: np.ndarray, ggml_type: int) -> int:
    """Returns the file offset of the tensor's data."""
    f.write(struct.pack("i", len(name.encode())))
    f.write(name.encode())
    f.write(struct.pack("i" * (2 + tensor.ndim), tensor.ndim, *tensor.shape, ggml_type))
    if ggml_type == F32:
        payload = tensor.astype(np.float32)
    elif ggml_type == F16:
        payload = tensor.astype(np.float16)
    elif ggml_type == Q8_0:
        payload = quantize_q8_0(tensor)
    elif ggml_type == Q4_0:
        payload = quantize_q4_0(tensor)
    else:
        raise NotImplementedError(ggml_type)
    aligned = (f.tell() + GGML_MEM_ALIGN - 1) // GGML_MEM_ALIGN * GGML_MEM_ALIGN
    f.write(b"\0" * (aligned - f.tell()))
    f.write(payload.tobytes())
    return aligned


def weight_names(model_type: int, n_layers: int, prefix: bool):
    if model_type == CHATGLM:
        names = ["transformer.word_embeddings.weight"]
        for i in range(n_layers):
            p = f"transformer.layers.{i}."
            names += [p + "input_layernorm.weight", p + "input_layernorm.bias", p + "attention.query_key_value.weight",
                      p + "attention.query_key_value.bias", p + "attention.dense.weight", p + "attention.dense.bias",
                      p + "post_attention_layernorm.weight", p + "post_attention_layernorm.bias",
                      p + "mlp.dense_h_to_4h.weight", p + "mlp.dense_h_to_4h.bias", p + "mlp.dense_4h_to_h.weight",
                      p + "mlp.dense_4h_to_h.bias"]
        return names + ["transformer.final_layernorm.weight", "transformer.final_layernorm.bias"]
    names = ["past_key_values"] if prefix else []
    names.append("transformer.embedding.word_embeddings.weight")
    for i in range(n_layers):
        p = f"transformer.encoder.layers.{i}."
        names += [p + "input_layernorm.weight", p + "self_attention.query_key_value.weight",
                  p + "self_attention.query_key_value.bias", p + "self_attention.dense.weight",
                  p + "post_attention_layernorm.weight", p + "mlp.dense_h_to_4h.weight", p + "mlp.dense_4h_to_h.weight"]
    return names + ["transformer.encoder.final_layernorm.weight", "transformer.output_layer.weight"]


def shape_of(name: str, cfg: dict):
    h, kvh, hd, inter, vocab = cfg["hidden_size"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"]
    qkv = h + 2 * kvh * hd
    if name == "past_key_values":
        return (2 * cfg["num_hidden_layers"], kvh, cfg["num_virtual_tokens"], hd)
    if name.endswith("word_embeddings.weight") or name.endswith("output_layer.weight"):
        return (vocab, h)
    if name.endswith("query_key_value.weight"):
        return (qkv, h)
    if name.endswith("query_key_value.bias"):
        return (qkv,)
    if name.endswith("dense.weight"):
        return (h, h)
    if name.endswith("dense_h_to_4h.weight"):
        return ((inter if cfg["model_type"] == CHATGLM else 2 * inter), h)
    if name.endswith("dense_h_to_4h.bias"):
        return (inter,)
    if name.endswith("dense_4h_to_h.weight"):
        return (h, inter)
    return (h,)   # norms and the remaining biases


def write_model(cfg: dict, ggml_type: int = F16, version: int = 2, seed: int = 0, tokenizer_blob: bytes = b"\x0atokenizer-blob"):
    """Returns (file bytes, {name: (array as written before quantisation, ggml type, data offset)})."""
    rng = np.random.default_rng(seed)
    f = io.BytesIO()
    f.write(b"ggml")
    f.write(struct.pack("i", cfg["model_type"]))
    if version == 2:
        f.write(struct.pack("iiiiiiiififiii", 2, ggml_type, cfg["vocab_size"], cfg["hidden_size"], cfg["num_attention_heads"],
                            cfg["num_key_value_heads"], cfg["num_hidden_layers"], cfg["intermediate_size"], cfg["norm_eps"],
                            cfg["num_virtual_tokens"], cfg["rope_theta"], cfg["max_length"], cfg["eos_token_id"],
                            cfg["pad_token_id"]))
    else:   # the older records (chatglm.h:51-71): ConfigRecordV1, plus num_key_value_heads for ChatGLM2/3
        vals = [ggml_type, cfg["vocab_size"], cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_hidden_layers"],
                cfg["intermediate_size"], cfg["max_length"], cfg["bos_token_id"], cfg["eos_token_id"], cfg["pad_token_id"],
                cfg["sep_token_id"]]
        if cfg["model_type"] != CHATGLM:
            vals.append(cfg["num_key_value_heads"])
        f.write(struct.pack("i" * (1 + len(vals)), 1, *vals))
    f.write(struct.pack("i", len(tokenizer_blob)))
    f.write(tokenizer_blob)
    written = {}
    for name in weight_names(cfg["model_type"], cfg["num_hidden_layers"], cfg["num_virtual_tokens"] > 0):
        shape = shape_of(name, cfg)
        x = rng.standard_normal(shape).astype(np.float32)
        if name == "past_key_values":
            t = F16
        elif len(shape) == 2:
            t = ggml_type
        else:
            t = F32
        off = dump_tensor(f, name, x, t)
        written[name] = (x, t, off)
    return f.getvalue(), written


GLM2_SMALL = dict(model_type=CHATGLM2, vocab_size=96, hidden_size=256, num_attention_heads=8, num_key_value_heads=2,
                  head_dim=32, num_hidden_layers=3, intermediate_size=64, norm_eps=1e-5, num_virtual_tokens=0,
                  rope_theta=10000.0, max_length=512, bos_token_id=-1, eos_token_id=2, pad_token_id=0, sep_token_id=-1)
GLM1_SMALL = dict(model_type=CHATGLM, vocab_size=64, hidden_size=128, num_attention_heads=4, num_key_value_heads=4,
                  head_dim=32, num_hidden_layers=2, intermediate_size=512, norm_eps=1e-5, num_virtual_tokens=0,
                  rope_theta=10000.0, max_length=128, bos_token_id=5, eos_token_id=6, pad_token_id=3, sep_token_id=7)
# a fused-decode shape with a P-Tuning v2 prefix: head_dim 128, capacity 56 + 8 = 64
GLM3_PTUNING = dict(model_type=CHATGLM3, vocab_size=32, hidden_size=512, num_attention_heads=4, num_key_value_heads=2,
                    head_dim=128, num_hidden_layers=2, intermediate_size=32, norm_eps=1e-5, num_virtual_tokens=8,
                    rope_theta=10000.0, max_length=56, bos_token_id=-1, eos_token_id=2, pad_token_id=0, sep_token_id=-1)
