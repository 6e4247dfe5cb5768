"""The model-file reader (include/cglm_model_file.h) against files written by a Python twin of the reference's
converter (tests/model_file_writer.py): config records of both versions and both families, tokenizer blob, tensor
table (names in file order, shapes, dtypes, 16-byte aligned data, contents), attention descriptor, broken files."""
import ctypes as C
import struct

import numpy as np
import pytest

import model_file_writer as W


def _open(blob: bytes):
    from chatglm_cpp_b200 import _lib
    L = _lib.lib()
    buf = C.create_string_buffer(blob, len(blob))
    h = C.c_void_p()
    rc = L.cglm_model_file_open_memory(buf, len(blob), C.byref(h))
    return rc, h, buf


def _tensors(h):
    from chatglm_cpp_b200 import _lib
    L = _lib.lib()
    out = []
    for i in range(L.cglm_model_file_n_tensors(h)):
        info = _lib.TensorInfo()
        assert L.cglm_model_file_tensor(h, i, C.byref(info)) == 0
        out.append((info.name.decode(), info.ndim, tuple(info.ne), info.dtype, info.offset, info.nbytes,
                    C.string_at(info.data, info.nbytes)))
    return out


@pytest.mark.parametrize("cfg,version,ggml_type", [
    (W.GLM2_SMALL, 2, W.F16), (W.GLM2_SMALL, 1, W.Q8_0), (W.GLM1_SMALL, 1, W.F32), (W.GLM1_SMALL, 2, W.Q4_0),
    (dict(W.GLM2_SMALL, model_type=W.CHATGLM4, rope_theta=5.0e6), 2, W.F16), (W.GLM3_PTUNING, 2, W.F16),
])
def test_reader_returns_what_the_writer_wrote(cfg, version, ggml_type):
    from chatglm_cpp_b200 import _lib
    L = _lib.lib()
    blob, written = W.write_model(cfg, ggml_type, version, seed=7, tokenizer_blob=b"\x01\x02tok\x00en")
    rc, h, keep = _open(blob)
    assert rc == 0, L.cglm_last_error_string()
    mc = _lib.ModelConfig()
    assert L.cglm_model_file_config(h, C.byref(mc)) == 0
    v1 = cfg["model_type"] == W.CHATGLM
    assert (mc.model_type, mc.version, mc.dtype) == (cfg["model_type"], version, ggml_type)
    for key in ("vocab_size", "hidden_size", "num_attention_heads", "num_hidden_layers", "intermediate_size", "max_length",
                "eos_token_id", "pad_token_id"):
        assert getattr(mc, key) == cfg[key], key
    assert mc.num_key_value_heads == cfg["num_key_value_heads"]
    if version == 1:   # records without these fields get the constructor's defaults (chatglm.cpp:1777,1801)
        assert (mc.bos_token_id, mc.sep_token_id) == (cfg["bos_token_id"], cfg["sep_token_id"])
        assert mc.norm_eps == np.float32(1e-5) and mc.rope_theta == 10000.0 and mc.num_virtual_tokens == 0
    else:
        assert (mc.bos_token_id, mc.sep_token_id) == (-1, -1)
        assert mc.rope_theta == np.float32(cfg["rope_theta"]) and mc.num_virtual_tokens == cfg["num_virtual_tokens"]
    # derived members of ModelConfig (chatglm.h:121-137)
    assert (mc.hidden_act, mc.use_qkv_bias, mc.use_dense_bias, mc.interleaved_qkv, mc.tie_word_embeddings) == \
        ((0, 1, 1, 1, 1) if v1 else (1, 1, 0, 0, 0))
    assert mc.rope_type == (_lib.ROPE_CHATGLM if v1 else _lib.ROPE_CHATGLM2)
    assert mc.attn_mask_type == (_lib.MASK_CHATGLM if v1 else _lib.MASK_CAUSAL)
    data, size = C.c_void_p(), C.c_size_t()
    assert L.cglm_model_file_tokenizer(h, C.byref(data), C.byref(size)) == 0
    assert C.string_at(data, size.value) == b"\x01\x02tok\x00en"
    # tensor table
    got = _tensors(h)
    virt = cfg["num_virtual_tokens"] if version == 2 else 0
    names = W.weight_names(cfg["model_type"], cfg["num_hidden_layers"], cfg["num_virtual_tokens"] > 0)
    assert [g[0] for g in got] == names
    for name, ndim, ne, dtype, offset, nbytes, payload in got:
        x, t, off = written[name]
        assert ndim == x.ndim and tuple(reversed(ne[:ndim])) == x.shape and all(e == 1 for e in ne[ndim:])
        assert dtype == t and offset == off and offset % 16 == 0
        if t == W.F32:
            want = x.astype(np.float32).tobytes()
        elif t == W.F16:
            want = x.astype(np.float16).tobytes()
        elif t == W.Q8_0:
            want = W.quantize_q8_0(x).tobytes()
        else:
            want = W.quantize_q4_0(x).tobytes()
        assert nbytes == len(want) and payload == want, name
    info = _lib.TensorInfo()
    qkv_name = C.create_string_buffer(128)
    assert L.cglm_model_file_attn_weight_name(h, 1, 0, qkv_name, 128) == 0
    assert L.cglm_model_file_find(h, qkv_name.value, C.byref(info)) == 0
    hd = cfg["head_dim"]
    assert tuple(info.ne[:2]) == (cfg["hidden_size"], cfg["hidden_size"] + 2 * cfg["num_key_value_heads"] * hd)
    assert L.cglm_model_file_attn_weight_name(h, 0, 3, qkv_name, 128) == (0 if v1 else _lib.ERR_INVALID_ARG)
    assert L.cglm_model_file_find(h, b"no.such.tensor", C.byref(info)) == _lib.ERR_INVALID_ARG
    # attention descriptor
    d = _lib.AttnDesc()
    assert L.cglm_model_file_attn_desc(h, 0, C.byref(d)) == 0
    assert (d.n_head, d.n_kv_head, d.head_dim, d.n_virtual) == (cfg["num_attention_heads"], cfg["num_key_value_heads"], hd, virt)
    assert d.max_len == cfg["max_length"] + virt and d.rope_type == mc.rope_type and d.mask_type == mc.attn_mask_type
    assert d.rope_theta == mc.rope_theta
    half = cfg["max_length"] // 2
    assert L.cglm_model_file_attn_desc(h, half, C.byref(d)) == 0 and d.max_len == half + virt
    assert L.cglm_model_file_attn_desc(h, cfg["max_length"] + 1, C.byref(d)) == _lib.ERR_INVALID_ARG   # chatglm.cpp:1755-1762
    assert L.cglm_model_file_close(h) == 0


def test_open_from_a_path(tmp_path):
    from chatglm_cpp_b200 import _lib
    L = _lib.lib()
    blob, written = W.write_model(W.GLM2_SMALL, W.F16, 2, seed=3)
    p = tmp_path / "model.bin"
    p.write_bytes(blob)
    h = C.c_void_p()
    assert L.cglm_model_file_open(str(p).encode(), C.byref(h)) == 0
    assert L.cglm_model_file_n_tensors(h) == len(written)
    assert L.cglm_model_file_close(h) == 0
    assert L.cglm_model_file_open(str(tmp_path / "missing.bin").encode(), C.byref(h)) == _lib.ERR_INVALID_ARG
    assert b"cannot open" in L.cglm_last_error_string()


def test_broken_files_are_refused_with_a_status():
    """Bad magic, unknown type or version, and every truncation point: a status code, never a crash or an over-read."""
    from chatglm_cpp_b200 import _lib
    L = _lib.lib()
    blob, _ = W.write_model(W.GLM1_SMALL, W.F16, 2, seed=1)
    rc, h, keep = _open(b"gguf" + blob[4:])
    assert rc == _lib.ERR_INVALID_ARG and b"bad magic" in L.cglm_last_error_string()
    rc, h, keep = _open(blob[:4] + struct.pack("i", 9) + blob[8:])
    assert rc == _lib.ERR_INVALID_ARG and b"invalid model type" in L.cglm_last_error_string()
    rc, h, keep = _open(blob[:8] + struct.pack("i", 3) + blob[12:])
    assert rc == _lib.ERR_INVALID_ARG and b"version" in L.cglm_last_error_string()
    glm4_v1 = blob[:4] + struct.pack("ii", W.CHATGLM4, 1) + blob[12:]
    assert _open(glm4_v1)[0] == _lib.ERR_INVALID_ARG
    rng = np.random.default_rng(0)
    cuts = sorted(set(int(c) for c in rng.integers(0, len(blob) - 1, 60)) | {0, 3, 4, 11, 12, 63, 64, 65, len(blob) - 1})
    for cut in cuts:
        rc, h, keep = _open(blob[:cut])
        assert rc == _lib.ERR_INVALID_ARG, cut
    # a tensor whose declared shape leaves the file
    head_len = blob.index(b"transformer.word_embeddings.weight") + len(b"transformer.word_embeddings.weight")
    huge = blob[:head_len] + struct.pack("iiii", 2, 2 ** 30, 2 ** 30, W.F16) + blob[head_len + 16:]
    rc, h, keep = _open(huge)
    assert rc == _lib.ERR_INVALID_ARG and b"exceeds the file" in L.cglm_last_error_string()
    bad_type = blob[:head_len] + struct.pack("iiii", 2, 64, 128, 99) + blob[head_len + 16:]
    rc, h, keep = _open(bad_type)
    assert rc == _lib.ERR_INVALID_ARG and b"unsupported ggml type" in L.cglm_last_error_string()


def test_cpp_reader_under_address_and_ub_sanitizers(tmp_path):
    """The C++ reader (chatglm::ModelFile, compiled into the test program with -fsanitize=address,undefined) over a
    good file, over every kind of broken file and over truncations: it parses or refuses, and never trips a sanitizer."""
    import subprocess

    from cpp.build_cpp import build_cpp_test
    exe = build_cpp_test("test_model_file", sanitize=True, extra_sources=["chatglm_cpp_b200/csrc/model_file.cu"])
    blob, written = W.write_model(W.GLM3_PTUNING, W.Q8_0, 2, seed=5)
    env = dict(**__import__("os").environ, ASAN_OPTIONS="detect_leaks=0:protect_shadow_gap=0")

    def run(data: bytes, *args):
        p = tmp_path / "m.bin"
        p.write_bytes(data)
        return subprocess.run([exe, str(p), *args], capture_output=True, text=True, env=env, timeout=120)

    r = run(blob)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "model_type=3 version=2 layers=2 heads=4 kv_heads=2 head_dim=128 max_len=64 virtual=8 rope=8 mask=0" in r.stdout
    assert f"tensors={len(written)} qkv0=transformer.encoder.layers.0.self_attention.query_key_value.weight" in r.stdout
    r = run(blob, "57")
    assert r.returncode == 3 and "exceeds the max possible model sequence length" in r.stdout
    rng = np.random.default_rng(2)
    for cut in [0, 5, 12, 60, 70] + [int(c) for c in rng.integers(64, len(blob) - 1, 12)]:
        r = run(blob[:cut])
        assert r.returncode == 3, (cut, r.stdout, r.stderr[-2000:])
    flipped = bytearray(blob)
    name_at = blob.index(b"past_key_values")
    flipped[name_at - 4:name_at] = struct.pack("i", -7)      # negative name length
    r = run(bytes(flipped))
    assert r.returncode == 3 and "invalid tensor name length" in r.stdout


@pytest.mark.gpu
def test_prefix_cache_from_a_model_file_lands_in_the_arena():
    """P-Tuning v2: the converter stores the prefix as f16 [2 * layers][kv_heads][virtual][head_dim]
    (chatglm_cpp/convert.py:212-222); load_prefix puts layer l's block into cache positions [0, virtual) of a slot,
    V transposed (chatglm.h:580-615).  Checked against the oracle's load_prefix_cache, then one decode step on top."""
    import torch

    from chatglm_cpp_b200 import _lib
    from chatglm_cpp_b200 import attention as A
    from gpu_util import download_cache, oracle_cfg, run_decode_batch  # noqa: F401
    from oracle import attn_oracle as O
    L = _lib.lib()
    cfg = W.GLM3_PTUNING
    blob, written = W.write_model(cfg, W.F16, 2, seed=11)
    rc, h, keep = _open(blob)
    assert rc == 0
    desc = _lib.AttnDesc()
    assert L.cglm_model_file_attn_desc(h, 0, C.byref(desc)) == 0
    n_layers = cfg["num_hidden_layers"]
    arena = A.KVArena(desc, n_layers)
    block = 2 * desc.n_kv_head * desc.n_virtual * desc.head_dim
    staging = torch.empty(block, dtype=torch.float16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    past = written["past_key_values"][0].astype(np.float16)            # [2L, G, V, D]
    ocfg = oracle_cfg(desc)
    for layer in range(n_layers):
        assert L.cglm_model_file_load_prefix(h, arena._h, layer, layer, staging.data_ptr(), stream) == 0
        torch.cuda.synchronize()                                        # the staging buffer is reused by the next layer
        kc, vc = O.new_caches(ocfg)
        O.load_prefix_cache(ocfg, past[2 * layer:2 * layer + 2], kc, vc)
        gk, gv = download_cache(arena, layer)
        np.testing.assert_array_equal(gk, kc)
        np.testing.assert_array_equal(gv, vc)
    assert L.cglm_model_file_load_prefix(h, arena._h, n_layers, 0, staging.data_ptr(), stream) == _lib.ERR_INVALID_ARG
    other = A.KVArena(_lib.AttnDesc(4, 2, 128, 64, 4, _lib.ROPE_CHATGLM2, 10000.0, _lib.MASK_CAUSAL), 1)
    assert L.cglm_model_file_load_prefix(h, other._h, 0, 0, staging.data_ptr(), stream) == _lib.ERR_INVALID_ARG
    L.cglm_model_file_close(h)


@pytest.mark.gpu
def test_attention_weights_from_a_model_file_drive_the_linears():
    """cglm_model_file_load_attn_weight: the four parameters of a layer's attention module go from the mapping to device
    memory with the bits the file holds (f16 weights, f32 biases), and the query_key_value Linear run on them matches
    the oracle's Linear on the same bits.  Absent tensors, wrong sizes and f32 checkpoints are refused."""
    import torch

    from chatglm_cpp_b200 import _lib
    from chatglm_cpp_b200 import attention as A
    from oracle import attn_oracle as O
    L = _lib.lib()
    cfg = W.GLM3_PTUNING
    blob, written = W.write_model(cfg, W.F16, 2, seed=12)
    rc, h, keep = _open(blob)
    assert rc == 0
    stream = torch.cuda.current_stream().cuda_stream
    hidden = cfg["hidden_size"]
    loaded = {}
    for layer in range(cfg["num_hidden_layers"]):
        for which in range(4):
            buf = C.create_string_buffer(256)
            named = L.cglm_model_file_attn_weight_name(h, layer, which, buf, 256) == 0   # GLM-2/3/4 have no dense bias
            name = buf.value.decode() if named else ""
            probe = torch.empty(16, dtype=torch.uint8, device="cuda")
            if name not in written:
                assert L.cglm_model_file_load_attn_weight(h, layer, which, probe.data_ptr(), 16, stream) == _lib.ERR_INVALID_ARG
                continue
            x, t, _ = written[name]
            want = x.astype(np.float16 if t == W.F16 else np.float32)
            dst = torch.empty(want.shape, dtype=torch.float16 if t == W.F16 else torch.float32, device="cuda")
            assert L.cglm_model_file_load_attn_weight(h, layer, which, dst.data_ptr(), want.nbytes - 4, stream) == _lib.ERR_INVALID_ARG
            assert L.cglm_model_file_load_attn_weight(h, layer, which, dst.data_ptr(), want.nbytes, stream) == 0, L.cglm_last_error_string()
            torch.cuda.synchronize()
            np.testing.assert_array_equal(dst.cpu().numpy().view(np.uint8), want.view(np.uint8))
            loaded[(layer, which)] = (dst, want)
    assert (0, 0) in loaded and (1, 2) in loaded
    assert L.cglm_model_file_load_attn_weight(h, cfg["num_hidden_layers"], 0, loaded[(0, 0)][0].data_ptr(), 16, stream) == _lib.ERR_INVALID_ARG
    # the Linear on the loaded parameters
    w_d, w = loaded[(1, 0)]
    bias = loaded.get((1, 1))
    rng = np.random.default_rng(5)
    xs = rng.standard_normal((3, hidden)).astype(np.float16)
    out = torch.empty(3, w.shape[0], device="cuda")
    desc = _lib.AttnDesc()
    assert L.cglm_model_file_attn_desc(h, 0, C.byref(desc)) == 0
    ws = A.Workspace(desc, 1, 1)
    rc = L.cglm_linear_forward(torch.from_numpy(xs).cuda().data_ptr(), 3, hidden, w_d.data_ptr(), w.shape[0],
                               bias[0].data_ptr() if bias else None, out.data_ptr(), 0, ws.ptr, ws.bytes, stream)
    assert rc == 0, L.cglm_last_error_string()
    torch.cuda.synchronize()
    want = O.linear(xs.astype(np.float32), w, bias[1] if bias else None)
    assert np.abs(out.cpu().numpy() - want).max() <= 2e-4 * max(1.0, float(np.abs(want).max()))
    L.cglm_model_file_close(h)
    # an f32 checkpoint: weights are refused, not converted behind the caller's back
    blob32, _ = W.write_model(cfg, W.F32, 2, seed=12)
    rc, h32, keep32 = _open(blob32)
    assert rc == 0
    assert L.cglm_model_file_load_attn_weight(h32, 0, 0, w_d.data_ptr(), w.nbytes * 2, stream) == _lib.ERR_UNSUPPORTED
    L.cglm_model_file_close(h32)


def test_attention_weight_loader_refuses_before_it_copies():
    """cglm_model_file_load_attn_weight validates against the file on the host: layer and selector ranges, tensors the
    model family does not have, sizes, and matrix types the Linear kernels do not take (no device is touched)."""
    from chatglm_cpp_b200 import _lib
    L = _lib.lib()
    cfg = W.GLM3_PTUNING
    dst = 0x1000   # never written: every call below is refused
    blob, written = W.write_model(cfg, W.F16, 2, seed=3)
    rc, h, keep = _open(blob)
    assert rc == 0
    n_w = written["transformer.encoder.layers.0.self_attention.query_key_value.weight"][0].size * 2
    assert L.cglm_model_file_load_attn_weight(h, -1, 0, dst, n_w, None) == _lib.ERR_INVALID_ARG
    assert L.cglm_model_file_load_attn_weight(h, cfg["num_hidden_layers"], 0, dst, n_w, None) == _lib.ERR_INVALID_ARG
    assert L.cglm_model_file_load_attn_weight(h, 0, 4, dst, n_w, None) == _lib.ERR_INVALID_ARG
    assert L.cglm_model_file_load_attn_weight(h, 0, 3, dst, 4 * cfg["hidden_size"], None) == _lib.ERR_INVALID_ARG   # no dense bias in GLM-3
    assert L.cglm_model_file_load_attn_weight(h, 0, 0, dst, n_w - 2, None) == _lib.ERR_INVALID_ARG                  # wrong size
    assert L.cglm_model_file_load_attn_weight(h, 0, 0, None, n_w, None) == _lib.ERR_INVALID_ARG
    L.cglm_model_file_close(h)
    for t in (W.F32, W.Q8_0, W.Q4_0):
        blob, _ = W.write_model(cfg, t, 2, seed=3)
        rc, h, keep = _open(blob)
        assert rc == 0
        assert L.cglm_model_file_load_attn_weight(h, 0, 0, dst, n_w, None) == _lib.ERR_UNSUPPORTED
        assert b"f16" in L.cglm_last_error_string()
        L.cglm_model_file_close(h)
