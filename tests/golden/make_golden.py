"""Generate the committed golden fixtures under tests/golden/ from the reference's own test data.

Run where the reference checkout is present:

    python tests/golden/make_golden.py [--reference /path/to/chatglm.cpp]

For each of the six 1-layer model fixtures that pin BasicAttention::forward
(tests/data/{glm,glm_ptuning_v2,glm2,glm3,glm3_ptuning_v2,glm4}_model.data, read as laid out by
chatglm_test.cpp:288-362 and written by tests/test_convert.py:318-323) it writes ``<name>.npz`` with
 - the model weights, the three inputs x1..x3 and the three golden outputs y1..y3 (HF PyTorch
   outputs, the reference's 5e-4 comparison targets),
 - the optional P-Tuning prefix cache,
 - the fused qkv activation of every step (what query_key_value.forward returns, chatglm.cpp:629),
 - an independent float64 numpy attention (not the C oracle) evaluated at the attention boundary:
   context_layer per step and the final f16 caches; it is accepted only if pushing it through the
   rest of the model reproduces y1..y3 within 5e-4.
It also writes ``rope_d128_hf.npz``: random head_dim-128 tensors pushed through the rotary
functions of ``transformers.models.glm`` (the HF-native GLM-4 model: interleaved pairs on the first
half of the head), which pins the pair pattern and the frequency ladder that the head_dim-4
fixtures cannot.
"""
import argparse
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import glm_tail  # noqa: E402

FIXTURES = {
    # name: (family, n_kv_head, ffn, n_virtual)   -- configs from chatglm_test.cpp:594-776
    "glm_model": ("glm1", 8, 128, 0),
    "glm_ptuning_v2_model": ("glm1", 8, 128, 5),
    "glm2_model": ("glm2", 2, 48, 0),
    "glm3_model": ("glm2", 2, 48, 0),
    "glm3_ptuning_v2_model": ("glm2", 2, 48, 5),
    "glm4_model": ("glm2", 2, 48, 0),
}
H, HID, VOCAB, MAX_LENGTH, SEQ_LEN = 8, 32, 5, 8, 3
D = HID // H


def _rd(f, n, dt=np.float32):
    return np.frombuffer(f.read(n * np.dtype(dt).itemsize), dtype=dt).copy()


def _rope_adjacent(x, pos, n_dims, theta):
    x = x.astype(np.float64).copy()
    for s in range(x.shape[0]):
        for i in range(n_dims // 2):
            a = pos[s] * theta ** (-2.0 * i / n_dims)
            c, sn = np.cos(a), np.sin(a)
            x0, x1 = x[s, :, 2 * i].copy(), x[s, :, 2 * i + 1].copy()
            x[s, :, 2 * i], x[s, :, 2 * i + 1] = x0 * c - x1 * sn, x0 * sn + x1 * c
    return x


def _rope_split(x, pos, theta=10000.0):
    x = x.astype(np.float64).copy()
    n = x.shape[-1]
    for s in range(x.shape[0]):
        for i in range(n // 2):
            a = pos[s] * theta ** (-2.0 * i / n)
            c, sn = np.cos(a), np.sin(a)
            x0, x1 = x[s, :, i].copy(), x[s, :, i + n // 2].copy()
            x[s, :, i], x[s, :, i + n // 2] = x0 * c - x1 * sn, x0 * sn + x1 * c
    return x


def numpy_attention(family, G, nvt, qkv, kc, vc, n_past, n_ctx):
    """float64 restatement used only to produce boundary vectors; caches are f16 arrays updated in place."""
    ql = qkv.shape[0]
    if family == "glm1":
        t = qkv.reshape(ql, H, 3, D)
        q, k, v = t[:, :, 0], t[:, :, 1], t[:, :, 2]
        p = np.arange(n_past, n_past + ql)
        p1, p2 = np.minimum(p, n_ctx - 2), np.maximum(p - (n_ctx - 2), 0)
        h = D // 2
        q = np.concatenate([_rope_split(q[..., :h], p1), _rope_split(q[..., h:], p2)], -1)
        k = np.concatenate([_rope_split(k[..., :h], p1), _rope_split(k[..., h:], p2)], -1)
    else:
        q = qkv[:, :HID].reshape(ql, H, D)
        k = qkv[:, HID:HID + G * D].reshape(ql, G, D)
        v = qkv[:, HID + G * D:].reshape(ql, G, D)
        pos = np.arange(n_past, n_past + ql)
        q, k = _rope_adjacent(q, pos, D // 2, 10000.0), _rope_adjacent(k, pos, D // 2, 10000.0)
    kc[:, nvt + n_past:nvt + n_past + ql, :] = k.transpose(1, 0, 2).astype(np.float32).astype(np.float16)
    vc[:, :, nvt + n_past:nvt + n_past + ql] = v.transpose(1, 2, 0).astype(np.float32).astype(np.float16)
    L = nvt + n_past + ql
    out = np.zeros((ql, H, D))
    for hh in range(H):
        g = hh // (H // G)
        K, Vt = kc[g, :L].astype(np.float64), vc[g, :, :L].astype(np.float64)
        sc = (q[:, hh, :] / np.sqrt(D)) @ K.T
        if n_past == 0:
            if family == "glm1":
                sc[:ql - 1, L - 1] = -np.inf
            else:
                for i in range(ql):
                    sc[i, nvt + i + 1:] = -np.inf
        pr = np.exp(sc - sc.max(-1, keepdims=True))
        pr /= pr.sum(-1, keepdims=True)
        out[:, hh, :] = pr @ Vt.T
    return out.reshape(ql, HID).astype(np.float32)


def convert(ref_dir, name):
    family, G, ffn, nvt = FIXTURES[name]
    dims = {"V": VOCAB, "hid": HID, "ffn": ffn, "qkv": HID + 2 * D * G}
    order = glm_tail.GLM1_WEIGHTS if family == "glm1" else glm_tail.GLM2_WEIGHTS
    out = {}
    with open(os.path.join(ref_dir, "tests", "data", name + ".data"), "rb") as f:
        if nvt:
            out["prefix"] = _rd(f, 2 * G * nvt * D, np.float16).reshape(2, G, nvt, D)
        w = {}
        for wn, shape in order:
            shp = tuple(dims[s] for s in shape)
            w[wn] = _rd(f, int(np.prod(shp))).reshape(shp)
        steps = []
        for s in (SEQ_LEN, 1, 1):
            x = _rd(f, s, np.int32)
            y = _rd(f, s * HID).reshape(s, HID)
            steps.append((x, y))
        assert f.read() == b"", "trailing bytes in " + name
    M = MAX_LENGTH + nvt
    kc, vc = np.zeros((G, M, D), np.float16), np.zeros((G, D, M), np.float16)
    if nvt:
        kc[:, :nvt, :] = out["prefix"][0]
        vc[:, :, :nvt] = out["prefix"][1].transpose(0, 2, 1)
    n_past, worst = 0, 0.0
    for i, (x, y) in enumerate(steps, 1):
        state, qkv = glm_tail.pre(family, w, x)
        ctx = numpy_attention(family, G, nvt, qkv.astype(np.float64), kc, vc, n_past, SEQ_LEN)
        err = float(np.abs(glm_tail.post(family, w, state, ctx) - y).max())
        assert err < 5e-4, (name, i, err)
        worst = max(worst, err)
        out.update({f"x{i}": x, f"y{i}": y, f"qkv{i}": qkv, f"ctx{i}": ctx, f"n_past{i}": np.int32(n_past)})
        n_past += len(x)
    out.update({"w_" + k: v for k, v in w.items()})
    out["k_cache_final"], out["v_cache_final"] = kc, vc
    out["meta"] = np.array(json.dumps({
        "family": family, "n_head": H, "n_kv_head": G, "head_dim": D, "hidden": HID, "max_length": MAX_LENGTH,
        "n_virtual": nvt, "n_ctx": SEQ_LEN, "interleaved_qkv": family == "glm1",
        "rope_type": 4 if family == "glm1" else 8, "mask_type": 1 if family == "glm1" else 0,
        "rope_theta": 10000.0, "source": f"tests/data/{name}.data", "numpy_twin_max_err": worst}))
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(f"{name}: numpy twin vs golden y max-abs {worst:.3e}")


def make_rope_hf():
    import torch
    from transformers.models.glm.configuration_glm import GlmConfig
    from transformers.models.glm.modeling_glm import GlmRotaryEmbedding, apply_rotary_pos_emb

    rng = np.random.default_rng(20240607)
    out = {}
    for tag, theta in (("t1e4", 10000.0), ("t5e6", 5.0e6)):
        try:
            cfg = GlmConfig(hidden_size=4096, num_attention_heads=32, num_key_value_heads=2, head_dim=128,
                            rope_parameters={"rope_type": "default", "rope_theta": theta,
                                             "partial_rotary_factor": 0.5})
        except TypeError:
            cfg = GlmConfig(hidden_size=4096, num_attention_heads=32, num_key_value_heads=2, head_dim=128,
                            rope_theta=theta, partial_rotary_factor=0.5)
        rot = GlmRotaryEmbedding(cfg)
        assert rot.inv_freq.numel() == 32, rot.inv_freq.shape
        pos = np.array([0, 1, 2, 7, 512, 1023, 8191, 131072], np.int64)
        q = rng.standard_normal((len(pos), 4, 128)).astype(np.float32)   # [s, heads, d]
        k = rng.standard_normal((len(pos), 2, 128)).astype(np.float32)
        tq, tk = torch.from_numpy(q).double()[None], torch.from_numpy(k).double()[None]  # [1, s, h, d]
        # float64 angles so that the fixture is a mathematical target rather than one f32 rounding path
        freqs = torch.from_numpy(pos).double()[:, None] * rot.inv_freq.double()[None, :]
        emb = torch.cat((freqs, freqs), dim=-1)[None]
        qe, ke = apply_rotary_pos_emb(tq, tk, emb.cos(), emb.sin(), unsqueeze_dim=2)
        out.update({f"{tag}_pos": pos.astype(np.int32), f"{tag}_q": q, f"{tag}_k": k,
                    f"{tag}_q_out": qe[0].numpy(), f"{tag}_k_out": ke[0].numpy(),
                    f"{tag}_theta": np.float32(theta)})
    np.savez_compressed(os.path.join(HERE, "rope_d128_hf.npz"), **out)
    print("rope_d128_hf.npz written")


def convert_linear(ref_dir):
    """tests/data/linear.data (tests/test_convert.py:192-207; read by chatglm_test.cpp:392-405): weight [32, 64], bias [32],
    x [2, 64], torch F.linear(x, w, b) [2, 32], then the same for the vector x[0]."""
    with open(os.path.join(ref_dir, "tests", "data", "linear.data"), "rb") as f:
        w = _rd(f, 32 * 64).reshape(32, 64)
        b = _rd(f, 32)
        x = _rd(f, 2 * 64).reshape(2, 64)
        y = _rd(f, 2 * 32).reshape(2, 32)
        vx = _rd(f, 64)
        vy = _rd(f, 32)
        assert f.read() == b""
    np.savez_compressed(os.path.join(HERE, "linear.npz"), w=w, b=b, x=x, y=y, vec_x=vx, vec_y=vy)
    print("linear.npz written")


def make_rope_modes_hf():
    """Full-head GPTJ and NEOX rotary and the ChatGLM-6B 2-D rotary at head_dim 128, through the rotary helpers of
    Hugging Face transformers (GPT-J: rotate_every_two; LLaMA / GPT-NeoX: rotate_half) with float64 angles.  The
    ladder inv_freq = theta^(-2i/n_dims) is the one both HF models build.  The 2-D form follows ChatGLM-6B's published
    formulation: the head is cut in two halves of D/2, each half is rotated NeoX-style (pairs (i, i + D/4)) over
    n_dims = D/2 with base 10000, the first by the position id and the second by the block position id."""
    import torch
    from transformers.models.gptj.modeling_gptj import apply_rotary_pos_emb as gptj_apply
    from transformers.models.llama.modeling_llama import apply_rotary_pos_emb as neox_apply

    rng = np.random.default_rng(20241125)
    D = 128
    pos = np.array([0, 1, 2, 7, 513, 2047, 8191, 40000], np.int64)
    blk = np.array([0, 0, 3, 1, 77, 1, 300, 2], np.int64)
    x = rng.standard_normal((len(pos), 3, D)).astype(np.float32)      # [s, heads, d]
    tx = torch.from_numpy(x).double()[None]                            # [1, s, h, d]
    out = {"pos": pos.astype(np.int32), "block": blk.astype(np.int32), "x": x}
    for theta in (10000.0, 50000.0):
        inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float64) / D))          # [D/2]
        ang = torch.from_numpy(pos).double()[:, None] * inv[None, :]                      # [s, D/2]
        y_gptj = gptj_apply(tx, ang.sin()[None], ang.cos()[None])                         # pairs (2i, 2i+1)
        emb = torch.cat((ang, ang), dim=-1)[None]
        y_neox, _ = neox_apply(tx, tx, emb.cos(), emb.sin(), unsqueeze_dim=2)             # pairs (i, i + D/2)
        tag = f"t{int(theta)}"
        out[f"gptj_{tag}"] = y_gptj[0].numpy()
        out[f"neox_{tag}"] = y_neox[0].numpy()
    half = D // 2
    inv = 1.0 / (10000.0 ** (torch.arange(0, half, 2, dtype=torch.float64) / half))      # [D/4]
    halves = []
    for ids, sl in ((pos, slice(0, half)), (blk, slice(half, D))):
        ang = torch.from_numpy(ids).double()[:, None] * inv[None, :]
        emb = torch.cat((ang, ang), dim=-1)[None]
        y, _ = neox_apply(tx[..., sl], tx[..., sl], emb.cos(), emb.sin(), unsqueeze_dim=2)
        halves.append(y)
    out["glm2d"] = torch.cat(halves, dim=-1)[0].numpy()
    np.savez_compressed(os.path.join(HERE, "rope_modes_d128_hf.npz"), **out)
    print("rope_modes_d128_hf.npz written")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("CHATGLM_CPP_REFERENCE"), required="CHATGLM_CPP_REFERENCE" not in os.environ,
                    help="checkout of li-plus/chatglm.cpp (or set CHATGLM_CPP_REFERENCE)")
    ap.add_argument("--skip-hf", action="store_true")
    a = ap.parse_args()
    for n in FIXTURES:
        convert(a.reference, n)
    convert_linear(a.reference)
    if not a.skip_hf:
        make_rope_hf()
        make_rope_modes_hf()
