"""The CPU oracle against the reference's golden vectors (CPU only).

Trust chain: reference fixtures (HF PyTorch outputs, tests/data/*_model.data) -> oracle at head_dim 4
for every family, with and without a P-Tuning prefix, over prefill + two decode steps -> the same
oracle code at head_dim 128 -> the CUDA kernels (GPU tests).
"""
import os

import numpy as np
import pytest

from golden_util import GOLDEN_ATOL, MODEL_FIXTURES, load_fixture, model_output, steps
from oracle import attn_oracle as O


def _cfg(meta, numerics):
    return O.make_cfg(meta["n_head"], meta["n_kv_head"], meta["head_dim"], meta["max_length"] + meta["n_virtual"],
                      meta["n_virtual"], meta["rope_type"], meta["rope_theta"], meta["mask_type"], numerics)


@pytest.mark.parametrize("numerics", ["ggml", "f32"])
@pytest.mark.parametrize("name", MODEL_FIXTURES)
def test_oracle_reproduces_reference_fixture(name, numerics):
    z, meta, w = load_fixture(name)
    cfg = _cfg(meta, numerics)
    kc, vc = O.new_caches(cfg)
    if meta["n_virtual"]:
        O.load_prefix_cache(cfg, z["prefix"], kc, vc)
    for i, x, y, qkv, ctx_twin, n_past in steps(z):
        ctx = O.attn_forward(cfg, qkv, meta["interleaved_qkv"], kc, vc, n_past, n_ctx=meta["n_ctx"])
        out = model_output(meta, w, x, ctx)
        assert np.isfinite(out).all()
        # the reference's own check: 1-layer model output within 5e-4 of the HF golden vector
        assert np.abs(out - y).max() < GOLDEN_ATOL, (name, i)
        # and at the attention boundary against the independent numpy restatement
        tol = 2e-3 if numerics == "ggml" else 1e-5
        assert np.abs(ctx - ctx_twin).max() < tol, (name, i)
    # caches: identical f16 bits to the numpy restatement's
    np.testing.assert_array_equal(kc, z["k_cache_final"].view(np.uint16))
    np.testing.assert_array_equal(vc, z["v_cache_final"].view(np.uint16))


# where a checkout of li-plus/chatglm.cpp is mounted, if anywhere (CHATGLM_CPP_REFERENCE=/path/to/checkout)
REFERENCE_DATA = os.path.join(os.environ.get("CHATGLM_CPP_REFERENCE", ""), "tests", "data")


@pytest.mark.skipif(not os.path.isdir(REFERENCE_DATA), reason="CHATGLM_CPP_REFERENCE does not point at a reference checkout")
@pytest.mark.parametrize("name", MODEL_FIXTURES)
def test_committed_fixture_matches_reference_file(name):
    """The committed .npz carries exactly the golden bytes of the reference's .data file."""
    z, meta, w = load_fixture(name)
    raw = np.fromfile(os.path.join(REFERENCE_DATA, name + ".data"), np.uint8)
    tail = np.concatenate([np.concatenate([z[f"x{i}"].view(np.uint8), z[f"y{i}"].reshape(-1).view(np.uint8)])
                           for i in (1, 2, 3)])
    np.testing.assert_array_equal(raw[-tail.size:], tail)


def test_oracle_linear_matches_reference_fixture():
    """Linear (chatglm.cpp:418-426) against the reference's tests/data/linear.data, with the reference's own
    tolerances per weight type (chatglm_test.cpp:430-436): f32 1e-5, f16 weights atol 1e-2 + rtol 5e-4."""
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "linear.npz"))
    for x, y in ((z["x"], z["y"]), (z["vec_x"][None], z["vec_y"][None])):
        got = O.linear(x, z["w"], z["b"])
        assert np.abs(got - y).max() <= 1e-5
        for round_x in (False, True):
            got16 = O.linear(x, z["w"].astype(np.float16), z["b"], round_x_f16=round_x)
            assert (np.abs(got16 - y) <= 1e-2 + 5e-4 * np.abs(y)).all()
        assert np.abs(O.linear(x, z["w"], None) + z["b"] - y).max() <= 1e-5


def test_f16_conversion_matches_ieee_rne():
    rng = np.random.default_rng(0)
    xs = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 20000),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001,
                  6.1e-5, 6.0975e-5, np.inf, -np.inf, 1.0009765625, 1.00048828125, 1.00146484375], np.float32)])
    want = xs.astype(np.float16).view(np.uint16)
    lib = O.lib()
    got = np.array([lib.oracle_f32_to_f16(float(x)) for x in xs], np.uint16)
    np.testing.assert_array_equal(got, want)
    hs = np.arange(0, 65536, 7, dtype=np.uint16)
    back = np.array([lib.oracle_f16_to_f32(int(h)) for h in hs], np.float32)
    ref = hs.view(np.float16).astype(np.float32)
    np.testing.assert_array_equal(back[~np.isnan(ref)], ref[~np.isnan(ref)])


@pytest.mark.parametrize("tag", ["t1e4", "t5e6"])
def test_oracle_rope_d128_matches_hf_glm(tag):
    """Pair pattern, partial-rotary width and frequency ladder at head_dim 128 (HF-native GLM-4 rotary)."""
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "rope_d128_hf.npz"))
    pos, theta = z[f"{tag}_pos"], float(z[f"{tag}_theta"])
    for which, nh in (("q", 4), ("k", 2)):
        cfg = O.make_cfg(nh, nh, 128, 8, 0, O.ROPE_CHATGLM2, theta)
        got = O.apply_rotary_emb(cfg, z[f"{tag}_{which}"], pos)
        want = z[f"{tag}_{which}_out"]
        # untouched half is bit-identical
        np.testing.assert_array_equal(got[..., 64:], z[f"{tag}_{which}"][..., 64:])
        # rotated half: f32 angle (iterated ladder) vs float64 angles; error grows with the position
        err = np.abs(got[..., :64] - want[..., :64]).max(axis=(1, 2))
        assert (err <= 2e-6 + 2e-7 * pos).all(), err


@pytest.mark.parametrize("mode", ["gptj_t10000", "gptj_t50000", "neox_t10000", "neox_t50000", "glm2d"])
def test_oracle_rope_modes_d128_match_hf_helpers(mode):
    """The full-head GPTJ / NEOX branches (apply_rotary_emb_basic, chatglm.cpp:523-537) and the ChatGLM-6B 2-D rotary
    (apply_rotary_emb_glm, chatglm.cpp:539-574) at head_dim 128 against vectors made with the rotary helpers of Hugging
    Face transformers (tests/golden/make_golden.py:make_rope_modes_hf): pair pattern, ladder, which half takes which id."""
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "rope_modes_d128_hf.npz"))
    x, pos, blk = z["x"], z["pos"], z["block"]
    if mode == "glm2d":
        cfg = O.make_cfg(3, 3, 128, 8, 0, O.ROPE_CHATGLM, 10000.0, O.MASK_CHATGLM)
        ids = np.concatenate([pos, blk]).astype(np.int32)      # [2S]: position ids, then block position ids
        scale = np.maximum(pos, blk)
    else:
        kind, tag = mode.split("_t")
        cfg = O.make_cfg(3, 3, 128, 8, 0, O.ROPE_GPTJ if kind == "gptj" else O.ROPE_NEOX, float(tag))
        ids, scale = pos.astype(np.int32), pos
    got = O.apply_rotary_emb(cfg, x, ids)
    want = z[mode]
    # f32 iterated-ladder angles (theta_scale rounded to f32, one more rounding per ladder step: a relative angle
    # error of about i * 6e-8 at step i) against float64 angles: the gap grows with the position and nothing else
    err = np.abs(got - want).max(axis=(1, 2))
    assert (err <= 2e-6 + 5e-7 * scale).all(), err
    # and a wrong pair pattern or ladder would be off by O(1)
    assert np.abs(want - x).max() > 0.5


def test_rope_modes_small_cases():
    """The four rope modes on hand-checkable inputs (chatglm.cpp:523-618)."""
    x = np.arange(1, 9, dtype=np.float32).reshape(1, 1, 8)
    ids = np.array([3], np.int32)
    # DISABLED: passthrough
    cfg = O.make_cfg(1, 1, 8, 4, 0, O.ROPE_DISABLED)
    np.testing.assert_array_equal(O.apply_rotary_emb(cfg, x, ids), x)
    # CHATGLM2: first 4 dims as adjacent pairs, angles 3*1e4^(-2i/4)
    cfg = O.make_cfg(1, 1, 8, 4, 0, O.ROPE_CHATGLM2)
    y = O.apply_rotary_emb(cfg, x, ids)[0, 0]
    for i, a in enumerate([3.0, 3.0 * 10000.0 ** -0.5]):
        c, s = np.cos(a), np.sin(a)
        np.testing.assert_allclose(y[2 * i], x[0, 0, 2 * i] * c - x[0, 0, 2 * i + 1] * s, rtol=1e-6)
        np.testing.assert_allclose(y[2 * i + 1], x[0, 0, 2 * i] * s + x[0, 0, 2 * i + 1] * c, rtol=1e-6)
    np.testing.assert_array_equal(y[4:], x[0, 0, 4:])
    # CHATGLM (2-D): dims [0,4) by ids[0], [4,8) by ids[1], split-half pairs (i, i+2) inside each half
    cfg = O.make_cfg(1, 1, 8, 4, 0, O.ROPE_CHATGLM)
    y = O.apply_rotary_emb(cfg, x, np.array([2, 5], np.int32))[0, 0]
    for base, p in ((0, 2.0), (4, 5.0)):
        for i, a in enumerate([p, p * 10000.0 ** -0.5]):
            c, s = np.cos(a), np.sin(a)
            x0, x1 = x[0, 0, base + i], x[0, 0, base + i + 2]
            np.testing.assert_allclose(y[base + i], x0 * c - x1 * s, rtol=2e-6)
            np.testing.assert_allclose(y[base + i + 2], x0 * s + x1 * c, rtol=2e-6)
    # GPTJ / NEOX over the full head
    for mode, pair in ((O.ROPE_GPTJ, lambda i: (2 * i, 2 * i + 1)), (O.ROPE_NEOX, lambda i: (i, i + 4))):
        cfg = O.make_cfg(1, 1, 8, 4, 0, mode)
        y = O.apply_rotary_emb(cfg, x, ids)[0, 0]
        for i in range(4):
            a = 3.0 * 10000.0 ** (-2.0 * i / 8)
            c, s = np.cos(a), np.sin(a)
            i0, i1 = pair(i)
            np.testing.assert_allclose(y[i0], x[0, 0, i0] * c - x[0, 0, i1] * s, rtol=2e-5, atol=1e-6)
            np.testing.assert_allclose(y[i1], x[0, 0, i0] * s + x[0, 0, i1] * c, rtol=2e-5, atol=1e-6)


def test_position_ids_and_mask_producers():
    np.testing.assert_array_equal(O.position_ids(O.make_cfg(1, 1, 4, 8), 3, 5), [5, 6, 7])
    cfg1 = O.make_cfg(1, 1, 4, 8, rope_type=O.ROPE_CHATGLM)
    # prefill of n_ctx=3 tokens: positions 0,1,1 / blocks 0,0,1 (chatglm.cpp:1147-1151)
    np.testing.assert_array_equal(O.position_ids(cfg1, 3, 0, 3), [0, 1, 1, 0, 0, 1])
    np.testing.assert_array_equal(O.position_ids(cfg1, 1, 4, 3), [1, 3])
    m = O.attention_mask_glm(3, 5)
    assert np.isneginf(m[0, 4]) and np.isneginf(m[1, 4]) and m[2, 4] == 0 and (m[:, :4] == 0).all()


def test_partial_combine_equals_full_attention():
    """Split-KV partials merged by log-sum-exp reproduce the one-pass attention."""
    rng = np.random.default_rng(5)
    H, G, D, M, P = 8, 2, 16, 96, 80
    cfg = O.make_cfg(H, G, D, M, numerics="f32")
    kc, vc = O.new_caches(cfg)
    kc[:, :P] = rng.standard_normal((G, P, D)).astype(np.float16).view(np.uint16)
    vc[:, :, :P] = rng.standard_normal((G, D, P)).astype(np.float16).view(np.uint16)
    qkv = rng.standard_normal((1, (H + 2 * G) * D)).astype(np.float32)
    full, qr, _ = O.attn_forward(cfg, qkv, False, kc, vc, P, want_roped=True)
    for cuts in ([0, P + 1], [0, 17, P + 1], [0, 1, 40, 41, P + 1]):
        parts = [O.attn_partial(cfg, qr[0], kc, vc, a, b) for a, b in zip(cuts[:-1], cuts[1:])]
        out = O.attn_combine(np.stack([p[0] for p in parts]), np.stack([p[1] for p in parts]),
                             np.stack([p[2] for p in parts]))
        np.testing.assert_allclose(out.reshape(-1), full[0], atol=2e-6, rtol=1e-5)
    # an empty slice contributes nothing
    empty = O.attn_partial(cfg, qr[0], kc, vc, 7, 7)
    whole = O.attn_partial(cfg, qr[0], kc, vc, 0, P + 1)
    out = O.attn_combine(np.stack([empty[0], whole[0]]), np.stack([empty[1], whole[1]]),
                         np.stack([empty[2], whole[2]]))
    np.testing.assert_allclose(out.reshape(-1), full[0], atol=2e-6, rtol=1e-5)


def test_decode_batch_matches_single_calls():
    rng = np.random.default_rng(11)
    H, G, D, M = 8, 2, 16, 40
    cfg = O.make_cfg(H, G, D, M)
    n_past = [0, 5, 39, 17]
    qs, ks, vs, kcs, vcs, want = [], [], [], [], [], []
    for P in n_past:
        kc, vc = O.new_caches(cfg)
        kc[:, :P] = rng.standard_normal((G, P, D)).astype(np.float16).view(np.uint16)
        vc[:, :, :P] = rng.standard_normal((G, D, P)).astype(np.float16).view(np.uint16)
        qkv = rng.standard_normal((1, (H + 2 * G) * D)).astype(np.float32)
        kc2, vc2 = kc.copy(), vc.copy()
        want.append((O.attn_forward(cfg, qkv, False, kc2, vc2, P)[0], kc2, vc2))
        qs.append(qkv[0, :H * D].copy()); ks.append(qkv[0, H * D:(H + G) * D].copy()); vs.append(qkv[0, (H + G) * D:].copy())
        kcs.append(kc); vcs.append(vc)
    outs = O.attn_decode_batch(cfg, qs, ks, vs, D, D, kcs, vcs, n_past, n_threads=2)
    for o, (w, kc2, vc2), kc, vc in zip(outs, want, kcs, vcs):
        np.testing.assert_array_equal(o, w)
        np.testing.assert_array_equal(kc, kc2)
        np.testing.assert_array_equal(vc, vc2)


def test_bad_arguments_are_rejected():
    cfg = O.make_cfg(8, 2, 4, 8)
    kc, vc = O.new_caches(cfg)
    qkv = np.zeros((1, 48), np.float32)
    with pytest.raises(ValueError):
        O.attn_forward(cfg, qkv, False, kc, vc, 8)  # n_past + qlen > max_len
