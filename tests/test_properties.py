"""Property tests of the CPU oracle over random shapes (hypothesis): an independent float64 numpy restatement of
chatglm.cpp:523-717 written here, size-independent identities of the path (split-KV partials merge to the whole,
a prompt fed token by token fills the cache with the same bits as the prompt fed at once), and the prefix loader.
Small shapes, so the whole file runs in seconds on CPU."""
import numpy as np
from hypothesis import given, settings, strategies as st

from oracle import attn_oracle as O


def rope_f64(x, pos, n_dims, theta, split):
    """x [S, heads, n_dims...]: rotate the first n_dims of every head; pairs (2i, 2i+1) or (i, i + n_dims/2)."""
    x = x.astype(np.float64).copy()
    i = np.arange(n_dims // 2)
    ang = pos[:, None].astype(np.float64) * theta ** (-2.0 * i / n_dims)[None, :]      # [S, n_dims/2]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = (i, i + n_dims // 2) if split else (2 * i, 2 * i + 1)
    x0, x1 = x[..., a].copy(), x[..., b].copy()
    x[..., a], x[..., b] = x0 * c - x1 * s, x0 * s + x1 * c
    return x


def twin_forward(H, G, D, V, rope, mask, theta, qkv, interleaved, kc, vc, n_past, n_ctx):
    """float64 attention over f16 caches (updated in place, f16 bits as uint16)."""
    S = qkv.shape[0]
    if interleaved:
        t = qkv.reshape(S, H, 3, D)
        q, k, v = t[:, :, 0], t[:, :, 1], t[:, :, 2]
    else:
        q = qkv[:, :H * D].reshape(S, H, D)
        k = qkv[:, H * D:(H + G) * D].reshape(S, G, D)
        v = qkv[:, (H + G) * D:].reshape(S, G, D)
    p = np.arange(n_past, n_past + S)
    if rope == O.ROPE_CHATGLM:
        p1, p2 = np.minimum(p, n_ctx - 2), np.maximum(p - (n_ctx - 2), 0)
        h = D // 2
        q = np.concatenate([rope_f64(q[..., :h], p1, h, 10000.0, True), rope_f64(q[..., h:], p2, h, 10000.0, True)], -1)
        k = np.concatenate([rope_f64(k[..., :h], p1, h, 10000.0, True), rope_f64(k[..., h:], p2, h, 10000.0, True)], -1)
    elif rope == O.ROPE_CHATGLM2:
        q, k = rope_f64(q, p, D // 2, theta, False), rope_f64(k, p, D // 2, theta, False)
    elif rope in (O.ROPE_GPTJ, O.ROPE_NEOX):
        q, k = rope_f64(q, p, D, theta, rope == O.ROPE_NEOX), rope_f64(k, p, D, theta, rope == O.ROPE_NEOX)
    k16 = k.astype(np.float32).astype(np.float16)
    v16 = v.astype(np.float32).astype(np.float16)
    kc[:, V + n_past:V + n_past + S, :] = k16.transpose(1, 0, 2).view(np.uint16)
    vc[:, :, V + n_past:V + n_past + S] = v16.transpose(1, 2, 0).view(np.uint16)
    L = V + n_past + S
    out = np.zeros((S, H, D))
    for h in range(H):
        g = h // (H // G)
        K = kc[g, :L].view(np.float16).astype(np.float64)
        Vt = vc[g, :, :L].view(np.float16).astype(np.float64)
        sc = (q[:, h, :].astype(np.float64) / np.sqrt(D)) @ K.T
        if n_past == 0:
            if mask == O.MASK_CHATGLM:
                sc[:S - 1, L - 1] = -np.inf
            else:
                for i in range(S):
                    sc[i, V + i + 1:] = -np.inf
        pr = np.exp(sc - sc.max(-1, keepdims=True))
        pr /= pr.sum(-1, keepdims=True)
        out[:, h, :] = pr @ Vt.T
    return out.reshape(S, H * D)


shapes = st.tuples(
    st.sampled_from([1, 2, 4]),                 # G
    st.sampled_from([1, 2, 4, 16]),             # R = H / G
    st.sampled_from([4, 8, 32, 128]),           # D
    st.integers(0, 6),                          # V
    st.sampled_from(["glm2", "glm1", "gptj", "neox", "none"]),
    st.integers(0, 40),                         # n_past
    st.integers(1, 9),                          # S
    st.integers(0, 2 ** 31 - 1),                # seed
)


@settings(max_examples=60, deadline=None)
@given(shapes)
def test_oracle_matches_numpy_twin_on_random_shapes(sh):
    G, R, D, V, fam, n_past, S, seed = sh
    H = G * R
    if fam == "glm1":
        G, H = H, H          # the v1 family is MHA with interleaved qkv (chatglm.cpp:637)
    if H * D > 2048:
        R = max(1, 2048 // (G * D)); H = G * R
        if fam == "glm1":
            G = H
    rope = {"glm2": O.ROPE_CHATGLM2, "glm1": O.ROPE_CHATGLM, "gptj": O.ROPE_GPTJ, "neox": O.ROPE_NEOX, "none": O.ROPE_DISABLED}[fam]
    mask = O.MASK_CHATGLM if fam == "glm1" else O.MASK_CAUSAL
    theta = 10000.0 if seed % 2 else 500000.0
    M = V + n_past + S + seed % 5
    rng = np.random.default_rng(seed)
    inter = fam == "glm1"
    width = 3 * H * D if inter else (H + 2 * G) * D
    n_ctx = max(2, n_past // 2 + 2)
    cfg = O.make_cfg(H, G, D, M, V, rope, theta, mask, "f32")
    kc = np.zeros((G, M, D), np.uint16)
    vc = np.zeros((G, D, M), np.uint16)
    kc[:, :V + n_past] = rng.standard_normal((G, V + n_past, D)).astype(np.float16).view(np.uint16)
    vc[:, :, :V + n_past] = rng.standard_normal((G, D, V + n_past)).astype(np.float16).view(np.uint16)
    qkv = rng.standard_normal((S, width)).astype(np.float32)
    kt, vt = kc.copy(), vc.copy()
    got = O.attn_forward(cfg, qkv, inter, kc, vc, n_past, n_ctx=n_ctx)
    want = twin_forward(H, G, D, V, rope, mask, theta, qkv, inter, kt, vt, n_past, n_ctx)
    assert np.abs(got - want).max() <= 2e-4 * (1 + 1e-3 * (n_past + S)), (sh, float(np.abs(got - want).max()))
    # the appended rows: V is a plain f16 rounding (bit-exact); a roped K value comes out of x0 c - x1 s with f32-ladder
    # angles on one side and float64 angles on the other, so it may land on a neighbouring f16 value (or, where the
    # two products cancel, a few ulps of a small number away): compare values, and bits wherever nothing was appended
    np.testing.assert_array_equal(vc, vt)
    kf, tf = kc.view(np.float16).astype(np.float32), kt.view(np.float16).astype(np.float32)
    assert np.abs(kf - tf).max() <= 4e-3 and (kc != kt).mean() < 0.02
    rows = np.r_[0:V + n_past, V + n_past + S:M]
    np.testing.assert_array_equal(kc[:, rows], kt[:, rows])


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 300), st.integers(2, 6), st.sampled_from([(4, 2, 32), (16, 1, 128), (3, 3, 8)]), st.integers(0, 2 ** 31 - 1))
def test_splitkv_partials_of_any_cut_merge_to_the_whole(L, n_cut, hgd, seed):
    """The LSE merge is order- and cut-independent (the identity the multi-GPU split rests on)."""
    H, G, D = hgd
    rng = np.random.default_rng(seed)
    cfg = O.make_cfg(H, G, D, L, 0, O.ROPE_DISABLED, 10000.0, O.MASK_CAUSAL, "f32")
    kc = rng.standard_normal((G, L, D)).astype(np.float16).view(np.uint16)
    vc = rng.standard_normal((G, D, L)).astype(np.float16).view(np.uint16)
    q = rng.standard_normal((H, D)).astype(np.float32)
    cuts = sorted(set([0, L] + [int(c) for c in rng.integers(0, L + 1, n_cut - 1)]))
    parts = [O.attn_partial(cfg, q, kc, vc, a, b) for a, b in zip(cuts[:-1], cuts[1:])]
    whole = O.attn_partial(cfg, q, kc, vc, 0, L)
    rng.shuffle(parts)
    acc = np.stack([p[0] for p in parts]); m = np.stack([p[1] for p in parts]); l = np.stack([p[2] for p in parts])
    got = O.attn_combine(acc, m, l)
    want = whole[0] / whole[2][:, None]
    assert np.abs(got - want).max() <= 1e-5 * (1 + np.abs(want).max())


@settings(max_examples=25, deadline=None)
@given(st.integers(2, 12), st.sampled_from(["glm2", "glm1"]), st.integers(0, 4), st.integers(0, 2 ** 31 - 1))
def test_prompt_fed_at_once_or_token_by_token_fills_the_cache_identically(S, fam, V, seed):
    """chatglm.cpp:664-675 appends per token; RoPE depends on the position only: the cache after a prompt of S tokens
    is the same whether the tokens came in one call or in S calls, and the last token's output agrees."""
    H, G, D = (4, 4, 16) if fam == "glm1" else (8, 2, 16)
    rope, mask = (O.ROPE_CHATGLM, O.MASK_CHATGLM) if fam == "glm1" else (O.ROPE_CHATGLM2, O.MASK_CAUSAL)
    inter = fam == "glm1"
    M = V + S + 3
    rng = np.random.default_rng(seed)
    cfg = O.make_cfg(H, G, D, M, V, rope, 10000.0, mask, "f32")
    width = 3 * H * D if inter else (H + 2 * G) * D
    qkv = rng.standard_normal((S, width)).astype(np.float32)
    pre_k = rng.standard_normal((G, V, D)).astype(np.float16).view(np.uint16)
    pre_v = rng.standard_normal((G, D, V)).astype(np.float16).view(np.uint16)
    caches = []
    outs = []
    for mode in ("once", "stepwise"):
        kc, vc = O.new_caches(cfg)
        kc[:, :V], vc[:, :, :V] = pre_k, pre_v
        if mode == "once":
            out = O.attn_forward(cfg, qkv, inter, kc, vc, 0, n_ctx=S)[-1]
        else:
            for t in range(S):
                out = O.attn_forward(cfg, qkv[t:t + 1], inter, kc, vc, t, n_ctx=S)[0]
        caches.append((kc, vc)); outs.append(out)
    np.testing.assert_array_equal(caches[0][0], caches[1][0])
    np.testing.assert_array_equal(caches[0][1], caches[1][1])
    # the last row of a causal prefill sees everything, like a decode step; the v1 mask also lets the last row see all
    assert np.abs(outs[0] - outs[1]).max() <= 1e-5


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 9), st.integers(1, 200), st.integers(1, 40), st.booleans(), st.booleans(), st.booleans(),
       st.integers(0, 2 ** 31 - 1))
def test_oracle_linear_matches_float64_numpy(n_tok, n_in, n_out, w_f16, round_x, use_bias, seed):
    """Linear::forward of the oracle (chatglm.cpp:418-426) against a float64 product of the same operands: f16 weights are
    widened exactly, round_x_f16 rounds the activation to f16 first, the bias is added once.  Bound: f32 accumulation of
    n_in products of unit scale."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n_tok, n_in)).astype(np.float32)
    w = rng.standard_normal((n_out, n_in)).astype(np.float16 if w_f16 else np.float32)
    b = rng.standard_normal(n_out).astype(np.float32) if use_bias else None
    got = O.linear(x, w, b, round_x_f16=round_x)
    xe = x.astype(np.float16).astype(np.float64) if round_x else x.astype(np.float64)
    want = xe @ w.astype(np.float64).T + (b.astype(np.float64) if use_bias else 0.0)
    assert got.shape == (n_tok, n_out) and got.dtype == np.float32
    assert np.abs(got - want).max() <= 4e-6 * n_in * max(1.0, float(np.abs(want).max()))
