"""numpy forms of the non-attention parts of the reference's 1-layer test models.

The reference pins BasicAttention::forward only through a whole 1-layer model
(chatglm_test.cpp:288-362): embedding -> block -> final norm.  To carry those golden vectors to the
attention boundary, these helpers compute what comes before the attention (``pre``: embedding, input
norm, fused qkv Linear) and after it (``post``: dense, residual, MLP, final norm) for the two
families: ChatGLM-6B v1 (GLMBlock, chatglm.cpp:1070-1087) and ChatGLM2/3/4 (BasicBlock,
chatglm.h:488-503).  Attention itself is deliberately absent.
"""
import numpy as np


def _rms(x, w, eps=1e-5):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def _ln(x, w, b, eps=1e-5):
    m = x.mean(-1, keepdims=True)
    v = ((x - m) ** 2).mean(-1, keepdims=True)
    return (x - m) / np.sqrt(v + eps) * w + b


def _silu(x):
    return x / (1 + np.exp(-x))


def _gelu(x):
    return 0.5 * x * (1 + np.tanh(0.7978845608028654 * x * (1 + 0.044715 * x * x)))


# weight order in the fixture files (chatglm_test.cpp:609-623 and :677-686)
GLM1_WEIGHTS = [("emb", ("V", "hid")), ("ln1_w", ("hid",)), ("ln1_b", ("hid",)), ("qkv_w", ("qkv", "hid")),
                ("qkv_b", ("qkv",)), ("dense_w", ("hid", "hid")), ("dense_b", ("hid",)), ("ln2_w", ("hid",)),
                ("ln2_b", ("hid",)), ("fc1_w", ("ffn", "hid")), ("fc1_b", ("ffn",)), ("fc2_w", ("hid", "ffn")),
                ("fc2_b", ("hid",)), ("lnf_w", ("hid",)), ("lnf_b", ("hid",))]
GLM2_WEIGHTS = [("emb", ("V", "hid")), ("ln1_w", ("hid",)), ("qkv_w", ("qkv", "hid")), ("qkv_b", ("qkv",)),
                ("dense_w", ("hid", "hid")), ("ln2_w", ("hid",)), ("gate_w", ("ffn", "hid")),
                ("up_w", ("ffn", "hid")), ("down_w", ("hid", "ffn")), ("lnf_w", ("hid",))]

GLM1_ALPHA = np.sqrt(2.0 * 28.0)  # GLMBlock alpha for the 28-layer ChatGLM-6B the fixture shrinks


def pre(family, w, x):
    """token ids -> (state the post step needs, fused qkv activation [qlen, qkv])."""
    h = w["emb"][x]
    if family == "glm1":
        a = _ln(h, w["ln1_w"], w["ln1_b"])
        return a, (a @ w["qkv_w"].T + w["qkv_b"]).astype(np.float32)
    a = _rms(h, w["ln1_w"])
    return h, (a @ w["qkv_w"].T + w["qkv_b"]).astype(np.float32)


def post(family, w, state, ctx):
    """context_layer [qlen, hid] -> model output [qlen, hid]."""
    if family == "glm1":
        a = state
        h = a * GLM1_ALPHA + (ctx @ w["dense_w"].T + w["dense_b"])
        m = _ln(h, w["ln2_w"], w["ln2_b"])
        h = m * GLM1_ALPHA + (_gelu(m @ w["fc1_w"].T + w["fc1_b"]) @ w["fc2_w"].T + w["fc2_b"])
        return _ln(h, w["lnf_w"], w["lnf_b"])
    h = state + ctx @ w["dense_w"].T
    m = _rms(h, w["ln2_w"])
    h = h + (_silu(m @ w["gate_w"].T) * (m @ w["up_w"].T)) @ w["down_w"].T
    return _rms(h, w["lnf_w"])
