"""Shared helpers of the GPU parity tests: run one case through the C ABI and through the CPU oracle."""
import numpy as np
import torch

from chatglm_cpp_b200 import attention as A
from chatglm_cpp_b200._lib import AttnDesc
from oracle import attn_oracle as O

# north-star tolerances for the attention output against the oracle in f32
OUT_ATOL, OUT_RTOL = 2e-3, 1e-2
ROPE_MAX_ULP = 2


def ulp_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in units in the last place between two f32 arrays."""
    def ordered(x):
        i = np.ascontiguousarray(x, np.float32).view(np.int32).astype(np.int64)
        return np.where(i < 0, -(i & 0x7FFFFFFF), i)
    return np.abs(ordered(a) - ordered(b))


def assert_out_close(got: np.ndarray, want: np.ndarray, what=""):
    """North-star gate: max-abs <= 2e-3 (and so within 2e-3 + 1e-2*|want|), plus a norm-wise sanity bound."""
    err = np.abs(got - want)
    assert np.isfinite(got).all(), what
    assert err.max() <= OUT_ATOL, (what, float(err.max()))
    assert (err <= OUT_ATOL + OUT_RTOL * np.abs(want)).all(), what
    rel = float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
    assert rel <= 2e-3, (what, rel)


def make_desc(H, G, D, M, V=0, rope=O.ROPE_CHATGLM2, theta=10000.0, mask=O.MASK_CAUSAL) -> AttnDesc:
    return AttnDesc(H, G, D, M, V, rope, theta, mask)


def oracle_cfg(desc: AttnDesc, numerics="ggml"):
    return O.make_cfg(desc.n_head, desc.n_kv_head, desc.head_dim, desc.max_len, desc.n_virtual, desc.rope_type,
                      desc.rope_theta, desc.mask_type, numerics)


def random_cache(rng, desc: AttnDesc, n_filled: int):
    """Host caches (uint16 views of f16) with N(0,1) in positions [0, n_filled) and a canary pattern elsewhere."""
    G, M, D = desc.n_kv_head, desc.max_len, desc.head_dim
    k = np.full((G, M, D), 0x3555, np.uint16)       # canary: f16 0.333
    v = np.full((G, D, M), 0xB555, np.uint16)       # canary: f16 -0.333
    k[:, :n_filled] = rng.standard_normal((G, n_filled, D)).astype(np.float16).view(np.uint16)
    v[:, :, :n_filled] = rng.standard_normal((G, D, n_filled)).astype(np.float16).view(np.uint16)
    return k, v


def upload_cache(arena: A.KVArena, slot: int, k: np.ndarray, v: np.ndarray):
    arena.k_cache(slot).copy_(torch.from_numpy(k.view(np.float16)).cuda())
    arena.v_cache(slot).copy_(torch.from_numpy(v.view(np.float16)).cuda())


def download_cache(arena: A.KVArena, slot: int):
    return (arena.k_cache(slot).cpu().numpy().view(np.uint16), arena.v_cache(slot).cpu().numpy().view(np.uint16))


def qkv_width(desc: AttnDesc, interleaved: bool) -> int:
    return 3 * desc.n_head * desc.head_dim if interleaved else (desc.n_head + 2 * desc.n_kv_head) * desc.head_dim


def run_decode_batch(desc: AttnDesc, n_past_list, seed=0, interleaved=False, n_ctx_list=None, check_rope=True,
                     n_past_on_device=False, f16_io=False):
    """One decode step for a batch through the CUDA path and the oracle; asserts the parity gates.
    n_past_on_device: the kernel reads every position from a device word (CGLM_SEQ_N_PAST_DEVICE); the host field
    then only carries an upper bound.
    f16_io: the activations go in as f16 and the output comes back as f16 (CGLM_SEQ_QKV_F16 | CGLM_SEQ_OUT_F16); the
    oracle is fed the same f16-representable values, so the cache bits and the RoPE bound do not change, and its
    output is compared after the one extra rounding."""
    rng = np.random.default_rng(seed)
    n = len(n_past_list)
    V = desc.n_virtual
    arena = A.KVArena(desc, n)
    ws = A.Workspace(desc, n, 1)
    calls, host = [], []
    n_past_dev = torch.tensor([int(p) for p in n_past_list], dtype=torch.int32, device="cuda")
    bound = desc.max_len - V - 1
    for i, P in enumerate(n_past_list):
        k, v = random_cache(rng, desc, V + P)
        upload_cache(arena, i, k, v)
        qkv = rng.standard_normal((1, qkv_width(desc, interleaved))).astype(np.float32)
        if f16_io:
            qkv = qkv.astype(np.float16).astype(np.float32)
        n_ctx = n_ctx_list[i] if n_ctx_list is not None else 0
        qkv_dev = torch.from_numpy(qkv).cuda()
        call = A.SeqCall(qkv=qkv_dev.half() if f16_io else qkv_dev, slot=i, n_past=bound if n_past_on_device else P, n_ctx=n_ctx,
                         out=torch.zeros(1, desc.n_head * desc.head_dim, device="cuda",
                                         dtype=torch.float16 if f16_io else torch.float32),
                         q_roped=torch.zeros(1, desc.n_head, desc.head_dim, device="cuda"),
                         k_roped=torch.zeros(1, desc.n_kv_head, desc.head_dim, device="cuda"),
                         flags=A.SEQ_N_PAST_DEVICE if n_past_on_device else 0,
                         n_past_dev=n_past_dev[i:i + 1] if n_past_on_device else None)
        calls.append(call)
        host.append((qkv, k, v, n_ctx))
    A.forward_batch(arena, ws, calls, interleaved)
    torch.cuda.synchronize()
    assert ws.status() == 0
    cfg_g, cfg_f = oracle_cfg(desc, "ggml"), oracle_cfg(desc, "f32")
    for i, (P, call, (qkv, k, v, n_ctx)) in enumerate(zip(n_past_list, calls, host)):
        kg, vg = k.copy(), v.copy()
        want_g, qr, kr = O.attn_forward(cfg_g, qkv, interleaved, kg, vg, P, n_ctx=n_ctx or None, want_roped=True)
        kf, vf = k.copy(), v.copy()
        want_f = O.attn_forward(cfg_f, qkv, interleaved, kf, vf, P, n_ctx=n_ctx or None)
        got = call.out.float().cpu().numpy()
        if f16_io:   # the path's own output rounding: half an f16 ulp of the value
            assert np.abs(got - want_f).max() <= OUT_ATOL + 2.0 ** -11 * np.abs(want_f).max()
            want_f = want_f.astype(np.float16).astype(np.float32)
            want_g = want_g.astype(np.float16).astype(np.float32)
        assert_out_close(got, want_f, f"seq {i} n_past {P} vs f32 oracle")
        assert_out_close(got, want_g, f"seq {i} n_past {P} vs ggml-numerics oracle")
        gk, gv = download_cache(arena, i)
        np.testing.assert_array_equal(gk, kg, err_msg=f"k_cache seq {i} n_past {P}")   # bit-exact, canaries included
        np.testing.assert_array_equal(gv, vg, err_msg=f"v_cache seq {i} n_past {P}")
        if check_rope:
            uq = ulp_distance(call.q_roped.cpu().numpy()[0], qr[0]).max()
            uk = ulp_distance(call.k_roped.cpu().numpy()[0], kr[0]).max()
            assert uq <= ROPE_MAX_ULP and uk <= ROPE_MAX_ULP, f"rope seq {i}: q {uq} ulp, k {uk} ulp"
    arena.close()
