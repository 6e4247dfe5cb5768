"""GPU parity: the CUDA path through the C ABI against the CPU oracle and the committed golden vectors."""
import ctypes as C

import numpy as np
import pytest
import torch

from golden_util import GOLDEN_ATOL, MODEL_FIXTURES, load_fixture, model_output, steps
from gpu_util import (OUT_ATOL, ROPE_MAX_ULP, assert_out_close, download_cache, make_desc, oracle_cfg, qkv_width,
                      random_cache, run_decode_batch, ulp_distance, upload_cache)
from oracle import attn_oracle as O

pytestmark = pytest.mark.gpu


def _A():
    from chatglm_cpp_b200 import attention as A
    return A


@pytest.mark.parametrize("name", MODEL_FIXTURES)
def test_reference_fixture_through_cuda(name):
    """The reference's own golden vectors (prefill 3, decode, decode; chatglm_test.cpp:329-361), CUDA attention."""
    A = _A()
    z, meta, w = load_fixture(name)
    desc = make_desc(meta["n_head"], meta["n_kv_head"], meta["head_dim"], meta["max_length"] + meta["n_virtual"],
                     meta["n_virtual"], meta["rope_type"], meta["rope_theta"], meta["mask_type"])
    arena, ws = A.KVArena(desc, 1), A.Workspace(desc, 1, 8)
    attn = A.BasicAttention(arena, 0, ws, meta["interleaved_qkv"])
    cfg = oracle_cfg(desc)
    kc, vc = O.new_caches(cfg)
    if meta["n_virtual"]:
        arena.load_prefix(0, torch.from_numpy(z["prefix"]).cuda())
        O.load_prefix_cache(cfg, z["prefix"], kc, vc)
    for i, x, y, qkv, ctx_twin, n_past in steps(z):
        ctx, qr, kr = attn.forward(torch.from_numpy(qkv).cuda(), n_past, n_ctx=meta["n_ctx"], want_roped=True)
        torch.cuda.synchronize()
        ctx = ctx.cpu().numpy()
        want, oqr, okr = O.attn_forward(cfg, qkv, meta["interleaved_qkv"], kc, vc, n_past, n_ctx=meta["n_ctx"],
                                        want_roped=True)
        assert np.abs(model_output(meta, w, x, ctx) - y).max() < GOLDEN_ATOL, (name, i)
        assert_out_close(ctx, want, f"{name} step {i}")
        assert np.abs(ctx - ctx_twin).max() < OUT_ATOL
        assert ulp_distance(qr.cpu().numpy(), oqr).max() <= ROPE_MAX_ULP
        assert ulp_distance(kr.cpu().numpy(), okr).max() <= ROPE_MAX_ULP
    gk, gv = download_cache(arena, 0)
    np.testing.assert_array_equal(gk, kc)
    np.testing.assert_array_equal(gv, vc)
    np.testing.assert_array_equal(gk, z["k_cache_final"].view(np.uint16))
    assert ws.status() == 0


def test_config1_glm3_decode_n_past_512():
    """benchmark configuration 1: ChatGLM3-6B layer, one decode step at n_past 512, max_length 2048."""
    run_decode_batch(make_desc(32, 2, 128, 2048), [512], seed=1001)


@pytest.mark.parametrize("n_past", [0, 1, 15, 16, 17, 62, 63, 64, 65, 127, 128, 129, 1000, 2046, 2047])
def test_decode_tile_edges(n_past):
    """Attended lengths around the 16-token warp slice and the 64-token tile, up to a full cache."""
    run_decode_batch(make_desc(32, 2, 128, 2048), [n_past], seed=n_past)


@pytest.mark.parametrize("seed", range(12))
def test_decode_random_shapes_grid(seed):
    """A seeded grid over what the decode path's geometry depends on: kv heads, q heads per kv head (1 ... 16 on the fused
    kernel, 32 on the generic one), virtual tokens, capacity (also not a multiple of 8), batch size and lengths from an
    empty cache to a full one, rope mode and qkv layout.  Small launches (fewer tiles than SMs) and large ones."""
    rng = np.random.default_rng(7000 + seed)
    G = int(rng.choice([1, 2, 4, 8]))
    R = int(rng.choice([1, 2, 4, 8, 16, 32] if G <= 2 else [1, 2, 4]))
    V = int(rng.choice([0, 0, 3, 8]))
    v1 = R == 1                                         # the v1 family: MHA, interleaved qkv, 2-D rope, its own mask
    M = int(rng.choice([256, 517, 1024, 2048 + V])) if not v1 else 512
    n_seq = int(rng.choice([1, 2, 5, 17]))
    cap = M - V - 1
    n_past = [int(x) for x in rng.integers(0, cap + 1, n_seq)]
    n_past[0] = cap if seed % 2 else 0                 # a full cache, or an empty one
    desc = make_desc(G * R, G, 128, M, V=V, rope=O.ROPE_CHATGLM if v1 else O.ROPE_CHATGLM2,
                     mask=O.MASK_CHATGLM if v1 else O.MASK_CAUSAL, theta=10000.0 if seed % 2 else 5.0e6)
    n_ctx = [max(2, p // 2 + 1) for p in n_past] if v1 else None
    run_decode_batch(desc, n_past, seed=seed, interleaved=v1, n_ctx_list=n_ctx, f16_io=seed % 4 == 3)


def test_decode_batch_mixed_lengths_spans_and_merges():
    """64 sequences of uniformly random length: spans cross item boundaries, items are merged from partials."""
    rng = np.random.default_rng(1003)
    n_past = rng.integers(1024, 8192, 64).tolist()
    run_decode_batch(make_desc(32, 2, 128, 8192, theta=10000.0), n_past, seed=3, check_rope=False)


def test_decode_single_long_sequence_many_parts():
    """One long sequence: every CTA holds a part of the same two items."""
    run_decode_batch(make_desc(32, 2, 128, 32768 + 64, theta=5.0e6), [32768], seed=4)


def test_decode_small_batch_fewer_tiles_than_ctas():
    run_decode_batch(make_desc(32, 2, 128, 256), [3, 70, 130], seed=5)


def test_decode_mha_v1_2d_rope_interleaved():
    """benchmark configuration 5 shape: ChatGLM-6B v1, 32 heads with their own K/V, 2-D RoPE, interleaved qkv."""
    run_decode_batch(make_desc(32, 32, 128, 4096, rope=O.ROPE_CHATGLM, mask=O.MASK_CHATGLM), [2048, 2048, 5, 300],
                     seed=1005, interleaved=True, n_ctx_list=[17, 2000, 4, 300])


def test_decode_gqa_r4_and_rope_disabled():
    run_decode_batch(make_desc(8, 2, 128, 512), [100, 400], seed=6)
    run_decode_batch(make_desc(16, 1, 128, 512, rope=O.ROPE_DISABLED), [77], seed=7)


def test_decode_virtual_tokens_d128():
    """P-Tuning prefix on the fast path: cache capacity max_length + n_virtual stays a multiple of 8."""
    run_decode_batch(make_desc(32, 2, 128, 1024 + 8, V=8), [0, 5, 900], seed=8)


def test_decode_ptuning_capacity_not_a_multiple_of_8_stays_on_the_fused_kernel():
    """max_length + num_virtual_tokens = 1029: the arena lays its rows out with a pitch of 1032 tokens, the views keep
    the reference's extents, the calls are checked against 1029 (the last position fills the cache exactly), and the
    step is ONE fused launch, not the generic path's two."""
    from chatglm_cpp_b200 import _lib
    before = _lib.lib().cglm_launch_count()
    run_decode_batch(make_desc(32, 2, 128, 1029, V=5), [0, 700, 1023], seed=9)
    assert _lib.lib().cglm_launch_count() - before == 1
    A = _A()
    desc = make_desc(32, 2, 128, 1029, V=5)
    arena = A.KVArena(desc, 1)
    assert arena.pitch == 1032 and tuple(arena.v_cache(0).shape) == (2, 128, 1029) and arena.v_cache(0).stride(1) == 1032
    ws = A.Workspace(desc, 1, 1)
    call = A.SeqCall(qkv=torch.zeros(1, qkv_width(desc, False), device="cuda"), slot=0, n_past=1024,
                     out=torch.zeros(1, 32 * 128, device="cuda"))
    with pytest.raises(_lib.CglmError):          # position 1024 would be token 1030 of a cache of 1029
        A.forward_batch(arena, ws, [call], False)
    arena.close()


def test_decode_generic_shapes():
    """Shapes only the generic kernel covers: head_dim 64, 32 q heads per kv head, full-head rope modes."""
    run_decode_batch(make_desc(8, 2, 64, 256), [100], seed=10)
    run_decode_batch(make_desc(32, 1, 128, 256), [100], seed=11)
    run_decode_batch(make_desc(4, 4, 32, 128, rope=O.ROPE_GPTJ), [50], seed=12)
    run_decode_batch(make_desc(4, 2, 32, 128, rope=O.ROPE_NEOX, theta=50000.0), [50], seed=13)


def test_long_context_rope_position_131072():
    """benchmark configuration 4's position: RoPE at 131072 with theta 5e6 stays within 2 ulp of the oracle."""
    desc = make_desc(32, 2, 128, 131072 + 64, theta=5.0e6)
    A = _A()
    arena, ws = A.KVArena(desc, 1), A.Workspace(desc, 1, 1)
    rng = np.random.default_rng(1004)
    P = 131072
    # fill the cache on the device, read it back for the oracle
    arena.k_cache(0)[:, :P].copy_(torch.randn(2, P, 128, device="cuda").half())
    arena.v_cache(0)[:, :, :P].copy_(torch.randn(2, 128, P, device="cuda").half())
    k, v = download_cache(arena, 0)
    qkv = rng.standard_normal((1, qkv_width(desc, False))).astype(np.float32)
    attn = A.BasicAttention(arena, 0, ws)
    out, qr, kr = attn.forward(torch.from_numpy(qkv).cuda(), P, want_roped=True)
    torch.cuda.synchronize()
    assert ws.status() == 0
    k, v = k.copy(), v.copy()
    want, oqr, okr = O.attn_forward(oracle_cfg(desc, "f32"), qkv, False, k, v, P, want_roped=True)
    assert ulp_distance(qr.cpu().numpy(), oqr).max() <= ROPE_MAX_ULP
    assert ulp_distance(kr.cpu().numpy(), okr).max() <= ROPE_MAX_ULP
    assert_out_close(out.cpu().numpy(), want, "n_past 131072")
    gk, gv = download_cache(arena, 0)
    np.testing.assert_array_equal(gk[:, P], k[:, P])
    np.testing.assert_array_equal(gv[:, :, P], v[:, :, P])
    arena.close()


@pytest.mark.parametrize("H,G,D,M,V,rope,mask,S", [
    (32, 2, 128, 2048, 0, O.ROPE_CHATGLM2, O.MASK_CAUSAL, 37),
    (8, 8, 128, 256, 0, O.ROPE_CHATGLM, O.MASK_CHATGLM, 19),
    (8, 2, 64, 128, 5, O.ROPE_CHATGLM2, O.MASK_CAUSAL, 16),
    (8, 8, 16, 77, 5, O.ROPE_CHATGLM, O.MASK_CHATGLM, 9),
])
def test_prefill_then_decode(H, G, D, M, V, rope, mask, S):
    """Prefill of S tokens at n_past 0 (both mask types, with and without a prefix), then two decode steps."""
    A = _A()
    desc = make_desc(H, G, D, M, V, rope, 10000.0, mask)
    inter = rope == O.ROPE_CHATGLM
    rng = np.random.default_rng(S)
    arena, ws = A.KVArena(desc, 1), A.Workspace(desc, 1, S)
    attn = A.BasicAttention(arena, 0, ws, inter)
    cfg = oracle_cfg(desc, "f32")
    k, v = random_cache(rng, desc, V)
    upload_cache(arena, 0, k, v)
    n_past = 0
    for qlen in (S, 1, 1):
        qkv = rng.standard_normal((qlen, qkv_width(desc, inter))).astype(np.float32)
        out, qr, kr = attn.forward(torch.from_numpy(qkv).cuda(), n_past, n_ctx=S, want_roped=True)
        torch.cuda.synchronize()
        want, oqr, okr = O.attn_forward(cfg, qkv, inter, k, v, n_past, n_ctx=S, want_roped=True)
        assert_out_close(out.cpu().numpy(), want, f"qlen {qlen} n_past {n_past}")
        assert ulp_distance(qr.cpu().numpy(), oqr).max() <= ROPE_MAX_ULP
        assert ulp_distance(kr.cpu().numpy(), okr).max() <= ROPE_MAX_ULP
        n_past += qlen
    gk, gv = download_cache(arena, 0)
    np.testing.assert_array_equal(gk, k)
    np.testing.assert_array_equal(gv, v)
    assert ws.status() == 0


@pytest.mark.parametrize("H,G,M,V,rope,mask,S", [
    (32, 2, 2048, 0, O.ROPE_CHATGLM2, O.MASK_CAUSAL, 1024),   # benchmark configuration 2
    (32, 2, 2048, 0, O.ROPE_CHATGLM2, O.MASK_CAUSAL, 128),
    (8, 2, 512, 0, O.ROPE_CHATGLM2, O.MASK_CAUSAL, 129),
    (8, 2, 512 + 8, 8, O.ROPE_CHATGLM2, O.MASK_CAUSAL, 300),  # P-Tuning prefix in front of the prompt
    (8, 2, 512 + 5, 5, O.ROPE_CHATGLM2, O.MASK_CAUSAL, 300),  # the same with a capacity that is not a multiple of 8
    (8, 8, 512, 0, O.ROPE_CHATGLM, O.MASK_CHATGLM, 200),      # v1: MHA, interleaved qkv, 2-D rope, prefix mask
    (4, 1, 264, 0, O.ROPE_DISABLED, O.MASK_CAUSAL, 256),
])
def test_prefill_tensor_core_path(H, G, M, V, rope, mask, S):
    """Prompts of >= 128 tokens at head_dim 128 take the tcgen05 kernel: parity of output, RoPE and cache, then a
    decode step on top of the cache it wrote."""
    A = _A()
    desc = make_desc(H, G, 128, M, V, rope, 10000.0, mask)
    inter = rope == O.ROPE_CHATGLM
    rng = np.random.default_rng(S + H)
    arena, ws = A.KVArena(desc, 1), A.Workspace(desc, 1, S)
    attn = A.BasicAttention(arena, 0, ws, inter)
    cfg = oracle_cfg(desc, "f32")
    k, v = random_cache(rng, desc, V)
    upload_cache(arena, 0, k, v)
    n_past = 0
    launches = []
    from chatglm_cpp_b200 import _lib
    for qlen in (S, 1):
        qkv = rng.standard_normal((qlen, qkv_width(desc, inter))).astype(np.float32)
        before = _lib.lib().cglm_launch_count()
        out, qr, kr = attn.forward(torch.from_numpy(qkv).cuda(), n_past, n_ctx=S, want_roped=True)
        torch.cuda.synchronize()
        launches.append(_lib.lib().cglm_launch_count() - before)
        assert ws.status() == 0
        want, oqr, okr = O.attn_forward(cfg, qkv, inter, k, v, n_past, n_ctx=S, want_roped=True)
        assert_out_close(out.cpu().numpy(), want, f"qlen {qlen} n_past {n_past}")
        assert ulp_distance(qr.cpu().numpy(), oqr).max() <= ROPE_MAX_ULP
        assert ulp_distance(kr.cpu().numpy(), okr).max() <= ROPE_MAX_ULP
        n_past += qlen
    gk, gv = download_cache(arena, 0)
    np.testing.assert_array_equal(gk, k)
    np.testing.assert_array_equal(gv, v)
    # prepare + tcgen05 attention (angles come from the arena's table), then one fused decode launch
    assert launches == [2, 1]
    arena.close()


def test_prefill_explicit_position_ids_take_their_own_angle_table():
    """Prefill with caller-supplied position ids (which need not lie inside the cache capacity) builds a table for
    the call (one more launch) and must agree bit for bit with ids derived from the token index."""
    A = _A()
    from chatglm_cpp_b200 import _lib
    S = 200
    desc = make_desc(8, 2, 128, 256, rope=O.ROPE_CHATGLM2, mask=O.MASK_CAUSAL)
    rng = np.random.default_rng(77)
    arena, ws = A.KVArena(desc, 2), A.Workspace(desc, 1, S)
    qkv = torch.from_numpy(rng.standard_normal((S, qkv_width(desc, False))).astype(np.float32)).cuda()
    ids = torch.arange(S, dtype=torch.int32, device="cuda")
    outs, counts = [], []
    for slot, pid in ((0, None), (1, ids)):
        before = _lib.lib().cglm_launch_count()
        outs.append(A.BasicAttention(arena, slot, ws).forward(qkv, 0, position_ids=pid))
        torch.cuda.synchronize()
        counts.append(_lib.lib().cglm_launch_count() - before)
    assert ws.status() == 0
    assert counts == [2, 3]
    assert torch.equal(outs[0], outs[1])
    assert torch.equal(arena.k_cache(0), arena.k_cache(1))
    assert torch.equal(arena.v_cache(0), arena.v_cache(1))
    arena.close()


def test_explicit_position_ids_match_derived():
    A = _A()
    desc = make_desc(32, 32, 128, 512, rope=O.ROPE_CHATGLM, mask=O.MASK_CHATGLM)
    rng = np.random.default_rng(21)
    arena, ws = A.KVArena(desc, 2), A.Workspace(desc, 2, 1)
    k, v = random_cache(rng, desc, 200)
    upload_cache(arena, 0, k, v)
    upload_cache(arena, 1, k, v)
    qkv = torch.from_numpy(rng.standard_normal((1, qkv_width(desc, True))).astype(np.float32)).cuda()
    ids = torch.tensor([48, 152], dtype=torch.int32, device="cuda")   # n_past 200, n_ctx 50 -> pos 48, block 152
    outs = [torch.zeros(1, 4096, device="cuda") for _ in range(2)]
    A.forward_batch(arena, ws, [A.SeqCall(qkv=qkv, slot=0, n_past=200, n_ctx=50, out=outs[0]),
                                A.SeqCall(qkv=qkv, slot=1, n_past=200, n_ctx=0, out=outs[1], position_ids=ids)], True)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])
    assert torch.equal(arena.k_cache(0), arena.k_cache(1))


def test_fused_splitkv_step_four_ranks_on_one_device():
    """cglm_attn_splitkv_step: attention over a slice, publication of the (acc, m, l) rows into every rank's exchange
    buffer and the log-sum-exp combine in ONE launch per rank.  Four ranks on one device: four exchange buffers, four
    arena slots holding contiguous slices of one sequence.  Ranks 0..2 only publish and rank 3, launched last, combines,
    so that no kernel waits for a later launch.  Two steps (both sets of the buffers; the owner of position n_past
    appends), checked against the one-pass oracle.  Then a step with a silent rank: the bounded wait runs out, the
    status says so, `out` stays untouched and the context stays usable.  Then the silent rank comes back one step
    late: its stale step number is not taken for the current one."""
    from chatglm_cpp_b200 import _lib, sharding
    A = _A()
    n_rank, H, G, D = 4, 32, 2, 128
    P0 = 4096 + 37
    cap = sharding.slice_capacity(P0 + 4, 0, n_rank) + 64
    full = make_desc(H, G, D, 8192, theta=5.0e6)
    local = make_desc(H, G, D, cap, theta=5.0e6)
    rng = np.random.default_rng(1004)
    k, v = random_cache(rng, full, P0)
    arena, ws = A.KVArena(local, n_rank), A.Workspace(local, 1, 1)
    for r in range(n_rank):
        sl = sharding.split_kv(P0, 0, n_rank, r)
        kl = np.zeros((G, cap, D), np.uint16); vl = np.zeros((G, D, cap), np.uint16)
        kl[:, :sl.n_local] = k[:, sl.begin:sl.begin + sl.n_local]
        vl[:, :, :sl.n_local] = v[:, :, sl.begin:sl.begin + sl.n_local]
        upload_cache(arena, r, kl, vl)
    bufs = [A.SplitKVExchange.new_buffer(n_rank, H, D) for _ in range(n_rank)]
    ranks = [A.SplitKVExchange(bufs, r, H, D) for r in range(n_rank)]
    cfg = oracle_cfg(full, "f32")

    def launch(r, P, qkv_d, out, combine, timeout_us=0):
        sl = sharding.split_kv(P, 0, n_rank, r)
        arr = (_lib.AttnSeq * 1)()
        flags = A.SEQ_USE_KV_LOCAL | (0 if sl.owns_new else A.SEQ_NO_APPEND)
        A.fill_seq(arr[0], local, A.SeqCall(qkv=qkv_d, slot=r, n_past=P, kv_local=sl.n_local, flags=flags), False)
        ranks[r].step(arena, ws, arr, out, combine=combine, timeout_us=timeout_us)
        return sl

    before = _lib.lib().cglm_launch_count()
    P = P0
    for step in range(2):
        qkv = rng.standard_normal((1, qkv_width(full, False))).astype(np.float32)
        qkv_d = torch.from_numpy(qkv).cuda()
        want = O.attn_forward(cfg, qkv, False, k, v, P)          # appends position P to k, v
        out = torch.zeros(H * D, device="cuda")
        owner = None
        for r in range(n_rank):
            sl = launch(r, P, qkv_d, out if r == n_rank - 1 else None, combine=(r == n_rank - 1))
            if sl.owns_new:
                owner = (r, sl)
        torch.cuda.synchronize()
        assert ws.status() == 0
        assert_out_close(out.cpu().numpy().reshape(1, -1), want, f"fused split-KV step {step}")
        r_own, sl = owner
        gk, gv = download_cache(arena, r_own)
        np.testing.assert_array_equal(gk[:, P - sl.begin], k[:, P])
        np.testing.assert_array_equal(gv[:, :, P - sl.begin], v[:, :, P])
        P += 1
    assert _lib.lib().cglm_launch_count() - before == 2 * n_rank      # one launch per rank and step
    for b in bufs:
        assert int(b[0]) == 2                                        # every rank has finished step 2
    words = ranks[3].read_words(32 + 2 * 16 * 32)                    # the diagnostics view: step counter, arrival words
    assert int(words[0]) == 2
    assert all(int(words[32 + (0 * 16 + r) * 32 + g]) == 2 for r in range(n_rank) for g in range(G))   # set 0 holds step 2
    assert all(int(words[32 + (1 * 16 + r) * 32 + g]) == 1 for r in range(n_rank) for g in range(G))   # set 1 holds step 1
    # rank 1 stays silent: rank 3 gives up after 2 ms
    out = torch.full((H * D,), 7.0, device="cuda")
    for r in (0, 2):
        launch(r, P, qkv_d, None, combine=False)
    launch(3, P, qkv_d, out, combine=True, timeout_us=2000)
    torch.cuda.synchronize()
    assert ws.status() == _lib.ERR_TIMEOUT
    assert ws.status() == 0                      # reading the status clears it
    assert torch.all(out == 7.0)                 # out untouched
    assert float(torch.ones(4, device="cuda").sum()) == 4.0   # the context still works
    # rank 1 comes back: it publishes step 3 while the others are at step 4; the stale number must not be accepted
    for r in (0, 1, 2):
        launch(r, P, qkv_d, None, combine=False)
    launch(3, P, qkv_d, out, combine=True, timeout_us=2000)
    torch.cuda.synchronize()
    assert [int(b[0]) for b in bufs] == [4, 3, 4, 4]
    assert ws.status() == _lib.ERR_TIMEOUT
    assert torch.all(out == 7.0)
    arena.close()


def test_fused_splitkv_step_single_rank_equals_plain_decode():
    """One rank: the step degenerates to decode + normalisation and must agree with cglm_attn_forward; a sequence short
    enough that one thread block holds a whole kv head takes the other publication path."""
    from chatglm_cpp_b200 import _lib
    A = _A()
    for n_past in (40, 3000):
        desc = make_desc(32, 2, 128, 4096)
        rng = np.random.default_rng(n_past)
        arena, ws = A.KVArena(desc, 2), A.Workspace(desc, 1, 1)
        k, v = random_cache(rng, desc, n_past)
        upload_cache(arena, 0, k, v)
        upload_cache(arena, 1, k, v)
        qkv = torch.from_numpy(rng.standard_normal((1, qkv_width(desc, False))).astype(np.float32)).cuda()
        ref = torch.zeros(1, 4096, device="cuda")
        A.forward_batch(arena, ws, [A.SeqCall(qkv=qkv, slot=0, n_past=n_past, out=ref)])
        x = A.SplitKVExchange([A.SplitKVExchange.new_buffer(1, 32, 128)], 0, 32, 128)
        arr = (_lib.AttnSeq * 1)()
        A.fill_seq(arr[0], desc, A.SeqCall(qkv=qkv, slot=1, n_past=n_past), False)
        out = torch.zeros(4096, device="cuda")
        for _ in range(3):                       # the same step three times: both buffer sets, the same result
            out.zero_()
            x.step(arena, ws, arr, out)
            torch.cuda.synchronize()
            assert ws.status() == 0
            assert_out_close(out.cpu().numpy().reshape(1, -1), ref.cpu().numpy(), f"n_past {n_past}")
        assert torch.equal(arena.k_cache(0), arena.k_cache(1)) and torch.equal(arena.v_cache(0), arena.v_cache(1))
        arena.close()


def test_splitkv_partials_combine_to_full_attention():
    """A long sequence cut into 4 contiguous KV slices held in 4 slots: partials + LSE combine == one-pass result."""
    A = _A()
    P, n_rank = 4096 + 37, 4
    chunk = (P + 1 + n_rank - 1) // n_rank
    M_local = (chunk + 63) // 64 * 64 + 64
    full = make_desc(32, 2, 128, 8192, theta=5.0e6)
    local = make_desc(32, 2, 128, M_local, theta=5.0e6)
    rng = np.random.default_rng(1004)
    k, v = random_cache(rng, full, P)
    qkv = rng.standard_normal((1, qkv_width(full, False))).astype(np.float32)
    kf, vf = k.copy(), v.copy()
    want = O.attn_forward(oracle_cfg(full, "f32"), qkv, False, kf, vf, P)
    arena, ws = A.KVArena(local, n_rank), A.Workspace(local, n_rank, 1)
    partials = torch.zeros(n_rank, 32, 130, device="cuda")
    qkv_d = torch.from_numpy(qkv).cuda()
    calls = []
    for r in range(n_rank):
        lo, hi = r * chunk, min((r + 1) * chunk, P + 1)
        owns_new = lo <= P < hi
        n_local = (min(hi, P) - lo)
        kl = np.zeros((2, M_local, 128), np.uint16); vl = np.zeros((2, 128, M_local), np.uint16)
        kl[:, :n_local] = k[:, lo:lo + n_local]; vl[:, :, :n_local] = v[:, :, lo:lo + n_local]
        upload_cache(arena, r, kl, vl)
        flags = A.SEQ_PARTIAL | A.SEQ_USE_KV_LOCAL | (0 if owns_new else A.SEQ_NO_APPEND)
        calls.append(A.SeqCall(qkv=qkv_d, slot=r, n_past=P, partial=partials[r], kv_local=n_local, flags=flags))
    A.forward_batch(arena, ws, calls)
    out = A.splitkv_combine(partials)
    torch.cuda.synchronize()
    assert ws.status() == 0
    assert_out_close(out.cpu().numpy().reshape(1, -1), want, "split-KV combine")
    # the owner of position P appended it at its local index
    r_own = P // chunk
    gk, gv = download_cache(arena, r_own)
    np.testing.assert_array_equal(gk[:, P - r_own * chunk], kf[:, P])
    np.testing.assert_array_equal(gv[:, :, P - r_own * chunk], vf[:, :, P])


@pytest.mark.parametrize("pinned", [True, False])
def test_forward_host_roundtrip_matches_device_call(pinned):
    """Host-buffer call against the plain device call, from pinned host buffers (asynchronous copies, the decode launch
    gated by the device word behind its input copy) and from pageable ones."""
    from chatglm_cpp_b200 import _lib
    A = _A()
    desc = make_desc(32, 2, 128, 1024)
    rng = np.random.default_rng(31)
    n, n_past = 3, [10, 500, 1023]
    arena, ws = A.KVArena(desc, 2 * n), A.Workspace(desc, n, 1)
    qkv = rng.standard_normal((n, qkv_width(desc, False))).astype(np.float32)
    outs = []
    for i, P in enumerate(n_past):
        k, v = random_cache(rng, desc, P)
        upload_cache(arena, i, k, v)
        upload_cache(arena, n + i, k, v)
    calls = [A.SeqCall(qkv=torch.from_numpy(qkv[i:i + 1]).cuda(), slot=i, n_past=P, out=torch.zeros(1, 4096, device="cuda"))
             for i, P in enumerate(n_past)]
    A.forward_batch(arena, ws, calls)
    qkv_pinned = torch.from_numpy(qkv).pin_memory() if pinned else torch.from_numpy(qkv.copy())
    out_pinned = torch.zeros(n, 4096).pin_memory() if pinned else torch.zeros(n, 4096)
    dev_qkv, dev_out = torch.empty(n, qkv.shape[1], device="cuda"), torch.empty(n, 4096, device="cuda")
    arr = (_lib.AttnSeq * n)()
    for i, P in enumerate(n_past):
        arr[i].slot, arr[i].qlen, arr[i].n_past = n + i, 1, P
    _lib.check(_lib.lib().cglm_attn_forward_host(arena._h, arr, n, 0, qkv_pinned.data_ptr(), out_pinned.data_ptr(),
                                                 dev_qkv.data_ptr(), dev_out.data_ptr(), ws.ptr, ws.bytes,
                                                 torch.cuda.current_stream().cuda_stream), "forward_host")
    _lib.check(_lib.lib().cglm_attn_host_drain(arena._h, torch.cuda.current_stream().cuda_stream), "host_drain")
    torch.cuda.current_stream().synchronize()
    for i in range(n):
        assert torch.equal(out_pinned[i], calls[i].out[0].cpu())
        assert torch.equal(arena.k_cache(i), arena.k_cache(n + i))
        assert torch.equal(arena.v_cache(i), arena.v_cache(n + i))


def test_forward_host_drain_on_another_stream_and_uninitialised_workspace():
    """The drain may be enqueued on a stream other than the one the host-buffer calls ran on: that stream then waits for
    the calls' device-to-host copies.  And a workspace that never went through cglm_attn_workspace_init is reported by
    the status query."""
    from chatglm_cpp_b200 import _lib
    A = _A()
    L = _lib.lib()
    desc = make_desc(32, 2, 128, 1024)
    rng = np.random.default_rng(32)
    n, n_past = 4, [900, 1000, 1023, 700]
    arena, ws = A.KVArena(desc, 2 * n), A.Workspace(desc, n, 1)
    qkv = rng.standard_normal((n, qkv_width(desc, False))).astype(np.float32)
    for i, P in enumerate(n_past):
        k, v = random_cache(rng, desc, P)
        upload_cache(arena, i, k, v)
        upload_cache(arena, n + i, k, v)
    calls = [A.SeqCall(qkv=torch.from_numpy(qkv[i:i + 1]).cuda(), slot=i, n_past=P, out=torch.zeros(1, 4096, device="cuda"))
             for i, P in enumerate(n_past)]
    A.forward_batch(arena, ws, calls)
    torch.cuda.synchronize()
    qkv_pinned, out_pinned = torch.from_numpy(qkv).pin_memory(), torch.zeros(n, 4096).pin_memory()
    dev_qkv, dev_out = torch.empty(n, qkv.shape[1], device="cuda"), torch.empty(n, 4096, device="cuda")
    arr = (_lib.AttnSeq * n)()
    for i, P in enumerate(n_past):
        arr[i].slot, arr[i].qlen, arr[i].n_past = n + i, 1, P
    work, other = torch.cuda.Stream(), torch.cuda.Stream()
    _lib.check(L.cglm_attn_forward_host(arena._h, arr, n, 0, qkv_pinned.data_ptr(), out_pinned.data_ptr(), dev_qkv.data_ptr(),
                                        dev_out.data_ptr(), ws.ptr, ws.bytes, work.cuda_stream), "forward_host")
    _lib.check(L.cglm_attn_host_drain(arena._h, other.cuda_stream), "host_drain")
    other.synchronize()                       # only the OTHER stream is waited for
    for i in range(n):
        assert torch.equal(out_pinned[i], calls[i].out[0].cpu())
    torch.cuda.synchronize()
    raw = torch.zeros(ws.bytes, dtype=torch.uint8, device="cuda")          # never initialised
    assert L.cglm_attn_workspace_status(raw.data_ptr(), None) == _lib.ERR_WORKSPACE
    arena.close()


def test_forward_host_pipeline_reuses_staging_buffers():
    """Six host-buffer calls in a row over two staging pairs (copies overlap neighbouring kernels): every call's
    output must equal the plain device call's, i.e. the reuse of a staging buffer is ordered correctly."""
    from chatglm_cpp_b200 import _lib
    A = _A()
    desc = make_desc(32, 2, 128, 2048)
    rng = np.random.default_rng(41)
    n_layers, n = 6, 8          # 8 x 18 KiB of activations per call
    n_past = [1500, 20, 700, 2047, 64, 1, 1023, 333]
    arena, ws = A.KVArena(desc, 2 * n_layers * n), A.Workspace(desc, n, 1)
    arena.k_all().normal_(); arena.v_all().normal_()
    half = n_layers * n
    arena.k_all()[half:].copy_(arena.k_all()[:half]); arena.v_all()[half:].copy_(arena.v_all()[:half])
    width = qkv_width(desc, False)
    qkv = torch.from_numpy(rng.standard_normal((n_layers, n, width)).astype(np.float32))
    qkv_pinned, out_pinned = qkv.pin_memory(), torch.zeros(n_layers, n, 4096).pin_memory()
    qkv_dev = qkv.cuda()
    out_ref = torch.zeros(n_layers, n, 4096, device="cuda")
    stage_in = [torch.empty(n, width, device="cuda") for _ in range(2)]
    stage_out = [torch.empty(n, 4096, device="cuda") for _ in range(2)]
    stream = torch.cuda.current_stream().cuda_stream
    for l in range(n_layers):
        A.forward_batch(arena, ws, [A.SeqCall(qkv=qkv_dev[l, i:i + 1], slot=l * n + i, n_past=n_past[i], out=out_ref[l, i:i + 1])
                                    for i in range(n)])
    for l in range(n_layers):
        arr = (_lib.AttnSeq * n)()
        for i in range(n):
            arr[i].slot, arr[i].qlen, arr[i].n_past = half + l * n + i, 1, n_past[i]
        _lib.check(_lib.lib().cglm_attn_forward_host(arena._h, arr, n, 0, qkv_pinned[l].data_ptr(), out_pinned[l].data_ptr(),
                                                     stage_in[l % 2].data_ptr(), stage_out[l % 2].data_ptr(), ws.ptr, ws.bytes,
                                                     stream), "forward_host")
    _lib.check(_lib.lib().cglm_attn_host_drain(arena._h, stream), "host_drain")
    torch.cuda.current_stream().synchronize()
    assert ws.status() == 0
    assert torch.equal(out_pinned, out_ref.cpu())
    assert torch.equal(arena.k_all()[:half], arena.k_all()[half:])


def test_forward_host_gates_with_one_staging_pair_two_launches_per_call_and_a_prompt_in_between():
    """Host-buffer calls of 130 sequences (two fused launches per call, both behind the same gate words) through ONE
    staging pair, so that every call has to find its input staged and the previous call's output copied back; the third
    call carries a prompt, which is served by kernels that wait on the stream instead.  Outputs and caches must equal the
    plain device calls'."""
    from chatglm_cpp_b200 import _lib
    A = _A()
    L = _lib.lib()
    desc = make_desc(32, 2, 128, 256)
    rng = np.random.default_rng(43)
    n_calls, n = 6, 130
    n_past = [int(x) for x in rng.integers(0, 255, n)]
    arena, ws = A.KVArena(desc, 2 * n), A.Workspace(desc, n, 64)
    arena.k_all().normal_(); arena.v_all().normal_()
    arena.k_all()[n:].copy_(arena.k_all()[:n]); arena.v_all()[n:].copy_(arena.v_all()[:n])
    width = qkv_width(desc, False)
    stream = torch.cuda.current_stream().cuda_stream
    stage_in, stage_out = torch.empty(n + 64, width, device="cuda"), torch.empty(n + 64, 4096, device="cuda")
    outs_host, outs_ref = [], []
    for c in range(n_calls):
        prompt = c == 2
        qlens = [40 if (prompt and i == 0) else 1 for i in range(n)]
        past = [0 if (prompt and i == 0) else n_past[i] for i in range(n)]
        tok = sum(qlens)
        qkv = torch.from_numpy(rng.standard_normal((tok, width)).astype(np.float32))
        qkv_pinned, out_pinned = qkv.pin_memory(), torch.zeros(tok, 4096).pin_memory()
        qkv_dev, out_ref = qkv.cuda(), torch.zeros(tok, 4096, device="cuda")
        calls, t0 = [], 0
        for i in range(n):
            calls.append(A.SeqCall(qkv=qkv_dev[t0:t0 + qlens[i]], slot=i, n_past=past[i], out=out_ref[t0:t0 + qlens[i]]))
            t0 += qlens[i]
        A.forward_batch(arena, ws, calls)
        arr = (_lib.AttnSeq * n)()
        for i in range(n):
            arr[i].slot, arr[i].qlen, arr[i].n_past = n + i, qlens[i], past[i]
        _lib.check(L.cglm_attn_forward_host(arena._h, arr, n, 0, qkv_pinned.data_ptr(), out_pinned.data_ptr(), stage_in.data_ptr(),
                                            stage_out.data_ptr(), ws.ptr, ws.bytes, stream), "forward_host")
        outs_host.append((qkv_pinned, out_pinned)); outs_ref.append(out_ref)
        if prompt:
            n_past[0] = 40
    _lib.check(L.cglm_attn_host_drain(arena._h, stream), "host_drain")
    torch.cuda.current_stream().synchronize()
    assert ws.status() == 0
    for (_, got), want in zip(outs_host, outs_ref):
        assert torch.equal(got, want.cpu())
    assert torch.equal(arena.k_all()[:n], arena.k_all()[n:]) and torch.equal(arena.v_all()[:n], arena.v_all()[n:])
    arena.close()


def test_decode_with_4_byte_aligned_activation_takes_the_generic_path_and_agrees():
    """The fused decode kernel reads q/k/v rows 16 bytes at a time; an activation that is only 4-byte aligned must be
    routed to the generic CUDA path (same launch count as any generic call) and give the same output and cache."""
    from chatglm_cpp_b200 import _lib
    A = _A()
    desc = make_desc(32, 2, 128, 512)
    rng = np.random.default_rng(314)
    arena, ws = A.KVArena(desc, 2), A.Workspace(desc, 1, 1)
    k, v = random_cache(rng, desc, 300)
    upload_cache(arena, 0, k, v)
    upload_cache(arena, 1, k, v)
    width = qkv_width(desc, False)
    flat = torch.from_numpy(rng.standard_normal(width + 1).astype(np.float32)).cuda()
    aligned = flat[:width].clone().view(1, width)          # 16-byte aligned copy of the same numbers
    shifted = torch.empty(width + 1, device="cuda")
    shifted[1:] = flat[:width]
    shifted = shifted[1:].view(1, width)                    # starts 4 bytes into the allocation
    assert aligned.data_ptr() % 16 == 0 and shifted.data_ptr() % 16 == 4
    outs, counts = [], []
    for slot, x in ((0, aligned), (1, shifted)):
        out = torch.zeros(1, 4096, device="cuda")
        before = _lib.lib().cglm_launch_count()
        A.forward_batch(arena, ws, [A.SeqCall(qkv=x, slot=slot, n_past=300, out=out)])
        torch.cuda.synchronize()
        counts.append(_lib.lib().cglm_launch_count() - before)
        outs.append(out)
    assert ws.status() == 0
    assert counts[0] == 1 and counts[1] == 2                # fused kernel; rope+append kernel and attend kernel
    assert_out_close(outs[1].cpu().numpy(), outs[0].cpu().numpy(), "generic vs fused decode")
    assert torch.equal(arena.k_cache(0), arena.k_cache(1))
    assert torch.equal(arena.v_cache(0), arena.v_cache(1))
    arena.close()


def test_f16_hand_off_decode_configs():
    """f16 activations in, f16 context out (the hand-off to f16 Linears either side of the path) on the decode shapes
    of benchmark configurations 1, 3 and 5 and on generic-path shapes: cache bits and RoPE as with f32 inputs of the same values."""
    run_decode_batch(make_desc(32, 2, 128, 2048), [512], seed=1001, f16_io=True)
    rng = np.random.default_rng(1003)
    run_decode_batch(make_desc(32, 2, 128, 8192), rng.integers(1024, 8192, 24).tolist(), seed=3, check_rope=False, f16_io=True)
    run_decode_batch(make_desc(32, 32, 128, 4096, rope=O.ROPE_CHATGLM, mask=O.MASK_CHATGLM), [2048, 300, 5],
                     seed=1005, interleaved=True, n_ctx_list=[17, 300, 4], f16_io=True)
    run_decode_batch(make_desc(8, 2, 64, 256), [100], seed=10, f16_io=True)
    run_decode_batch(make_desc(32, 2, 128, 1029, V=5), [0, 700], seed=9, f16_io=True)
    run_decode_batch(make_desc(32, 2, 128, 2048), [33, 1999], seed=12, n_past_on_device=True, f16_io=True)


@pytest.mark.parametrize("S,rope,mask,H,G", [(1024, O.ROPE_CHATGLM2, O.MASK_CAUSAL, 32, 2), (200, O.ROPE_CHATGLM, O.MASK_CHATGLM, 8, 8),
                                             (37, O.ROPE_CHATGLM2, O.MASK_CAUSAL, 32, 2)])
def test_f16_hand_off_prefill(S, rope, mask, H, G):
    """benchmark configuration 2 (and a v1 prompt, and a prompt short enough for the generic path) with f16 in / f16 out."""
    A = _A()
    desc = make_desc(H, G, 128, 2048, 0, rope, 10000.0, mask)
    inter = rope == O.ROPE_CHATGLM
    rng = np.random.default_rng(S)
    arena, ws = A.KVArena(desc, 1), A.Workspace(desc, 1, S)
    attn = A.BasicAttention(arena, 0, ws, inter)
    k, v = random_cache(rng, desc, 0)
    upload_cache(arena, 0, k, v)
    qkv = rng.standard_normal((S, qkv_width(desc, inter))).astype(np.float16)
    out, qr, kr = attn.forward(torch.from_numpy(qkv).cuda(), 0, n_ctx=S, want_roped=True, out_dtype=torch.float16)
    torch.cuda.synchronize()
    assert ws.status() == 0 and out.dtype == torch.float16
    want, oqr, okr = O.attn_forward(oracle_cfg(desc, "f32"), qkv.astype(np.float32), inter, k, v, 0, n_ctx=S, want_roped=True)
    assert_out_close(out.float().cpu().numpy(), want.astype(np.float16).astype(np.float32), f"prefill {S} f16")
    assert ulp_distance(qr.cpu().numpy(), oqr).max() <= ROPE_MAX_ULP
    assert ulp_distance(kr.cpu().numpy(), okr).max() <= ROPE_MAX_ULP
    gk, gv = download_cache(arena, 0)
    np.testing.assert_array_equal(gk, k)
    np.testing.assert_array_equal(gv, v)
    arena.close()


@pytest.mark.parametrize("n", [3, 16])
def test_f16_hand_off_through_host_buffers(n):
    """cglm_attn_forward_host with CGLM_HOST_F16 (half the bytes across the bus) against the device call with f16
    tensors, for a small and a larger call."""
    from chatglm_cpp_b200 import _lib
    A = _A()
    desc = make_desc(32, 2, 128, 1024)
    rng = np.random.default_rng(n)
    n_past = [int(p) for p in rng.integers(1, 1023, n)]
    arena, ws = A.KVArena(desc, 2 * n), A.Workspace(desc, n, 1)
    for i, P in enumerate(n_past):
        k, v = random_cache(rng, desc, P)
        upload_cache(arena, i, k, v)
        upload_cache(arena, n + i, k, v)
    qkv = torch.from_numpy(rng.standard_normal((n, qkv_width(desc, False))).astype(np.float16))
    qkv_dev = qkv.cuda()
    ref = torch.zeros(n, 4096, device="cuda", dtype=torch.float16)
    A.forward_batch(arena, ws, [A.SeqCall(qkv=qkv_dev[i:i + 1], slot=i, n_past=P, out=ref[i:i + 1]) for i, P in enumerate(n_past)])
    qkv_pinned, out_pinned = qkv.pin_memory(), torch.zeros(n, 4096, dtype=torch.float16).pin_memory()
    dev_qkv, dev_out = torch.empty_like(qkv_dev), torch.empty_like(ref)
    arr = (_lib.AttnSeq * n)()
    for i, P in enumerate(n_past):
        arr[i].slot, arr[i].qlen, arr[i].n_past = n + i, 1, P
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(_lib.lib().cglm_attn_forward_host(arena._h, arr, n, _lib.HOST_F16, qkv_pinned.data_ptr(), out_pinned.data_ptr(),
                                                 dev_qkv.data_ptr(), dev_out.data_ptr(), ws.ptr, ws.bytes, stream), "forward_host")
    _lib.check(_lib.lib().cglm_attn_host_drain(arena._h, stream), "host_drain")
    torch.cuda.current_stream().synchronize()
    assert ws.status() == 0
    assert torch.equal(out_pinned, ref.cpu())
    for i in range(n):
        assert torch.equal(arena.k_cache(i), arena.k_cache(n + i)) and torch.equal(arena.v_cache(i), arena.v_cache(n + i))
    arena.close()


@pytest.mark.parametrize("n_seq,rope", [(1, O.ROPE_CHATGLM2), (9, O.ROPE_CHATGLM2), (64, O.ROPE_CHATGLM2), (128, O.ROPE_DISABLED)])
def test_fused_qkv_linear_feeds_the_decode_kernel(n_seq, rope):
    """cglm_qkv_linear_forward (tcgen05 GEMM of the layer input with the f16 query_key_value weight, bias, RoPE and the
    K/V append in its epilogue) followed by the attention call with CGLM_SEQ_Q_ROPED | CGLM_SEQ_NO_APPEND, against the
    oracle's Linear (chatglm.cpp:418-426) followed by its attention path.  The GEMM's f32 sums differ from the oracle's
    in the last bits (another summation order), so the appended f16 rows may differ by one f16 ulp in a few places."""
    from chatglm_cpp_b200 import _lib
    A = _A()
    L = _lib.lib()
    H, G, D, M, hidden = 32, 2, 128, 1024, 4096
    desc = make_desc(H, G, D, M, rope=rope)
    rng = np.random.default_rng(1000 + n_seq)
    n_past = [int(p) for p in rng.integers(0, M - 1, n_seq)]
    arena, ws = A.KVArena(desc, n_seq), A.Workspace(desc, n_seq, 1)
    host = []
    for i, P in enumerate(n_past):
        k, v = random_cache(rng, desc, P)
        upload_cache(arena, i, k, v)
        host.append((k, v))
    x = rng.standard_normal((n_seq, hidden)).astype(np.float16)
    w = (rng.standard_normal(((H + 2 * G) * D, hidden)) / np.sqrt(hidden)).astype(np.float16)
    bias = rng.standard_normal((H + 2 * G) * D).astype(np.float32)
    x_d, w_d, b_d = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), torch.from_numpy(bias).cuda()
    q_roped = torch.zeros(n_seq, H * D, device="cuda")
    out = torch.zeros(n_seq, H * D, device="cuda")
    arr = (_lib.AttnSeq * n_seq)()
    for i, P in enumerate(n_past):
        arr[i].slot, arr[i].qlen, arr[i].n_past = i, 1, P
    stream = torch.cuda.current_stream().cuda_stream
    before = L.cglm_launch_count()
    rc = L.cglm_qkv_linear_forward(arena._h, arr, n_seq, x_d.data_ptr(), hidden, w_d.data_ptr(), b_d.data_ptr(),
                                   q_roped.data_ptr(), ws.ptr, ws.bytes, stream)
    assert rc == 0, L.cglm_last_error_string()
    calls = [A.SeqCall(qkv=q_roped[i:i + 1], slot=i, n_past=P, out=out[i:i + 1], kv_local=P + 1,
                       flags=A.SEQ_NO_APPEND | A.SEQ_USE_KV_LOCAL | _lib.SEQ_Q_ROPED) for i, P in enumerate(n_past)]
    arr2 = (_lib.AttnSeq * n_seq)()
    for i, c in enumerate(calls):       # q only: k and v alias q and are not read
        base = c.qkv.data_ptr()
        arr2[i].q = arr2[i].k = arr2[i].v = base
        arr2[i].q_head_stride = arr2[i].kv_head_stride = D
        arr2[i].q_tok_stride = arr2[i].kv_tok_stride = H * D
        arr2[i].slot, arr2[i].qlen, arr2[i].n_past, arr2[i].kv_local = i, 1, c.n_past, c.kv_local
        arr2[i].flags, arr2[i].out = c.flags, c.out.data_ptr()
    _lib.check(L.cglm_attn_forward(arena._h, arr2, n_seq, ws.ptr, ws.bytes, stream), "cglm_attn_forward")
    torch.cuda.synchronize()
    assert ws.status() == 0
    assert L.cglm_launch_count() - before == 2          # the Linear and the decode kernel
    qkv = O.linear(x.astype(np.float32), w, bias)        # [n, (H + 2G) D] f32
    cfg = oracle_cfg(desc, "f32")
    n_bad = 0
    for i, P in enumerate(n_past):
        k, v = host[i]
        want, qr, kr = O.attn_forward(cfg, qkv[i:i + 1], False, k, v, P, want_roped=True)
        got_q = q_roped[i].cpu().numpy().reshape(H, D)
        assert np.abs(got_q - qr[0]).max() <= 2e-3, i
        gk, gv = download_cache(arena, i)
        for got, exp in ((gk[:, P], k[:, P]), (gv[:, :, P], v[:, :, P])):
            gf, ef = got.view(np.float16).astype(np.float32), exp.view(np.float16).astype(np.float32)
            assert np.abs(gf - ef).max() <= 4e-3, (i, float(np.abs(gf - ef).max()))   # a neighbouring f16 value at most
            n_bad += int((got != exp).sum())
        np.testing.assert_array_equal(np.delete(gk, P, axis=1), np.delete(k, P, axis=1))   # nothing else was touched
        np.testing.assert_array_equal(np.delete(gv, P, axis=2), np.delete(v, P, axis=2))
        assert_out_close(out[i:i + 1].cpu().numpy(), want, f"seq {i} n_past {P}")
    assert n_bad <= 0.02 * n_seq * 2 * G * D
    # shapes the fused Linear does not take are refused, not served by another path
    v1 = A.KVArena(make_desc(8, 8, 128, 256, rope=O.ROPE_CHATGLM, mask=O.MASK_CHATGLM), 1)
    assert L.cglm_qkv_linear_forward(v1._h, arr, 1, x_d.data_ptr(), hidden, w_d.data_ptr(), None, q_roped.data_ptr(),
                                     ws.ptr, ws.bytes, stream) == _lib.ERR_UNSUPPORTED
    arena.close()


@pytest.mark.parametrize("n_tok,n_in,n_out,use_bias,out_f16", [
    (1, 4096, 4096, True, False),       # dense of one decode token (chatglm.cpp:719)
    (64, 4096, 4096, False, True),
    (128, 256, 96, True, False),
    (200, 512, 160, True, True),        # two token tiles, the second ragged
    (300, 1024, 4608, True, True),      # query_key_value of a prompt: three token tiles, unsplit
    (200, 512, 3072, True, False),      # two token tiles, k split over two thread blocks per tile
    (129, 4096, 256, False, True),      # second token tile holds one token; k split over four
])
def test_linear_forward_matches_oracle(n_tok, n_in, n_out, use_bias, out_f16):
    """cglm_linear_forward (Linear::forward, chatglm.cpp:418-426, as a tcgen05 GEMM with f16 operands and f32 sums)
    against the oracle's Linear, which the reference's linear.data pins.  Tolerance: the two sum the same f32 products
    in another order (2e-4 on outputs of unit variance); an f16 output adds half an f16 ulp (2e-3 at |y| < 4)."""
    from chatglm_cpp_b200 import _lib
    A = _A()
    L = _lib.lib()
    rng = np.random.default_rng(n_tok * 7 + n_out)
    x = rng.standard_normal((n_tok, n_in)).astype(np.float16)
    w = (rng.standard_normal((n_out, n_in)) / np.sqrt(n_in)).astype(np.float16)
    bias = rng.standard_normal(n_out).astype(np.float32) if use_bias else None
    x_d, w_d = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    b_d = torch.from_numpy(bias).cuda() if use_bias else None
    # guard rows either side: the kernel must not write outside [n_tok][n_out]
    buf = torch.full((n_tok + 2, n_out), 7.0, device="cuda", dtype=torch.float16 if out_f16 else torch.float32)
    ws = A.Workspace(make_desc(32, 2, 128, 1024), 1, 1)
    stream = torch.cuda.current_stream().cuda_stream
    before = L.cglm_launch_count()
    rc = L.cglm_linear_forward(x_d.data_ptr(), n_tok, n_in, w_d.data_ptr(), n_out, b_d.data_ptr() if use_bias else None,
                               buf[1:].data_ptr(), int(out_f16), ws.ptr, ws.bytes, stream)
    assert rc == 0, L.cglm_last_error_string()
    torch.cuda.synchronize()
    assert ws.status() == 0
    assert L.cglm_launch_count() - before == 1
    want = O.linear(x.astype(np.float32), w, bias)
    got = buf[1:n_tok + 1].float().cpu().numpy()
    tol = 2e-4 + (2e-3 * np.maximum(1.0, np.abs(want) / 4) if out_f16 else 0.0)
    assert (np.abs(got - want) <= tol).all(), float(np.abs(got - want).max())
    assert (buf[0] == 7).all() and (buf[n_tok + 1] == 7).all()
    if use_bias:
        # a bias that is only 4-byte aligned (one kernel reads it four features at a time; the call must not hand it one)
        shifted = torch.cat([torch.zeros(1, device="cuda"), b_d])[1:]
        assert shifted.data_ptr() % 16 == 4
        buf.fill_(7.0)
        rc = L.cglm_linear_forward(x_d.data_ptr(), n_tok, n_in, w_d.data_ptr(), n_out, shifted.data_ptr(), buf[1:].data_ptr(),
                                   int(out_f16), ws.ptr, ws.bytes, stream)
        assert rc == 0, L.cglm_last_error_string()
        torch.cuda.synchronize()
        assert ws.status() == 0
        got = buf[1:n_tok + 1].float().cpu().numpy()
        assert (np.abs(got - want) <= tol).all(), float(np.abs(got - want).max())
    # refused, not served by another path
    assert L.cglm_linear_forward(x_d.data_ptr(), n_tok, n_in - 32, w_d.data_ptr(), n_out, None, buf[1:].data_ptr(),
                                 int(out_f16), ws.ptr, ws.bytes, stream) == _lib.ERR_UNSUPPORTED
    assert L.cglm_linear_forward(x_d.data_ptr(), n_tok, n_in, w_d.data_ptr(), n_out - 8, None, buf[1:].data_ptr(),
                                 int(out_f16), ws.ptr, ws.bytes, stream) == _lib.ERR_UNSUPPORTED


def test_convert_f32_to_f16_rounds_like_numpy():
    """cglm_convert_f32_to_f16 (the cast in front of an f16 Linear) against numpy's round-to-nearest-even cast, on a
    length that is not a multiple of 4 and at an address that is not 16-byte aligned."""
    from chatglm_cpp_b200 import _lib
    L = _lib.lib()
    rng = np.random.default_rng(77)
    x = np.concatenate([rng.standard_normal(5001).astype(np.float32) * 50,
                        np.array([0.0, -0.0, 65504.0, 1e-8, 6.1e-5, 1.00048828125], np.float32)])
    src = torch.from_numpy(np.concatenate([[0.0], x]).astype(np.float32)).cuda()
    dst = torch.zeros(x.size + 1, device="cuda", dtype=torch.float16)
    stream = torch.cuda.current_stream().cuda_stream
    assert L.cglm_convert_f32_to_f16(src[1:].data_ptr(), dst[1:].data_ptr(), x.size, stream) == 0
    torch.cuda.synchronize()
    np.testing.assert_array_equal(dst[1:].cpu().numpy().view(np.uint16), x.astype(np.float16).view(np.uint16))
    assert dst[0] == 0


def test_decode_with_settled_caches_streams_early_and_gives_the_same_bits():
    """CGLM_SEQ_CACHE_SETTLED lets a launch read cache tiles while the previous launch of the stream drains.  Eight
    layer calls back to back, each on its own slots, with and without the flag: same output bits, same caches, and
    parity with the oracle for the flagged run."""
    from chatglm_cpp_b200 import _lib
    A = _A()
    desc = make_desc(32, 2, 128, 4096)
    rng = np.random.default_rng(515)
    n_layer, n_past = 8, [4000, 130, 2500, 64, 3333, 1, 700, 2047, 1999, 3071]
    n = len(n_past)
    arena, ws = A.KVArena(desc, 2 * n_layer * n), A.Workspace(desc, n, 1)
    host = []
    for s in range(n_layer * n):
        k, v = random_cache(rng, desc, n_past[s % n])
        upload_cache(arena, s, k, v)
        upload_cache(arena, n_layer * n + s, k, v)
        host.append((k, v))
    width = qkv_width(desc, False)
    qkv_h = rng.standard_normal((n_layer, n, width)).astype(np.float32)
    qkv = torch.from_numpy(qkv_h).cuda()
    outs = [torch.zeros(n_layer, n, 4096, device="cuda") for _ in range(2)]
    torch.cuda.synchronize()
    for run, flags in enumerate((0, A.SEQ_CACHE_SETTLED)):
        for layer in range(n_layer):
            A.forward_batch(arena, ws, [A.SeqCall(qkv=qkv[layer, i:i + 1], slot=run * n_layer * n + layer * n + i,
                                                  n_past=n_past[i], out=outs[run][layer, i:i + 1], flags=flags)
                                        for i in range(n)])
        torch.cuda.synchronize()
        assert ws.status() == 0
    assert torch.equal(outs[0], outs[1])
    half = n_layer * n
    assert torch.equal(arena.k_all()[:half], arena.k_all()[half:])
    assert torch.equal(arena.v_all()[:half], arena.v_all()[half:])
    cfg = oracle_cfg(desc, "f32")
    for layer in (0, n_layer - 1):
        for i in range(n):
            k, v = host[layer * n + i]
            want = O.attn_forward(cfg, qkv_h[layer, i:i + 1], False, k, v, n_past[i])
            assert_out_close(outs[1][layer, i:i + 1].cpu().numpy(), want, f"layer {layer} seq {i}")
            gk, gv = download_cache(arena, half + layer * n + i)
            np.testing.assert_array_equal(gk, k)
            np.testing.assert_array_equal(gv, v)
    arena.close()


def test_decode_batch_with_device_side_positions_mixed_lengths():
    """The instantiation of the decode kernel that reads n_past from device words, on a batch whose spans cross item
    boundaries and whose grid (sized from the host's upper bounds) is larger than the real number of tiles needs."""
    desc = make_desc(32, 2, 128, 2048)
    rng = np.random.default_rng(4242)
    n_past = [int(x) for x in rng.integers(1, 2000, size=48)]
    run_decode_batch(desc, n_past, seed=17, n_past_on_device=True)
    v1 = make_desc(8, 8, 128, 512, rope=O.ROPE_CHATGLM, mask=O.MASK_CHATGLM)
    run_decode_batch(v1, [100, 257, 31], seed=18, interleaved=True, n_ctx_list=[40, 200, 10], n_past_on_device=True)


def test_decode_step_graph_with_device_side_position_replays_for_new_tokens():
    """The step loop of the reference (chatglm.cpp:726-755, 886-925) rebuilds its graph for every token.  Here the
    layer calls of one decode step (two layers, three sequences of different lengths) are captured ONCE in a CUDA
    graph with n_past read from device words, and replayed for four tokens; every replay must match the oracle run
    token by token, caches included."""
    from chatglm_cpp_b200 import _lib
    A = _A()
    H, G, D, M, n_layer = 32, 2, 128, 512, 2
    desc = make_desc(H, G, D, M)
    starts = [130, 63, 300]
    n = len(starts)
    rng = np.random.default_rng(99)
    arena, ws = A.KVArena(desc, n_layer * n), A.Workspace(desc, n, 1)
    cfg = oracle_cfg(desc, "f32")
    host = {}
    for layer in range(n_layer):
        for i, P in enumerate(starts):
            k, v = random_cache(rng, desc, P)
            upload_cache(arena, layer * n + i, k, v)
            host[(layer, i)] = (k, v)
    width = qkv_width(desc, False)
    qkv = torch.zeros(n_layer, n, width, device="cuda")                 # the graph's input buffers
    outs = torch.zeros(n_layer, n, H * D, device="cuda")
    n_past_dev = torch.tensor(starts, dtype=torch.int32, device="cuda")
    bound = max(starts) + 8                                              # host-side upper bound of the positions
    arrs = []
    for layer in range(n_layer):
        arr = (_lib.AttnSeq * n)()
        for i in range(n):
            A.fill_seq(arr[i], desc, A.SeqCall(qkv=qkv[layer, i:i + 1], slot=layer * n + i, n_past=bound,
                                               out=outs[layer, i:i + 1], flags=A.SEQ_N_PAST_DEVICE,
                                               n_past_dev=n_past_dev[i:i + 1]), False)
        arrs.append(arr)
    L = _lib.lib()

    def step():
        stream = torch.cuda.current_stream().cuda_stream
        for layer in range(n_layer):
            assert L.cglm_attn_forward(arena._h, arrs[layer], n, ws.ptr, ws.bytes, stream) == 0
        assert L.cglm_seq_advance(n_past_dev.data_ptr(), n, 1, stream) == 0

    side = torch.cuda.Stream()                  # one eager step first (token 0), as torch wants before a capture
    side.wait_stream(torch.cuda.current_stream())
    tokens = [rng.standard_normal((n_layer, n, width)).astype(np.float32) for _ in range(5)]
    results = []
    with torch.cuda.stream(side):
        qkv.copy_(torch.from_numpy(tokens[0]))
        step()
        results.append(outs.clone())
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()                                   # captured, not executed
    for t in range(1, 5):
        qkv.copy_(torch.from_numpy(tokens[t]))
        graph.replay()
        results.append(outs.clone())
    torch.cuda.synchronize()
    assert ws.status() == 0
    assert n_past_dev.cpu().tolist() == [p + 5 for p in starts]
    for t in range(5):
        for layer in range(n_layer):
            for i, P in enumerate(starts):
                k, v = host[(layer, i)]
                want = O.attn_forward(cfg, tokens[t][layer, i:i + 1], False, k, v, P + t)   # appends into k, v
                assert_out_close(results[t][layer, i:i + 1].cpu().numpy(), want, f"token {t} layer {layer} seq {i}")
    for layer in range(n_layer):
        for i in range(n):
            gk, gv = download_cache(arena, layer * n + i)
            np.testing.assert_array_equal(gk, host[(layer, i)][0])
            np.testing.assert_array_equal(gv, host[(layer, i)][1])
    # a position beyond the capacity is clamped and reported, never followed
    n_past_dev.fill_(M + 5)
    step()
    torch.cuda.synchronize()
    assert ws.status() == _lib.ERR_INVALID_ARG
    arena.close()


@pytest.mark.parametrize("H,G,D,M,V,rope,mask", [
    (32, 2, 128, 512, 0, O.ROPE_CHATGLM2, O.MASK_CAUSAL),
    (8, 8, 64, 200, 5, O.ROPE_CHATGLM, O.MASK_CHATGLM),
])
def test_chunked_prompt_second_chunk_attends_everything(H, G, D, M, V, rope, mask):
    """qlen > 1 with n_past > 0 (a prompt fed in two chunks): the reference builds no mask then (chatglm.cpp:689),
    so every row of the second chunk sees the whole cache including the chunk's later tokens.  Same here."""
    A = _A()
    desc = make_desc(H, G, D, M, V, rope, 10000.0, mask)
    inter = rope == O.ROPE_CHATGLM
    rng = np.random.default_rng(H + D)
    arena, ws = A.KVArena(desc, 1), A.Workspace(desc, 1, 64)
    attn = A.BasicAttention(arena, 0, ws, inter)
    cfg = oracle_cfg(desc, "f32")
    k, v = random_cache(rng, desc, V)
    upload_cache(arena, 0, k, v)
    n_past = 0
    for qlen in (40, 23, 1):
        qkv = rng.standard_normal((qlen, qkv_width(desc, inter))).astype(np.float32)
        out, qr, kr = attn.forward(torch.from_numpy(qkv).cuda(), n_past, n_ctx=63, want_roped=True)
        torch.cuda.synchronize()
        want, oqr, okr = O.attn_forward(cfg, qkv, inter, k, v, n_past, n_ctx=63, want_roped=True)
        assert_out_close(out.cpu().numpy(), want, f"qlen {qlen} n_past {n_past}")
        assert ulp_distance(qr.cpu().numpy(), oqr).max() <= ROPE_MAX_ULP
        assert ulp_distance(kr.cpu().numpy(), okr).max() <= ROPE_MAX_ULP
        n_past += qlen
    gk, gv = download_cache(arena, 0)
    np.testing.assert_array_equal(gk, k)
    np.testing.assert_array_equal(gv, v)
    assert ws.status() == 0


@pytest.mark.parametrize("with_table", [True, False])
def test_adopted_caches_behave_like_an_arena_of_the_librarys_own(with_table):
    """cglm_kv_arena_adopt: tensor maps (and optionally the angle table) over caller-owned cache memory.  Prefill on
    tensor cores, decode steps and a chunk on the generic path give the same bits as on an allocated arena, and the
    caller's tensors hold the caches."""
    from chatglm_cpp_b200 import _lib
    A = _A()
    desc = make_desc(32, 2, 128, 1024)
    n_slots = 3
    k_all = torch.zeros(n_slots, 2, 1024, 128, dtype=torch.float16, device="cuda")
    v_all = torch.zeros(n_slots, 2, 128, 1024, dtype=torch.float16, device="cuda")
    table = torch.empty(_lib.lib().cglm_kv_angle_table_bytes(C.byref(desc)), dtype=torch.uint8, device="cuda") if with_table else None
    own, mine = A.KVArena(desc, n_slots), A.KVArena(desc, n_slots, adopt=(k_all, v_all, table))
    ws = A.Workspace(desc, 2, 256)
    rng = np.random.default_rng(8)
    n_past = 0
    for qlen in (200, 1, 1, 5):
        qkv = torch.from_numpy(rng.standard_normal((qlen, qkv_width(desc, False))).astype(np.float32)).cuda()
        outs = [A.BasicAttention(arena, 1, ws).forward(qkv, n_past) for arena in (own, mine)]
        torch.cuda.synchronize()
        assert torch.equal(outs[0], outs[1]), (qlen, n_past)
        n_past += qlen
    assert ws.status() == 0
    assert torch.equal(own.k_all(), k_all) and torch.equal(own.v_all(), v_all)
    assert k_all[1, :, :n_past].abs().sum() > 0 and k_all[0].abs().sum() == 0 and k_all[2].abs().sum() == 0
    mine.close()
    assert k_all[1, :, :n_past].abs().sum() > 0          # the memory is still the caller's
    h = C.c_void_p()
    L = _lib.lib()
    assert L.cglm_kv_arena_adopt(C.byref(desc), n_slots, k_all.data_ptr() + 2, v_all.data_ptr(), None, C.byref(h)) == _lib.ERR_INVALID_ARG
    host = torch.zeros(16, dtype=torch.float16).pin_memory()
    assert L.cglm_kv_arena_adopt(C.byref(desc), 1, host.data_ptr(), v_all.data_ptr(), None, C.byref(h)) == _lib.ERR_INVALID_ARG


def test_second_device_in_one_process_gets_its_own_kernel_attributes():
    """One host process driving two GPUs: the opt-in to large dynamic shared memory is a per-device attribute of a
    kernel, so the first fused launch on each device must set it there.  Decode and tensor-core prefill on device 0,
    then the same on device 1, must agree bit for bit.  (Skipped on a one-GPU box.)"""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs in one process")
    from chatglm_cpp_b200 import _lib
    A = _A()
    desc = make_desc(32, 2, 128, 1024)
    rng = np.random.default_rng(2)
    qkv_p = rng.standard_normal((300, qkv_width(desc, False))).astype(np.float32)
    qkv_d = rng.standard_normal((1, qkv_width(desc, False))).astype(np.float32)
    results = []
    for dev in (0, 1):
        with torch.cuda.device(dev):
            arena, ws = A.KVArena(desc, 1), A.Workspace(desc, 1, 300)
            attn = A.BasicAttention(arena, 0, ws)
            o1 = attn.forward(torch.from_numpy(qkv_p).cuda(), 0)
            o2 = attn.forward(torch.from_numpy(qkv_d).cuda(), 300)
            torch.cuda.synchronize()
            assert ws.status() == 0
            results.append((o1.cpu(), o2.cpu(), arena.k_cache(0).cpu(), arena.v_cache(0).cpu()))
            # an arena of another device is refused by the call that carries its own scratch
            arr = (_lib.AttnSeq * 1)()
            A.fill_seq(arr[0], desc, A.SeqCall(qkv=torch.from_numpy(qkv_d).cuda(), slot=0, n_past=301,
                                               out=torch.zeros(1, 4096, device="cuda")), False)
            with torch.cuda.device(1 - dev):
                assert _lib.lib().cglm_attn_decode_static(arena._h, arr, 1, 1, None) == _lib.ERR_INVALID_ARG
            arena.close()
    for a, b in zip(*results):
        assert torch.equal(a, b)


def test_argument_errors_return_codes():
    from chatglm_cpp_b200 import _lib
    A = _A()
    L = _lib.lib()
    desc = make_desc(32, 2, 128, 256)
    arena, ws = A.KVArena(desc, 1), A.Workspace(desc, 1, 1)
    qkv = torch.zeros(1, qkv_width(desc, False), device="cuda")
    out = torch.zeros(1, 4096, device="cuda")
    with pytest.raises(_lib.CglmError) as e:   # n_past + 1 > capacity
        A.forward_batch(arena, ws, [A.SeqCall(qkv=qkv, slot=0, n_past=256, out=out)])
    assert e.value.status == _lib.ERR_INVALID_ARG
    with pytest.raises(_lib.CglmError):        # slot out of range
        A.forward_batch(arena, ws, [A.SeqCall(qkv=qkv, slot=1, n_past=0, out=out)])
    arr = (_lib.AttnSeq * 1)()
    A.fill_seq(arr[0], desc, A.SeqCall(qkv=qkv, slot=0, n_past=0, out=out), False)
    assert L.cglm_attn_forward(arena._h, arr, 1, ws.ptr, 1024, None) == _lib.ERR_WORKSPACE
    assert L.cglm_attn_forward(arena._h, arr, 1, None, 0, None) == _lib.ERR_WORKSPACE
    bad = make_desc(32, 3, 128, 256)
    h = C.c_void_p()
    assert L.cglm_kv_arena_create(C.byref(bad), 1, C.byref(h)) == _lib.ERR_INVALID_ARG
    assert ws.status() == 0
