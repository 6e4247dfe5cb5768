"""The decode entry point that carries its own scratch memory, against the regular one.

Some hosts cannot give the library a workspace when they call it (their allocator owns the whole GPU, or the
plugin interface forbids cudaMalloc), so cglm_attn_decode_static keeps the scratch of the split-sequence merge
in a fixed array inside the library.  This test drives both entry points through the C ABI with the same
inputs, twice in a row (the second call finds the array as the first one left it), and expects the same
outputs and the same cache contents.  It lives in a file that pytest collects last.
"""
import numpy as np
import pytest
import torch

from gpu_util import OUT_ATOL, make_desc, qkv_width, random_cache, upload_cache

pytestmark = pytest.mark.gpu


def test_static_scratch_decode_matches_workspace_decode_twice():
    from chatglm_cpp_b200 import _lib
    from chatglm_cpp_b200 import attention as A
    L = _lib.lib()
    desc = make_desc(32, 2, 128, 4096)
    rng = np.random.default_rng(77)
    # lengths long enough that every sequence is split across thread blocks: partial slots and counters are used
    n_past = [3000, 1500, 4000, 777, 2048, 63, 3500, 2600]
    n = len(n_past)
    arena = A.KVArena(desc, 2 * n)                 # slots [0, n): regular entry point, [n, 2n): static-scratch one
    ws = A.Workspace(desc, n, 1)
    for i, P in enumerate(n_past):
        k, v = random_cache(rng, desc, P)
        upload_cache(arena, i, k, v)
        upload_cache(arena, n + i, k, v)
    stream = torch.cuda.current_stream().cuda_stream
    for step in range(2):                          # two decode steps in a row: n_past, then n_past + 1
        qkv = torch.from_numpy(rng.standard_normal((n, qkv_width(desc, False))).astype(np.float32)).cuda()
        out_ref = torch.zeros(n, 4096, device="cuda")
        out_new = torch.full((n, 4096), float("nan"), device="cuda")
        ref_calls, arr = [], (_lib.AttnSeq * n)()
        for i, P in enumerate(n_past):
            ref_calls.append(A.SeqCall(qkv=qkv[i:i + 1], slot=i, n_past=P + step, out=out_ref[i:i + 1]))
            A.fill_seq(arr[i], desc, A.SeqCall(qkv=qkv[i:i + 1], slot=n + i, n_past=P + step, out=out_new[i:i + 1]), False)
        A.forward_batch(arena, ws, ref_calls)
        rc = L.cglm_attn_decode_static(arena._h, arr, n, 1, stream)   # waits and returns the device-side status
        assert rc == 0, L.cglm_status_string(rc)
        torch.cuda.synchronize()
        assert ws.status() == 0
        assert torch.isfinite(out_new).all()
        assert (out_new - out_ref).abs().max().item() <= OUT_ATOL
        assert torch.equal(out_new, out_ref)       # same kernel, same split: the bits agree as well
        for i in range(n):
            assert torch.equal(arena.k_cache(i), arena.k_cache(n + i))
            assert torch.equal(arena.v_cache(i), arena.v_cache(n + i))


def test_static_scratch_limits_are_refused():
    from chatglm_cpp_b200 import _lib
    from chatglm_cpp_b200 import attention as A
    L = _lib.lib()
    desc = make_desc(32, 2, 128, 256)
    arena = A.KVArena(desc, 1)
    n = 129                                        # one more sequence than the static scratch covers
    qkv = torch.zeros(1, qkv_width(desc, False), device="cuda")
    out = torch.zeros(1, 4096, device="cuda")
    arr = (_lib.AttnSeq * n)()
    for i in range(n):
        A.fill_seq(arr[i], desc, A.SeqCall(qkv=qkv, slot=0, n_past=1, out=out), False)
    assert L.cglm_attn_decode_static(arena._h, arr, n, 0, None) == _lib.ERR_WORKSPACE
    assert b"128 sequences" in L.cglm_last_error_string()
    # a slot outside the arena or a position beyond the cache capacity is refused by return code: nothing is launched
    before = L.cglm_launch_count()
    one = (_lib.AttnSeq * 1)()
    for slot, n_past in ((-1, 1), (1, 1), (0, 255), (0, 256), (0, 2**31 - 1)):
        A.fill_seq(one[0], desc, A.SeqCall(qkv=qkv, slot=slot, n_past=n_past, out=out), False)
        want = _lib.OK if (slot, n_past) == (0, 255) else _lib.ERR_INVALID_ARG
        assert L.cglm_attn_decode_static(arena._h, one, 1, 1, None) == want, (slot, n_past)
    assert L.cglm_launch_count() == before + 1
    # shapes outside the fused decode kernel are refused, not served by another path
    small = A.KVArena(make_desc(8, 2, 64, 256), 1)
    arr1 = (_lib.AttnSeq * 1)()
    A.fill_seq(arr1[0], small.desc, A.SeqCall(qkv=torch.zeros(1, 12 * 64, device="cuda"), slot=0, n_past=1,
                                              out=torch.zeros(1, 512, device="cuda")), False)
    assert L.cglm_attn_decode_static(small._h, arr1, 1, 0, None) == _lib.ERR_UNSUPPORTED
