"""CPU-only checks of the drop-in boundary: the built library loads and exports what the C headers under include/
declare."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = set()
    for header in ("cglm_attn.h", "cglm_model_file.h"):
        text = open(os.path.join(ROOT, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(cglm_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_header_symbols_are_exported_and_bound():
    from chatglm_cpp_b200 import _lib, build
    build.build()
    handle = C.CDLL(_lib.LIB_PATH)
    declared = _declared_symbols()
    assert len(declared) >= 15
    for name in declared:
        assert hasattr(handle, name), f"{name} declared under include/ but not exported"
        assert name in _lib.SYMBOLS, f"{name} has no ctypes binding"
    assert set(_lib.SYMBOLS) == set(declared)


def test_struct_layouts_match_header():
    from chatglm_cpp_b200 import _lib
    assert C.sizeof(_lib.AttnDesc) == 32
    # the same numbers are static_asserted against the C structs in csrc/cglm_attn_api.cu
    assert C.sizeof(_lib.AttnSeq) == 128
    assert _lib.AttnSeq.position_ids.offset == 72 and _lib.AttnSeq.partial.offset == 112


def test_host_only_entry_points_without_a_gpu():
    """Pure host functions answer without a device; compute entry points refuse politely."""
    from chatglm_cpp_b200 import _lib
    L = _lib.lib()
    d = _lib.AttnDesc(32, 2, 128, 2048, 0, _lib.ROPE_CHATGLM2, 10000.0, _lib.MASK_CAUSAL)
    assert L.cglm_kv_slot_bytes(C.byref(d)) == 4 * 2 * 2048 * 128
    assert L.cglm_attn_workspace_bytes(C.byref(d), 64, 1) > 0
    assert L.cglm_status_string(_lib.ERR_TIMEOUT) == b"device-side wait timed out"
    assert L.cglm_launch_count() == 0 or L.cglm_launch_count() > 0
    bad = _lib.AttnDesc(32, 5, 128, 2048, 0, _lib.ROPE_CHATGLM2, 10000.0, _lib.MASK_CAUSAL)
    assert L.cglm_kv_slot_bytes(C.byref(bad)) == 0
    import torch
    if not torch.cuda.is_available():
        h = C.c_void_p()
        assert L.cglm_kv_arena_create(C.byref(d), 1, C.byref(h)) == _lib.ERR_NO_DEVICE
        from chatglm_cpp_b200 import attention as A
        with pytest.raises(RuntimeError):
            A.KVArena(d, 1)


def test_linear_kernel_plan_stays_inside_its_buffers():
    """cglm_linear_kernel_plan over a grid of shapes: what the launcher would ask of shared memory, tensor memory, the
    workspace scratch and the tile counters stays inside what exists (a plan outside them would fault on the device)."""
    from chatglm_cpp_b200 import _lib
    L = _lib.lib()
    scratch = L.cglm_linear_workspace_bytes() - 256
    smem_per_cta = 232448
    taken = 0
    for n_sm in (148, 132, 64):
        for n_tok in (1, 7, 8, 16, 17, 32, 33, 64, 100, 128, 129, 200, 256, 1000, 1024, 4096, 8192):
            for n_in in (64, 128, 512, 1024, 4096, 4160, 13696):
                for n_out in (128, 256, 1536, 3072, 4096, 4608, 8192, 27392):
                    plan = (C.c_int * 8)()
                    if not L.cglm_linear_kernel_plan(n_tok, n_in, n_out, n_sm, plan):
                        continue
                    taken += 1
                    n_box, tiles, ttiles, ksplit, blocks, kb, stages, cols = list(plan)
                    what = (n_sm, n_tok, n_in, n_out, list(plan))
                    assert n_box % 16 == 0 and 16 <= n_box <= 128 and n_box >= min(n_tok, 128), what
                    assert tiles * 128 == n_out and ttiles == (n_tok + 127) // 128, what
                    assert ksplit in (1, 2, 4) and blocks * ksplit * 64 == n_in, what
                    assert kb >= 1 and blocks % kb == 0 and 1 <= stages <= 8 and stages <= blocks // kb, what
                    stage_bytes = kb * (n_box * 128 + 128 * 128)
                    assert 2048 + stages * stage_bytes <= smem_per_cta, what
                    assert cols in (32, 64, 128) and cols >= n_box, what
                    if ksplit > 1:
                        ctas = tiles * ttiles * ksplit
                        assert ctas <= n_sm and tiles * ttiles <= 60, what
                        assert ctas * n_box * 128 * 4 <= scratch, what
                    else:
                        assert stages * stage_bytes >= n_box * 128 * 4, what       # the sums pass through the ring
    assert taken > 500
    # out-features that are not a multiple of 128, or in-features that are not a multiple of 64: the other kernel
    plan = (C.c_int * 8)()
    assert L.cglm_linear_kernel_plan(8, 4096, 96, 148, plan) == 0
    assert L.cglm_linear_kernel_plan(8, 4000, 4096, 148, plan) == 0


def test_linear_entry_points_validate_before_they_touch_a_device():
    """Argument checks of the Linear entry points answer on a machine without a GPU: null pointers, shapes the kernels
    do not take, a workspace that cannot even hold the status word, misaligned operands."""
    from chatglm_cpp_b200 import _lib
    L = _lib.lib()
    assert L.cglm_linear_workspace_bytes() == 256 + 148 * 128 * 128 * 4
    ok = 0x1000   # a plausible, 16-byte aligned address; never dereferenced by the checks
    big = L.cglm_linear_workspace_bytes()
    assert L.cglm_linear_forward(None, 1, 64, ok, 32, None, ok, 0, ok, big, None) == _lib.ERR_INVALID_ARG
    assert L.cglm_linear_forward(ok, 0, 64, ok, 32, None, ok, 0, ok, big, None) == _lib.ERR_INVALID_ARG
    assert L.cglm_linear_forward(ok, 1, 64, ok, 32, None, ok, 0, None, big, None) == _lib.ERR_WORKSPACE
    assert L.cglm_linear_forward(ok, 1, 64, ok, 32, None, ok, 0, ok, 128, None) == _lib.ERR_WORKSPACE
    assert L.cglm_linear_forward(ok, 1, 96, ok, 32, None, ok, 0, ok, big, None) == _lib.ERR_UNSUPPORTED     # in % 64
    assert L.cglm_linear_forward(ok, 1, 64, ok, 40, None, ok, 0, ok, big, None) == _lib.ERR_UNSUPPORTED     # out % 32
    assert L.cglm_linear_forward(ok + 8, 1, 64, ok, 32, None, ok, 0, ok, big, None) == _lib.ERR_INVALID_ARG   # x alignment
    assert L.cglm_linear_forward(ok, 1, 64, ok, 32, None, ok + 4, 0, ok, big, None) == _lib.ERR_INVALID_ARG   # out alignment
    assert L.cglm_convert_f32_to_f16(None, ok, 4, None) == _lib.ERR_INVALID_ARG
    assert L.cglm_convert_f32_to_f16(ok, ok, 0, None) == 0                                                     # nothing to do
    plan = (C.c_int * 8)()
    assert L.cglm_linear_kernel_plan(8, 4096, 4096, 0, plan) == 0 and L.cglm_linear_kernel_plan(8, 4096, 4096, 148, None) == 0
