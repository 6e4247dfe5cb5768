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
