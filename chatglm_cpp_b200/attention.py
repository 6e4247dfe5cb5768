"""Python face of the C ABI (include/cglm_attn.h) for tests and benchmarks.

PyTorch appears here only as the owner of device buffers and streams; every computation goes through
libcglm_attn.so.  The classes mirror the reference's objects: ``KVArena`` is ModelContext's kv buffer
(chatglm.h:337,345,627-628) and ``BasicAttention`` keeps the constructor arguments, public cache members
and ``forward(qkv, n_past, n_ctx)`` call shape of chatglm::BasicAttention (chatglm.h:440-472) for the part
between its two Linears.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import (AttnDesc, AttnSeq, MASK_CAUSAL, MASK_CHATGLM, ROPE_CHATGLM, ROPE_CHATGLM2, ROPE_DISABLED,  # noqa: F401
                   ROPE_GPTJ, ROPE_NEOX, SEQ_CACHE_SETTLED, SEQ_NO_APPEND, SEQ_N_PAST_DEVICE, SEQ_PARTIAL, SEQ_USE_KV_LOCAL, check)


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


class _DevView:
    """Zero-copy torch view of library-owned device memory."""

    def __init__(self, ptr: int, shape, typestr: str, strides=None):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3}
        if strides is not None:
            self.__cuda_array_interface__["strides"] = tuple(strides)   # bytes


class KVArena:
    """All k_cache / v_cache pairs of a model (layers x sequences) in one device allocation."""

    def __init__(self, desc: AttnDesc, n_slots: int, adopt=None):
        """adopt: (k_all, v_all[, angle_table]) caller-owned device tensors in the arena's layout (cglm_kv_arena_adopt);
        the arena then allocates nothing and the tensors must outlive it."""
        if not torch.cuda.is_available():
            raise RuntimeError("KVArena needs a CUDA device: this package has no CPU fallback")
        self.desc = desc
        self.n_slots = n_slots
        handle = C.c_void_p()
        if adopt is None:
            check(_lib.lib().cglm_kv_arena_create(C.byref(desc), n_slots, C.byref(handle)), "cglm_kv_arena_create")
        else:
            self._adopted = adopt
            table = adopt[2].data_ptr() if len(adopt) > 2 and adopt[2] is not None else None
            check(_lib.lib().cglm_kv_arena_adopt(C.byref(desc), n_slots, adopt[0].data_ptr(), adopt[1].data_ptr(), table,
                                                 C.byref(handle)), "cglm_kv_arena_adopt")
        self._h = handle
        # tokens between two cache rows as laid out (>= max_len: see cglm_kv_arena_pitch); the views below keep the
        # reference's extents and carry the pitch in their strides
        self.pitch = int(_lib.lib().cglm_kv_arena_pitch(self._h))

    def _k_view(self, ptr, lead):
        d, P = self.desc, self.pitch
        shape = lead + (d.n_kv_head, d.max_len, d.head_dim)
        strides = ((d.n_kv_head * P * d.head_dim * 2,) if lead else ()) + (P * d.head_dim * 2, d.head_dim * 2, 2)
        return torch.as_tensor(_DevView(ptr, shape, "<f2", None if P == d.max_len else strides), device="cuda")

    def _v_view(self, ptr, lead):
        d, P = self.desc, self.pitch
        shape = lead + (d.n_kv_head, d.head_dim, d.max_len)
        strides = ((d.n_kv_head * P * d.head_dim * 2,) if lead else ()) + (d.head_dim * P * 2, P * 2, 2)
        return torch.as_tensor(_DevView(ptr, shape, "<f2", None if P == d.max_len else strides), device="cuda")

    def close(self):
        if self._h:
            _lib.lib().cglm_kv_arena_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def k_cache(self, slot: int) -> torch.Tensor:
        """f16 [n_kv_head, max_len, head_dim] view of the slot's k_cache (chatglm.h:470)."""
        d = self.desc
        ptr = _lib.lib().cglm_kv_arena_k_cache(self._h, slot)
        return self._k_view(ptr, ())

    def v_cache(self, slot: int) -> torch.Tensor:
        """f16 [n_kv_head, head_dim, max_len] view of the slot's transposed v_cache (chatglm.h:471)."""
        d = self.desc
        ptr = _lib.lib().cglm_kv_arena_v_cache(self._h, slot)
        return self._v_view(ptr, ())

    def k_all(self) -> torch.Tensor:
        """f16 [n_slots, n_kv_head, max_len, head_dim] view of every k_cache (the arena keeps them contiguous)."""
        d = self.desc
        ptr = _lib.lib().cglm_kv_arena_k_cache(self._h, 0)
        return self._k_view(ptr, (self.n_slots,))

    def v_all(self) -> torch.Tensor:
        """f16 [n_slots, n_kv_head, head_dim, max_len] view of every v_cache."""
        d = self.desc
        ptr = _lib.lib().cglm_kv_arena_v_cache(self._h, 0)
        return self._v_view(ptr, (self.n_slots,))

    def load_prefix(self, slot: int, past_kv: torch.Tensor) -> None:
        """past_kv: f16 [2, n_kv_head, n_virtual, head_dim] on the device (chatglm.h:580-615)."""
        assert past_kv.is_cuda and past_kv.dtype == torch.float16 and past_kv.is_contiguous()
        check(_lib.lib().cglm_kv_load_prefix(self._h, slot, past_kv.data_ptr(), _stream_ptr()), "cglm_kv_load_prefix")


class Workspace:
    def __init__(self, desc: AttnDesc, n_seq: int, max_qlen: int = 1):
        n = _lib.lib().cglm_attn_workspace_bytes(C.byref(desc), n_seq, max_qlen)
        if n == 0:
            raise ValueError("bad descriptor for workspace")
        self.buf = torch.empty(n, dtype=torch.uint8, device="cuda")
        self.bytes = n
        check(_lib.lib().cglm_attn_workspace_init(self.buf.data_ptr(), n, _stream_ptr()), "cglm_attn_workspace_init")

    @property
    def ptr(self) -> int:
        return self.buf.data_ptr()

    def status(self) -> int:
        return _lib.lib().cglm_attn_workspace_status(self.ptr, _stream_ptr())


@dataclass
class SeqCall:
    """One sequence of a batched forward: a fused qkv activation on the device plus its cache slot."""
    qkv: torch.Tensor                 # f32 or f16 [qlen, (H+2G)*D] (blocked) or [qlen, 3*H*D] (interleaved)
    slot: int
    n_past: int
    n_ctx: int = 0
    out: Optional[torch.Tensor] = None        # f32 or f16 [qlen, H*D]
    position_ids: Optional[torch.Tensor] = None
    q_roped: Optional[torch.Tensor] = None
    k_roped: Optional[torch.Tensor] = None
    partial: Optional[torch.Tensor] = None
    kv_local: int = 0
    flags: int = 0
    n_past_dev: Optional[torch.Tensor] = None  # int32 device word(s); with SEQ_N_PAST_DEVICE the kernel reads n_past here


def fill_seq(dst: AttnSeq, desc: AttnDesc, call: SeqCall, interleaved: bool) -> None:
    H, G, D = desc.n_head, desc.n_kv_head, desc.head_dim
    qkv = call.qkv
    assert qkv.is_cuda and qkv.dtype in (torch.float32, torch.float16) and qkv.is_contiguous() and qkv.dim() == 2
    base, esz = qkv.data_ptr(), qkv.element_size()
    row = qkv.shape[1]
    if interleaved:   # chatglm.cpp:638-644
        assert row == 3 * H * D and H == G
        dst.q, dst.k, dst.v = base, base + D * esz, base + 2 * D * esz
        dst.q_head_stride = dst.kv_head_stride = 3 * D
    else:             # chatglm.cpp:646-652
        assert row == (H + 2 * G) * D
        dst.q, dst.k, dst.v = base, base + H * D * esz, base + (H + G) * D * esz
        dst.q_head_stride = dst.kv_head_stride = D
    dst.q_tok_stride = dst.kv_tok_stride = row
    dst.slot, dst.qlen, dst.n_past, dst.n_ctx = call.slot, qkv.shape[0], call.n_past, call.n_ctx
    dst.position_ids = call.position_ids.data_ptr() if call.position_ids is not None else None
    dst.out = call.out.data_ptr() if call.out is not None else None
    dst.q_roped = call.q_roped.data_ptr() if call.q_roped is not None else None
    dst.k_roped = call.k_roped.data_ptr() if call.k_roped is not None else None
    dst.partial = call.partial.data_ptr() if call.partial is not None else None
    dst.kv_local, dst.flags = call.kv_local, call.flags
    if qkv.dtype == torch.float16:
        dst.flags |= _lib.SEQ_QKV_F16
    if call.out is not None and call.out.dtype == torch.float16:
        dst.flags |= _lib.SEQ_OUT_F16
    dst.n_past_dev = call.n_past_dev.data_ptr() if call.n_past_dev is not None else None


def forward_batch(arena: KVArena, ws: Workspace, calls: Sequence[SeqCall], interleaved: bool = False,
                  seq_array=None) -> None:
    """cglm_attn_forward over a batch of sequences; asynchronous on the current stream."""
    n = len(calls)
    arr = seq_array if seq_array is not None else (AttnSeq * n)()
    for i, c in enumerate(calls):
        fill_seq(arr[i], arena.desc, c, interleaved)
    check(_lib.lib().cglm_attn_forward(arena._h, arr, n, ws.ptr, ws.bytes, _stream_ptr()), "cglm_attn_forward")


class BasicAttention:
    """The cache-owning attention module of one layer for one sequence (chatglm.h:440-472).

    ``forward`` takes what query_key_value.forward returns (chatglm.cpp:629) and returns what dense.forward
    consumes (chatglm.cpp:719).
    """

    def __init__(self, arena: KVArena, slot: int, ws: Workspace, interleaved_qkv: bool = False):
        d = arena.desc
        self.arena, self.slot, self.ws = arena, slot, ws
        self.num_attention_heads = d.n_head
        self.num_key_value_heads = d.n_kv_head
        self.interleaved_qkv = interleaved_qkv
        self.rope_type = d.rope_type
        self.rope_theta = d.rope_theta
        self.attn_mask_type = d.mask_type
        self.num_virtual_tokens = d.n_virtual
        self.k_cache = arena.k_cache(slot)   # [#kvh, s, d]
        self.v_cache = arena.v_cache(slot)   # [#kvh, d, s]

    def forward(self, qkv: torch.Tensor, n_past: int, n_ctx: int = 0, position_ids: Optional[torch.Tensor] = None,
                want_roped: bool = False, out_dtype: torch.dtype = torch.float32):
        d = self.arena.desc
        qlen = qkv.shape[0]
        out = torch.empty(qlen, d.n_head * d.head_dim, dtype=out_dtype, device="cuda")
        qr = kr = None
        if want_roped:
            qr = torch.empty(qlen, d.n_head, d.head_dim, dtype=torch.float32, device="cuda")
            kr = torch.empty(qlen, d.n_kv_head, d.head_dim, dtype=torch.float32, device="cuda")
        call = SeqCall(qkv=qkv, slot=self.slot, n_past=n_past, n_ctx=n_ctx, out=out, position_ids=position_ids,
                       q_roped=qr, k_roped=kr)
        forward_batch(self.arena, self.ws, [call], self.interleaved_qkv)
        return (out, qr, kr) if want_roped else out


class SplitKVExchange:
    """One rank's side of the fused split-KV step (cglm_attn_splitkv_step).  ``buffers`` holds every rank's exchange
    buffer as a tensor valid on this device (entry ``rank`` is the local one); how the peers' buffers were mapped
    (CUDA IPC between processes, plain tensors inside one process) is the caller's business."""

    def __init__(self, buffers: Sequence, rank: int, n_head: int, head_dim: int):
        """buffers: per rank a tensor on this device, or a raw device pointer (int) valid on this device."""
        self.n_rank, self.rank, self.n_head, self.head_dim = len(buffers), rank, n_head, head_dim
        need = self.bytes(self.n_rank, n_head, head_dim)
        ptrs = []
        for b in buffers:
            if isinstance(b, torch.Tensor):
                assert b.is_cuda and b.is_contiguous() and b.numel() * b.element_size() >= need
                ptrs.append(b.data_ptr())
            else:
                ptrs.append(int(b))
        self.buffers = list(buffers)   # keeps tensors alive
        self._local = ptrs[rank]
        self._ptrs = (C.c_void_p * self.n_rank)(*ptrs)

    @staticmethod
    def alloc_exported(n_rank: int, n_head: int, head_dim: int):
        """Allocates this rank's zero-filled buffer outside torch's allocator and returns (pointer, 64-byte IPC handle)."""
        ptr = C.c_void_p()
        check(_lib.lib().cglm_xchg_alloc(SplitKVExchange.bytes(n_rank, n_head, head_dim), C.byref(ptr)), "cglm_xchg_alloc")
        handle = C.create_string_buffer(64)
        check(_lib.lib().cglm_xchg_export(ptr, handle), "cglm_xchg_export")
        return ptr.value, handle.raw

    @staticmethod
    def import_handle(handle: bytes, owner_device: int) -> int:
        """Maps a peer's buffer into the current device's context; returns the device pointer."""
        ptr = C.c_void_p()
        check(_lib.lib().cglm_xchg_import(handle, owner_device, C.byref(ptr)), "cglm_xchg_import")
        return ptr.value

    @staticmethod
    def bytes(n_rank: int, n_head: int, head_dim: int) -> int:
        return int(_lib.lib().cglm_attn_splitkv_xchg_bytes(n_rank, n_head, head_dim))

    @staticmethod
    def new_buffer(n_rank: int, n_head: int, head_dim: int) -> torch.Tensor:
        return torch.zeros((SplitKVExchange.bytes(n_rank, n_head, head_dim) + 3) // 4, dtype=torch.int32, device="cuda")

    def read_words(self, n: int):
        """The first n 32-bit words of the local buffer (step counter, arrival words), for diagnostics."""
        host = torch.empty(n, dtype=torch.int32)
        buf = self.buffers[self.rank]
        if isinstance(buf, torch.Tensor):
            torch.cuda.synchronize()
            return buf.view(torch.int32)[:n].cpu().numpy().view("uint32")
        check(_lib.lib().cglm_xchg_read(C.c_void_p(self._local), host.data_ptr(), n * 4), "cglm_xchg_read")
        return host.numpy().view("uint32")

    def step(self, arena: "KVArena", ws: "Workspace", seq_array, out: Optional[torch.Tensor], combine: bool = True,
             timeout_us: int = 0) -> None:
        """One fused launch: attention over this rank's slice, rows published to every rank, merged into ``out``."""
        check(_lib.lib().cglm_attn_splitkv_step(arena._h, seq_array, self._ptrs, self.n_rank, self.rank,
                                                out.data_ptr() if out is not None else None, int(combine), timeout_us,
                                                ws.ptr, ws.bytes, _stream_ptr()), "cglm_attn_splitkv_step")


def splitkv_combine(partials: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """partials: f32 [n_part, H, D+2] (acc | m | l) on this device -> f32 [H*D]."""
    assert partials.is_cuda and partials.dtype == torch.float32 and partials.is_contiguous()
    n, H, Dp2 = partials.shape
    if out is None:
        out = torch.empty(H * (Dp2 - 2), dtype=torch.float32, device="cuda")
    check(_lib.lib().cglm_attn_splitkv_combine(partials.data_ptr(), n, H, Dp2 - 2, out.data_ptr(), _stream_ptr()),
          "cglm_attn_splitkv_combine")
    return out
