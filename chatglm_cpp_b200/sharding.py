"""Host-side partitioning of the attention KV-cache path across the GPUs of one box.

Two cases shard naturally (the reference itself is single-device and single-sequence, chatglm.cpp:400,624-625):
 - independent sequences of a batch go to different GPUs and exchange nothing;
 - one very long context is split along its KV length: rank r holds a contiguous range of cache positions,
   produces an un-normalised partial (acc, m, l) per q head, and the partials are merged by a log-sum-exp
   combine after one all-gather of n_head * (head_dim + 2) floats per rank.
Pure Python, no device code: usable in CPU tests with any torch.distributed backend.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple


def shard_sequences(n_seq: int, world: int, rank: int) -> List[int]:
    """Round-robin assignment of sequence indices to ranks (sequence i -> rank i % world)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad rank/world")
    return list(range(rank, n_seq, world))


@dataclass(frozen=True)
class KvSlice:
    begin: int        # first global cache position held by this rank
    end: int          # one past the last position this rank may hold (capacity of its slice)
    n_local: int      # positions of [0, n_past) that fall into this rank's range
    owns_new: bool    # this rank appends position n_past


def split_kv(n_past: int, n_virtual: int, world: int, rank: int, align: int = 64) -> KvSlice:
    """Contiguous split of the attended range [0, n_virtual + n_past] (the last position is appended now).

    Every rank gets ceil(L / world) positions rounded up to `align` (the decode kernel's tile), so slices start on
    tile boundaries; trailing ranks may be empty.
    """
    if world <= 0 or not 0 <= rank < world or n_past < 0:
        raise ValueError("bad arguments")
    total = n_virtual + n_past + 1
    chunk = -(-total // world)
    chunk = -(-chunk // align) * align
    begin = min(rank * chunk, total)
    end = min(begin + chunk, total)
    new_pos = n_virtual + n_past
    owns_new = begin <= new_pos < end
    n_local = max(0, min(end, new_pos) - begin)
    return KvSlice(begin, begin + chunk, n_local, owns_new)


def slice_capacity(n_past_max: int, n_virtual: int, world: int, align: int = 64) -> int:
    """Cache capacity (tokens) each rank must provide to hold its slice of a context of n_past_max tokens."""
    total = n_virtual + n_past_max + 1
    chunk = -(-total // world)
    return -(-chunk // align) * align


def kv_ranges(n_past: int, n_virtual: int, world: int, align: int = 64) -> List[Tuple[int, int]]:
    """[begin, begin + n_local (+1 if the rank appends)) of every rank: a partition of [0, n_virtual + n_past]."""
    out = []
    for r in range(world):
        s = split_kv(n_past, n_virtual, world, r, align)
        out.append((s.begin, s.begin + s.n_local + (1 if s.owns_new else 0)))
    return out
