"""Host-side multi-rank logic on CPU: partitioning rules, and a world_size-2 gloo run of the split-KV flow
(per-rank partial -> all_gather -> log-sum-exp combine) with the CPU oracle standing in for the device kernels."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from chatglm_cpp_b200 import sharding
from oracle import attn_oracle as O


def test_shard_sequences_is_a_partition():
    for n, w in ((64, 1), (64, 8), (4, 8), (7, 3)):
        seen = sorted(i for r in range(w) for i in sharding.shard_sequences(n, w, r))
        assert seen == list(range(n))
    with pytest.raises(ValueError):
        sharding.shard_sequences(4, 2, 2)


@pytest.mark.parametrize("n_past,nv,world", [(131072, 0, 8), (131072, 0, 1), (5, 0, 4), (0, 0, 2), (1000, 5, 3), (63, 0, 2), (64, 0, 2)])
def test_split_kv_covers_every_position_once(n_past, nv, world):
    ranges = sharding.kv_ranges(n_past, nv, world)
    total = nv + n_past + 1
    covered = [p for b, e in ranges for p in range(b, e)] if total < 5000 else None
    if covered is not None:
        assert covered == list(range(total))
    assert sum(e - b for b, e in ranges) == total
    owners = [r for r in range(world) if sharding.split_kv(n_past, nv, world, r).owns_new]
    assert len(owners) == 1
    cap = sharding.slice_capacity(n_past, nv, world)
    for r in range(world):
        s = sharding.split_kv(n_past, nv, world, r)
        assert s.begin % 64 == 0 or s.n_local == 0
        assert s.n_local + (1 if s.owns_new else 0) <= cap


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_past, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    H, G, D = 8, 2, 16
    rng = np.random.default_rng(99)                      # same data on every rank
    M = n_past + 8
    cfg = O.make_cfg(H, G, D, M, numerics="f32")
    k = np.zeros((G, M, D), np.uint16); v = np.zeros((G, D, M), np.uint16)
    k[:, :n_past] = rng.standard_normal((G, n_past, D)).astype(np.float16).view(np.uint16)
    v[:, :, :n_past] = rng.standard_normal((G, D, n_past)).astype(np.float16).view(np.uint16)
    qkv = rng.standard_normal((1, (H + 2 * G) * D)).astype(np.float32)
    full, qr, _ = O.attn_forward(cfg, qkv, False, k, v, n_past, want_roped=True)   # appends position n_past
    # this rank attends only its slice of the (now complete) cache
    b, e = sharding.kv_ranges(n_past, 0, world, align=4)[rank]
    acc, m, l = O.attn_partial(cfg, qr[0], k, v, b, e)
    mine = torch.from_numpy(np.concatenate([acc, m[:, None], l[:, None]], axis=1))   # [H, D+2]
    gathered = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    parts = torch.stack(gathered).numpy()
    out = O.attn_combine(parts[:, :, :D].copy(), parts[:, :, D].copy(), parts[:, :, D + 1].copy())
    out_q.put((rank, float(np.abs(out.reshape(-1) - full[0]).max())))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("n_past", [37, 3])
def test_split_kv_flow_world_size_2_gloo(n_past):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n_past, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err in results:
        assert err < 2e-6, (rank, err)
