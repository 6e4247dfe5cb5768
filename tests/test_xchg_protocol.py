"""The epoch protocol of the fused split-KV exchange, on CPU: a word-for-word model (tests/xchg_model.py) driven
through random interleavings (two buffer sets suffice; a combine only ever sees rows of its own step), through a
silent rank (bounded wait runs out, counter still advances, every later step of the others times out too: the host
must stop) and through a late rank (a stale step number is never taken for the current one); then the same between
two gloo processes that exchange the buffer writes as messages."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from hypothesis import given, settings, strategies as st

from xchg_model import OK, TIMEOUT, Rank, RankBuffer


def _make(n_rank, n_kv=2, payload=3):
    bufs = [RankBuffer(n_rank, n_kv, payload) for _ in range(n_rank)]
    return [Rank(r, bufs) for r in range(n_rank)], bufs


def _rows(rank, step, n_kv=2, payload=3):
    return [np.full(payload, 1000.0 * step + 10 * rank + g) for g in range(n_kv)]


@settings(max_examples=200, deadline=None)
@given(st.integers(2, 5), st.integers(1, 6), st.lists(st.integers(0, 10 ** 6), min_size=1, max_size=200))
def test_any_interleaving_keeps_steps_apart(n_rank, n_steps, choices):
    """Each rank runs publish(1), combine(1), publish(2), ... in order; a scheduler picks any rank whose next action is
    enabled (a combine is enabled once its arrival words are all there).  Whatever the schedule: nobody deadlocks, and a
    combine returns exactly the rows every rank published for THAT step, although only two slot sets exist."""
    ranks, _ = _make(n_rank)
    step = [1] * n_rank            # next step of each rank
    phase = [0] * n_rank           # 0: publish next, 1: combine next
    pick = iter(choices)
    done = 0
    while done < n_rank:
        enabled = [r for r in range(n_rank) if step[r] <= n_steps and (phase[r] == 0 or ranks[r].arrived())]
        assert enabled, "deadlock"
        r = enabled[next(pick, 0) % len(enabled)]
        if phase[r] == 0:
            assert ranks[r].publish(_rows(r, step[r])) == step[r]
            phase[r] = 1
        else:
            status, rows = ranks[r].combine()
            assert status == OK
            for p in range(n_rank):
                for g in range(2):
                    assert (rows[p, g] == _rows(p, step[r])[g]).all(), (r, p, step[r])
            phase[r] = 0
            step[r] += 1
            if step[r] > n_steps:
                done += 1
    assert all(rk.local.counter == n_steps for rk in ranks)


def test_silent_rank_times_out_and_the_ranks_fall_out_of_step():
    ranks, bufs = _make(3)
    for r in ranks:
        r.publish(_rows(r.rank, 1))
    assert all(r.combine()[0] == OK for r in ranks)
    # step 2: rank 1 is silent
    for r in (ranks[0], ranks[2]):
        r.publish(_rows(r.rank, 2))
    for r in (ranks[0], ranks[2]):
        assert not r.arrived()
        status, rows = r.combine(timed_out=True)
        assert status == TIMEOUT and rows is None
    assert [b.counter for b in bufs] == [2, 1, 2]
    # rank 1 comes back and publishes ITS step 2 while the others publish step 3: stale numbers are not accepted,
    # and rank 1 itself never sees the others' step 2 again (their words moved on) -- the host has to stop
    ranks[1].publish(_rows(1, 2))
    for r in (ranks[0], ranks[2]):
        r.publish(_rows(r.rank, 3))
    assert not ranks[0].arrived() and not ranks[2].arrived()
    assert ranks[1].arrived()          # set 0 still holds the others' step 2 words: rank 1 completes its late step 2 ...
    status, rows = ranks[1].combine()
    assert status == OK and (rows[0, 0] == _rows(0, 2)[0]).all()
    ranks[1].publish(_rows(1, 3))      # ... and catches up: now step 3 is complete everywhere
    assert all(r.arrived() for r in ranks)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_q):
    """Two processes; a "peer store" is a message.  Each process applies the stores it receives to its own buffer in
    arrival order.  Step 1 normal; at step 2 rank 1 publishes nothing, rank 0 must report TIMEOUT and stop."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n_kv, payload = 2, 4
    mine = RankBuffer(world, n_kv, payload)
    peer = 1 - rank
    log = []

    def exchange(e, rows):
        """rows = None: this rank stays silent in this step."""
        msg = torch.zeros(2 + n_kv * payload, dtype=torch.float64)
        if rows is not None:
            msg[0], msg[1] = 1.0, float(e)
            msg[2:] = torch.from_numpy(np.concatenate(rows))
        got = [torch.zeros_like(msg) for _ in range(world)]
        dist.all_gather(got, msg)                      # the transport; ordering = slots before arrival words
        for src in range(world):
            if got[src][0] == 1.0:
                se = int(got[src][1])
                mine.slots[se & 1, src] = got[src][2:].numpy().reshape(n_kv, payload)
                mine.flags[se & 1, src] = se

    for step, silent in ((1, False), (2, rank == 1)):
        e = mine.counter + 1
        exchange(e, None if silent else _rows(rank, step, n_kv, payload))
        if silent:
            log.append("silent")
            continue
        ok = bool((mine.flags[e & 1] == e).all())
        mine.counter = e
        if not ok:
            log.append(TIMEOUT)
            break                                        # the host stops at the first timeout
        rows = mine.slots[e & 1]
        assert (rows[peer, 1] == _rows(peer, step, n_kv, payload)[1]).all()
        log.append(OK)
    out_q.put((rank, log))
    dist.barrier()
    dist.destroy_process_group()


def test_epoch_protocol_world_size_2_gloo_with_a_silent_rank():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results[0] == [OK, TIMEOUT]
    assert results[1] == [OK, "silent"]
