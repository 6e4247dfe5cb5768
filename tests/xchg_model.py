"""Host-side model of the split-KV exchange protocol of cglm_attn_splitkv_step, word for word: every rank owns a
buffer with a step counter, two sets (alternating by step) of arrival words [rank][kv head] and two sets of partial
slots; a step publishes rows + the step number into every buffer, a combining rank waits until all arrival words of
the local buffer hold the step number.  The model lets CPU tests drive the protocol through interleavings and
failures that cannot be staged on a GPU without making a kernel wait for a later launch."""
from __future__ import annotations

import numpy as np

OK, TIMEOUT = 0, -5      # CGLM_OK, CGLM_ERR_TIMEOUT


class RankBuffer:
    def __init__(self, n_rank: int, n_kv: int, payload: int):
        self.counter = 0
        self.flags = np.zeros((2, n_rank, n_kv), np.int64)
        self.slots = np.zeros((2, n_rank, n_kv, payload), np.float64)


class Rank:
    """One rank's view: its own buffer and references to the peers' (the mapped peer memory)."""

    def __init__(self, rank: int, buffers):
        self.rank, self.buffers = rank, buffers
        self.local = buffers[rank]
        self.epoch = None           # step in flight (published, not yet combined)

    def publish(self, rows_of_kv_head):
        """First half of a step: e = local counter + 1; rows then the step number into every rank's buffer."""
        e = self.local.counter + 1
        for g, rows in enumerate(rows_of_kv_head):
            for b in self.buffers:
                b.slots[e & 1, self.rank, g] = rows          # plain stores ... fence ...
            for b in self.buffers:
                b.flags[e & 1, self.rank, g] = e             # ... then the arrival word (release)
        self.epoch = e
        return e

    def arrived(self) -> bool:
        return bool((self.local.flags[self.epoch & 1] == self.epoch).all())

    def combine(self, timed_out: bool = False):
        """Second half: called when arrived() holds, or with timed_out when the bounded wait ran out.  Returns
        (status, payloads of every rank for this step or None); advances the counter either way."""
        e = self.epoch
        if not timed_out:
            assert self.arrived()
        rows = None if timed_out else self.local.slots[e & 1].copy()
        self.local.counter = e
        self.epoch = None
        return (TIMEOUT if timed_out else OK), rows
