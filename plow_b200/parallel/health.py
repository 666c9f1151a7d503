"""Rank-group supervision on the host: heartbeats, an abort flag and a pre-launch gate.

Every rank of a tensor/expert-parallel group posts a monotonically increasing heartbeat to a key/value store
(the ``torch.distributed`` TCPStore used for rendezvous, or any object with ``set``/``get``) between steps.
Before a rank launches a step whose kernels wait on peers it calls :meth:`RankHealth.gate`: if a peer's
heartbeat is older than ``timeout_s`` or the group's abort flag is set, the gate raises
:class:`RankFailure` *before* anything is launched, so no kernel is left waiting for a rank that is gone
(device-side waits are bounded as well and report through the status word; this is the host half).
A rank that hits a fatal error calls :meth:`abort`, which the others see at their next gate.

Reference: leader/worker supervision and the abort flag of the process rank group
(crates/plowrt/src/exec/proc_group.rs:251, crates/plowrt/src/serve/cuda_group.rs:1-8) and the counter
monitor (crates/plowrt/src/exec/health.rs).
"""
from __future__ import annotations

import time


class RankFailure(RuntimeError):
    def __init__(self, msg, dead=(), aborted_by=None):
        super().__init__(msg)
        self.dead, self.aborted_by = tuple(dead), aborted_by


class DictStore:
    """In-process stand-in for a TCPStore (tests, single-process groups)."""

    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k):
        return self.d[k]

    def check(self, keys):
        return all(k in self.d for k in keys)


class RankHealth:
    def __init__(self, store, rank: int, world: int, timeout_s: float = 5.0, prefix: str = "plow/health", clock=time.monotonic):
        self.store, self.rank, self.world, self.timeout_s, self.prefix, self.clock = store, rank, world, timeout_s, prefix, clock
        self.step = 0
        self._seen = {}          # rank -> (last value, local time it changed)
        self.beat()

    def _key(self, r):
        return f"{self.prefix}/hb/{r}"

    def beat(self) -> None:
        self.step += 1
        self.store.set(self._key(self.rank), str(self.step))

    def abort(self, reason: str = "") -> None:
        self.store.set(f"{self.prefix}/abort", f"{self.rank}:{reason}")

    def aborted(self):
        k = f"{self.prefix}/abort"
        if self.store.check([k]):
            v = self.store.get(k).decode()
            r, _, why = v.partition(":")
            return int(r), why
        return None

    def dead_ranks(self) -> list:
        now, dead = self.clock(), []
        for r in range(self.world):
            if r == self.rank:
                continue
            k = self._key(r)
            v = self.store.get(k).decode() if self.store.check([k]) else None
            last = self._seen.get(r)
            if last is None or last[0] != v:
                self._seen[r] = (v, now)
            elif now - last[1] > self.timeout_s:
                dead.append(r)
        return dead

    def gate(self) -> None:
        """Call between steps, before launching work that waits on peers."""
        self.beat()
        ab = self.aborted()
        if ab is not None and ab[0] != self.rank:
            raise RankFailure(f"rank {ab[0]} aborted the group: {ab[1]}", aborted_by=ab[0])
        dead = self.dead_ranks()
        if dead:
            raise RankFailure(f"no heartbeat from rank(s) {dead} for {self.timeout_s}s", dead=dead)
