"""Rank groups for serving a model over several GPUs of one node: one process per GPU.

Two ways of running a step together, chosen by how the packet was sharded:

* **Lockstep group** (expert parallelism with data-parallel attention).  Every rank owns its own requests,
  scheduler and KV pages, but the MoE layers of a step are collective, so all ranks must launch the *same
  program* the same number of times.  Before each launch the ranks agree (one tiny all-reduce on a CPU
  process group) on the role and row count of the step: if any rank prefills, all run the prefill program that
  covers the largest row count; a rank with nothing to do joins with an empty batch.  :class:`StepGroup`.
* **Leader / follower group** (tensor parallelism).  All ranks run the same token batch.  Rank 0 owns the
  scheduler and the page bookkeeping; before each launch it broadcasts the step (program, rows, page-table rows
  that changed) and the followers replay it.  :class:`LeaderGroup`.

Both carry a stop flag, so a leader that shuts down (or fails) releases the other ranks instead of leaving them
in a collective, and both use bounded waits: a rank that never shows up ends the wait with an error after
``timeout_s`` (the process-group timeout).

Reference counterparts: crates/plowrt/src/serve/cuda_group.rs:1-8 (leader + `plowrt rank-worker`),
exec/proc_group.rs:251-339 (arm barrier with a plan fingerprint, fails instead of hanging),
docs/arch/09-multi-gpu.md:214-260.
"""
from __future__ import annotations

import datetime
import pickle

import numpy as np
import torch
import torch.distributed as dist


class GroupStopped(RuntimeError):
    """The group was told to stop (or a peer failed); no further steps will run."""


class StepGroup:
    """Per-step agreement between ranks that each schedule their own requests."""

    # fields of the agreement vector (all reduced with MAX)
    _PREFILL, _ROWS, _BUSY, _STOP, _SAMPLES = range(5)

    def __init__(self, rank: int, world: int, timeout_s: float = 60.0, pg=None):
        self.rank, self.world = rank, world
        self.pg = pg if pg is not None else dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))
        self._buf = torch.zeros(5, dtype=torch.int64)
        self.steps = 0
        self.stopped = False

    def agree(self, decode: bool, rows: int, busy: bool, stop: bool = False, samples: int = 0):
        """Returns (decode, rows, any_busy, samples) for the step every rank will now run.  Raises GroupStopped when
        any rank asked to stop."""
        if self.stopped:
            raise GroupStopped("group already stopped")
        b = self._buf
        b[self._PREFILL] = 0 if (decode or not busy) else 1
        b[self._ROWS] = rows if busy else 0
        b[self._BUSY] = 1 if busy else 0
        b[self._STOP] = 1 if stop else 0
        b[self._SAMPLES] = samples if busy else 0
        try:
            dist.all_reduce(b, op=dist.ReduceOp.MAX, group=self.pg)
        except RuntimeError as e:           # a peer died or never arrived: the timeout ends the wait
            self.stopped = True
            raise GroupStopped(f"rank group lost a member: {e}") from None
        if int(b[self._STOP]):
            self.stopped = True
            raise GroupStopped("stop requested")
        self.steps += 1
        return (not bool(int(b[self._PREFILL]))), int(b[self._ROWS]), bool(int(b[self._BUSY])), int(b[self._SAMPLES])

    def stop(self) -> None:
        """Tell the other ranks to stop at their next agreement (best effort)."""
        if not self.stopped:
            try:
                self.agree(True, 0, False, stop=True)
            except GroupStopped:
                pass


class LeaderGroup:
    """Rank 0 decides every step; the other ranks replay it."""

    def __init__(self, rank: int, world: int, timeout_s: float = 60.0, pg=None):
        self.rank, self.world = rank, world
        self.pg = pg if pg is not None else dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))
        self.stopped = False

    def _bcast(self, payload: bytes | None) -> bytes:
        n = torch.zeros(1, dtype=torch.int64)
        if self.rank == 0:
            n[0] = len(payload)
        dist.broadcast(n, src=0, group=self.pg)
        buf = torch.frombuffer(bytearray(payload), dtype=torch.uint8) if self.rank == 0 else torch.empty(int(n[0]), dtype=torch.uint8)
        if int(n[0]):
            dist.broadcast(buf, src=0, group=self.pg)
        return bytes(buf.numpy().tobytes())

    def publish(self, step: dict) -> None:
        """Leader: send one step description ({"stop": True} ends the followers' loops)."""
        try:
            self._bcast(pickle.dumps(step, protocol=pickle.HIGHEST_PROTOCOL))
        except RuntimeError as e:
            self.stopped = True
            raise GroupStopped(f"rank group lost a member: {e}") from None

    def receive(self) -> dict:
        """Follower: wait for the leader's next step."""
        try:
            step = pickle.loads(self._bcast(None))
        except RuntimeError as e:
            self.stopped = True
            raise GroupStopped(f"leader lost: {e}") from None
        if step.get("stop"):
            self.stopped = True
            raise GroupStopped("stop requested")
        return step

    def stop(self) -> None:
        if self.rank == 0 and not self.stopped:
            try:
                self.publish({"stop": True})
            except GroupStopped:
                pass
            self.stopped = True


def follower_loop(engine, group: LeaderGroup) -> int:
    """Body of a tensor-parallel follower rank: replay the leader's steps until it stops.  Returns the step count."""
    from ..runtime.engine import TokenBatch
    n = 0
    while True:
        try:
            step = group.receive()
        except GroupStopped:
            return n
        for slot, row in step.get("pages", {}).items():
            engine.set_page_row(int(slot), np.asarray(row, dtype=np.int32))
        b = step["batch"]
        engine.step(TokenBatch(b["ids"], b["pos"], b["seq"], b["sample_rows"], decode=b["decode"], want_logits=b["want_logits"]),
                    replay=True)
        n += 1
