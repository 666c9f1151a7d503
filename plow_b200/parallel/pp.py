"""Pipeline parallelism over point-to-point sends (NCCL p2p on GPUs, gloo on CPU): each rank runs a contiguous stage
of the model on micro-batches and hands the activation to the next rank with ``isend`` while it starts the next
micro-batch, so the transfer overlaps compute.  Stages are any callables (an engine restricted to a layer range, a
module): the runner owns only the schedule and the transport.  Reference: the stage hand-off buffer of the process
rank group (crates/plowrt/src/exec/proc_group.rs:88-120); the reference ships the design, not a PP executor."""
from __future__ import annotations

import torch
import torch.distributed as dist


class PipelineRunner:
    def __init__(self, stage_fn, rank: int, world: int, act_shape, dtype=torch.float32, device="cpu", group=None):
        self.fn, self.rank, self.world = stage_fn, rank, world
        self.act_shape, self.dtype, self.device, self.group = tuple(act_shape), dtype, device, group

    def run(self, micro_batches: list | None, n_micro: int) -> list:
        """Rank 0 feeds ``micro_batches``; the last rank returns the outputs (others return [])."""
        outs, pending = [], []
        for m in range(n_micro):
            if self.rank == 0:
                x = micro_batches[m]
            else:
                x = torch.empty(self.act_shape, dtype=self.dtype, device=self.device)
                dist.recv(x, src=self.rank - 1, group=self.group)
            y = self.fn(x)
            if self.rank == self.world - 1:
                outs.append(y)
            else:
                # the send of micro-batch m overlaps the compute of micro-batch m+1
                pending.append((dist.isend(y.contiguous(), dst=self.rank + 1, group=self.group), y))
                pending = [(w, t) for (w, t) in pending if not w.is_completed()]
        for w, _ in pending:
            w.wait()
        return outs
