"""Tensor parallelism over the GPUs of one node (Megatron layout: q/k/v/gate/up column-parallel,
o/down row-parallel, norms replicated; reference: crates/plowrt/src/asset/shard.rs:1-40).

The row-parallel projections end in an all-reduce.  On the product path that reduction happens
*inside* the GEMM kernel (``csrc/cuda/gemm_tc.cuh``, `ar_*` phases): every rank's partial tile goes to
its own slice of a symmetric buffer, the owner of a tile (tile mod world) sums the ranks' partials in
rank order straight out of peer memory, rounds once to bf16 and stores the result into every rank's
output, and the kernel on each rank retires only when all tiles have landed — one launch, no NCCL
call, bit-identical results on all ranks (the reference's numerics: runtime/nvidia/op_collective.cuh:18-20).
``impl="nccl"`` keeps the same GEMM and calls ``all_reduce`` instead (baseline arm).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import gemm as gemm_ops, native

BF16 = torch.bfloat16


def _align(x, a=256):
    return (x + a - 1) // a * a


class TpComm:
    def __init__(self, rank: int, world: int, max_rows: int = 128, max_n: int = 16384, impl: str = "fused", deadline_ms: int = 2000):
        self.rank, self.world, self.impl = rank, world, impl
        self.dev = torch.device("cuda", torch.cuda.current_device())
        self.max_rows, self.max_n, self.deadline_ms = max_rows, max_n, deadline_ms
        if impl != "fused":
            return
        import torch.distributed._symmetric_memory as symm
        tiles = (max_n + 127) // 128
        lay, off = {}, 0
        for name, nbytes in (("part", tiles * 128 * 128 * 2), ("flag", tiles * 8 * 4), ("done", 128), ("y", max_rows * max_n * 2)):
            lay[name] = off
            off = _align(off + nbytes)
        self.lay = lay
        self.buf = symm.empty(off, dtype=torch.uint8, device=self.dev)
        self.buf.zero_()
        self.hdl = symm.rendezvous(self.buf, dist.group.WORLD)
        torch.cuda.synchronize()
        dist.barrier()
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.peers = list(self.hdl.buffer_ptrs)

    def gemm_allreduce(self, x, w, n_out, sx=None, sw=None, residual=None):
        """y = all_reduce_sum(x_shard @ w_shard.T) (+ residual).  x [M, K/tp], w [N, K/tp]; M <= 128.
        Returns a [M, N] bf16 view of the symmetric output area (valid until the next call)."""
        M = x.shape[0]
        assert M <= self.max_rows and n_out <= self.max_n
        bn = gemm_ops._pick_bn_swap(M, sx is not None, False)
        if self.impl == "fused" and bn <= 64:
            y = self.buf[self.lay["y"]:self.lay["y"] + M * n_out * 2].view(BF16).view(M, n_out)
            ar = dict(peers=self.peers, part_ofs=self.lay["part"], flag_ofs=self.lay["flag"], done_ofs=self.lay["done"],
                      y_ofs=self.lay["y"], epoch_ptr=self.epoch.data_ptr(), world=self.world, me=self.rank,
                      deadline_ms=self.deadline_ms)
            gemm_ops.gemm(x, w, sx=sx, sw=sw, n_out=n_out, swap=True, bn=bn, out=y, residual=residual, ar=ar)
            return y
        y = gemm_ops.gemm(x, w, sx=sx, sw=sw, n_out=n_out, swap=M <= 128, bn=bn if M <= 128 else None, splits=1)
        dist.all_reduce(y)
        if residual is not None:
            y = y + residual
        return y
