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
    def __init__(self, rank: int, world: int, max_rows: int = 128, max_n: int = 16384, impl: str = "fused", deadline_ms: int = 2000,
                 max_k: int = 16384, oneshot_bytes: int = 4 << 20, form: str = "auto", ar_rows: int = 512, ar_width: int = 8192):
        """form: "auto" (NVSwitch multicast reduce at 4+ ranks when the mapping exists, else one-shot for decode-size
        messages, else two-shot), or "oneshot" / "twoshot" / "nvls" to force one."""
        self.rank, self.world, self.impl, self.form = rank, world, impl, form
        self.oneshot_bytes = oneshot_bytes     # messages up to this size use the one-shot form (decode), larger ones two-shot
        self.dev = torch.device("cuda", torch.cuda.current_device())
        self.max_rows, self.max_n, self.deadline_ms = max_rows, max_n, deadline_ms
        self.max_k = max_k
        # stand-alone all-reduce (+ add + norm) over peer memory: rows x hidden width at most.  The one-shot form reads every
        # rank's partial on every rank, which wins while the message is latency-bound (measured on 2 GPUs: 21.6 us against
        # 45.6 us for NCCL + the norm kernel at 64 x 4096) and loses to NCCL's bandwidth-optimal ring once it is not
        # (93.6 us against 68.8 us at 1500 x 4096): larger row counts keep NCCL.
        self.ar_rows, self.ar_width = ar_rows, ar_width
        if impl != "fused":
            return
        import torch.distributed._symmetric_memory as symm
        tiles = (max_n + 127) // 128
        lay, off = {}, 0
        self.half_bytes = _align(tiles * world * 128 * 64 * 2)        # one-shot slots: [tile][source rank][128][<=64 tokens] bf16
        for name, nbytes in (("part", max(tiles * 128 * 128 * 2, 2 * self.half_bytes)), ("flag", tiles * 8 * 4), ("done", 128), ("tdone", tiles * 4), ("y", max_rows * max_n * 2),
                             ("ag_ctr", 128), ("ag_rel", 128), ("xg0", max_rows * max_k * 2),
                             ("ar_flag", world * ar_rows * 4), ("ar_part", 2 * _align(ar_rows * ar_width * 2))):
            lay[name] = off
            off = _align(off + nbytes)
        self.lay = lay
        self.buf = symm.empty(off, dtype=torch.uint8, device=self.dev)
        self.buf.zero_()
        self.hdl = symm.rendezvous(self.buf, dist.group.WORLD)
        torch.cuda.synchronize()
        dist.barrier()
        self.epoch = torch.zeros(4, dtype=torch.int32, device=self.dev)      # [launch counter, arrivals seen, CTAs through, -]
        self.ar_epoch = torch.zeros(2, dtype=torch.int32, device=self.dev)   # [call counter, CTAs through]
        self.ag_epoch = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.ag_done = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.peers = list(self.hdl.buffer_ptrs)
        try:
            self.mc_ptr = int(self.hdl.multicast_ptr) if self.hdl.has_multicast_support(self.dev.type, self.dev.index) else 0
        except Exception:
            self.mc_ptr = int(getattr(self.hdl, "multicast_ptr", 0) or 0)
        import ctypes
        self._peer_arr = (ctypes.c_void_p * 8)(*(self.peers + [None] * (8 - len(self.peers))))

    def gemm_allreduce(self, x, w, n_out, sx=None, sw=None, residual=None, out=None):
        """y = all_reduce_sum(x_shard @ w_shard.T) (+ residual).  x [M, K/tp], w [N, K/tp]; M <= 128.
        Returns a [M, N] bf16 view of the symmetric output area (valid until the next call)."""
        M = x.shape[0]
        bn = gemm_ops._pick_bn_swap(M, sx is not None, False) if M <= 128 else 128
        if self.impl == "fused" and M <= 64 and bn <= 64 and M <= self.max_rows and n_out <= self.max_n and n_out % 8 == 0:
            form = self.form
            if form == "auto":
                form = "nvls" if (self.mc_ptr and self.world >= 4) else ("oneshot" if (self.world - 1) * M * n_out * 2 <= self.oneshot_bytes else "twoshot")
            if form == "nvls" and not self.mc_ptr:
                raise RuntimeError("this symmetric allocation has no NVSwitch multicast mapping")
            oneshot = form == "oneshot"
            ar = dict(peers=self.peers, part_ofs=self.lay["part"], flag_ofs=self.lay["flag"], done_ofs=self.lay["done"],
                      y_ofs=self.lay["y"], epoch_ptr=self.epoch.data_ptr(), world=self.world, me=self.rank,
                      deadline_ms=self.deadline_ms, oneshot={"oneshot": 1, "twoshot": 0, "nvls": 2}[form], half_bytes=self.half_bytes,
                      mc_ptr=self.mc_ptr, tdone_ofs=self.lay["tdone"])
            if oneshot:
                # every rank reduces locally, so the result can land in any tensor of this rank
                y = out if out is not None else torch.empty(M, n_out, dtype=BF16, device=self.dev)
            else:
                y = self.buf[self.lay["y"]:self.lay["y"] + M * n_out * 2].view(BF16).view(M, n_out)
            gemm_ops.gemm(x, w, sx=sx, sw=sw, n_out=n_out, swap=True, bn=bn, out=y, residual=residual, ar=ar)
            if out is not None and not oneshot:
                out.copy_(y)
                return out
            return y
        y = gemm_ops.gemm(x, w, sx=sx, sw=sw, n_out=n_out, swap=M <= 128, bn=bn if M <= 128 else None, splits=1)
        if self._ar_fits(y):
            # larger row counts: the partial is reduced by the row kernel over peer memory (and the residual added there)
            return self.allreduce_add_norm(y, residual, None, out if out is not None else torch.empty_like(y), None)
        dist.all_reduce(y)
        if residual is not None:
            y = y + residual
        if out is not None:
            out.copy_(y)
            return out
        return y

    def _ar_fits(self, x) -> bool:
        return (self.impl == "fused" and x.dim() == 2 and x.dtype == BF16 and x.shape[0] <= self.ar_rows and x.shape[1] <= self.ar_width
                and x.shape[1] % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0)

    def allreduce_add_norm(self, partial, x_in, gamma, x_out, h_out, eps: float = 1e-6, plus_one: bool = False):
        """x_out = (x_in +) sum over ranks of ``partial``; with ``gamma``: h_out = rmsnorm(x_out) * gamma.  One kernel over
        peer memory (csrc/comm/tp_ar.cu); every rank gets bit-identical results.  Returns x_out."""
        M, H = partial.shape
        assert self._ar_fits(partial) and x_out.is_contiguous() and (x_in is None or x_in.is_contiguous())
        native.call("plow_tp_allreduce_norm", self._peer_arr, self.lay["ar_part"], _align(self.ar_rows * self.ar_width * 2),
                    self.lay["ar_flag"], self.ar_epoch, self.world, self.rank, self.ar_rows, partial, partial.stride(0), x_in, gamma,
                    x_out, h_out, M, H, float(eps), int(plus_one), self.deadline_ms, native.status_word(self.dev))
        return x_out

    def allgather_gemm(self, x_band, w, n_out, dual=False):
        """y = gather_rows(x_band over ranks) @ w.T for a column-parallel w [N/tp(*2), K] (bf16).

        x_band [rows/tp, K] is this rank's band of the sequence-parallel activation.  The band is pushed into
        every rank's gathered buffer by one kernel (csrc/comm/tp_ag.cu) and the GEMM waits for all bands from
        inside the kernel; ``impl="nccl"`` gathers with all_gather_into_tensor and runs the same GEMM."""
        band, K = x_band.shape
        M = band * self.world
        assert x_band.dtype == BF16 and x_band.is_contiguous()
        if self.impl != "fused":
            xg = torch.empty(M, K, dtype=BF16, device=self.dev)
            dist.all_gather_into_tensor(xg, x_band)
            return gemm_ops.gemm(xg, w, dual=dual, n_out=n_out)
        # one gathered buffer: the push of a call waits (on the device, bounded) until every rank has released the
        # previous call's rows, which each rank does right after its GEMM; no host-side state, so a captured graph replays
        ofs = self.lay["xg0"]
        assert M <= self.max_rows and K <= self.max_k
        native.call("plow_ag_push", self._peer_arr, ofs, self.lay["ag_ctr"], self.ag_epoch, self.ag_done, self.world,
                    self.rank, x_band, K * 2, band, K * 2, self.lay["ag_rel"], self.deadline_ms, native.status_word(self.dev))
        xg = self.buf[ofs:ofs + M * K * 2].view(BF16).view(M, K)
        ctr = self.buf.data_ptr() + self.lay["ag_ctr"]
        y = gemm_ops.gemm(xg, w, dual=dual, n_out=n_out, wait=(ctr, self.ag_epoch.data_ptr(), self.world, self.deadline_ms))
        native.call("plow_ag_release", self._peer_arr, self.lay["ag_rel"], self.world, self.rank)
        return y

    def all_reduce(self, x):
        """Stand-alone all-reduce (instructions the compiler did not fuse into a GEMM), in place: the peer-memory row
        kernel when the tensor fits its buffers, NCCL otherwise (and in the baseline arm)."""
        if self._ar_fits(x) and x.is_contiguous():
            return self.allreduce_add_norm(x, None, None, x, None)
        dist.all_reduce(x)
        return x
