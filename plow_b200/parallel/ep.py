"""Expert parallelism over the GPUs of one node: attention is data-parallel, every rank owns a
contiguous range of routed experts.

Two arms share the model code:

* ``fused`` — the product path.  Quantised token rows are pushed straight into the owning rank's
  expert-sorted buffer over NVLink peer memory (``csrc/comm/ep.cu``), the grouped tcgen05 GEMM of
  the owner gates on the arrival counter from inside the kernel, and the combine kernel pulls the
  expert outputs from the owners and forms the top-k weighted sum.  No host or stream
  synchronisation between dispatch, expert GEMMs and combine; flags are device-side epochs, so the
  whole layer sequence replays from a CUDA graph.
* ``nccl`` — the baseline arm: all-gather of the activations and routing tables, each rank runs its
  experts over every token routed to them, reduce-scatter of the partial outputs (whole experts per
  rank + reduction combine is what the reference's experimental EP does,
  crates/devgen/src/mla.rs:13016-13021).

Symmetric memory comes from ``torch.distributed._symmetric_memory`` (CUDA VMM handles exchanged
through the process group); only plain peer loads / stores are issued by this build's kernels.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import gemm as gemm_ops, native, rowops

FP8, BF16, F32, I32 = torch.float8_e4m3fn, torch.bfloat16, torch.float32, torch.int32


class EpArgs(C.Structure):
    _fields_ = [("peer", C.c_uint64 * 8), ("cnt_all", C.c_uint64), ("cnt_flag", C.c_uint64), ("data_ctr", C.c_uint64),
                ("y_flag", C.c_uint64), ("recv_x", C.c_uint64), ("recv_sx", C.c_uint64), ("y", C.c_uint64),
                ("W", C.c_int32), ("me", C.c_int32), ("E", C.c_int32), ("e_local", C.c_int32), ("Rmax", C.c_int32),
                ("H", C.c_int32), ("epoch", C.c_uint64), ("status", C.c_uint64), ("deadline_ns", C.c_uint64),
                ("trace", C.c_uint64)]


def _align(x, a=256):
    return (x + a - 1) // a * a


class EpComm:
    def __init__(self, rank: int, world: int, spec, max_rows: int, impl: str = "fused", deadline_ms: int = 2000, n_cta: int = 148):
        self.rank, self.world, self.impl = rank, world, impl
        self.dev = torch.device("cuda", torch.cuda.current_device())
        moe = next(l.ffn for l in spec.layers if l.ffn.kind == "moe")
        self.E, self.k, self.H = moe.n_experts, moe.top_k, spec.hidden
        self.e_local = self.E // world
        self.n_cta = n_cta
        self.deadline_ms = deadline_ms
        self.Rmax = world * max_rows * self.k + max_rows      # routed rows from every rank + this rank's own rows for a stacked shared expert
        self.timing = None            # set to a dict to collect CUDA-event phase times (debug aid, eager mode only)
        if impl != "fused":
            return
        import torch.distributed._symmetric_memory as symm
        KB = self.H // 128
        off, lay = 0, {}
        for name, nbytes in (("cnt_all", world * self.E * 4), ("cnt_flag", world * 128), ("data_ctr", 128), ("y_flag", world * 128),
                             ("recv_x", self.Rmax * self.H), ("recv_sx", KB * self.Rmax * 4), ("y", self.Rmax * self.H * 2)):
            lay[name] = off
            off = _align(off + nbytes)
        self.buf = symm.empty(off, dtype=torch.uint8, device=self.dev)
        self.buf.zero_()
        self.hdl = symm.rendezvous(self.buf, dist.group.WORLD)
        torch.cuda.synchronize()
        dist.barrier()
        self.lay = lay
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.cursor = torch.zeros(self.E + 1, dtype=I32, device=self.dev)   # +1: CTA counter of the push kernel
        self.grp_off = torch.zeros(self.e_local + 2, dtype=I32, device=self.dev)        # +1: stacked shared expert
        self.tile_prefix = torch.zeros(self.e_local + 2, dtype=I32, device=self.dev)
        self.pair_dest = torch.zeros(max_rows * self.k, dtype=I32, device=self.dev)
        a = EpArgs()
        ptrs = list(self.hdl.buffer_ptrs)
        for i in range(8):
            a.peer[i] = ptrs[i] if i < world else 0
        for name in ("cnt_all", "cnt_flag", "data_ctr", "y_flag", "recv_x", "recv_sx", "y"):
            setattr(a, name, lay[name])
        a.W, a.me, a.E, a.e_local, a.Rmax, a.H = world, rank, self.E, self.e_local, self.Rmax, self.H
        a.epoch = self.epoch.data_ptr()
        a.status = native.status_word(self.dev).data_ptr()
        a.deadline_ns = deadline_ms * 1_000_000
        a.trace = 0
        self.args = a
        self.recv_x = self.buf[lay["recv_x"]:lay["recv_x"] + self.Rmax * self.H].view(FP8).view(self.Rmax, self.H)
        self.recv_sx = self.buf[lay["recv_sx"]:lay["recv_sx"] + KB * self.Rmax * 4].view(F32).view(KB, self.Rmax)
        self.y = self.buf[lay["y"]:lay["y"] + self.Rmax * self.H * 2].view(BF16).view(self.Rmax, self.H)
        self.data_ctr_ptr = self.buf.data_ptr() + lay["data_ctr"]

    # ---- fused arm -----------------------------------------------------------------------------
    def dispatch(self, eng, st, ins, counts_done=False):
        """Counts + push for the MoE instruction `ins`; called as soon as the routing table exists so
        the transfer overlaps the shared-expert GEMMs that sit between router and experts.  ``counts_done``: the fused
        routing kernel already published this rank's counts (its last CTA does what the counts kernel does)."""
        if self.impl != "fused":
            return
        h, table = eng.tensor(st, ins.t[1]), eng.tensor(st, ins.t[2])
        T, k, H = st.rows, self.k, self.H
        xq, sx = eng._quant_of(st, ins.t[1], 0, H, h)
        ap = C.addressof(self.args)
        self._mark("t0")
        if not counts_done:
            native.call("plow_ep_counts", ap, table, T * k, self.cursor)
        self._mark("counts")
        native.call("plow_ep_push", ap, table, T * k, k, xq, sx, sx.stride(0), self.cursor, self.grp_off, self.tile_prefix,
                    self.pair_dest, self.n_cta, T if ins.i[6] else 0)
        self._mark("push")
        st.scratch["ep_dispatched"] = ins.i[7]

    def args_ptr(self) -> int:
        return C.addressof(self.args)

    def device_trace(self, on: bool):
        """Debug aid: device-side (tag, globaltimer) marks of the EP kernels.  Only effective for eager launches
        issued after the call (captured graphs keep the arguments they were captured with)."""
        if on:
            self._trace = torch.zeros(1 + 2 * 4000, dtype=torch.int64, device=self.dev)
            self.args.trace = self._trace.data_ptr()
        else:
            self.args.trace = 0

    def device_trace_rows(self):
        t = self._trace.cpu()
        n = min(int(t[0]), 4000)
        return [(int(t[1 + 2 * i]), int(t[2 + 2 * i])) for i in range(n)]

    def _mark(self, name):
        if self.timing is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.timing.setdefault("_ev", []).append((name, ev))

    def timing_report(self):
        evs = self.timing.pop("_ev", [])
        torch.cuda.synchronize()
        out = {}
        for (n0, e0), (n1, e1) in zip(evs, evs[1:]):
            if n1 != "t0":
                out.setdefault(n1, []).append(e0.elapsed_time(e1) * 1e3)
        return {k: round(sum(v) / len(v), 1) for k, v in out.items()}

    def moe_experts(self, eng, st, ins):
        if self.impl == "nccl":
            return self._moe_nccl(eng, st, ins)
        y_out, h, table = (eng.tensor(st, ins.t[k]) for k in range(3))
        shared = eng.tensor(st, ins.t[5]) if ins.t[5] != 0xFFFF else None
        F = ins.i[3]
        sg = bool(ins.i[6])               # shared expert stacked behind the local routed experts (group e_local)
        ng = self.e_local + (1 if sg else 0)
        T, k, H = st.rows, self.k, self.H
        ap = C.addressof(self.args)
        if st.scratch.get("ep_dispatched") != ins.i[7]:
            self.dispatch(eng, st, ins)
        st.scratch["ep_dispatched"] = None
        self._mark("shared_etc")
        w1, s1 = eng.static_q[ins.t[3]]
        w2, s2 = eng.static_q[ins.t[4]]
        wait = (self.data_ctr_ptr, self.epoch.data_ptr(), self.world, self.deadline_ms)
        per = max(1, self.world * T * k // self.E)
        R = self.world * T * k + (T if sg else 0)   # rows this rank can receive for this program
        rx, rsx, ry = self.recv_x[:R], self.recv_sx, self.y[:R]
        if per <= 64:
            bn = 32 if per <= 32 else 64
            hq, shq = gemm_ops.gemm(rx, w1, sx=rsx, sw=s1, dual=True, n_out=F, n_experts=ng, grp_off=self.grp_off,
                                    swap=True, bn=bn, quant_out=True, ld_syq=R, wait=wait)
            self._mark("gemm1")
            gemm_ops.gemm(hq, w2, sx=shq, sw=s2, n_out=H, n_experts=ng, grp_off=self.grp_off, swap=True, bn=bn, out=ry)
            self._mark("gemm2")
        else:
            hb = gemm_ops.gemm(rx, w1, sx=rsx, sw=s1, dual=True, n_out=F, n_experts=ng, grp_off=self.grp_off,
                               tile_prefix=self.tile_prefix, swap=False, bn=64, wait=wait)
            hq, shq = rowops.quant_act(hb)
            gemm_ops.gemm(hq, w2, sx=shq, sw=s2, n_out=H, n_experts=ng, grp_off=self.grp_off,
                          tile_prefix=self.tile_prefix, swap=False, bn=128, out=ry)
        # the combine kernel first signals that this rank's outputs can be pulled, then waits for the other ranks' signals
        native.call("plow_ep_combine", ap, y_out, shared, table, self.pair_dest, T, k, self.grp_off[self.e_local:] if sg else None, 1)
        self._mark("combine")

    # ---- NCCL baseline arm ---------------------------------------------------------------------
    def _moe_nccl(self, eng, st, ins):
        y_out, h, table = (eng.tensor(st, ins.t[k]) for k in range(3))
        shared = eng.tensor(st, ins.t[5]) if ins.t[5] != 0xFFFF else None
        F = ins.i[3]
        T, k, H, W = st.rows, self.k, self.H, self.world
        hg = torch.empty(W * T, H, dtype=BF16, device=self.dev)
        tg = torch.empty(W * T, k, 2, dtype=I32, device=self.dev)
        dist.all_gather_into_tensor(hg, h.contiguous())
        dist.all_gather_into_tensor(tg, table.contiguous())
        sg = bool(ins.i[6])               # shared expert stacked behind the local routed experts: its rows are this rank's tokens
        ng = self.e_local + (1 if sg else 0)
        n_rows = W * T * k + (T if sg else 0)
        grp_off, tile_prefix, row_of_pair, pair_of_row = rowops.moe_align(tg, self.rank * self.e_local, self.e_local,
                                                                          shared_rows=T if sg else 0, shared_tok_base=self.rank * T)
        xq, sx = rowops.quant_act(hg)
        xs, sxs = rowops.moe_gather(xq, sx, pair_of_row, grp_off[ng:], n_rows, k)
        w1, s1 = eng.static_q[ins.t[3]]
        w2, s2 = eng.static_q[ins.t[4]]
        per = max(1, W * T * k // self.E)
        if per <= 64:
            bn = 32 if per <= 32 else 64
            hq, shq = gemm_ops.gemm(xs, w1, sx=sxs, sw=s1, dual=True, n_out=F, n_experts=ng, grp_off=grp_off,
                                    swap=True, bn=bn, quant_out=True, ld_syq=n_rows)
            yo = gemm_ops.gemm(hq, w2, sx=shq, sw=s2, n_out=H, n_experts=ng, grp_off=grp_off, swap=True, bn=bn)
        else:
            hb = gemm_ops.gemm(xs, w1, sx=sxs, sw=s1, dual=True, n_out=F, n_experts=ng, grp_off=grp_off,
                               tile_prefix=tile_prefix, swap=False, bn=64)
            hq, shq = rowops.quant_act(hb)
            yo = gemm_ops.gemm(hq, w2, sx=shq, sw=s2, n_out=H, n_experts=ng, grp_off=grp_off, tile_prefix=tile_prefix,
                               swap=False, bn=128)
        part = rowops.moe_combine(yo, None, tg, row_of_pair, W * T, H)
        mine = torch.empty(T, H, dtype=BF16, device=self.dev)
        dist.reduce_scatter_tensor(mine, part)
        if sg:
            idx = grp_off[self.e_local:self.e_local + 1].long() + torch.arange(T, device=self.dev)
            torch.add(mine, torch.index_select(yo, 0, idx), out=y_out)
        elif shared is not None:
            torch.add(mine, shared, out=y_out)
        else:
            y_out.copy_(mine)
