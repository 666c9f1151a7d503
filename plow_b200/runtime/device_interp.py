"""Host side of the persistent sm_100a interpreter (csrc/cuda/interp_sm100.cu).

Uploads a program's tables exactly as the packet stores them (instructions, per-unit streams, waits,
successors), resolves every tensor handle of the program to a device pointer once, and launches one
cooperative interpreter kernel per *row segment*: a maximal run of consecutive instructions whose opcodes
have a body inside the interpreter.  GEMM / attention / collective instructions stay role kernels that the
engine launches between interpreter segments (reference: crates/plow-asset/src/segment_roles.rs,
runtime/nvidia/interp_sm120.cu).
"""
from __future__ import annotations

import struct

import numpy as np
import torch

from ..compiler import packet as pk
from ..compiler.packet import Op
from ..ops import native

ROW_OPS = {Op.NOP, Op.EMBED, Op.RMSNORM, Op.ADD_NORM, Op.RESIDUAL, Op.GLU, Op.ROW_GATHER, Op.ARGMAX}


def _dev_bytes(b: bytes, device):
    return torch.frombuffer(bytearray(b if b else b"\0" * 8), dtype=torch.uint8).to(device)


class DeviceInterp:
    def __init__(self, packet, prog, tensor_of, rows: int, samples: int, device, deadline_ms: int = 2000, trace: bool = False):
        """``tensor_of(handle)`` returns the torch tensor bound to a handle for this program (or None)."""
        self.prog, self.device, self.deadline_ms = prog, device, deadline_ms
        self.insts = _dev_bytes(b"".join(i.pack() for i in prog.insts), device)
        self.stream = _dev_bytes(b"".join(s.pack() for s in prog.stream), device)
        self.cu_ofs = torch.tensor(prog.cu_ofs, dtype=torch.int32, device=device)
        self.waits = _dev_bytes(b"".join(struct.pack("<II", c, t) for c, t in prog.waits), device)
        self.succs = torch.tensor(prog.succs if prog.succs else [0], dtype=torch.int32, device=device)
        ptrs = np.zeros(len(packet.tensors), dtype=np.uint64)
        self._keep = []
        for h in range(len(packet.tensors)):
            t = tensor_of(h)
            if t is not None:
                ptrs[h] = t.data_ptr()
                self._keep.append(t)
        self.tensors = torch.from_numpy(ptrs.view(np.int64)).to(device)
        aux = np.zeros((len(prog.insts), 2), dtype=np.int32)
        for k, ins in enumerate(prog.insts):
            out = packet.tensors[ins.t[0]] if ins.t[0] != pk.T_NONE else None
            d0 = int(out.dims[0]) if out is not None else -1
            aux[k, 0] = rows if d0 == -1 else samples if d0 == -2 else d0
            aux[k, 1] = int(out.dims[1]) if out is not None and len(out.dims) > 1 else 0
        self.aux = torch.from_numpy(aux).to(device)
        self.ctr = torch.zeros(max(1, prog.n_ctr) * 32, dtype=torch.int32, device=device)
        self.trace = torch.zeros(len(prog.stream), 40, dtype=torch.uint8, device=device) if trace else None
        self.n_cu = prog.n_cu
        self.launches = 0
        self._pc0 = {}

    def _pc0_for(self, lo: int):
        """Per unit, the first stream index whose instruction is >= lo (streams are ordered by instruction)."""
        if lo not in self._pc0:
            import bisect
            prog = self.prog
            insts = [s.inst for s in prog.stream]
            v = [bisect.bisect_left(insts, lo, prog.cu_ofs[c], prog.cu_ofs[c + 1]) for c in range(prog.n_cu)]
            self._pc0[lo] = torch.tensor(v, dtype=torch.int32, device=self.device)
        return self._pc0[lo]

    @staticmethod
    def segments(prog, eligible=None):
        """[(lo, hi, on_device)] covering the program: maximal runs of interpreter ops vs single role instructions."""
        out, k, n = [], 0, len(prog.insts)
        ok = lambda j: Op(prog.insts[j].op) in ROW_OPS and (eligible is None or eligible(j))
        while k < n:
            if ok(k):
                j = k
                while j < n and ok(j):
                    j += 1
                out.append((k, j, True))
                k = j
            else:
                out.append((k, k + 1, False))
                k += 1
        return out

    def run(self, lo: int, hi: int) -> None:
        native.call("plow_interp_run", self.insts, self.stream, self.cu_ofs, self.waits, self.succs, self.tensors, self.aux,
                    self._pc0_for(lo), self.ctr, self.trace, native.status_word(self.device), lo, hi, self.n_cu, self.deadline_ms)
        self.launches += 1

    def trace_records(self):
        """Decoded PlowTraceRec entries of the entries that ran (t_end != 0)."""
        if self.trace is None:
            return []
        raw = self.trace.cpu().numpy().tobytes()
        recs = []
        for k in range(len(self.prog.stream)):
            cu, pc, inst, op, ta, tr, te = struct.unpack_from("<IIIIQQQ", raw, 40 * k)
            if te:
                recs.append(dict(cu=cu, pc=pc, inst=inst, op=Op(op).name, t_arrive=ta, t_ready=tr, t_end=te))
        return recs
