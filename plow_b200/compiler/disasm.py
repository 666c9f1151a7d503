"""Packet disassembler: one line per instruction with tensor names and immediates
(reference: crates/packet/src/disasm.rs, `plowrt disasm`)."""
from __future__ import annotations

from . import packet as pk


def disasm(pkt: pk.Packet, program: int = 0, limit: int = 200) -> str:
    p = pkt.programs[program]
    n_entries = [0] * len(p.insts)
    units = [set() for _ in p.insts]
    for c in range(p.n_cu):
        for e in p.stream[p.cu_ofs[c]:p.cu_ofs[c + 1]]:
            n_entries[e.inst] += 1
            units[e.inst].add(c)
    first_wait = {}
    for e in p.stream:
        first_wait.setdefault(e.inst, [w[0] for w in p.waits[e.wait_ofs:e.wait_ofs + e.n_wait]])
    lines = [f"; program {program}: role={pk.Role(p.role).name} rows={p.rows} rank={p.rank} insts={len(p.insts)} "
             f"stream={len(p.stream)} ctr={p.n_ctr} seg={p.n_seg} arena={p.arena_bytes}"]
    for k, ins in enumerate(p.insts[:limit]):
        try:
            name = pk.Op(ins.op).name
        except ValueError:
            name = f"OP{ins.op}"
        ts = " ".join(f"t{j}={pkt.tensors[h].name}" for j, h in enumerate(ins.t) if h != pk.T_NONE)
        iv = ",".join(str(v) for v in ins.i)
        fv = ",".join(f"{v:g}" for v in ins.f)
        lines.append(f"{k:5d} {name:<18} slices={ins.nslice:<4} units={len(units[k]):<4} waits={first_wait.get(k, [])} "
                     f"i=[{iv}] f=[{fv}] {ts}")
    if len(p.insts) > limit:
        lines.append(f"; ... {len(p.insts) - limit} more")
    return "\n".join(lines)
