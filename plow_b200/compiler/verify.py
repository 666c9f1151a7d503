"""Packet verifier: structural proofs obligations checked before anything is written.

The reference discharges these with a Lean checker over JSON IPC (crates/lean_verify, lean-plow/):
checkpoint D (queue order topological over counter edges), C (memory fit), E (wire format), F
(address map).  Here they are executable checks over the in-memory packet:

* **D / protocol** — every program's per-unit streams are in instruction order, every wait names a
  counter of an *earlier* instruction with the producer's exact entry count, and a host-side
  simulation of the counter protocol completes (no deadlock with all units resident).
* **C / memory**   — activation tensors whose lifetimes overlap never share arena bytes.
* **E / wire**     — serialise + parse round trip preserves every field.
* **F / address**  — every tensor handle an instruction names exists and is bound by class.
"""
from __future__ import annotations

import tempfile
from pathlib import Path

from . import packet as pk, schedule


def _check_protocol(p: pk.Program) -> list:
    bad = []
    n_entries = [0] * len(p.insts)
    for e in p.stream:
        n_entries[e.inst] += 1
    for c in range(p.n_cu):
        prev = -1
        for e in p.stream[p.cu_ofs[c]:p.cu_ofs[c + 1]]:
            if e.inst < prev:
                bad.append(f"unit {c}: stream not in instruction order")
                break
            prev = e.inst
    for e in p.stream:
        for (ctr, tgt) in p.waits[e.wait_ofs:e.wait_ofs + e.n_wait]:
            if ctr >= e.inst:
                bad.append(f"inst {e.inst} waits on later counter {ctr}")
            elif tgt != n_entries[ctr]:
                bad.append(f"inst {e.inst} waits for {tgt} arrivals of {ctr}, producer has {n_entries[ctr]} entries")
    if not schedule.simulate(p)["completed"]:
        bad.append("counter protocol simulation did not complete")
    return bad


def _check_memory(p: pk.Program, tensors: list, samples_of_rows) -> list:
    bad = []
    first, last = {}, {}
    for k, ins in enumerate(p.insts):
        for h in ins.t:
            if h != pk.T_NONE and tensors[h].tclass == pk.TClass.ACT:
                first.setdefault(h, k)
                last[h] = k
    acts = sorted(first)
    sizes = {h: schedule._bound_bytes(tensors[h], p.rows, samples_of_rows(p)) for h in acts}
    for i, a in enumerate(acts):
        if p.actmap[a] == pk.U64_MAX:
            bad.append(f"activation {tensors[a].name} has no arena offset")
            continue
        if p.actmap[a] + sizes[a] > p.arena_bytes:
            bad.append(f"activation {tensors[a].name} exceeds the arena")
        for b in acts[i + 1:]:
            if first[b] <= last[a] and first[a] <= last[b]:
                if p.actmap[a] < p.actmap[b] + sizes[b] and p.actmap[b] < p.actmap[a] + sizes[a]:
                    bad.append(f"live activations {tensors[a].name} and {tensors[b].name} overlap")
    return bad


def verify_packet(pkt: pk.Packet) -> dict:
    failures = []
    buckets = (pkt.section_json("serve.json") or {}).get("buckets", {})
    max_seqs = buckets.get("max_seqs", 64)

    def samples(p):
        return p.rows if p.role == pk.Role.DECODE else max(1, min(p.rows, max_seqs))

    for p in pkt.programs:
        tag = f"program(role={p.role},rows={p.rows},rank={p.rank})"
        try:
            pk.validate_program(p, len(pkt.tensors))
        except pk.PacketError as e:
            failures.append(f"{tag}: {e}")
            continue
        failures += [f"{tag}: {m}" for m in _check_protocol(p)]
        failures += [f"{tag}: {m}" for m in _check_memory(p, pkt.tensors, samples)]
    # wire round trip
    with tempfile.TemporaryDirectory() as d:
        f = Path(d) / "rt.pkt"
        pk.write_packet(pkt, f)
        try:
            back = pk.read_packet(f)
            if len(back.tensors) != len(pkt.tensors) or len(back.programs) != len(pkt.programs):
                failures.append("wire: table sizes changed in the round trip")
            else:
                for a, b in zip(pkt.programs, back.programs):
                    if [i.pack() for i in a.insts] != [i.pack() for i in b.insts] or a.waits != [tuple(w) for w in b.waits]:
                        failures.append("wire: program bytes changed in the round trip")
        except pk.PacketError as e:
            failures.append(f"wire: {e}")
    return dict(ok=not failures, failures=failures[:20], checks=["D:protocol", "C:memory", "E:wire", "F:address"],
                programs=len(pkt.programs))
