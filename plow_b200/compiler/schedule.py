"""Scheduling: slices, per-compute-unit streams, the counter DAG and the activation arena.

Input: a lowered instruction list with per-instruction read/write sets (tensor indices).
Output: a :class:`packet.Program`.

* **Dependencies**: RAW/WAW/WAR over tensor indices *and* over arena byte ranges (two
  activation tensors that share arena bytes are ordered through their readers), then a
  transitive reduction so an entry polls as few counters as possible.
* **Counters**: one per instruction; every stream entry bumps its instruction's counter once
  when its slices are globally visible; a consumer waits until the producer's counter reaches
  the producer's entry count (coarse dependency).
* **Streams**: a list scheduler hands the slices of each instruction to the compute units
  with the earliest estimated finish time (cost model), contiguous slice ranges per unit, so
  each unit's stream is in instruction order — which is what makes spin-waiting deadlock-free
  when all units are co-resident.
* **Arena**: first-fit over liveness intervals, 256-byte aligned.

Reference counterpart: crates/schedule (passes.rs, memory.rs, emit.rs) and the packet Builder's
``finish()`` (crates/packet/src/devbuild.rs:2003: transitive reduction, streams, waits/succs).
"""
from __future__ import annotations

from dataclasses import dataclass, field

from . import packet as pk

ALIGN = 256


@dataclass
class LInst:
    """A lowered instruction before scheduling."""
    inst: pk.Inst
    reads: list
    writes: list
    cost_us: float = 1.0
    work: int = 1            # independent work items available for slicing
    seg_class: str = "row"   # row | gemm | attn | comm — consecutive equal classes share a segment


def plan_arena(tensors: list, linsts: list, rows: int, samples: int):
    """Assign arena offsets to ACT tensors for one program.  Returns (actmap, arena_bytes,
    alias_deps) where alias_deps are extra (earlier_inst, later_inst) orderings required because
    two tensors share bytes."""
    n = len(tensors)
    first = [None] * n
    last = [None] * n
    for k, li in enumerate(linsts):
        for t in li.reads + li.writes:
            if t is None or t == pk.T_NONE:
                continue
            if first[t] is None:
                first[t] = k
            last[t] = k
    actmap = [pk.U64_MAX] * n
    live = []   # (ofs, size, tensor)
    placed = []  # (ofs, size, first, last, tensor)
    arena = 0
    order = sorted((t for t in range(n) if tensors[t].tclass == pk.TClass.ACT and first[t] is not None),
                   key=lambda t: first[t])
    alias_deps = []
    for t in order:
        size = _bound_bytes(tensors[t], rows, samples)
        size = (size + ALIGN - 1) // ALIGN * ALIGN
        # first fit among gaps left by tensors whose lifetime ended strictly before first[t]
        busy = sorted((o, s) for (o, s, f, l, _) in placed if not (l < first[t]))
        ofs = 0
        for o, s in busy:
            if ofs + size <= o:
                break
            ofs = max(ofs, o + s)
        for (o, s, f, l, u) in placed:
            if l < first[t] and o < ofs + size and ofs < o + s:
                alias_deps.append((u, t))
        placed.append((ofs, size, first[t], last[t], t))
        actmap[t] = ofs
        arena = max(arena, ofs + size)
    _ = live
    return actmap, arena, alias_deps


def _bound_bytes(t: pk.TensorEnt, rows: int, samples: int) -> int:
    n = pk.DTYPE_BYTES[pk.DType(t.dtype)]
    for d in t.dims:
        n *= rows if d == -1 else samples if d == -2 else d
    return n


def build_deps(linsts: list, alias_deps: list) -> list:
    """Per instruction, the set of earlier instructions it must wait for (transitively reduced)."""
    n = len(linsts)
    last_write: dict[int, int] = {}
    readers: dict[int, list] = {}
    deps = [set() for _ in range(n)]
    users_of: dict[int, list] = {}
    for k, li in enumerate(linsts):
        for t in li.reads:
            if t in last_write:
                deps[k].add(last_write[t])               # RAW
        for t in li.writes:
            if t in last_write:
                deps[k].add(last_write[t])               # WAW
            for r in readers.get(t, []):
                if r != k:
                    deps[k].add(r)                       # WAR
        for t in li.reads:
            readers.setdefault(t, []).append(k)
        for t in li.writes:
            last_write[t] = k
            readers[t] = []
        for t in li.reads + li.writes:
            users_of.setdefault(t, []).append(k)
    # arena aliasing: every user of the older tensor precedes the first writer of the newer one
    for old_t, new_t in alias_deps:
        new_users = users_of.get(new_t, [])
        if not new_users:
            continue
        w = new_users[0]
        for u in users_of.get(old_t, []):
            if u < w:
                deps[w].add(u)
    # transitive reduction with reachability bitsets
    reach = [0] * n
    out = []
    for k in range(n):
        ds = sorted(deps[k], reverse=True)
        keep = []
        acc = 0
        for d in ds:
            if not (acc >> d) & 1:
                keep.append(d)
                acc |= reach[d] | (1 << d)
        reach[k] = acc
        out.append(sorted(keep))
    return out


def schedule(linsts: list, n_cu: int, role: int, rows: int, rank: int, tensors: list, samples: int,
             max_slices: int | None = None) -> pk.Program:
    actmap, arena, alias_deps = plan_arena(tensors, linsts, rows, samples)
    deps = build_deps(linsts, alias_deps)
    n = len(linsts)
    # slices per instruction: as many as there is independent work, at most one per unit
    cap = max_slices or n_cu
    for li in linsts:
        li.inst.nslice = max(1, min(cap, li.work, 0xFFFF))
    # list scheduling: contiguous slice ranges to the units that free up first
    ready = [0.0] * n_cu
    finish = [0.0] * n
    per_cu = [[] for _ in range(n_cu)]   # (inst, slice0, nslice)
    n_entries = [0] * n
    seg_of = []
    seg = -1
    prev_cls = None
    for k, li in enumerate(linsts):
        if li.seg_class != prev_cls:
            seg += 1
            prev_cls = li.seg_class
        seg_of.append(seg)
        start = max([finish[d] for d in deps[k]] + [0.0])
        ns = li.inst.nslice
        units = sorted(range(n_cu), key=lambda c: (max(ready[c], start), c))[:min(ns, n_cu)]
        units.sort()
        base, extra = divmod(ns, len(units))
        s0 = 0
        per_slice = li.cost_us / ns
        for j, c in enumerate(units):
            cnt = base + (1 if j < extra else 0)
            if cnt == 0:
                continue
            per_cu[c].append((k, s0, cnt))
            t0 = max(ready[c], start)
            ready[c] = t0 + per_slice * cnt
            finish[k] = max(finish[k], ready[c])
            n_entries[k] += 1
            s0 += cnt
    # waits / succs
    waits, succs, stream, cu_ofs = [], [], [], [0]
    wait_ofs_of = {}
    for k in range(n):
        wait_ofs_of[k] = len(waits)
        for d in deps[k]:
            waits.append((d, n_entries[d]))
    succ_ofs_of = {}
    for k in range(n):
        succ_ofs_of[k] = len(succs)
        succs.append(k)
    for c in range(n_cu):
        for (k, s0, cnt) in per_cu[c]:
            stream.append(pk.StreamEnt(inst=k, slice0=s0, nslice=cnt, wait_ofs=wait_ofs_of[k],
                                       succ_ofs=succ_ofs_of[k], n_wait=len(deps[k]), n_succ=1, seg=seg_of[k]))
        cu_ofs.append(len(stream))
    prog = pk.Program(role=role, rows=rows, rank=rank, n_cu=n_cu, insts=[li.inst for li in linsts], stream=stream,
                      cu_ofs=cu_ofs, waits=waits, succs=succs, n_ctr=n, n_seg=seg + 1, actmap=actmap,
                      arena_bytes=arena)
    prog.est_us = max(finish) if finish else 0.0
    pk.validate_program(prog, len(tensors))
    return prog


def simulate(prog: pk.Program) -> dict:
    """Walk the streams with counter semantics on the host (no data): proves the program cannot
    deadlock when every unit is resident, and returns the op-major completion order.  The
    reference's `plowrt simulate` does the same over its packets (crates/plowrt/src/sim/mod.rs)."""
    ctr = [0] * prog.n_ctr
    pc = [prog.cu_ofs[c] for c in range(prog.n_cu)]
    order = []
    progressed = True
    while progressed:
        progressed = False
        for c in range(prog.n_cu):
            while pc[c] < prog.cu_ofs[c + 1]:
                e = prog.stream[pc[c]]
                if any(ctr[w] < tgt for (w, tgt) in prog.waits[e.wait_ofs:e.wait_ofs + e.n_wait]):
                    break
                for s in prog.succs[e.succ_ofs:e.succ_ofs + e.n_succ]:
                    ctr[s] += 1
                order.append((c, e.inst))
                pc[c] += 1
                progressed = True
    done = all(pc[c] == prog.cu_ofs[c + 1] for c in range(prog.n_cu))
    return dict(completed=done, order=order, counters=ctr)
