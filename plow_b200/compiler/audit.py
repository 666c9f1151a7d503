"""Packet audits that complement the verifier: which backend has a body for every opcode a packet uses, and which
counters of a program do no work.

* :func:`audit_ops` classifies every opcode of every program against the body tables of a backend and refuses what is
  unclassified, before anything runs (the CPU interpreter would otherwise stop mid-step with "op not implemented").
  The CPU table is checked against the interpreter's own dispatch in the tests, the sm_100a table is the engine's
  handler map plus the row ops of the on-device interpreter.
* :func:`counter_report` walks a program's counter protocol: counters nobody waits on (their arrivals are wasted
  traffic unless the instruction is a sink), waits already implied by an earlier wait of the same unit (redundant
  polling), and the longest wait chain (the program's dependency depth).

Reference: crates/plowc/src/opaudit.rs:1-30 (refuse unclassified opcodes), crates/schedule/src/analysis/counters.rs
(dead-counter report).
"""
from __future__ import annotations

from . import packet as pk
from .packet import Op

# opcodes with a golden body in csrc/cpu/interp.cpp
CPU_OPS = frozenset({Op.NOP, Op.EMBED, Op.RMSNORM, Op.ADD_NORM, Op.GEMM, Op.ROPE_KV, Op.ATTN, Op.ROW_GATHER, Op.ARGMAX, Op.RESIDUAL,
                     Op.GLU, Op.MLA_KV_WRITE, Op.MLA_DECODE, Op.MLA_PREFILL, Op.DSA_INDEX, Op.DSA_TOPK, Op.ROUTER_TOPK, Op.MOE_GEMM,
                     Op.GDN_STEP, Op.GATED_NORM, Op.SIGMOID_GATE})
CLASSES = {
    "row": {Op.NOP, Op.EMBED, Op.RMSNORM, Op.ADD_NORM, Op.ROPE_KV, Op.ROW_GATHER, Op.ARGMAX, Op.SAMPLE, Op.RESIDUAL, Op.GLU, Op.QUANT_ACT,
            Op.MLA_KV_WRITE, Op.MLA_Q_ROPE, Op.MLA_ABSORB_Q, Op.MLA_FOLD_V, Op.DSA_INDEX, Op.ROUTER_TOPK, Op.MOE_ALIGN, Op.MOE_GATHER,
            Op.MOE_COMBINE, Op.GDN_CONV, Op.GDN_GATES, Op.GATED_NORM, Op.SIGMOID_GATE},
    "gemm": {Op.GEMM, Op.MOE_GEMM},
    "attention": {Op.ATTN, Op.MLA_DECODE, Op.MLA_PREFILL, Op.DSA_TOPK, Op.GDN_STEP, Op.GDN_CHUNK},
    "collective": {Op.XREDUCE, Op.XREDUCE_ADD_NORM, Op.XGATHER, Op.XREDUCE_SCATTER, Op.XA2A_DISPATCH, Op.XA2A_COMBINE, Op.XARGMAX_FIN,
                   Op.GEMM_XREDUCE, Op.XGATHER_GEMM},
}


def op_class(op: int) -> str | None:
    for name, ops in CLASSES.items():
        if op in ops:
            return name
    return None


def gpu_ops() -> frozenset:
    """Opcodes the sm_100a engine has a handler for (read from the engine's own table, so the audit cannot drift)."""
    from ..runtime import gpu_engine
    table = getattr(gpu_engine.GpuEngine, "_HANDLERS", None) or getattr(gpu_engine.GpuEngine, "HANDLERS", {})
    ext = {getattr(Op, n[5:].upper()) for n in dir(gpu_engine.GpuEngine) if n.startswith("_ext_") and hasattr(Op, n[5:].upper())}
    return frozenset(set(table) | ext)


# operand variants of an opcode that only the CPU interpreter implements: (name, predicate over an instruction).  The sm_100a
# engine refuses a packet that carries one when it loads it; the audit names them ahead of that.
CPU_ONLY_VARIANTS = (
    ("GEMM bias", lambda i: i.op in (Op.GEMM, Op.GEMM_XREDUCE) and bool(i.i[2] & pk.GEMM_BIAS)),
    ("GELU gate", lambda i: i.op in (Op.GEMM, Op.GEMM_XREDUCE) and bool(i.i[2] & (pk.GEMM_ACT_GELU_TANH | pk.GEMM_ACT_GELU_ERF))
     or i.op == Op.GLU and bool(i.i[0])),
    ("attention sinks", lambda i: i.op == Op.ATTN and i.t[5] != pk.T_NONE),
    ("biased clamped-GLU experts", lambda i: i.op == Op.MOE_GEMM and i.t[6] != pk.T_NONE),
    ("Kimi Delta Attention", lambda i: i.op == Op.GDN_STEP and i.i[4] == 1),
)


def cpu_only_variants(pkt: pk.Packet) -> list:
    return sorted({name for p in pkt.programs for ins in p.insts for name, pred in CPU_ONLY_VARIANTS if pred(ins)})


def audit_ops(pkt: pk.Packet, backend: str) -> dict:
    have = CPU_OPS if backend == "cpu" else gpu_ops()
    used, missing, unclassified = {}, set(), set()
    for p in pkt.programs:
        for ins in p.insts:
            op = Op(ins.op) if ins.op in Op._value2member_map_ else None
            if op is None or op_class(op) is None:
                unclassified.add(int(ins.op))
                continue
            used[op.name] = used.get(op.name, 0) + 1
            if op not in have:
                missing.add(op.name)
    variants = cpu_only_variants(pkt) if backend != "cpu" else []
    return dict(backend=backend, ok=not missing and not unclassified and not variants, cpu_only_variants=variants, used=dict(sorted(used.items())),
                by_class={c: sorted(n for n in used if op_class(Op[n]) == c) for c in CLASSES},
                missing=sorted(missing), unclassified=sorted(unclassified))


def counter_report(p: pk.Program) -> dict:
    """Counter i counts the entries of instruction i that have finished."""
    waited = set()
    redundant = 0
    depth = [0] * len(p.insts)
    for c in range(p.n_cu):
        seen: dict = {}                                  # counter -> highest target this unit has already waited for
        for e in p.stream[p.cu_ofs[c]:p.cu_ofs[c + 1]]:
            for (ctr, tgt) in p.waits[e.wait_ofs:e.wait_ofs + e.n_wait]:
                waited.add(ctr)
                if seen.get(ctr, -1) >= tgt:
                    redundant += 1
                seen[ctr] = max(seen.get(ctr, -1), tgt)
                depth[e.inst] = max(depth[e.inst], depth[ctr] + 1)
    produced = {e.inst for e in p.stream}
    last = len(p.insts) - 1
    dead = sorted(i for i in produced if i not in waited and i != last)
    return dict(counters=len(produced), waited=len(waited), dead=dead, redundant_waits=redundant,
                dependency_depth=max(depth) if depth else 0, waits=len(p.waits))
