"""Kernel capability registry: which hand-written sm_100a kernels exist, what shapes they accept and what they
cost in registers / shared memory / TMEM, so the emitter selects only what the runtime can run.

Specs are declared here; resources are filled from the build's ptxas report (``-Xptxas -v`` lines captured by
``plow_b200/build.py``) and the exported entry points are probed from the built library.
Reference: crates/kernelcaps/src/{select,probe,resource}.rs."""
from __future__ import annotations

import re
from dataclasses import dataclass, field


@dataclass
class KernelSpec:
    name: str                 # exported launcher symbol
    op: str                   # graph / packet op it implements
    dtypes: tuple             # operand dtypes accepted
    constraints: dict = field(default_factory=dict)   # attr -> allowed values / (lo, hi) range / callable
    uses: tuple = ()          # ISA features: tcgen05, tmem, tma, peer
    smem_bytes: int = 0
    tmem_cols: int = 0
    regs: int = 0             # filled from the ptxas report
    alias_group: str = ""     # kernels that may stand in for one another


REGISTRY = [
    KernelSpec("plow_gemm", "linear", ("bf16", "e4m3"), dict(k_multiple=64), ("tcgen05", "tmem", "tma"), 203776, 512, alias_group="gemm"),
    KernelSpec("plow_gemm", "linear_glu", ("bf16", "e4m3"), dict(n_multiple=128), ("tcgen05", "tmem", "tma"), 203776, 512, alias_group="gemm"),
    KernelSpec("plow_gemm", "moe_experts", ("bf16", "e4m3"), dict(n_multiple=128), ("tcgen05", "tmem", "tma"), 203776, 512, alias_group="gemm"),
    KernelSpec("plow_gemm", "gemm_xreduce", ("bf16", "e4m3"), dict(rows=(1, 64), n_multiple=8), ("tcgen05", "tmem", "tma", "peer"), 203776, 512),
    KernelSpec("plow_gqa_attention", "attention", ("bf16",), dict(head_dim=(128, 256), group_pow2=True), ("tcgen05", "tmem", "tma"), 198656, 256),
    KernelSpec("plow_rope_kv", "rope_kv", ("bf16",), dict(head_dim_multiple=8)),
    KernelSpec("plow_mla_decode", "mla_attention", ("e4m3",), dict(heads=(128,), kv_lora=(512,), qk_rope=(64,)), ("tcgen05", "tmem", "tma"), 203776, 512),
    KernelSpec("plow_mla_absorb", "mla_attention", ("bf16",), dict(qk_nope=(128,)), ("tcgen05", "tmem", "tma")),
    KernelSpec("plow_mla_fold", "mla_attention", ("bf16",), dict(v_head=(128,), max_splits=(1, 8)), ("tcgen05", "tmem", "tma")),
    KernelSpec("plow_mla_kv_write", "mla_kv_write", ("e4m3",)),
    KernelSpec("plow_dsa_k_write", "dsa_k_write", ("e4m3",), dict(dim=(128,))),
    KernelSpec("plow_dsa_select", "dsa_topk", ("e4m3",), dict(heads=(64,), dim=(128,), max_len=(1, 1 << 20)), ("tcgen05", "tmem", "tma"), 26048, 64),
    KernelSpec("plow_gdn", "gdn", ("bf16",), dict(head_dim=(128,), conv=(4,))),
    KernelSpec("plow_gated_norm", "gated_norm", ("bf16",)),
    KernelSpec("plow_router_topk", "router_topk", ("f32",), dict(n_experts=(1, 1024))),
    KernelSpec("plow_sample", "sample", ("f32",)),
    KernelSpec("plow_rmsnorm", "rmsnorm", ("bf16",)),
    KernelSpec("plow_add_norm", "add_norm", ("bf16",)),
    KernelSpec("plow_interp_run", "row_segment", ("bf16",), dict(ops=("embed", "rmsnorm", "add_norm", "add", "silu_mul", "row_gather", "argmax"))),
    KernelSpec("plow_ep_push", "xa2a_dispatch", ("e4m3",), dict(world=(2, 8)), ("peer",)),
    KernelSpec("plow_ep_combine", "xa2a_combine", ("bf16",), dict(world=(2, 8)), ("peer",)),
    KernelSpec("plow_ag_push", "xgather_gemm", ("bf16",), dict(world=(2, 8)), ("peer",)),
]


def _ok(rule, v) -> bool:
    if callable(rule):
        return bool(rule(v))
    if isinstance(rule, tuple) and len(rule) == 2 and all(isinstance(x, int) for x in rule) and rule[0] < rule[1] and v not in rule:
        return rule[0] <= v <= rule[1]
    if isinstance(rule, tuple):
        return v in rule
    return v == rule


def select_kernel(op: str, dtype: str, isa_caps=("tcgen05", "tmem", "tma", "peer"), **attrs):
    """First registered kernel of ``op`` whose dtype, ISA needs and constraints accept ``attrs``; None when nothing fits
    (the emitter then reports the op as unsupported instead of emitting an instruction nothing can run)."""
    for k in REGISTRY:
        if k.op != op or dtype not in k.dtypes or any(u not in isa_caps for u in k.uses):
            continue
        good = True
        for name, rule in k.constraints.items():
            if name.endswith("_multiple"):
                a = name[:-9]
                if a in attrs and attrs[a] % rule:
                    good = False
            elif name == "group_pow2":
                g = attrs.get("group")
                if g is not None and (g & (g - 1)):
                    good = False
            elif name in attrs and not _ok(rule, attrs[name]):
                good = False
        if good:
            return k
    return None


def apply_ptxas_report(text: str) -> dict:
    """Parse ``ptxas info`` lines: {kernel symbol fragment -> (registers, spill bytes, static smem)}."""
    out, cur = {}, None
    for line in text.splitlines():
        m = re.search(r"Compiling entry function '([^']+)'", line)
        if m:
            cur = m.group(1)
            continue
        m = re.search(r"Used (\d+) registers", line)
        if m and cur:
            sm = re.search(r"(\d+) bytes smem", line)
            out[cur] = dict(regs=int(m.group(1)), smem=int(sm.group(1)) if sm else 0, spill=out.get(cur, {}).get("spill", 0))
        m = re.search(r"(\d+) bytes spill stores", line)
        if m and cur:
            out.setdefault(cur, {})["spill"] = int(m.group(1))
    return out


def resource_gate(report: dict, max_regs: int = 255, max_spill: int = 512) -> list:
    """Kernels of a build that violate the resource budget (spilling hot kernels are build failures in CI)."""
    return [k for k, v in report.items() if v.get("regs", 0) > max_regs or v.get("spill", 0) > max_spill]


def probe(lib) -> dict:
    """Which registered launchers the loaded library really exports."""
    return {k.name: hasattr(lib, k.name) for k in REGISTRY}
