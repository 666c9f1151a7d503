"""Graph rewriting: fuse primitive ops into the ISA's fused vocabulary.

Each rule is a small pattern matcher over the node list that replaces a group of nodes by one
fused node and records a *site* name.  Rules are tried to a fixed point; a rule only fires when
the cost model says the fused form moves fewer bytes / launches fewer kernels, and when every
intermediate value it swallows has no other consumer.  The applied sites are reported in
``build.json`` (fusion coverage), and the negative cases (a second consumer, mismatched shapes)
are covered by tests.

Reference counterpart: crates/rewrite (egglog rules in egl/rules.egg: rmsnorm-linear-fuse :25,
gated-mlp-fuse :52, residual-rmsnorm-fuse :100 ...).  There the rules run as equality
saturation; here they are directed rewrites with a cost gate, which is what reaches the
emitter in both systems (only fused-site names cross into code generation).
"""
from __future__ import annotations

from dataclasses import dataclass

from . import costmodel
from .graph import Graph, Node, R


@dataclass
class Site:
    rule: str
    layer: int
    saved_bytes_per_row: int
    nodes_removed: int


def _single_use(cons, v, by: Node) -> bool:
    c = cons.get(v, [])
    return len(c) == 1 and c[0] is by


def _cat_weight(g: Graph, names: list, tag: str) -> str:
    """Derived weight: row-wise concatenation of checkpoint tensors (all share K)."""
    ws = [g.values[n] for n in names]
    tail = tuple(ws[0].shape[1:])                  # (K,) for matrices, () for bias vectors
    assert all(tuple(w.shape[1:]) == tail for w in ws)
    rows = sum(w.shape[0] for w in ws)
    base, kind = names[0].rsplit(".", 2)[0], names[0].rsplit(".", 1)[1]
    name = f"cat/{base}.{tag}.{kind}"
    g.value(name, (rows,) + tail, ws[0].dtype, "derived",
            meta=dict(op="cat", axis=0, parts=list(names), shard_axis=ws[0].shard_axis),
            shard_axis=ws[0].shard_axis)
    return name


def _replace(g: Graph, old: list, new: list, at: str = "last") -> None:
    """Swap `old` nodes for `new`.  ``at="last"`` puts the fused nodes where the last swallowed
    node was (every input is produced by then); ``at="first"`` where the first one was (for
    rules whose inputs all precede the group and whose outputs are needed early)."""
    first = min(g.nodes.index(n) for n in old)
    last = max(g.nodes.index(n) for n in old)
    for n in old:
        g.nodes.remove(n)
    pos = first if at == "first" else last - (len(old) - 1)
    g.nodes[pos:pos] = new


# ------------------------------------------------------------------------------------------------
def rule_qkv_fuse(g: Graph, sites: list) -> bool:
    """linear(h,Wq), linear(h,Wk), linear(h,Wv) on the same input -> one linear over [Wq;Wk;Wv]."""
    cons = g.consumers()
    for n in g.nodes:
        if n.op != "linear" or not n.inputs[1].endswith("q_proj.weight"):
            continue
        h = n.inputs[0]
        sib = [m for m in cons.get(h, []) if m.op == "linear" and m.layer == n.layer]
        k = next((m for m in sib if m.inputs[1].endswith("k_proj.weight")), None)
        v = next((m for m in sib if m.inputs[1].endswith("v_proj.weight")), None)
        if k is None or v is None:
            continue
        nb = sum(len(x.inputs) > 2 for x in (n, k, v))
        if nb not in (0, 3):
            continue
        w = _cat_weight(g, [n.inputs[1], k.inputs[1], v.inputs[1]], "qkv_proj")
        bias = [_cat_weight(g, [n.inputs[2], k.inputs[2], v.inputs[2]], "qkv_proj")] if nb else []
        widths = [g.values[x.outputs[0]].shape[1] for x in (n, k, v)]
        y = g.tmp("qkv", (R, sum(widths)))
        fused = Node("linear", [h, w] + bias, [y], dict(split=widths), n.layer, "qkv-fuse")
        views = []
        ofs = 0
        for x, wd in zip((n, k, v), widths):
            views.append(Node("view", [y], [x.outputs[0]], dict(col_ofs=ofs, width=wd), n.layer))
            ofs += wd
        _replace(g, [n, k, v], [fused] + views, at="first")
        es = costmodel.dtype_bytes(g.values[h].dtype)
        sites.append(Site("qkv-fuse", n.layer, 2 * g.values[h].shape[1] * es, 2))
        return True
    return False


def rule_rope_kv_fuse(g: Graph, sites: list) -> bool:
    """view(q,k,v) [+ headnorm] + rope(q) + rope(k) + kv_write -> rope_kv on the fused qkv rows."""
    prod = g.producers()
    cons = g.consumers()
    for n in g.nodes:
        if n.op != "kv_write":
            continue
        kr, v = n.inputs[0], n.inputs[1]
        rk = prod.get(kr)
        if rk is None or rk.op != "rope":
            continue
        rq = next((m for m in g.nodes if m.op == "rope" and m.layer == n.layer and m is not rk), None)
        if rq is None:
            continue
        k_in, q_in = rk.inputs[0], rq.inputs[0]
        qn = kn = None
        hq, hk = prod.get(q_in), prod.get(k_in)
        swallowed = [rq, rk, n]
        has_norm = hq is not None and hq.op == "headnorm" and hk is not None and hk.op == "headnorm"
        q_user, k_user = (hq, hk) if has_norm else (rq, rk)
        if has_norm:
            qn, kn = hq.inputs[1], hk.inputs[1]
            q_in, k_in = hq.inputs[0], hk.inputs[0]
            swallowed += [hq, hk]
        # gated attention: the q projection carries [Q | gate] per head; the split is folded into the fused op
        gate_out = None
        sg = prod.get(q_in)
        if sg is not None and sg.op == "split_q_gate":
            if not _single_use(cons, sg.outputs[0], q_user):
                continue
            gate_out, q_in, q_user = sg.outputs[1], sg.inputs[0], sg
            swallowed.append(sg)
        vq, vk, vv = prod.get(q_in), prod.get(k_in), prod.get(v)
        if not all(x is not None and x.op == "view" for x in (vq, vk, vv)):
            continue
        if len({x.inputs[0] for x in (vq, vk, vv)}) != 1:
            continue
        if not (_single_use(cons, vq.outputs[0], q_user) and _single_use(cons, vk.outputs[0], k_user)
                and _single_use(cons, vv.outputs[0], n)):
            continue
        qkv = vq.inputs[0]
        swallowed += [vq, vk, vv]
        fused = Node("rope_kv", [qkv, qn, kn, rq.inputs[1], "in.pos", "in.seq"],
                     [rq.outputs[0], n.outputs[0], n.outputs[1]] + ([gate_out] if gate_out else []),
                     dict(gated=bool(gate_out), heads=rq.attrs["heads"], kv_heads=rk.attrs["heads"], head_dim=rq.attrs["head_dim"],
                          rot_dim=rq.attrs["rot_dim"], pair_mode=rq.attrs["pair_mode"],
                          eps=(hq.attrs["eps"] if has_norm else 0.0),
                          plus_one=(hq.attrs.get("plus_one", False) if has_norm else False),
                          kv_scales=n.attrs.get("kv_scales")),
                     n.layer, "rope-kv-fuse")
        _replace(g, swallowed, [fused])
        es = costmodel.dtype_bytes(g.values[qkv].dtype)
        sites.append(Site("rope-kv-fuse", n.layer, 2 * g.values[qkv].shape[1] * es, len(swallowed) - 1))
        return True
    return False


def rule_gated_mlp_fuse(g: Graph, sites: list) -> bool:
    """silu_mul(linear(h,Wg), linear(h,Wu)) -> linear_glu(h, [Wg;Wu])."""
    prod = g.producers()
    cons = g.consumers()
    for n in g.nodes:
        if n.op != "silu_mul":
            continue
        a, b = prod.get(n.inputs[0]), prod.get(n.inputs[1])
        if a is None or b is None or a.op != "linear" or b.op != "linear" or a.inputs[0] != b.inputs[0]:
            continue
        if not (_single_use(cons, a.outputs[0], n) and _single_use(cons, b.outputs[0], n)):
            continue
        w = _cat_weight(g, [a.inputs[1], b.inputs[1]], "gate_up_proj")
        fused = Node("linear_glu", [a.inputs[0], w], [n.outputs[0]], dict(act=n.attrs.get("act", "silu")), n.layer, "gated-mlp-fuse")
        _replace(g, [a, b, n], [fused])
        es = costmodel.dtype_bytes(g.values[a.outputs[0]].dtype)
        sites.append(Site("gated-mlp-fuse", n.layer, 4 * g.values[a.outputs[0]].shape[1] * es, 2))
        return True
    return False


def rule_residual_rmsnorm_fuse(g: Graph, sites: list) -> bool:
    """add(x, d) -> x2 ; rmsnorm(x2, γ) -> h   ==>   add_norm(x, d, γ) -> (x2, h)."""
    cons = g.consumers()
    for n in g.nodes:
        if n.op != "add":
            continue
        users = cons.get(n.outputs[0], [])
        norm = next((m for m in users if m.op == "rmsnorm" and m.inputs[0] == n.outputs[0]), None)
        if norm is None:
            continue
        # both outputs stay live: the sum feeds the next residual, the norm the next block
        fused = Node("add_norm", [n.inputs[0], n.inputs[1], norm.inputs[1]], [n.outputs[0], norm.outputs[0]],
                     dict(norm.attrs), norm.layer, "residual-rmsnorm-fuse")
        _replace(g, [n, norm], [fused])
        es = costmodel.dtype_bytes(g.values[n.outputs[0]].dtype)
        sites.append(Site("residual-rmsnorm-fuse", n.layer, g.values[n.outputs[0]].shape[1] * es, 1))
        return True
    return False


def rule_xreduce_add_norm_fuse(g: Graph, sites: list) -> bool:
    """xreduce(v) -> add_norm(x, ·, γ)  ==>  xreduce_add_norm(x, v, γ): the reduction, the residual
    add and the RMSNorm run in one pass over the peers' partials."""
    prod = g.producers()
    cons = g.consumers()
    for n in g.nodes:
        if n.op != "add_norm":
            continue
        xr = prod.get(n.inputs[1])
        if xr is None or xr.op != "xreduce" or not _single_use(cons, xr.outputs[0], n):
            continue
        fused = Node("xreduce_add_norm", [n.inputs[0], xr.inputs[0], n.inputs[2]], list(n.outputs),
                     dict(n.attrs), n.layer, "xreduce-add-norm-fuse")
        _replace(g, [xr, n], [fused])
        sites.append(Site("xreduce-add-norm-fuse", n.layer, 2 * g.values[n.outputs[0]].shape[1] * 2, 1))
        return True
    return False


def rule_gemm_xreduce_fuse(g: Graph, sites: list) -> bool:
    """linear(a, W_rowparallel) -> xreduce  ==>  gemm_xreduce: partial tiles are reduced through
    peer memory from inside the GEMM epilogue."""
    prod = g.producers()
    cons = g.consumers()
    for n in g.nodes:
        if n.op not in ("xreduce", "xreduce_add_norm"):
            continue
        src = n.inputs[0] if n.op == "xreduce" else n.inputs[1]
        lin = prod.get(src)
        if lin is None or lin.op != "linear" or not _single_use(cons, src, n) or n.op != "xreduce":
            continue
        fused = Node("gemm_xreduce", list(lin.inputs), list(n.outputs), dict(lin.attrs), n.layer, "gemm-xreduce-fuse")
        _replace(g, [lin, n], [fused])
        sites.append(Site("gemm-xreduce-fuse", n.layer, 2 * g.values[src].shape[1] * 2, 1))
        return True
    return False


def rule_mla_down_fuse(g: Graph, sites: list) -> bool:
    """q_a_proj and kv_a_proj_with_mqa share their input: one GEMM over [W_qa; W_kva]."""
    cons = g.consumers()
    for n in g.nodes:
        if n.op != "linear" or not n.inputs[1].endswith("q_a_proj.weight"):
            continue
        sib = next((m for m in cons.get(n.inputs[0], []) if m.op == "linear" and m.layer == n.layer
                    and m.inputs[1].endswith("kv_a_proj_with_mqa.weight")), None)
        if sib is None:
            continue
        w = _cat_weight(g, [n.inputs[1], sib.inputs[1]], "qkv_a_proj")
        widths = [g.values[n.outputs[0]].shape[1], g.values[sib.outputs[0]].shape[1]]
        y = g.tmp("qkv_a", (R, sum(widths)))
        fused = Node("linear", [n.inputs[0], w], [y], dict(split=widths), n.layer, "mla-down-fuse")
        views = [Node("view", [y], [n.outputs[0]], dict(col_ofs=0, width=widths[0]), n.layer),
                 Node("view", [y], [sib.outputs[0]], dict(col_ofs=widths[0], width=widths[1]), n.layer)]
        _replace(g, [n, sib], [fused] + views, at="first")
        sites.append(Site("mla-down-fuse", n.layer, g.values[n.inputs[0]].shape[1] * 2, 1))
        return True
    return False


def rule_moe_shared_group_fuse(g: Graph, sites: list) -> bool:
    """linear_glu(h, W_sh_gate_up) -> linear(., W_sh_down) -> moe_experts(h, ..., shared)  ==>  moe_experts with the
    shared expert stacked behind the routed ones as one more group that every row belongs to.  A shared expert with the
    routed experts' shape is then two more tiles' worth of work inside the grouped GEMMs instead of two few-tile
    launches of its own (decode: ~47 us of latency-bound kernels per layer become ~12 us of streamed weights)."""
    prod = g.producers()
    cons = g.consumers()
    if g.tp > 1:
        return False
    for n in g.nodes:
        if n.op != "moe_experts" or not n.attrs.get("has_shared") or n.attrs.get("shared_group"):
            continue
        h, table, w1, w2, shared = n.inputs
        down = prod.get(shared)
        if down is None or down.op != "linear" or not _single_use(cons, shared, n):
            continue
        glu = prod.get(down.inputs[0])
        if glu is None or glu.op != "linear_glu" or glu.inputs[0] != h or not _single_use(cons, glu.outputs[0], down):
            continue
        F, H = n.attrs["inter"], g.values[h].shape[1]
        wgu, wd = g.values[glu.inputs[1]], g.values[down.inputs[1]]
        if wgu.shape != (2 * F, H) or wd.shape != (H, F) or wgu.meta.get("op") != "cat":
            continue
        e_local = n.attrs["e_local"]
        m1, m2 = dict(g.values[w1].meta), dict(g.values[w2].meta)
        m1["tail"], m2["tail"] = list(wgu.meta["parts"]), [down.inputs[1]]
        base = w1[len("cat/"):].rsplit(".experts.", 1)[0]
        w1s = g.value(f"cat/{base}.experts_shared.gate_up.weight", ((e_local + 1) * 2 * F, H), g.values[w1].dtype, "derived", meta=m1)
        w2s = g.value(f"cat/{base}.experts_shared.down.weight", ((e_local + 1) * H, F), g.values[w2].dtype, "derived", meta=m2)
        attrs = dict(n.attrs)
        attrs["has_shared"], attrs["shared_group"] = False, True
        fused = Node("moe_experts", [h, table, w1s, w2s], list(n.outputs), attrs, n.layer, "moe-shared-group-fuse")
        _replace(g, [glu, down, n], [fused])
        sites.append(Site("moe-shared-group-fuse", n.layer, 2 * (F + H) * 2, 2))
        return True
    return False


# Of the two collective rules the add+norm fold goes first: a reduction that feeds a residual add and RMSNorm becomes
# one peer-memory kernel (all-reduce + add + norm, csrc/comm/tp_ar.cu) after a plain GEMM.  Measured on the dense 8B
# model at TP2, 64 decode rows: 6.40 ms per step this way, 7.28 ms with the reduction inside the GEMM epilogue
# (gemm-xreduce: its tile-by-tile exchange keeps the GEMM's CTAs waiting on peers) and 6.90 ms with NCCL.  gemm-xreduce
# still takes the reductions that no add+norm follows.
RULES = [rule_qkv_fuse, rule_rope_kv_fuse, rule_gated_mlp_fuse, rule_residual_rmsnorm_fuse,
         rule_xreduce_add_norm_fuse, rule_gemm_xreduce_fuse, rule_mla_down_fuse, rule_moe_shared_group_fuse]


def fuse(g: Graph, disable: set | None = None, max_iters: int = 100000) -> list:
    """Apply every enabled rule to a fixed point; returns the list of applied sites."""
    sites: list[Site] = []
    disable = disable or set()
    rules = [r for r in RULES if r.__name__.replace("rule_", "").replace("_", "-") not in disable]
    for _ in range(max_iters):
        if not any(r(g, sites) for r in rules):
            break
    g.check_topological()
    return sites


def coverage(sites: list) -> dict:
    out: dict[str, int] = {}
    for s in sites:
        out[s.rule] = out.get(s.rule, 0) + 1
    return out
