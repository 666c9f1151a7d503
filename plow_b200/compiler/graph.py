"""Model-agnostic op-graph IR and the model zoo that builds it from a :class:`ModelSpec`.

A graph is a topologically ordered list of :class:`Node` over named :class:`Value` s.  Shapes are
symbolic in the row count (``R`` = rows of the token batch, ``S`` = sampled rows), which the
scheduler binds per program (prefill bucket / decode rung).  Builders emit *primitive* ops
(linear, rmsnorm, rope, add ...); :mod:`plow_b200.compiler.rewrite` fuses them into the ISA's
vocabulary.  Weight values carry the checkpoint tensor name — names are the weight contract.

Reference counterpart: crates/nn-graph (op.rs, graph.rs, builder.rs, models/*.rs).
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..models.config import ModelSpec
from ..utils.rope import mla_softmax_factor

R = "R"   # rows of the running program
S = "S"   # sampled rows (one per sequence that finishes a chunk)


@dataclass
class Value:
    name: str
    shape: tuple
    dtype: str                 # f32 | bf16 | e4m3 | i32
    kind: str = "act"          # weight | derived | gen | kv | state | act | input | output | peer
    shard_axis: int | None = None   # tensor-parallel shard axis of a weight
    meta: dict = field(default_factory=dict)


@dataclass
class Node:
    op: str
    inputs: list
    outputs: list
    attrs: dict = field(default_factory=dict)
    layer: int = -1
    site: str = ""             # fusion site name once rewritten


class Graph:
    def __init__(self, spec: ModelSpec, tp: int = 1, ep: int = 1, rank: int = 0):
        self.spec = spec
        self.tp, self.ep, self.rank = tp, ep, rank
        self.values: dict[str, Value] = {}
        self.nodes: list[Node] = []
        self._n = 0

    # ---- construction ---------------------------------------------------------------------
    def value(self, name, shape, dtype, kind="act", **kw) -> str:
        if name in self.values:
            return name
        self.values[name] = Value(name, tuple(shape), dtype, kind, **kw)
        return name

    def tmp(self, base, shape, dtype=None) -> str:
        self._n += 1
        return self.value(f"act.{base}.{self._n}", shape, dtype or self.spec.dtype)

    def add(self, op, inputs, outputs, layer=-1, **attrs) -> Node:
        for v in list(inputs) + list(outputs):
            if v is not None and v not in self.values:
                raise KeyError(f"{op}: unknown value {v}")
        n = Node(op, list(inputs), list(outputs), attrs, layer)
        self.nodes.append(n)
        return n

    def weight(self, name, shape, shard_axis=None, dtype=None) -> str:
        return self.value(name, shape, dtype or self.weight_dtype(), "weight", shard_axis=shard_axis)

    def weight_dtype(self) -> str:
        return self.spec.dtype

    # ---- queries --------------------------------------------------------------------------
    def producers(self) -> dict:
        return {o: n for n in self.nodes for o in n.outputs}

    def consumers(self) -> dict:
        c: dict[str, list] = {}
        for n in self.nodes:
            for i in n.inputs:
                if i is not None:
                    c.setdefault(i, []).append(n)
        return c

    def check_topological(self) -> None:
        seen = {k for k, v in self.values.items() if v.kind != "act"}
        for n in self.nodes:
            for i in n.inputs:
                if i is not None and self.values[i].kind == "act" and i not in seen:
                    raise ValueError(f"{n.op} reads {i} before it is produced")
            seen.update(n.outputs)

    def bind(self, shape, rows, samples):
        return tuple(rows if d == R else samples if d == S else d for d in shape)


# ------------------------------------------------------------------------------------------------
# builders
# ------------------------------------------------------------------------------------------------
def build_graph(spec: ModelSpec, tp: int = 1, ep: int = 1, rank: int = 0, emit_hidden: bool = False) -> Graph:
    """``emit_hidden`` makes the decoder's normed hidden state of every row an output (``out.hidden`` [R, H]): the input
    of a prediction-module drafter.  A spec with ``role == "mtp"`` (ModelSpec.drafter_spec) builds that drafter: rows
    carry a token and a hidden state (``in.hidden``), ``x = eh_proj([enorm(embed(token)) | hnorm(hidden)])`` runs through
    one decoder block with a KV cache of its own, and the outputs are the draft ids / logits and the block's hidden state
    of the sampled rows (``out.hidden`` [S, H]) for the next draft of the chain
    (reference: crates/devgen/src/mtp.rs, crates/plowrt/src/exec/gpu/spec.rs:1-12)."""
    g = Graph(spec, tp, ep, rank)
    H, V = spec.hidden, spec.vocab
    ndt = "f32" if spec.dtype == "f32" else "bf16"
    ids = g.value("in.ids", (R,), "i32", "input")
    g.value("in.pos", (R,), "i32", "input")
    g.value("in.seq", (R,), "i32", "input")
    g.value("in.sample_rows", (S,), "i32", "input")
    emb = g.weight("model.embed_tokens.weight", (V, H))
    x = g.tmp("x", (R, H))
    g.add("embed", [emb, ids], [x], scale=spec.embed_scale)
    mtp = spec.role == "mtp"
    if mtp:
        p0 = f"model.layers.{spec.name_base}"
        hid = g.value("in.hidden", (R, H), spec.dtype, "input")
        en, hn = g.tmp("en", (R, H)), g.tmp("hn", (R, H))
        g.add("rmsnorm", [x, g.weight(f"{p0}.enorm.weight", (H,), dtype=ndt)], [en], eps=spec.rms_eps, plus_one=spec.norm_plus_one)
        g.add("rmsnorm", [hid, g.weight(f"{p0}.hnorm.weight", (H,), dtype=ndt)], [hn], eps=spec.rms_eps, plus_one=spec.norm_plus_one)
        # eh_proj([e | h]) as two projections over the column halves of the checkpoint matrix: no concatenation pass
        halves = []
        for nm, src, lo in (("e", en, 0), ("h", hn, H)):
            w = g.value(f"cols/{p0}.eh_proj.weight.{nm}", (H, H), g.weight_dtype(), "derived",
                        meta=dict(op="cols", src=f"{p0}.eh_proj.weight", start=lo, stop=lo + H))
            y = g.tmp("y", (R, H))
            g.add("linear", [src, w], [y])
            halves.append(y)
        x = g.tmp("x", (R, H))
        g.add("add", halves, [x])
    for li, layer in enumerate(spec.layers):
        x = _decoder_layer(g, li, f"model.layers.{spec.name_base + li}", x, layer)
    fn = g.weight(f"model.layers.{spec.name_base}.shared_head.norm.weight" if mtp else "model.norm.weight", (H,), dtype=ndt)
    hf = g.value("out.hidden", (R, H), spec.dtype, "output") if emit_hidden and not mtp else g.tmp("h", (R, H))
    g.add("rmsnorm", [x, fn], [hf], eps=spec.rms_eps, plus_one=spec.norm_plus_one)
    if mtp:
        g.add("row_gather", [x, "in.sample_rows"], [g.value("out.hidden", (S, H), spec.dtype, "output")])
    hs = g.tmp("hs", (S, H))
    g.add("row_gather", [hf, "in.sample_rows"], [hs])
    logits = g.value("out.logits", (S, V), "f32", "output")
    out_ids = g.value("out.ids", (S,), "i32", "output")
    if tp > 1 and not spec.tie_embeddings and V % (tp * 128) == 0:
        # vocabulary-sharded lm_head: each rank streams V/tp rows, takes the arg-max of its shard as a packed
        # (score, ~global index) key and the ranks fold the keys; full logits are gathered for sampled requests
        # (reference: asset/shard.rs:1-40 "lm_head replicated or vocab-sharded + XArgmaxFin", dev_isa.h:224-238)
        head = g.weight("lm_head.weight", (V // tp, H), shard_axis=0)
        local = g.tmp("logits_l", (S, V // tp), "f32")
        g.add("linear", [hs, head], [local], out_f32=True)
        keys = g.tmp("amax_key", (S,), "i64")
        g.add("argmax", [local], [keys], packed=True, vocab_ofs=g.rank * (V // tp))
        g.add("xargmax_fin", [keys], [out_ids])
        g.add("xgather", [local], [logits], width=V // tp)
    else:
        head = emb if spec.tie_embeddings else g.weight("lm_head.weight", (V, H))
        g.add("linear", [hs, head], [logits], out_f32=True)
        g.add("argmax", [logits], [out_ids])
    g.check_topological()
    return g


def _decoder_layer(g: Graph, li: int, p: str, x: str, layer) -> str:
    """One pre-norm decoder block: ``li`` indexes its KV cache / recurrent state, ``p`` names its checkpoint tensors."""
    spec, tp = g.spec, g.tp
    H = spec.hidden
    ndt = "f32" if spec.dtype == "f32" else "bf16"
    ln1 = g.weight(f"{p}.input_layernorm.weight", (H,), dtype=ndt)
    h = g.tmp("h", (R, H))
    g.add("rmsnorm", [x, ln1], [h], layer=li, eps=spec.rms_eps, plus_one=spec.norm_plus_one)
    if layer.attn.kind == "gqa":
        o = _gqa_attention(g, li, p, h, layer.attn)
    elif layer.attn.kind == "mla":
        o = _mla_attention(g, li, p, h, layer.attn)
    elif layer.attn.kind == "kda":
        o = _kda_attention(g, li, p, h, layer.attn)
    else:
        o = _gdn_attention(g, li, p, h, layer.attn)
    if tp > 1:
        o = _xreduce(g, o, li)
    if spec.sandwich_norms:
        # four norms per layer: the attention output is normed before it joins the residual, and the MLP reads a norm of
        # its own (pre_feedforward) and is normed again behind (post_feedforward)
        on = g.tmp("h", (R, H))
        g.add("rmsnorm", [o, g.weight(f"{p}.post_attention_layernorm.weight", (H,), dtype=ndt)], [on], layer=li, eps=spec.rms_eps,
              plus_one=spec.norm_plus_one)
        o = on
    x2 = g.tmp("x", (R, H))
    g.add("add", [x, o], [x2], layer=li)
    ln2 = g.weight(f"{p}.{'pre_feedforward' if spec.sandwich_norms else 'post_attention'}_layernorm.weight", (H,), dtype=ndt)
    h2 = g.tmp("h", (R, H))
    g.add("rmsnorm", [x2, ln2], [h2], layer=li, eps=spec.rms_eps, plus_one=spec.norm_plus_one)
    if layer.ffn.kind == "dense":
        d = _dense_ffn(g, li, f"{p}.mlp", h2, layer.ffn.inter, act=layer.ffn.act)
        if tp > 1:
            d = _xreduce(g, d, li)
    else:
        d = _moe_ffn(g, li, f"{p}.{layer.ffn.block}", h2, layer.ffn)
    if spec.sandwich_norms:
        dn = g.tmp("h", (R, H))
        g.add("rmsnorm", [d, g.weight(f"{p}.post_feedforward_layernorm.weight", (H,), dtype=ndt)], [dn], layer=li, eps=spec.rms_eps,
              plus_one=spec.norm_plus_one)
        d = dn
    x3 = g.tmp("x", (R, H))
    g.add("add", [x2, d], [x3], layer=li)
    return x3


def _xreduce(g: Graph, v: str, li: int) -> str:
    out = g.tmp("xr", g.values[v].shape)
    g.add("xreduce", [v], [out], layer=li)
    return out


def _linear(g: Graph, li, x, wname, n_out, k_in, shard_axis=None, rows=R, bias=False, **attrs) -> str:
    """y = x . w^T (+ bias).  A column-parallel projection shards its bias with its rows; a row-parallel one is summed over
    the ranks afterwards, so only rank 0 adds the bias."""
    tp = g.tp
    n_l = n_out // tp if shard_axis == 0 else n_out
    k_l = k_in // tp if shard_axis == 1 else k_in
    w = g.weight(wname, (n_l, k_l), shard_axis=shard_axis)
    y = g.tmp("y", (rows, n_l), "f32" if attrs.get("out_f32") else None)     # the arena slot must match what the GEMM writes
    ins = [x, w]
    if bias and (shard_axis != 1 or g.rank == 0):
        ins.append(g.weight(wname[:-len("weight")] + "bias", (n_l,), shard_axis=0 if shard_axis == 0 else None,
                            dtype="f32" if g.spec.dtype == "f32" else "bf16"))
    g.add("linear", ins, [y], layer=li, **attrs)
    return y


def _gqa_attention(g: Graph, li, p, h, a) -> str:
    spec, tp = g.spec, g.tp
    H = spec.hidden
    nq, nkv, hd = a.n_heads // tp, max(1, a.n_kv_heads // tp), a.head_dim
    qd = a.n_heads * hd * (2 if a.gated else 1)
    q = _linear(g, li, h, f"{p}.self_attn.q_proj.weight", qd, H, shard_axis=0, bias=a.qkv_bias)
    k = _linear(g, li, h, f"{p}.self_attn.k_proj.weight", a.n_kv_heads * hd, H, shard_axis=0, bias=a.qkv_bias)
    v = _linear(g, li, h, f"{p}.self_attn.v_proj.weight", a.n_kv_heads * hd, H, shard_axis=0, bias=a.qkv_bias)
    gate = None
    if a.gated:
        qs, gate = g.tmp("q", ("R", nq * hd)), g.tmp("gate", (R, nq * hd))
        g.add("split_q_gate", [q], [qs, gate], layer=li, heads=nq, head_dim=hd)
        q = qs
    if a.qk_norm:
        qn = g.weight(f"{p}.self_attn.q_norm.weight", (hd,), dtype="f32" if spec.dtype == "f32" else "bf16")
        kn = g.weight(f"{p}.self_attn.k_norm.weight", (hd,), dtype="f32" if spec.dtype == "f32" else "bf16")
        q2, k2 = g.tmp("q", (R, nq * hd)), g.tmp("k", (R, nkv * hd))
        g.add("headnorm", [q, qn], [q2], layer=li, heads=nq, head_dim=hd, eps=spec.rms_eps, plus_one=spec.norm_plus_one)
        g.add("headnorm", [k, kn], [k2], layer=li, heads=nkv, head_dim=hd, eps=spec.rms_eps, plus_one=spec.norm_plus_one)
        q, k = q2, k2
    if a.rope_theta and a.rope_theta != spec.rope.theta:
        # a layer with a rotary base of its own (no scaling: the long-context scaling belongs to the global layers)
        rope = g.value("gen.rope.local", (spec.rope.max_pos, max(2, spec.rope.rot_dim)), "f32", "gen",
                       meta=dict(theta=a.rope_theta, rot_dim=spec.rope.rot_dim, scaling=None))
    else:
        rope = g.value("gen.rope", (spec.rope.max_pos, max(2, spec.rope.rot_dim)), "f32", "gen",
                       meta=dict(theta=spec.rope.theta, rot_dim=spec.rope.rot_dim, scaling=spec.rope.scaling))
    qr, kr = g.tmp("q", (R, nq * hd)), g.tmp("k", (R, nkv * hd))
    g.add("rope", [q, rope, "in.pos"], [qr], layer=li, heads=nq, head_dim=hd, rot_dim=spec.rope.rot_dim, pair_mode=spec.rope.pair_mode)
    g.add("rope", [k, rope, "in.pos"], [kr], layer=li, heads=nkv, head_dim=hd, rot_dim=spec.rope.rot_dim, pair_mode=spec.rope.pair_mode)
    kc = g.value(f"kv.{li}.k", ("P", 64, nkv, hd), spec.kv_dtype if spec.kv_dtype != "fp8" else "e4m3", "kv")
    vc = g.value(f"kv.{li}.v", ("P", 64, nkv, hd), spec.kv_dtype if spec.kv_dtype != "fp8" else "e4m3", "kv")
    # e4m3 cache: one f32 scale per (token, kv head) next to the cells, k scales then v scales of a token
    # (reference: runtime/common/dev_isa.h:388-398, the fp8 twins of HEADNORM_ROPE / FLASH_DECODE / FLASH_PREFILL)
    ksc = g.value(f"kv.{li}.s", ("P", 64, 2 * nkv), "f32", "kv") if spec.kv_dtype == "fp8" else None
    g.add("kv_write", [kr, v, "in.pos", "in.seq"], [kc, vc], layer=li, heads=nkv, head_dim=hd, kv_scales=ksc)
    ao = g.tmp("attn", (R, nq * hd))
    sinks = g.weight(f"{p}.self_attn.sinks", (nq,), shard_axis=0, dtype="f32") if a.sinks else None
    g.add("attention", [qr, kc, vc], [ao], layer=li, heads=nq, kv_heads=nkv, head_dim=hd, window=a.window,
          scale=a.scale or hd ** -0.5, kv_scales=ksc, sinks=sinks)
    if gate is not None:
        ag = g.tmp("attn", (R, nq * hd))
        g.add("sigmoid_gate", [ao, gate], [ag], layer=li)
        ao = ag
    return _linear(g, li, ao, f"{p}.self_attn.o_proj.weight", H, a.n_heads * hd, shard_axis=1, bias=a.o_bias)


def _dense_ffn(g: Graph, li, p, h, inter, rows=R, act="silu") -> str:
    H = g.spec.hidden
    gt = _linear(g, li, h, f"{p}.gate_proj.weight", inter, H, shard_axis=0, rows=rows)
    up = _linear(g, li, h, f"{p}.up_proj.weight", inter, H, shard_axis=0, rows=rows)
    m = g.tmp("glu", (rows, inter // g.tp))
    g.add("silu_mul", [gt, up], [m], layer=li, act=act)        # act(gate) * up; the op keeps its historical name
    return _linear(g, li, m, f"{p}.down_proj.weight", H, inter, shard_axis=1, rows=rows)


def _mla_attention(g: Graph, li, p, h, a) -> str:
    """Multi-head latent attention in absorbed form for decode (scores against the latent cache)
    and materialised K/V for prefill; both are expressed by one ``mla_attention`` node whose
    lowering picks the kernel per program role (reference: crates/devgen/src/mla.rs:6211-6323)."""
    spec, tp = g.spec, g.tp
    H = spec.hidden
    nh = a.n_heads // tp
    qh = a.qk_nope + a.qk_rope
    nd = "f32" if spec.dtype == "f32" else "bf16"
    if a.q_lora:
        qa = _linear(g, li, h, f"{p}.self_attn.q_a_proj.weight", a.q_lora, H)
        qn = g.weight(f"{p}.self_attn.q_a_layernorm.weight", (a.q_lora,), dtype=nd)
        qan = g.tmp("qa", (R, a.q_lora))
        g.add("rmsnorm", [qa, qn], [qan], layer=li, eps=spec.rms_eps, plus_one=False)
        q = _linear(g, li, qan, f"{p}.self_attn.q_b_proj.weight", a.n_heads * qh, a.q_lora, shard_axis=0)
    else:
        q = _linear(g, li, h, f"{p}.self_attn.q_proj.weight", a.n_heads * qh, H, shard_axis=0)
    kva = _linear(g, li, h, f"{p}.self_attn.kv_a_proj_with_mqa.weight", a.kv_lora + a.qk_rope, H)
    kvn = g.weight(f"{p}.self_attn.kv_a_layernorm.weight", (a.kv_lora,), dtype=nd)
    rope = g.value("gen.rope", (spec.rope.max_pos, max(2, spec.rope.rot_dim)), "f32", "gen",
                   meta=dict(theta=spec.rope.theta, rot_dim=spec.rope.rot_dim, scaling=spec.rope.scaling))
    kvd = "e4m3" if spec.kv_dtype == "fp8" else spec.kv_dtype
    cache = g.value(f"kv.{li}.latent", ("P", 64, a.kv_lora + a.qk_rope), kvd, "kv")
    inputs = [kva, kvn, rope, "in.pos", "in.seq"]
    outs = [cache]
    if spec.kv_dtype == "fp8":
        outs.append(g.value(f"kv.{li}.latent_scale", ("P", 64), "f32", "kv"))
    g.add("mla_kv_write", inputs, outs, layer=li, kv_lora=a.kv_lora, qk_rope=a.qk_rope, eps=spec.rms_eps,
          pair_mode=spec.rope.pair_mode)
    wkv_b = g.weight(f"{p}.self_attn.kv_b_proj.weight", (nh * (a.qk_nope + a.v_head), a.kv_lora), shard_axis=0)
    ao = g.tmp("attn", (R, nh * a.v_head))
    extra = []
    if a.index_heads:
        extra = [_dsa_select(g, li, p, h, qan if a.q_lora else h, a)]
    g.add("mla_attention", [q, rope, "in.pos", wkv_b] + outs + extra, [ao], layer=li, heads=nh, kv_lora=a.kv_lora,
          qk_nope=a.qk_nope, qk_rope=a.qk_rope, v_head=a.v_head, scale=qh ** -0.5 * mla_softmax_factor(spec.rope.scaling),
          pair_mode=spec.rope.pair_mode,
          sparse=bool(a.index_heads), topk=a.index_topk)
    return _linear(g, li, ao, f"{p}.self_attn.o_proj.weight", H, a.n_heads * a.v_head, shard_axis=1)


def _dsa_select(g: Graph, li, p, h, q_in, a) -> str:
    """DSA lightning indexer: per-token top-k KV positions (reference: runtime/nvidia/op_dsa.cuh,
    dev_isa.h:516-534)."""
    spec = g.spec
    H = spec.hidden
    qi = _linear(g, li, q_in, f"{p}.self_attn.indexer.wq_b.weight", a.index_heads * a.index_dim,
                 a.q_lora if a.q_lora else H)
    ki = _linear(g, li, h, f"{p}.self_attn.indexer.wk.weight", a.index_dim, H)
    wts = _linear(g, li, h, f"{p}.self_attn.indexer.weights_proj.weight", a.index_heads, H, out_f32=True)
    kn_w = g.weight(f"{p}.self_attn.indexer.k_norm.weight", (a.index_dim,), dtype="f32")
    kn_b = g.weight(f"{p}.self_attn.indexer.k_norm.bias", (a.index_dim,), dtype="f32")
    kcache = g.value(f"kv.{li}.index_k", ("P", 64, a.index_dim), "e4m3" if spec.kv_dtype == "fp8" else spec.kv_dtype, "kv")
    ksc = g.value(f"kv.{li}.index_k_scale", ("P", 64), "f32", "kv")
    g.add("dsa_k_write", [ki, kn_w, kn_b, "gen.rope", "in.pos", "in.seq"], [kcache, ksc], layer=li,
          dim=a.index_dim, rot_dim=spec.rope.rot_dim)
    sel = g.tmp("dsa_sel", (R, a.index_topk), "i32")
    g.add("dsa_topk", [qi, wts, kcache, ksc, "gen.rope", "in.pos", "in.seq"], [sel], layer=li,
          heads=a.index_heads, dim=a.index_dim, topk=a.index_topk, rot_dim=spec.rope.rot_dim)
    return sel


def _moe_ffn(g: Graph, li, p, h, f) -> str:
    """Router -> (dispatch) -> grouped expert GLU/down -> (combine) + shared expert.
    Expert weights are stacked per layer as derived tensors ``cat/<p>.experts.{gate_up,down}``;
    under expert parallelism a rank holds a contiguous range of experts (reference planner:
    crates/packet/src/moe_ep.rs)."""
    spec, ep = g.spec, g.ep
    H = spec.hidden
    E, k, F = f.n_experts, f.top_k, f.moe_inter
    e_local = E // ep
    if f.fused_experts:
        return _moe_fused_experts(g, li, p, h, f)
    gate_w = g.weight(f"{p}.gate.weight", (E, H), dtype="f32" if spec.dtype == "f32" else "bf16")
    logits = g.tmp("router", (R, E), "f32")
    g.add("linear", [h, gate_w], [logits], layer=li, out_f32=True, router=True)
    inputs = [logits]
    if f.has_bias:
        inputs.append(g.weight(f"{p}.gate.e_score_correction_bias", (E,), dtype="f32"))
    table = g.tmp("route", (R, k, 2), "i32")
    g.add("router_topk", inputs, [table], layer=li, n_experts=E, top_k=k, n_group=f.n_group,
          topk_group=f.topk_group, score=f.score, norm_topk=f.norm_topk, route_scale=f.route_scale)
    gate_n, up_n, down_n = ("w1", "w3", "w2") if f.expert_names == "w123" else ("gate_proj", "up_proj", "down_proj")
    w1 = g.value(f"cat/{p}.experts.gate_up.weight", (e_local * 2 * F, H), g.weight_dtype(), "derived",
                 meta=dict(op="stack_experts", parts=[gate_n, up_n], prefix=f"{p}.experts", n=E,
                           ep=ep, rank=g.rank))
    w2 = g.value(f"cat/{p}.experts.down.weight", (e_local * H, F), g.weight_dtype(), "derived",
                 meta=dict(op="stack_experts", parts=[down_n], prefix=f"{p}.experts", n=E, ep=ep, rank=g.rank))
    y = g.tmp("moe", (R, H))
    shared = None
    if f.n_shared:
        shared = _dense_ffn(g, li, f"{p}.shared_experts" if spec.family == "mla_moe" else f"{p}.shared_expert",
                            h, F * f.n_shared)
    g.add("moe_experts", [h, table, w1, w2] + ([shared] if shared else []), [y], layer=li, n_experts=E,
          e_local=e_local, top_k=k, inter=F, ep=ep, has_shared=bool(shared))
    return y


def _moe_fused_experts(g: Graph, li, p, h, f) -> str:
    """gpt_oss experts: a biased router, then experts that live in one checkpoint tensor per projection.  The derived
    tensors bring them into the stacked layout the expert op reads (per expert: gate rows, up rows | down rows) and the
    biases into the same order; the op's two float operands carry the GLU's clamp and its sigmoid slope."""
    spec, ep = g.spec, g.ep
    H = spec.hidden
    E, k, F = f.n_experts, f.top_k, f.moe_inter
    e_local = E // ep
    logits = _linear(g, li, h, f"{p}.router.weight", E, H, bias=True, out_f32=True, router=True)
    table = g.tmp("route", (R, k, 2), "i32")
    g.add("router_topk", [logits], [table], layer=li, n_experts=E, top_k=k, n_group=1, topk_group=1, score=f.score,
          norm_topk=f.norm_topk, route_scale=f.route_scale)

    def derived(tag, shape, kind, src, dtype=None):
        return g.value(f"cat/{p}.experts.{tag}", shape, dtype or g.weight_dtype(), "derived",
                       meta=dict(op="fused_experts", kind=kind, src=f"{p}.experts.{src}", n=E, ep=ep, rank=g.rank))

    bdt = "f32" if spec.dtype == "f32" else "bf16"
    w1 = derived("gate_up.weight", (e_local * 2 * F, H), "gate_up", "gate_up_proj")
    w2 = derived("down.weight", (e_local * H, F), "down", "down_proj")
    b1 = derived("gate_up.bias", (e_local * 2 * F,), "gate_up_bias", "gate_up_proj_bias", bdt)
    b2 = derived("down.bias", (e_local * H,), "down_bias", "down_proj_bias", bdt)
    y = g.tmp("moe", (R, H))
    g.add("moe_experts", [h, table, w1, w2], [y], layer=li, n_experts=E, e_local=e_local, top_k=k, inter=F, ep=ep,
          has_shared=False, bias1=b1, bias2=b2, swiglu_limit=f.swiglu_limit, swiglu_alpha=f.swiglu_alpha)
    return y


def _kda_attention(g: Graph, li, p, h, a) -> str:
    """Kimi Delta Attention (reference contract: runtime/common/dev_isa.h:711-840; emitter crates/devgen/src/kda.rs).
    One GEMM over [q_proj; k_proj; v_proj; b_proj], the low-rank forget-gate and output-gate projections, then one
    recurrent op per layer: short causal convolutions + SiLU on q | k | v, L2-normalised q / k, per-(head, key-channel)
    decay exp(g), delta-rule update of the [H, D, D] state, read of the updated state; a per-head RMSNorm gated by the
    sigmoid of the output-gate projection closes it.  Heads are not sharded: the op runs at TP 1."""
    spec = g.spec
    if g.tp != 1:
        raise ValueError("Kimi Delta Attention layers are not sharded: compile kimi_linear with --parallel ep or one GPU")
    H = spec.hidden
    nh, d = a.gdn_v_heads, a.gdn_head_dim
    sa = f"{p}.self_attn"
    for nm, shp in (("q_proj", (nh * d, H)), ("k_proj", (nh * d, H)), ("v_proj", (nh * d, H)), ("b_proj", (nh, H))):
        g.weight(f"{sa}.{nm}.weight", shp)
    wcat = g.value(f"cat/{sa}.qkvb_proj.weight", (3 * nh * d + nh, H), g.weight_dtype(), "derived",
                   meta=dict(op="cat", axis=0, parts=[f"{sa}.{n}.weight" for n in ("q_proj", "k_proj", "v_proj", "b_proj")], shard_axis=None))
    qkvb = g.tmp("qkvb", (R, 3 * nh * d + nh))
    g.add("linear", [h, wcat], [qkvb], layer=li)
    graw = _linear(g, li, _linear(g, li, h, f"{sa}.f_a_proj.weight", d, H), f"{sa}.f_b_proj.weight", nh * d, d)
    gate = _linear(g, li, _linear(g, li, h, f"{sa}.g_a_proj.weight", d, H), f"{sa}.g_b_proj.weight", nh * d, d)
    for nm in ("q_conv1d", "k_conv1d", "v_conv1d"):
        g.weight(f"{sa}.{nm}.weight", (nh * d, a.gdn_conv), dtype="f32")
    conv_w = g.value(f"cat/{sa}.qkv_conv1d.weight", (3 * nh * d, a.gdn_conv), "f32", "derived",
                     meta=dict(op="cat", axis=0, parts=[f"{sa}.{n}.weight" for n in ("q_conv1d", "k_conv1d", "v_conv1d")], shard_axis=None))
    a_log = g.weight(f"{sa}.A_log", (nh,), dtype="f32")
    dt_bias = g.weight(f"{sa}.dt_bias", (nh * d,), dtype="f32")
    conv_state = g.value(f"state.{li}.conv", ("B", 3 * nh * d, a.gdn_conv - 1), "f32", "state")
    ssm_state = g.value(f"state.{li}.ssm", ("B", nh, d, d), "f32", "state")
    o = g.tmp("kda", (R, nh * d))
    g.add("kda", [qkvb, graw, conv_w, a_log, dt_bias, "in.pos", "in.seq"], [o, conv_state, ssm_state], layer=li,
          heads=nh, head_dim=d, conv=a.gdn_conv, kda_mode=1, gate_floor=a.kda_gate_floor)
    nw = g.weight(f"{sa}.o_norm.weight", (d,), dtype="f32")
    on = g.tmp("kda", (R, nh * d))
    g.add("gated_norm", [o, gate, nw], [on], layer=li, heads=nh, head_dim=d, eps=spec.rms_eps, z_offset=0, gate_sigmoid=1)
    return _linear(g, li, on, f"{sa}.o_proj.weight", H, nh * d)


def _gdn_attention(g: Graph, li, p, h, a) -> str:
    """Gated delta-rule linear attention (reference semantics: runtime/nvidia/op_qwen_gdn.cuh,
    dev_isa.h:1259-1280): causal depthwise conv + SiLU over packed qkv, L2-normalised q/k,
    state S[V,K] per (sequence, v-head), gated RMSNorm on the way out."""
    spec, tp = g.spec, g.tp
    H = spec.hidden
    hk, hv, d = a.gdn_k_heads // tp, a.gdn_v_heads // tp, a.gdn_head_dim
    if a.gdn_split_proj:
        # qwen3_5 ships [q | k | v], z, b and a as four matrices: stacked, they are the two operands the recurrent op reads
        if tp != 1:
            raise ValueError("split gated-delta-rule projections (qwen3_5) are not sharded: compile with one GPU or --parallel ep")
        la = f"{p}.linear_attn"
        kd, vd = a.gdn_k_heads * d, a.gdn_v_heads * d
        wq = g.value(f"cat/{la}.in_proj_qkvz.weight", (2 * kd + 2 * vd, H), g.weight_dtype(), "derived",
                     meta=dict(op="cat", axis=0, parts=[f"{la}.in_proj_qkv.weight", f"{la}.in_proj_z.weight"], shard_axis=None))
        wb = g.value(f"cat/{la}.in_proj_ba.weight", (2 * a.gdn_v_heads, H), g.weight_dtype(), "derived",
                     meta=dict(op="cat", axis=0, parts=[f"{la}.in_proj_b.weight", f"{la}.in_proj_a.weight"], shard_axis=None))
        qkvz, ba = g.tmp("y", (R, 2 * kd + 2 * vd)), g.tmp("y", (R, 2 * a.gdn_v_heads))
        g.add("linear", [h, wq], [qkvz], layer=li)
        g.add("linear", [h, wb], [ba], layer=li)
    else:
        qkvz = _linear(g, li, h, f"{p}.linear_attn.in_proj_qkvz.weight", 2 * a.gdn_k_heads * d + 2 * a.gdn_v_heads * d, H, shard_axis=0)
        ba = _linear(g, li, h, f"{p}.linear_attn.in_proj_ba.weight", 2 * a.gdn_v_heads, H, shard_axis=0)
    conv_w = g.weight(f"{p}.linear_attn.conv1d.weight", ((2 * hk + hv) * d, a.gdn_conv), dtype="f32")
    a_log = g.weight(f"{p}.linear_attn.A_log", (hv,), dtype="f32")
    dt_bias = g.weight(f"{p}.linear_attn.dt_bias", (hv,), dtype="f32")
    conv_state = g.value(f"state.{li}.conv", ("B", (2 * hk + hv) * d, a.gdn_conv - 1), "f32", "state")
    ssm_state = g.value(f"state.{li}.ssm", ("B", hv, d, d), "f32", "state")
    o = g.tmp("gdn", (R, hv * d))
    g.add("gdn", [qkvz, ba, conv_w, a_log, dt_bias, "in.pos", "in.seq"], [o, conv_state, ssm_state], layer=li,
          k_heads=hk, v_heads=hv, head_dim=d, conv=a.gdn_conv)
    nw = g.weight(f"{p}.linear_attn.norm.weight", (d,), dtype="f32")
    on = g.tmp("gdn", (R, hv * d))
    g.add("gated_norm", [o, qkvz, nw], [on], layer=li, heads=hv, head_dim=d, eps=spec.rms_eps,
          z_offset=2 * hk * d + hv * d)
    return _linear(g, li, on, f"{p}.linear_attn.out_proj.weight", H, a.gdn_v_heads * d, shard_axis=1)
