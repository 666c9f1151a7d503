"""Lowering: fused graph -> tensor table + instruction list -> scheduled programs -> packet.

One program is emitted per (role, row count, rank): prefill buckets and decode rungs, each with
its own streams, counters and arena map.  Weight tensors are declared by checkpoint name (the
names are the binding contract); derived tensors (row-concatenated projections, stacked expert
matrices, fp8 twins) carry a recipe in ``derived_weights.json`` that the loader executes.

Reference counterpart: crates/devgen (emit_dense_gqa lib.rs:10812, emit_glm_mla mla.rs:6081,
emit_glm_moe_ffn mla.rs:12981), Builder::{tensor,emit,finish} (crates/packet/src/devbuild.rs).
"""
from __future__ import annotations

import json

from . import costmodel, packet as pk, schedule
from .graph import Graph, R, S
from .hwspec import GpuSpec
from .packet import Op

DIM_ROWS, DIM_SAMPLES, DIM_PAGES, DIM_SLOTS = -1, -2, -3, -4
_SYM = {R: DIM_ROWS, S: DIM_SAMPLES, "P": DIM_PAGES, "B": DIM_SLOTS}
_DT = {"f32": pk.DType.F32, "bf16": pk.DType.BF16, "f16": pk.DType.F16, "e4m3": pk.DType.E4M3,
       "i32": pk.DType.I32, "u8": pk.DType.U8, "fp8": pk.DType.E4M3, "i64": pk.DType.I64}
_TC = {"weight": pk.TClass.WEIGHT, "derived": pk.TClass.DERIVED, "gen": pk.TClass.GEN, "kv": pk.TClass.KV,
       "state": pk.TClass.STATE, "act": pk.TClass.ACT, "input": pk.TClass.INPUT, "output": pk.TClass.OUTPUT,
       "peer": pk.TClass.PEER}
PAIR_MODE = {"half": 0, "interleaved": 1}


class Lowering:
    def __init__(self, g: Graph, hw: GpuSpec):
        self.g, self.hw = g, hw
        self.tensors: list[pk.TensorEnt] = []
        self.index: dict[str, int] = {}
        self.views: dict[str, tuple] = {}      # value -> (base value, col_ofs)
        self.derived: dict[str, dict] = {}
        self.gen: dict[str, dict] = {}
        for n in g.nodes:
            if n.op == "view":
                self.views[n.outputs[0]] = (n.inputs[0], n.attrs["col_ofs"])

    # ---- tensors -------------------------------------------------------------------------------
    def t(self, name) -> int:
        if name is None:
            return pk.T_NONE
        if name in self.views:
            name = self.views[name][0]
        if name not in self.index:
            v = self.g.values[name]
            dims = tuple(_SYM.get(d, d) for d in v.shape)
            ent = pk.TensorEnt(name=name, dtype=int(_DT[v.dtype]), tclass=int(_TC[v.kind]), dims=dims,
                               shard_axis=0xFFFFFFFF if v.shard_axis is None else v.shard_axis)
            if all(isinstance(d, int) and d >= 0 for d in dims):
                ent.bytes = ent.nbytes(0)
            self.index[name] = len(self.tensors)
            self.tensors.append(ent)
            if v.kind == "derived":
                self.derived[name] = v.meta
            if v.kind == "gen":
                self.gen[name] = v.meta
        return self.index[name]

    def xview(self, name) -> tuple:
        """(col offset, pitch) of an activation input; (0, 0) for a dense tensor."""
        if name in self.views:
            base, ofs = self.views[name]
            return ofs, self.g.values[base].shape[1]
        return 0, 0

    def width(self, name) -> int:
        return self.g.values[name].shape[-1]

    # ---- instructions --------------------------------------------------------------------------
    def lower(self, rows: int, samples: int, role: int) -> list:
        out = []
        g = self.g
        fp8w = g.spec.weight_quant == "fp8_block128"
        es = costmodel.dtype_bytes(g.spec.dtype)

        def rd(*names):
            return [self.t(x) for x in names if x is not None]

        def nrows(v):
            s0 = g.values[v].shape[0]
            return rows if s0 == R else samples if s0 == S else s0

        for n in g.nodes:
            a = n.attrs
            if n.op == "view":
                continue
            if n.op == "embed":
                ins = pk.Inst(Op.EMBED, f=(a.get("scale", 1.0), 0, 0), t=[self.t(n.outputs[0]), self.t(n.inputs[0]), self.t(n.inputs[1])],
                              i=[self.width(n.outputs[0])])
                out.append(schedule.LInst(ins, rd(n.inputs[0], n.inputs[1]), rd(n.outputs[0]),
                                          costmodel.rowwise_cost(rows, g.spec.hidden, 2, es).time_us(self.hw), rows))
            elif n.op == "rmsnorm":
                co, pitch = self.xview(n.inputs[0])
                ins = pk.Inst(Op.RMSNORM, f=(a["eps"], 0, 0), t=[self.t(n.outputs[0]), self.t(n.inputs[0]), self.t(n.inputs[1])],
                              i=[self.width(n.outputs[0]), int(a.get("plus_one", False)), 0, 0, 0, 0, co, pitch])
                out.append(schedule.LInst(ins, rd(n.inputs[0], n.inputs[1]), rd(n.outputs[0]),
                                          costmodel.rowwise_cost(nrows(n.outputs[0]), self.width(n.outputs[0]), 2, es).time_us(self.hw), nrows(n.outputs[0])))
            elif n.op == "add_norm":
                x_in, delta, gamma = n.inputs
                x_out, h_out = n.outputs
                ins = pk.Inst(Op.ADD_NORM, f=(a["eps"], 0, 0),
                              t=[self.t(h_out), self.t(x_in), self.t(delta), self.t(gamma), self.t(x_out)],
                              i=[self.width(h_out), int(a.get("plus_one", False))])
                out.append(schedule.LInst(ins, rd(x_in, delta, gamma), rd(h_out, x_out),
                                          costmodel.rowwise_cost(rows, self.width(h_out), 4, es).time_us(self.hw), rows))
            elif n.op == "add":
                ins = pk.Inst(Op.RESIDUAL, t=[self.t(n.outputs[0]), self.t(n.inputs[0]), self.t(n.inputs[1])],
                              i=[self.width(n.outputs[0])])
                out.append(schedule.LInst(ins, rd(*n.inputs), rd(n.outputs[0]),
                                          costmodel.rowwise_cost(rows, self.width(n.outputs[0]), 3, es).time_us(self.hw), rows))
            elif n.op in ("linear", "linear_glu", "gemm_xreduce"):
                x, w = n.inputs[0], n.inputs[1]
                wv = g.values[w]
                dual = n.op == "linear_glu"
                N = wv.shape[0] // (2 if dual else 1)
                K = wv.shape[1]
                m = nrows(n.outputs[0])
                quant = fp8w and wv.kind in ("weight", "derived") and not a.get("router") and not a.get("out_f32") \
                    and N % 128 == 0 and K % 128 == 0 and len(wv.shape) == 2
                flags = (pk.GEMM_DUAL_SILU | pk.ACT_FLAGS[a.get("act", "silu")] if dual else 0) | (pk.GEMM_OUT_F32 if a.get("out_f32") else 0) \
                    | (pk.GEMM_FP8_BLOCK if quant else 0)
                bias = n.inputs[2] if len(n.inputs) > 2 else None
                if bias and (dual or n.op == "gemm_xreduce" and g.rank != 0):
                    raise ValueError("a bias on a gated pair, or on a summed projection outside rank 0, has no lowering")
                flags |= pk.GEMM_BIAS if bias else 0
                co, pitch = self.xview(x)
                tile = costmodel.pick_gemm_tile(m, N, quant, dual)
                op = Op.GEMM_XREDUCE if n.op == "gemm_xreduce" else Op.GEMM
                ins = pk.Inst(op, t=[self.t(n.outputs[0]), self.t(x), self.t(w)] + ([self.t(None)] * 4 + [self.t(bias)] if bias else []),
                              i=[N, K, flags, int(tile["swap"]), tile["bn"], g.tp, co, pitch])
                c = costmodel.gemm_cost(m, N * (2 if dual else 1), K, 1 if quant else es, es)
                if op == Op.GEMM_XREDUCE:
                    c.link_bytes = costmodel.allreduce_cost(m, N, g.tp, es).link_bytes
                out.append(schedule.LInst(ins, rd(x, w, bias), rd(n.outputs[0]), c.time_us(self.hw, "e4m3" if quant else g.spec.dtype),
                                          max(1, N // 64), "gemm" if op == Op.GEMM else "comm"))
            elif n.op == "rope_kv":
                qkv, qn, kn, rope = n.inputs[0], n.inputs[1], n.inputs[2], n.inputs[3]
                q_out, kc, vc = n.outputs[:3]
                gate = n.outputs[3] if len(n.outputs) > 3 else None
                ksc = a.get("kv_scales")
                if ksc and gate:
                    raise ValueError("an e4m3 KV cache under gated attention is not supported (no operand slot left for the scales)")
                ins = pk.Inst(Op.ROPE_KV, f=(a.get("eps", 0.0), 0, 0),
                              t=[self.t(q_out), self.t(qkv), self.t(kc), self.t(vc), self.t(qn), self.t(kn), self.t(rope)]
                              + ([self.t(gate)] if gate else [self.t(ksc)] if ksc else []),
                              i=[a["heads"], a["kv_heads"], a["head_dim"], a["rot_dim"], PAIR_MODE[a["pair_mode"]],
                                 n.layer, int(a.get("plus_one", False)), int(bool(gate))])
                out.append(schedule.LInst(ins, rd(qkv, qn, kn, rope), rd(q_out, kc, vc, gate),
                                          costmodel.rowwise_cost(rows, self.width(qkv), 2, es).time_us(self.hw), rows))
            elif n.op == "attention":
                q, kc, vc = n.inputs
                mode = pk.ATTN_DECODE if role == pk.Role.DECODE else pk.ATTN_CAUSAL
                ins = pk.Inst(Op.ATTN, f=(a["scale"], 0, 0), t=[self.t(n.outputs[0]), self.t(q), self.t(kc), self.t(vc)]
                              + ([self.t(a.get("kv_scales")), self.t(a["sinks"])] if a.get("sinks") else
                                 [self.t(a["kv_scales"])] if a.get("kv_scales") else []),
                              i=[a["heads"], a["kv_heads"], a["head_dim"], a.get("window", 0), mode, n.layer])
                cost = costmodel.attention_decode_cost(rows * 2048, a["heads"], a["kv_heads"], a["head_dim"], a["head_dim"], es) \
                    if role == pk.Role.DECODE else costmodel.attention_prefill_cost(rows, rows, a["heads"], a["head_dim"], a["head_dim"])
                out.append(schedule.LInst(ins, rd(q, kc, vc), rd(n.outputs[0]), cost.time_us(self.hw),
                                          rows * a["heads"], "attn"))
            elif n.op == "row_gather":
                ins = pk.Inst(Op.ROW_GATHER, t=[self.t(n.outputs[0]), self.t(n.inputs[0]), self.t(n.inputs[1])],
                              i=[self.width(n.outputs[0])])
                out.append(schedule.LInst(ins, rd(*n.inputs), rd(n.outputs[0]), 1.0, samples))
            elif n.op == "argmax":
                ins = pk.Inst(Op.ARGMAX, t=[self.t(n.outputs[0]), self.t(n.inputs[0])],
                              i=[self.width(n.inputs[0]), int(a.get("packed", False)), int(a.get("vocab_ofs", 0))])
                out.append(schedule.LInst(ins, rd(n.inputs[0]), rd(n.outputs[0]), 2.0, samples))
            elif n.op == "xargmax_fin":
                ins = pk.Inst(Op.XARGMAX_FIN, t=[self.t(n.outputs[0]), self.t(n.inputs[0])], i=[g.tp])
                out.append(schedule.LInst(ins, rd(n.inputs[0]), rd(n.outputs[0]), 5.0, samples, "comm"))
            elif n.op == "xgather":
                ins = pk.Inst(Op.XGATHER, t=[self.t(n.outputs[0]), self.t(n.inputs[0])], i=[a["width"], g.tp])
                out.append(schedule.LInst(ins, rd(n.inputs[0]), rd(n.outputs[0]),
                                          costmodel.allreduce_cost(samples, a["width"] * g.tp, g.tp, 4).time_us(self.hw), samples, "comm"))
            elif n.op in ("xreduce", "xreduce_add_norm"):
                if n.op == "xreduce":
                    ins = pk.Inst(Op.XREDUCE, t=[self.t(n.outputs[0]), self.t(n.inputs[0])],
                                  i=[self.width(n.outputs[0]), g.tp])
                    reads, writes = rd(n.inputs[0]), rd(n.outputs[0])
                else:
                    x_in, part, gamma = n.inputs
                    x_out, h_out = n.outputs
                    ins = pk.Inst(Op.XREDUCE_ADD_NORM, f=(a["eps"], 0, 0),
                                  t=[self.t(h_out), self.t(x_in), self.t(part), self.t(gamma), self.t(x_out)],
                                  i=[self.width(h_out), int(a.get("plus_one", False)), g.tp])
                    reads, writes = rd(x_in, part, gamma), rd(h_out, x_out)
                out.append(schedule.LInst(ins, reads, writes,
                                          costmodel.allreduce_cost(rows, g.spec.hidden, g.tp, es).time_us(self.hw), rows, "comm"))
            else:
                out.append(self._lower_generic(n, rows, samples, role, rd))
        return out

    # Ops of the MLA / MoE / DSA / gated-delta families carry their parameters in the same fixed
    # fields; the table below names opcode, integer attributes and float attributes in order.
    _GENERIC = {
        "mla_kv_write": (Op.MLA_KV_WRITE, ["kv_lora", "qk_rope", "pair_mode"], ["eps"], "row"),
        "mla_attention": (Op.MLA_DECODE, ["heads", "kv_lora", "qk_nope", "qk_rope", "v_head", "pair_mode", "sparse", "topk"], ["scale"], "attn"),
        "dsa_k_write": (Op.DSA_INDEX, ["dim", "rot_dim"], [], "row"),
        "dsa_topk": (Op.DSA_TOPK, ["heads", "dim", "topk", "rot_dim"], [], "attn"),
        "router_topk": (Op.ROUTER_TOPK, ["n_experts", "top_k", "n_group", "topk_group", "score", "norm_topk"], ["route_scale"], "row"),
        "moe_experts": (Op.MOE_GEMM, ["n_experts", "e_local", "top_k", "inter", "ep", "has_shared", "shared_group"],
                        ["swiglu_limit", "swiglu_alpha"], "gemm"),
        "gdn": (Op.GDN_STEP, ["k_heads", "v_heads", "head_dim", "conv"], [], "attn"),
        "kda": (Op.GDN_STEP, ["heads", "heads", "head_dim", "conv", "kda_mode"], ["gate_floor"], "attn"),
        "gated_norm": (Op.GATED_NORM, ["heads", "head_dim", "z_offset", "gate_sigmoid"], ["eps"], "row"),
        "sigmoid_gate": (Op.SIGMOID_GATE, [], [], "row"),
        "split_q_gate": (Op.NOP, ["heads", "head_dim"], [], "row"),
        "headnorm": (Op.RMSNORM, ["head_dim", "plus_one", "heads"], ["eps"], "row"),
        "silu_mul": (Op.GLU, ["act_flag"], [], "row"),
        "rope": (Op.MLA_Q_ROPE, ["heads", "head_dim", "rot_dim", "pair_mode"], [], "row"),
        "kv_write": (Op.ROPE_KV, ["heads", "head_dim"], [], "row"),
    }

    def _lower_generic(self, n, rows, samples, role, rd) -> schedule.LInst:
        if n.op not in self._GENERIC:
            raise NotImplementedError(f"no lowering for graph op '{n.op}'")
        op, ikeys, fkeys, cls = self._GENERIC[n.op]
        if n.op == "mla_attention" and role != pk.Role.DECODE:
            op = Op.MLA_PREFILL

        def iv(k):
            v = n.attrs.get(k, 0)
            if k == "pair_mode":
                return PAIR_MODE[v]
            if k == "score":
                return 1 if v == "sigmoid" else 0
            if k == "act_flag":
                return pk.ACT_FLAGS[n.attrs.get("act", "silu")]
            return int(v)

        handles = [self.t(x) for x in (n.outputs + n.inputs)][:8]
        ivals = ([iv(k) for k in ikeys] + [0] * 7)[:7]
        fvals = [float(n.attrs.get(k, 0.0)) for k in fkeys] + [0.0] * (3 - len(fkeys))
        if n.op == "moe_experts" and n.attrs.get("bias1"):
            handles = (handles + [pk.T_NONE] * 6)[:6] + [self.t(n.attrs["bias1"]), self.t(n.attrs["bias2"])]
        if n.op == "mla_kv_write":
            # the latent row is usually a column range of the fused [q_a | kv_a] projection
            ivals[5], ivals[6] = self.xview(n.inputs[0])
        if n.op in ("mla_attention", "dsa_topk"):
            fvals[1] = float(n.attrs.get("topk", 0))
        ins = pk.Inst(op, f=tuple(fvals[:3]), t=handles + [pk.T_NONE] * (8 - len(handles)), i=ivals + [n.layer & 0xFFFF])
        return schedule.LInst(ins, rd(*n.inputs), rd(*n.outputs), 5.0, max(1, rows), cls)


def default_buckets(max_rows: int = 8192) -> dict:
    """Prefill bucket ladder and decode rung ladder (reference presets: crates/plowc/src/main.rs:404-432,
    crates/devgen/src/lib.rs:9173-9188)."""
    pf = [b for b in (128, 256, 512, 1024, 2048, 4096, 8192) if b <= max_rows]
    return dict(prefill=pf, decode=[1, 2, 4, 8, 16, 32, 64, 128, 256, 512])


def emit_packet(g: Graph, sites: list, hw: GpuSpec, n_cu: int, buckets: dict, extra_sections: dict | None = None,
                rank: int = 0) -> pk.Packet:
    low = Lowering(g, hw)
    programs = []
    for role, rows_list in ((pk.Role.PREFILL, buckets["prefill"]), (pk.Role.DECODE, buckets["decode"])):
        for rows in rows_list:
            samples = rows if role == pk.Role.DECODE else max(1, min(rows, buckets.get("max_seqs", 64)))
            linsts = low.lower(rows, samples, int(role))
            programs.append(schedule.schedule(linsts, n_cu, int(role), rows, rank, low.tensors, samples))
    spec = g.spec
    sections = {
        "model.json": spec.to_json().encode(),
        "derived_weights.json": json.dumps(low.derived, sort_keys=True).encode(),
        "gen_tensors.json": json.dumps(low.gen, sort_keys=True).encode(),
        "live_kv": json.dumps(dict(page=pk.KV_PAGE, dtype=spec.kv_dtype, bytes_per_token=spec.kv_bytes_per_token(),
                                   layers=spec.n_layers)).encode(),
        "weight_shards.json": json.dumps(dict(tp=g.tp, ep=g.ep, rank=rank)).encode(),
        "serve.json": json.dumps(dict(
            chat=dict(template=None), stop_token_ids=spec.eos_token_ids,
            sampling=dict(temperature=1.0, top_p=1.0, top_k=0),
            kv=dict(page=pk.KV_PAGE, dtype=spec.kv_dtype, max_ctx=spec.max_ctx),
            buckets=buckets)).encode(),
        "abi.json": json.dumps(dict(
            contract="plow-b200-packet", version=pk.VERSION, target=hw.arch,
            must_understand=["live_kv", "derived_weights.json", "weight_shards.json"],
            bindings=["in.ids", "in.pos", "in.seq", "in.sample_rows", "in.page_table", "in.kvlen",
                      "out.logits", "out.ids"])).encode(),
    }
    if any(l.attn.kind in ("gdn", "kda") for l in spec.layers):
        sections["recurrent_state"] = json.dumps(dict(kind=next(l.attn.kind for l in spec.layers if l.attn.kind in ("gdn", "kda")),
                                                      layers=[i for i, l in enumerate(spec.layers) if l.attn.kind in ("gdn", "kda")])).encode()
        abi = json.loads(sections["abi.json"])
        abi["must_understand"].append("recurrent_state")
        sections["abi.json"] = json.dumps(abi).encode()
    sections.update(extra_sections or {})
    return pk.Packet(tensors=low.tensors, programs=programs, sections=sections, n_cu=n_cu)
