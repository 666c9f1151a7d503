"""sm_100a backend: executes packet programs with the hand-written kernels in ``libplow_cuda.so``.

A program's instruction list is walked in order and every opcode is dispatched to a launcher
(`role objects`: tcgen05 GEMMs, attention kernels, row-wise kernels); the whole walk for a decode
rung is captured once in a CUDA graph and replayed, so a decode step costs one graph launch, one
H2D copy of the step inputs from pinned memory and one D2H read of the sampled ids.  Activations
live at the arena offsets the compiler planned (stable addresses make the capture valid);
padding rows of a rung point at a scratch slot so they never touch live KV.

Weights come from a :class:`WeightSource`: the checkpoint (names are the contract; block-scaled
e4m3 twins are produced on the device at load) or a synthetic on-device generator for benches at
the 671B shape, where no checkpoint exists.  Reference counterpart: crates/plowrt/src/exec/gpu.rs
(GpuEngine::load :4164, step_slots :9593, segment roles exec/gpu/*.rs).
"""
from __future__ import annotations

import json
import math
import os
from pathlib import Path

import numpy as np
import torch

from ..compiler import packet as pk
from ..compiler.packet import Op
from ..ops import dsa as dsa_ops, gdn as gdn_ops, gemm as gemm_ops, gqa as gqa_ops, mla as mla_ops, native, quant, rowops
from ..utils.rope import rope_table
from .device_interp import DeviceInterp
from .engine import EngineBase, EngineError, StepResult, TokenBatch
from .kv_pages import PAGE

BF16, FP8, F32, I32 = torch.bfloat16, torch.float8_e4m3fn, torch.float32, torch.int32
_TORCH_DT = {pk.DType.F32: F32, pk.DType.BF16: BF16, pk.DType.E4M3: FP8, pk.DType.I32: I32, pk.DType.U8: torch.uint8,
             pk.DType.I64: torch.int64}


# ------------------------------------------------------------------------------------------------
class WeightSource:
    """Provides device tensors for WEIGHT / DERIVED packet entries."""

    def bf16(self, ent, recipe) -> torch.Tensor:
        raise NotImplementedError

    def fp8(self, ent, recipe):
        """(e4m3 [N, K], f32 scales [N/128, K/128])"""
        w = self.bf16(ent, recipe)
        q, s = quant.quant_weight_128x128(w)
        return q, s


class CheckpointWeights(WeightSource):
    def __init__(self, ckpt_dir, device, tp=1, rank=0):
        from .weights import open_checkpoint
        self.ckpt = open_checkpoint(ckpt_dir)
        self.device, self.tp, self.rank = device, tp, rank
        self.twins = None              # pre-quantised e4m3 twins next to the packet (runtime/fp8_dir.py), set by the engine

    def fp8(self, ent, recipe):
        got = self.twins.get(ent.name, self.device) if self.twins else None
        if got is None:
            # a checkpoint that is already block-quantised (e4m3 codes + _scale_inv): its own codes, not a second rounding
            from .weights import fp8_codes
            got = fp8_codes(ent.name, ent, recipe, self.ckpt, self.tp, self.rank)
            if got is not None:
                got = (got[0].to(self.device), got[1].to(self.device))
        return got if got is not None else super().fp8(ent, recipe)

    def bf16(self, ent, recipe):
        from .weights import materialize
        w = materialize(ent.name, ent, recipe, self.ckpt, self.tp, self.rank)
        dt = F32 if pk.DType(ent.dtype) == pk.DType.F32 else BF16
        return w.to(device=self.device, dtype=dt).contiguous()


class SyntheticWeights(WeightSource):
    """N(0, std) weights generated on the device (norm weights 1, biases 0).  e4m3 tensors are
    drawn directly in the quantised domain with one constant block scale, so a 100 GB shard is
    produced in about a minute without a bf16 copy ever existing."""

    def __init__(self, device, seed=0, std=0.02, scaled_init_layers: int = 0):
        """`scaled_init_layers` = L > 0 selects the usual depth-scaled random init: unit-variance
        embeddings and residual-output projections (o_proj, down_proj) drawn with std / (2 L).  With
        plain N(0, std) everywhere the hidden states of different tokens become collinear after a few
        dozen random layers and every token routes to the same experts, which no trained
        (load-balanced) checkpoint does; the scaled init keeps routing token-specific.  Shapes, dtypes
        and bytes moved are identical either way."""
        self.device, self.std = device, std
        self.L = scaled_init_layers
        self.gen = torch.Generator(device=device).manual_seed(seed)

    def _std_for(self, name: str) -> float:
        if not self.L:
            return self.std
        if name.endswith("embed_tokens.weight"):
            return 1.0
        if name.endswith("o_proj.weight") or name.endswith("down_proj.weight") or name.endswith("experts.down.weight") \
                or name.endswith("out_proj.weight"):
            return self.std / (2.0 * self.L)
        return self.std

    def _shape(self, ent):
        return tuple(int(d) for d in ent.dims)

    def bf16(self, ent, recipe):
        shape = self._shape(ent)
        dt = F32 if pk.DType(ent.dtype) == pk.DType.F32 else BF16
        n = ent.name
        if n.endswith("norm.weight") or n.endswith("layernorm.weight"):
            return torch.ones(shape, dtype=dt, device=self.device)
        if n.endswith("bias"):
            return torch.zeros(shape, dtype=dt, device=self.device)
        out = torch.empty(shape, dtype=dt, device=self.device)
        flat = out.view(-1)
        step = 1 << 28
        for i in range(0, flat.numel(), step):
            flat[i:i + step] = torch.randn(min(step, flat.numel() - i), device=self.device, generator=self.gen) * self._std_for(n)
        return out

    def fp8(self, ent, recipe):
        n, k = self._shape(ent)
        clip = 4.0
        q = torch.empty(n, k, dtype=FP8, device=self.device)
        flat = q.view(-1)
        step = 1 << 28
        for i in range(0, flat.numel(), step):
            m = min(step, flat.numel() - i)
            flat[i:i + m] = (torch.randn(m, device=self.device, generator=self.gen).clamp_(-clip, clip) * (448.0 / clip)).to(FP8)
        s = torch.full(((n + 127) // 128, (k + 127) // 128), self._std_for(ent.name) * clip / 448.0, dtype=F32, device=self.device)
        return q, s


# ------------------------------------------------------------------------------------------------
class _Prog:
    """Per-program device state: arena views, quant side buffers, captured graph."""

    def __init__(self):
        self.t = {}          # handle -> tensor
        self.q = {}          # handle -> (xq, sx) for activations consumed by e4m3 GEMMs
        self.graph = None
        self.needs_q = set()
        self.scratch = {}
        self.interp = None
        self.segments = None


class GpuEngine(EngineBase):
    def __init__(self, assets_dir=None, packet=None, weights: WeightSource | None = None, max_slots=64, n_pages=None,
                 max_ctx=8192, kv_fraction=0.9, prefix_cache=True, cuda_graphs=True, device=None, rank=0,
                 comm=None, rungs=None, device_interp=None, tp_comm=None, step_group=None, leader_group=None):
        if not torch.cuda.is_available():
            raise EngineError("GpuEngine needs a CUDA device", fatal=True)
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        torch.cuda.set_device(self.device)
        native.cuda_lib()     # raises loudly when the kernel library is missing
        if packet is None:
            name = "model.pkt" if rank == 0 else f"model.rank{rank}.pkt"
            packet = pk.read_packet(Path(assets_dir) / name)
        self.rank, self.comm, self.tp_comm = rank, comm, tp_comm
        self.assets_dir = assets_dir
        # rank groups (plow_b200/parallel/group.py): step_group = every rank schedules its own requests and the ranks
        # agree on the program before each launch (expert parallelism with data-parallel attention); leader_group =
        # rank 0 schedules, the others replay its steps (tensor parallelism)
        self.step_group, self.leader_group = step_group, leader_group
        self.lockstep = step_group is not None
        # row-class segments run inside the persistent on-device interpreter (PLOW_DEVICE_INTERP=0 turns it off)
        self.device_interp = (os.environ.get("PLOW_DEVICE_INTERP", "1") != "0") if device_interp is None else bool(device_interp)
        shards = packet.section_json("weight_shards.json") or {}
        self.tp, self.ep = shards.get("tp", 1), shards.get("ep", 1)
        if weights is None:
            weights = CheckpointWeights(Path(assets_dir) / "checkpoint", self.device, self.tp, rank)
        self.weights = weights
        self.cuda_graphs = cuda_graphs
        self.derived = packet.section_json("derived_weights.json") or {}
        self.gen_meta = packet.section_json("gen_tensors.json") or {}
        pages_per_seq = (max_ctx + PAGE - 1) // PAGE
        if n_pages is None:
            n_pages = max_slots * pages_per_seq
        if any(t.tclass == pk.TClass.STATE for t in packet.tensors):
            prefix_cache = False      # recurrent state is per slot, not per page: a prefix hit would skip its update
        super().__init__(packet, max_slots, n_pages, max_ctx, prefix_cache)
        self.scratch_slot = max_slots                  # padding rows of a rung live here
        self.scratch_page = n_pages                    # one extra page nobody else maps
        self._load_static()
        self.progs: dict[int, _Prog] = {}
        self.step_ms_last = 0.0
        self.launches_last = 0
        self.profile_ops = os.environ.get("PLOW_PROFILE_OPS") == "1"     # per-instruction device times of eager steps
        self.taps: dict | None = None      # when a dict: copies of selected intermediates of eager steps, keyed (name, layer)
        self.op_times_last: list = []

    # ---- static tensors ------------------------------------------------------------------------
    def _load_static(self) -> None:
        dev = self.device
        pkt = self.packet
        self.static: dict[int, torch.Tensor] = {}
        self.static_q: dict[int, tuple] = {}
        if any(ins.op in (Op.GEMM, Op.GEMM_XREDUCE) and ins.i[2] & (pk.GEMM_ACT_GELU_TANH | pk.GEMM_ACT_GELU_ERF)
               or ins.op == Op.GLU and ins.i[0] for p in pkt.programs for ins in p.insts):
            raise EngineError("this packet's gated MLP uses a GELU gate: the sm_100a GEMM epilogue and GLU row op implement SiLU only "
                              "(the CPU backend runs it)", fatal=True)
        if any(ins.op == Op.GDN_STEP and ins.i[4] == 1 for p in pkt.programs for ins in p.insts):
            raise EngineError("this packet has Kimi Delta Attention layers: the sm_100a recurrent kernel implements the scalar-gated delta "
                              "rule only (the CPU backend runs it)", fatal=True)
        if any(ins.op == Op.ATTN and ins.t[5] != pk.T_NONE or ins.op == Op.MOE_GEMM and ins.t[6] != pk.T_NONE
               for p in pkt.programs for ins in p.insts):
            raise EngineError("this packet uses attention sinks / biased clamped-GLU experts (gpt_oss): the sm_100a attention and expert "
                              "kernels have neither (the CPU backend runs it)", fatal=True)
        if any(ins.op in (Op.GEMM, Op.GEMM_XREDUCE) and ins.i[2] & pk.GEMM_BIAS for p in pkt.programs for ins in p.insts):
            raise EngineError("this packet's projections carry biases: the sm_100a GEMM epilogue has no bias term (the CPU backend runs it)",
                              fatal=True)
        from .fp8_dir import Fp8Dir, fp8_weight_handles
        fp8_handles = fp8_weight_handles(pkt, self.spec.weight_quant)
        if isinstance(self.weights, CheckpointWeights) and self.weights.twins is None and getattr(self, "assets_dir", None):
            self.weights.twins = Fp8Dir(self.assets_dir, pkt, self.weights.rank)
        max_rows = max(p.rows for p in pkt.programs)
        self.max_rows_all = max_rows
        n_slots = self.max_slots + 1
        # host mirror of the page table in pinned memory; rows touched since the last step are uploaded at the start of
        # the next one (one async copy per row, or one for the whole table when many changed)
        self.h_page_table = torch.zeros(n_slots, self.max_pages_per_seq, dtype=I32).pin_memory()
        self.h_page_table[self.scratch_slot, :] = self.scratch_page
        self.page_table = self.h_page_table.numpy()
        self.d_page_table = self.h_page_table.to(dev)
        self._dirty_slots: set = set()
        # step inputs: one pinned staging block + one device block, copied with a single H2D
        self.h_in = torch.zeros(4, max_rows, dtype=I32).pin_memory()
        self.d_in = torch.zeros(4, max_rows, dtype=I32, device=dev)      # ids, pos, seq, sample_rows
        self.d_kvlen_row = torch.zeros(max_rows, dtype=I32, device=dev)   # pos + 1 per row
        self.h_out = torch.zeros(max_rows, dtype=I32).pin_memory()
        self.d_out_ids = torch.zeros(max_rows, dtype=I32, device=dev)
        self.d_logits = None
        # hidden-state input (a prediction-module drafter's rows) and output (what such a drafter reads): bound per
        # program as row views in _prepare
        self.d_hidden_in = self.d_hidden_out = None
        self.hidden_rows = None           # "rows" | "samples": which rows out.hidden carries
        for h, t in enumerate(pkt.tensors):
            tc = t.tclass
            if tc in (pk.TClass.WEIGHT, pk.TClass.DERIVED):
                recipe = self.derived.get(t.name)
                if h in fp8_handles:
                    self.static_q[h] = self.weights.fp8(t, recipe)
                else:
                    self.static[h] = self.weights.bf16(t, recipe)
            elif tc == pk.TClass.GEN:
                m = self.gen_meta[t.name]
                tab = rope_table(min(int(t.dims[0]), max(self.max_ctx, 64)), m["rot_dim"], m["theta"], m.get("scaling"))
                self.static[h] = torch.from_numpy(tab).to(dev)
            elif tc == pk.TClass.KV:
                dims = [self.pool.n_pages + 1 if d == -3 else int(d) for d in t.dims]
                dt = _TORCH_DT[pk.DType(t.dtype)]
                self.static[h] = torch.zeros(dims, dtype=dt, device=dev) if dt != FP8 else torch.zeros(dims, dtype=torch.uint8, device=dev).view(FP8)
            elif tc == pk.TClass.STATE:
                # recurrent state, one entry per slot (+ the scratch slot padding rows point at)
                dims = [self.max_slots + 1 if d == -4 else int(d) for d in t.dims]
                self.static[h] = torch.zeros(dims, dtype=_TORCH_DT[pk.DType(t.dtype)], device=dev)
            elif tc == pk.TClass.INPUT:
                if t.name == "in.hidden":
                    self.d_hidden_in = torch.zeros(max_rows, self.spec.hidden, dtype=_TORCH_DT[pk.DType(t.dtype)], device=dev)
                    self.static[h] = self.d_hidden_in
                    continue
                self.static[h] = self.d_in[{"in.ids": 0, "in.pos": 1, "in.seq": 2, "in.sample_rows": 3}[t.name]]
            elif tc == pk.TClass.OUTPUT:
                if t.name == "out.ids":
                    self.static[h] = self.d_out_ids
                elif t.name == "out.hidden":
                    self.d_hidden_out = torch.zeros(max_rows, self.spec.hidden, dtype=_TORCH_DT[pk.DType(t.dtype)], device=dev)
                    self.static[h] = self.d_hidden_out
                    self.hidden_rows = "rows" if t.dims[0] == -1 else "samples"
                else:
                    self.d_logits = torch.zeros(max(p.rows if p.role == pk.Role.DECODE else min(p.rows, self.buckets.get("max_seqs", 64))
                                                    for p in pkt.programs), self.spec.vocab, dtype=F32, device=dev)
                    self.static[h] = self.d_logits
        # per-page scale upper bounds for fp8 latent caches (one per layer cache)
        self.kv_smax: dict[int, torch.Tensor] = {}
        self._mla_derived: dict[int, tuple] = {}
        self._mla_ws = None
        # materialised prefill (K / V rebuilt from the latent once per layer for long runs of new rows)
        self._mla_pf_ws = None
        self._mla_plan = None
        self._route_ticket = None
        self._multi_out = self._h_multi_out = None
        self._mla_plan_rows = 0
        self._has_mla = any(l.attn.kind == "mla" for l in self.spec.layers)
        self._has_gdn = any(l.attn.kind == "gdn" for l in self.spec.layers)
        self._gdn_plan = None
        self._dsa_topk = max((l.attn.index_topk for l in self.spec.layers if l.attn.index_heads), default=0)
        self.h_plan = torch.zeros(2 * max_rows + 4 * n_slots, dtype=I32).pin_memory()
        self.d_plan = torch.zeros(2 * max_rows + 4 * n_slots, dtype=I32, device=dev)

    # ---- program preparation -------------------------------------------------------------------
    def _prepare(self, idx: int) -> _Prog:
        if idx in self.progs:
            return self.progs[idx]
        prog = self.packet.programs[idx]
        st = _Prog()
        dev = self.device
        rows = prog.rows
        samples = rows if prog.role == pk.Role.DECODE else max(1, min(rows, self.buckets.get("max_seqs", 64)))
        st.rows, st.samples, st.role = rows, samples, prog.role
        arena = torch.empty(max(prog.arena_bytes, 256), dtype=torch.uint8, device=dev)
        st.arena = arena
        for h, t in enumerate(self.packet.tensors):
            if t.tclass == pk.TClass.ACT and prog.actmap[h] != pk.U64_MAX:
                dims = [rows if d == -1 else samples if d == -2 else int(d) for d in t.dims]
                dt = _TORCH_DT[pk.DType(t.dtype)]
                n = int(np.prod(dims)) * torch.empty((), dtype=dt).element_size()
                st.t[h] = arena[prog.actmap[h]:prog.actmap[h] + n].view(dt).view(dims)
            elif t.name in ("in.hidden", "out.hidden"):
                st.t[h] = self.static[h][:samples if t.dims[0] == -2 else rows]      # handlers take the row count from the shape
        # which activations feed an e4m3 GEMM: their producer emits the quantised twin in the same pass
        for ins in prog.insts:
            if ins.op in (Op.GEMM, Op.GEMM_XREDUCE) and ins.i[2] & pk.GEMM_FP8_BLOCK:
                st.needs_q.add((ins.t[1], ins.i[6], ins.i[1]))      # (handle, col offset, K)
            if ins.op == Op.MOE_GEMM and self.spec.weight_quant == "fp8_block128":
                st.needs_q.add((ins.t[1], 0, self.spec.hidden))
        self._plan_route_fusion(st, prog)
        self.progs[idx] = st
        return st

    ROUTE_FUSE_MAX_ROWS = int(os.environ.get("PLOW_ROUTE_FUSE_MAX_ROWS", "256"))

    def _plan_route_fusion(self, st: _Prog, prog) -> None:
        """Decode-size programs: a router projection GEMM followed by ROUTER_TOPK (and the align step of a local MOE_GEMM)
        runs as one launch (csrc/cuda/rowops.cu, moe_route_kernel).  Records which GEMM instructions to skip and what
        the top-k instruction does instead."""
        st.skip, st.route = set(), {}
        if prog.rows > self.ROUTE_FUSE_MAX_ROWS:
            return
        insts = prog.insts
        for i, g in enumerate(insts[:-1]):
            tk = insts[i + 1]
            if g.op != Op.GEMM or tk.op != Op.ROUTER_TOPK or tk.t[1] != g.t[0]:
                continue
            N, K, flags, co = g.i[0], g.i[1], g.i[2], g.i[6]
            w = self.static.get(g.t[2])
            x = st.t.get(g.t[1])
            if (flags & (pk.GEMM_FP8_BLOCK | pk.GEMM_DUAL_SILU)) or co != 0 or w is None or w.dtype != BF16 or x is None \
                    or x.dtype != BF16 or x.shape[1] != K or N != tk.i[0] or K % 8 or N > 1024:
                continue
            k_top, n_grp = tk.i[1], max(1, tk.i[2])
            if k_top > 32 or n_grp > 32 or N % n_grp or (K + 3 * N) * 4 > 190 * 1024:
                continue                                  # outside what the routing kernel handles: keep the three kernels
            if any(o is not g and o is not tk and g.t[0] in o.t for o in insts):
                continue                                  # something else reads the logits
            moe = next((m for m in insts if m.op == Op.MOE_GEMM and m.t[2] == tk.t[0]), None)
            st.skip.add(id(g))
            st.route[id(tk)] = (g, moe)

    def tensor(self, st: _Prog, h: int):
        if h == pk.T_NONE:
            return None
        return st.t[h] if h in st.t else self.static[h]

    # ---- op handlers ---------------------------------------------------------------------------
    def _wants_q(self, st, h, co=0):
        return any(k[0] == h and k[1] == co for k in st.needs_q)

    def _quant_of(self, st, h, co, K, x):
        """e4m3 twin of activation columns [co, co+K) of handle h (made on demand if the producer did not)."""
        key = (h, co)
        if key not in st.q:
            xin = x if (co == 0 and x.shape[1] == K) else x[:, co:co + K]
            st.q[key] = rowops.quant_act(xin) if xin.is_contiguous() else rowops.quant_act(xin.contiguous())
        return st.q[key]

    def _op_embed(self, st, ins):
        native.call("plow_embed", self.tensor(st, ins.t[0]), self.tensor(st, ins.t[1]), self.tensor(st, ins.t[2]),
                    st.rows, ins.i[0], float(ins.f[0]))

    def _norm_common(self, st, out_h, fn):
        want = self._wants_q(st, out_h)
        res = fn(want)
        if want:
            st.q[(out_h, 0)] = (res[-2], res[-1])

    def _op_rmsnorm(self, st, ins):
        out, x, g = self.tensor(st, ins.t[0]), self.tensor(st, ins.t[1]), self.tensor(st, ins.t[2])
        W, co = ins.i[0], ins.i[6]
        R = out.shape[0]
        want = self._wants_q(st, ins.t[0]) and W % 128 == 0
        xq = sx = None
        if want:
            xq = torch.empty(R, W, dtype=FP8, device=self.device)
            sx = torch.empty(W // 128, R, dtype=F32, device=self.device)
            st.q[(ins.t[0], 0)] = (xq, sx)
        xin = x if co == 0 else x[:, co:]
        native.call("plow_rmsnorm", out, xq, sx, R, xin, g, R, W, x.stride(0), float(ins.f[0]), int(ins.i[1]))

    def _op_add_norm(self, st, ins):
        h_out, x_in, delta, g, x_out = (self.tensor(st, ins.t[k]) for k in range(5))
        R, W = h_out.shape
        want = self._wants_q(st, ins.t[0]) and W % 128 == 0
        xq = sx = None
        if want:
            xq = torch.empty(R, W, dtype=FP8, device=self.device)
            sx = torch.empty(W // 128, R, dtype=F32, device=self.device)
            st.q[(ins.t[0], 0)] = (xq, sx)
        native.call("plow_add_norm", h_out, xq, sx, R, x_out, x_in, delta, g, R, W, float(ins.f[0]), int(ins.i[1]))

    def _op_residual(self, st, ins):
        out, a, b = (self.tensor(st, ins.t[k]) for k in range(3))
        native.call("plow_eltwise2", out, a, b, out.numel(), 0)

    def _op_glu(self, st, ins):
        # only reached when gated-mlp fusion is disabled at compile time and the interpreter is off
        out, g, u = (self.tensor(st, ins.t[k]) for k in range(3))
        native.call("plow_eltwise2", out, g, u, out.numel(), 1)

    def _op_gemm(self, st, ins):
        if id(ins) in st.skip:
            return                     # a router projection computed inside the fused routing kernel
        y, x = self.tensor(st, ins.t[0]), self.tensor(st, ins.t[1])
        N, K, flags, swap, bn, co = ins.i[0], ins.i[1], ins.i[2], ins.i[3], ins.i[4], ins.i[6]
        dual = bool(flags & pk.GEMM_DUAL_SILU)
        M = y.shape[0]
        if flags & pk.GEMM_FP8_BLOCK:
            wq, sw = self.static_q[ins.t[2]]
            xq, sx = self._quant_of(st, ins.t[1], co, K, x)
            wide = dual and gemm_ops._WIDE_DEFAULT and not swap and bn == 64       # gemm() widens these tiles to 128
            want = self._wants_q(st, ins.t[0]) and (swap or bn == 128 or wide) and N % 128 == 0
            if want:
                # SwiGLU / projection result re-quantised in the GEMM epilogue for the next e4m3 GEMM
                yq, syq = gemm_ops.gemm(xq[:M], wq, sx=sx, sw=sw, dual=dual, n_out=N, swap=bool(swap), bn=bn, quant_out=True)
                st.q[(ins.t[0], 0)] = (yq, syq)
                # the bf16 value is still part of the program's dataflow when another op reads it
                if self._bf16_needed(st, ins.t[0]):
                    gemm_ops.gemm(xq[:M], wq, sx=sx, sw=sw, dual=dual, n_out=N, swap=bool(swap), bn=bn, out=y)
            else:
                gemm_ops.gemm(xq[:M], wq, sx=sx, sw=sw, dual=dual, n_out=N, swap=bool(swap), bn=bn, out=y,
                              out_f32=bool(flags & pk.GEMM_OUT_F32))
        else:
            w = self.static[ins.t[2]]
            xin = x if co == 0 and x.shape[1] == K else x[:, co:co + K]
            if w.dtype != BF16:
                w = self._bf16_weight(ins.t[2])
            gemm_ops.gemm(xin, w, dual=dual, n_out=N, swap=bool(swap), bn=min(bn, 128) if swap else bn, out=y,
                          out_f32=bool(flags & pk.GEMM_OUT_F32))

    def _bf16_weight(self, h):
        key = ("bf16", h)
        if key not in self.static:
            self.static[key] = self.static[h].to(BF16)
        return self.static[key]

    def _bf16_needed(self, st, h) -> bool:
        prog = st.prog
        for ins in prog.insts:
            reads = ins.t[1:]
            if h in reads:
                if ins.op in (Op.GEMM, Op.GEMM_XREDUCE) and ins.i[2] & pk.GEMM_FP8_BLOCK and ins.t[1] == h:
                    continue
                return True
        return False

    def _op_row_gather(self, st, ins):
        out, x, rows = (self.tensor(st, ins.t[k]) for k in range(3))
        native.call("plow_row_gather", out, x, rows, st.samples, ins.i[0])

    def _op_argmax(self, st, ins):
        out, lg = self.tensor(st, ins.t[0]), self.tensor(st, ins.t[1])
        if ins.i[1]:        # vocabulary-sharded lm_head: packed (score, ~global index) key of this rank's shard
            native.call("plow_argmax_key", out, lg, st.samples, ins.i[0], ins.i[2])
        else:
            native.call("plow_argmax", out, lg, st.samples, ins.i[0])

    def _ext_xargmax_fin(self, st, ins):
        """Fold the ranks' packed arg-max keys: a tiny all-gather, then a max per row (lowest global index on ties)."""
        import torch.distributed as dist
        out, keys = self.tensor(st, ins.t[0]), self.tensor(st, ins.t[1])
        world = ins.i[0]
        buf = st.scratch.setdefault(("amax_all", ins.t[1]), torch.empty(world, keys.shape[0], dtype=torch.int64, device=self.device))
        dist.all_gather_into_tensor(buf.view(-1), keys.contiguous())
        native.call("plow_argmax_fin", out, buf, st.samples, world)

    def _ext_xgather(self, st, ins):
        """out[:, r*width:(r+1)*width] = rank r's block (full logits for the host sampler)."""
        import torch.distributed as dist
        out, local = self.tensor(st, ins.t[0]), self.tensor(st, ins.t[1])
        width, world = ins.i[0], ins.i[1]
        buf = st.scratch.setdefault(("xg", ins.t[1]), torch.empty(world, local.shape[0], width, dtype=local.dtype, device=self.device))
        dist.all_gather_into_tensor(buf.view(-1), local.contiguous().view(-1))
        out[:local.shape[0]].view(local.shape[0], world, width).copy_(buf.permute(1, 0, 2))

    # -- MLA
    def _mla_prep(self, layer: int, wkv_b_h: int, heads: int, kv_lora: int, nope: int, v_head: int):
        """Per-head absorbed projections from kv_b_proj: W_uk^T [h][kv_lora][nope] and W_uv [h][v][kv_lora]."""
        if layer not in self._mla_derived:
            w = self.static[wkv_b_h] if wkv_b_h in self.static else quant.dequant_weight_128x128(*self.static_q[wkv_b_h]).to(BF16)
            w3 = w.view(heads, nope + v_head, kv_lora)
            wuk_t = w3[:, :nope, :].transpose(1, 2).contiguous().view(heads * kv_lora, nope).to(BF16)
            wuv = w3[:, nope:, :].contiguous().view(heads * v_head, kv_lora).to(BF16)
            self._mla_derived[layer] = (wuk_t, wuv)
        return self._mla_derived[layer]

    def _op_mla_kv_write(self, st, ins):
        fp8 = self.spec.kv_dtype == "fp8"
        if not fp8:
            raise EngineError("bf16 latent cache has no sm_100a body yet; compile with plow_kv_dtype=fp8")
        cache, scale, kva, gamma, rope = (self.tensor(st, ins.t[k]) for k in range(5))
        layer = ins.i[7]
        if layer not in self.kv_smax:
            self.kv_smax[layer] = torch.zeros(cache.shape[0], 4, dtype=F32, device=self.device)
        mla_ops.kv_write(cache, scale, self.kv_smax[layer], kva, ins.i[5], gamma, rope, self.d_in[1], self.d_in[2],
                         self.d_page_table, ins.i[0], ins.i[1], float(ins.f[0]), ins.i[2])

    # A run of at least this many consecutive new rows of one request attends over K / V rebuilt from the latent
    # (plain multi-head attention: 192-wide keys, 128-wide values) instead of the absorbed form (576 / 512 wide).
    MLA_PREFILL_MIN_RUN = int(os.environ.get("PLOW_MLA_PREFILL_MIN_RUN", "64"))
    # cached tokens (summed over the step's prefilling requests) whose K / V one layer may rebuild: 64 KiB per token
    MLA_PREFILL_BUDGET = int(os.environ.get("PLOW_MLA_PREFILL_BUDGET", "16384"))

    def _plan_mla_prefill(self, batch: TokenBatch, R: int):
        """Host side of the materialised prefill: which runs of rows take it, where each request's rebuilt K / V start.
        Returns None when no run qualifies.  Rows outside the chosen runs (decode riders, short runs, padding) stay on
        the absorbed kernel: they see kvlen 0 there if chosen, and position -1 here if not."""
        if self.MLA_PREFILL_MIN_RUN <= 0 or batch.rows < self.MLA_PREFILL_MIN_RUN:
            return None
        rows, seq, pos = batch.rows, batch.seq, batch.pos
        brk = np.flatnonzero((seq[1:] != seq[:-1]) | (pos[1:] != pos[:-1] + 1)) + 1
        starts = np.concatenate(([0], brk))
        ends = np.concatenate((brk, [rows]))
        budget = min(self.MLA_PREFILL_BUDGET, ((self.max_ctx + PAGE + 63) // 64) * 64 * 4)
        pos_mat = np.full(R, -1, np.int32)
        kv_abs = np.zeros(R, np.int32)
        kv_abs[:rows] = pos + 1
        spans, base, seen, max_tiles = [], 0, set(), 0
        for r0, r1 in zip(starts.tolist(), ends.tolist()):
            slot, L = int(seq[r0]), int(pos[r1 - 1]) + 1
            need = -(-L // 64) * 64
            if r1 - r0 < self.MLA_PREFILL_MIN_RUN or slot in seen or base + need > budget:
                continue
            seen.add(slot)
            spans.append((slot, L, base, 0))
            pos_mat[r0:r1] = pos[r0:r1]
            kv_abs[r0:r1] = 0
            base += need
            max_tiles = max(max_tiles, need // 64)
        if not spans:
            return None
        n_sp = len(spans)
        hp = self.h_plan.numpy()
        hp[:R] = pos_mat
        hp[R:2 * R] = kv_abs
        hp[2 * R:2 * R + 4 * n_sp] = np.asarray(spans, np.int32).reshape(-1)
        n = 2 * R + 4 * n_sp
        self.d_plan[:n].copy_(self.h_plan[:n], non_blocking=True)
        return dict(R=R, n_spans=n_sp, total=base, max_tiles=max_tiles, riders=bool((kv_abs[:rows] > 0).any()),
                    pos=self.d_plan[:R], kvlen=self.d_plan[R:2 * R], spans=self.d_plan[2 * R:2 * R + 4 * n_sp], budget=budget,
                    gathered=False)

    # Runs of at least this many new rows take the chunked gated-delta-rule prefill (0 = off, the default: that path is
    # batched matrix algebra through cuBLAS / cuSOLVER, and the serving default keeps the hand-written token-by-token
    # kernel on this op; set PLOW_GDN_CHUNKED_MIN_RUN=128 to trade that for a several times faster long-prompt prefill).
    GDN_CHUNKED_MIN_RUN = int(os.environ.get("PLOW_GDN_CHUNKED_MIN_RUN", "0"))

    def _plan_gdn_prefill(self, batch: TokenBatch, R: int):
        """Which runs of this (eager) step's rows take the chunked gated-delta-rule prefill; None when none does."""
        if self.GDN_CHUNKED_MIN_RUN <= 0 or batch.rows < self.GDN_CHUNKED_MIN_RUN:
            return None
        rows, seq, pos = batch.rows, batch.seq, batch.pos
        brk = np.flatnonzero((seq[1:] != seq[:-1]) | (pos[1:] != pos[:-1] + 1)) + 1
        starts = np.concatenate(([0], brk)).tolist()
        ends = np.concatenate((brk, [rows])).tolist()
        chunked, rest, seen = [], [], set()
        for r0, r1 in zip(starts, ends):
            slot = int(seq[r0])
            if r1 - r0 >= self.GDN_CHUNKED_MIN_RUN and slot not in seen:
                seen.add(slot)
                chunked.append((slot, r0, r1, int(pos[r0]) == 0))
            elif rest and rest[-1][1] == r0:
                rest[-1] = (rest[-1][0], r1)
            else:
                rest.append((r0, r1))
        if not chunked:
            return None
        if R > rows:                                  # the program's padding rows
            if rest and rest[-1][1] == rows:
                rest[-1] = (rest[-1][0], R)
            else:
                rest.append((rows, R))
        return dict(R=R, chunked=chunked, rest=rest)

    def _mla_prefill(self, st, ins, plan, ao, q, rope_tab, cache, scale):
        """Materialised prefill of one layer (see csrc/cuda/mla_prefill.cu)."""
        heads, kv_lora, nope, qk_rope, pair = ins.i[0], ins.i[1], ins.i[2], ins.i[3], ins.i[5]
        wh = ins.t[4]
        fp8_w = wh in self.static_q
        ws = self._mla_pf_ws
        if ws is None or ws.budget < plan["budget"] or ws.fp8 != fp8_w:
            ws = self._mla_pf_ws = mla_ops.PrefillWorkspace(plan["budget"], self.max_rows_all, self.max_slots + 1, self.max_pages_per_seq,
                                                            heads=heads, latent=kv_lora, rope=qk_rope, fp8_weight=fp8_w, device=self.device)
        n = plan["total"]
        mla_ops.latent_gather(ws, cache, scale, self.d_page_table, plan["spans"], plan["n_spans"], plan["max_tiles"])
        if fp8_w:
            wq, sw = self.static_q[wh]
            gemm_ops.gemm(ws.lat8[:n, :kv_lora], wq, sx=ws.lat_scale, sw=sw, out=ws.kvb[:n], swap=False)
        else:
            gemm_ops.gemm(ws.lat16[:n], self.static[wh], out=ws.kvb[:n], swap=False)
        mla_ops.q_rope(q, rope_tab, plan["pos"], heads, nope, qk_rope, pair)
        mla_ops.prefill_attention(q, ws, n, self.d_in[2], plan["pos"], float(ins.f[0]), ao)

    def _op_mla_attention(self, st, ins):
        ao, q, rope, _pos, wkv_b = (self.tensor(st, ins.t[k]) for k in range(5))
        cache, scale = self.tensor(st, ins.t[5]), self.tensor(st, ins.t[6])
        heads, kv_lora, nope, qk_rope, v_head, pair = ins.i[0], ins.i[1], ins.i[2], ins.i[3], ins.i[4], ins.i[5]
        layer = ins.i[7]
        if heads != 128 or kv_lora != 512 or qk_rope != 64:
            raise EngineError("the sm_100a MLA kernel is specialised for 128 heads, 512 latent and 64 rope dims per rank")
        T = st.rows
        if nope != 128 or v_head != 128:
            raise EngineError("the fused MLA projection kernels are specialised for 128 nope / 128 v dims")
        plan = self._mla_plan
        # sparse attention applies unless this (eager) step's positions all lie below top_k, where the indexer would
        # select every key anyway and the dense forms compute the same thing for less
        sparse = bool(ins.i[6]) and ins.t[7] != pk.T_NONE and not st.scratch.get("dsa_dense_ok", False)
        if plan is not None and (plan["R"] != T or sparse):
            plan = None
        kvlen_dense = self.d_kvlen_row if plan is None else plan["kvlen"]
        if plan is not None and not plan["riders"]:
            # every live row is in a materialised run: the absorbed kernels have nothing to do
            if T > self._mla_plan_rows:
                ao[self._mla_plan_rows:T].zero_()
            self._mla_prefill(st, ins, plan, ao, q, rope, cache, scale)
            if self._wants_q(st, ins.t[0]):
                st.q[(ins.t[0], 0)] = rowops.quant_act(ao)
            return
        wuk_t, wuv = self._mla_prep(layer, ins.t[4], heads, kv_lora, nope, v_head)
        blockwise = sparse and T > self.SPARSE_MAX_ROWS
        if not blockwise:
            q8, sq = mla_ops.absorb(q, wuk_t, rope, self.d_in[1], heads, pair)
        if self._mla_ws is None or self._mla_ws.opart.shape[0] < T:
            # up to 16 splits per request (the fold kernel's limit); a request's tiles are dealt evenly over its splits
            max_tiles = (self.max_ctx + PAGE + 63) // 64
            self._mla_ws = mla_ops.DecodeWorkspace(max(T, self.max_rows_all), self.max_ctx + PAGE,
                                                   tiles_per_split=max(int(os.environ.get('PLOW_MLA_TPS', '32')), -(-max_tiles // mla_ops.MAX_SPLITS)),
                                                   device=self.device)
        if self._mla_ws.max_splits > mla_ops.MAX_SPLITS:
            raise EngineError(f"max_ctx needs more than {mla_ops.MAX_SPLITS} KV splits; raise tiles_per_split")
        if blockwise:
            # large prefill buckets: the same select -> gather -> decode -> fold chain, one block of rows at a time (the
            # compact cache holds top_k tokens per row, so its size is bounded by the block, not by the bucket)
            sel_all = self.tensor(st, ins.t[7])
            top_k, B = sel_all.shape[1], self.SPARSE_MAX_ROWS
            key = ("dsa_cc", B, top_k)
            if key not in st.scratch:
                st.scratch[key] = dsa_ops.CompactCache(B, top_k, cache.shape[2], self.device)
            cc = st.scratch[key]
            pos_d, seq_d = self.d_in[1], self.d_in[2]
            for r0 in range(0, T, B):
                r1 = min(T, r0 + B)
                n = r1 - r0
                q8b, sqb = mla_ops.absorb(q[r0:r1], wuk_t, rope, pos_d[r0:r1], heads, pair)
                dsa_ops.gather(cc, sel_all[r0:r1], cache, scale, pos_d[r0:r1], seq_d[r0:r1], self.d_page_table)
                mla_ops.decode(q8b, sqb, cc.kv, cc.scale, cc.smax, cc.page_table[:n], cc.slot_of[:n], cc.kvlen[:n], self._mla_ws,
                               float(ins.f[0]), merge=False)
                mla_ops.fold(self._mla_ws, cc.kvlen[:n], wuv, n, heads, ao[r0:r1], want_fp8=False)
            st.scratch["mla_items"] = False
            if self._wants_q(st, ins.t[0]):
                st.q[(ins.t[0], 0)] = rowops.quant_act(ao)
            return
        if sparse:
            # sparse attention: the indexer's selection is gathered into a compact per-row cache and the same decode
            # kernel walks it (reference: runtime/nvidia/op_dsa.cuh, crates/devgen/src/mla.rs:7093)
            top_k = self.tensor(st, ins.t[7]).shape[1]
            key = ("dsa_cc", T, top_k)
            if key not in st.scratch:
                st.scratch[key] = dsa_ops.CompactCache(T, top_k, cache.shape[2], self.device)
            cc = st.scratch[key]
            dsa_ops.gather(cc, self.tensor(st, ins.t[7]), cache, scale, self.d_in[1], self.d_in[2], self.d_page_table)
            mla_ops.decode(q8, sq, cc.kv, cc.scale, cc.smax, cc.page_table, cc.slot_of, cc.kvlen, self._mla_ws, float(ins.f[0]), merge=False)
            kvlen = cc.kvlen
            st.scratch["mla_items"] = False
        else:
            # the work list depends on the rows' lengths only: the first dense attention of a walk builds it for all layers
            if not st.scratch.get("mla_items") or os.environ.get("PLOW_MLA_ITEMS_PER_LAYER") == "1":
                mla_ops.build_items(kvlen_dense, T, self._mla_ws)
                st.scratch["mla_items"] = True
            mla_ops.decode(q8, sq, cache, scale, self.kv_smax[layer], self.d_page_table, self.d_in[2], kvlen_dense,
                           self._mla_ws, float(ins.f[0]), merge=False, build_items=False, claim_slot=layer)
            kvlen = kvlen_dense
        want = self._wants_q(st, ins.t[0]) and plan is None
        aq, saq = mla_ops.fold(self._mla_ws, kvlen, wuv, T, heads, ao, want_fp8=want)
        if want:
            st.q[(ins.t[0], 0)] = (aq, saq)
        if plan is not None:
            # the runs chosen for the materialised form overwrite their rows (the absorbed kernels saw length 0 there)
            self._mla_prefill(st, ins, plan, ao, q, rope, cache, scale)
            if self._wants_q(st, ins.t[0]):
                st.q[(ins.t[0], 0)] = rowops.quant_act(ao)

    # -- tensor parallel (row-parallel projections end in an all-reduce)
    def _need_tp(self):
        if self.tp_comm is None:
            raise EngineError("this packet was compiled for tensor parallelism; pass tp_comm=TpComm(...)")
        return self.tp_comm

    def _ext_gemm_xreduce(self, st, ins):
        tp = self._need_tp()
        y, x = self.tensor(st, ins.t[0]), self.tensor(st, ins.t[1])
        N, K, flags, co = ins.i[0], ins.i[1], ins.i[2], ins.i[6]
        if flags & pk.GEMM_FP8_BLOCK:
            wq, sw = self.static_q[ins.t[2]]
            xq, sx = self._quant_of(st, ins.t[1], co, K, x)
            tp.gemm_allreduce(xq[:y.shape[0]], wq, N, sx=sx, sw=sw, out=y)
        else:
            w = self.static[ins.t[2]]
            xin = x if co == 0 and x.shape[1] == K else x[:, co:co + K]
            tp.gemm_allreduce(xin, w if w.dtype == BF16 else self._bf16_weight(ins.t[2]), N, out=y)

    def _ext_xreduce(self, st, ins):
        out, x = self.tensor(st, ins.t[0]), self.tensor(st, ins.t[1])
        if out.data_ptr() != x.data_ptr():
            out.copy_(x)
        self._need_tp().all_reduce(out)

    def _ext_xreduce_add_norm(self, st, ins):
        # emitted when the GEMM -> all-reduce fusion is disabled at compile time: reduce the partial in place, then the
        # same residual + RMSNorm row kernel as ADD_NORM (same operand order: h_out, x_in, partial, gamma, x_out)
        tp = self._need_tp()
        h_out, x_in, part, g, x_out = (self.tensor(st, ins.t[k]) for k in range(5))
        if tp._ar_fits(part) and g is not None and g.dtype == BF16 and x_in.is_contiguous() and x_out.is_contiguous():
            # one kernel over peer memory: all-reduce of the partial, residual add and RMSNorm (csrc/comm/tp_ar.cu); the
            # e4m3 twin of the normalised rows, when a consumer wants one, is made on demand
            tp.allreduce_add_norm(part, x_in, g, x_out, h_out, float(ins.f[0]), bool(ins.i[1]))
            return
        tp.all_reduce(part)
        self._op_add_norm(st, ins)

    # -- GQA
    def _op_rope_kv(self, st, ins):
        q_out, qkv, kc, vc = (self.tensor(st, ins.t[k]) for k in range(4))
        qn = self.tensor(st, ins.t[4]) if ins.t[4] != pk.T_NONE else None
        kn = self.tensor(st, ins.t[5]) if ins.t[5] != pk.T_NONE else None
        rope = self.tensor(st, ins.t[6])
        nq, nkv, hd, rot, pair, plus_one = ins.i[0], ins.i[1], ins.i[2], ins.i[3], ins.i[4], ins.i[6]
        gate = self.tensor(st, ins.t[7]) if ins.i[7] and ins.t[7] != pk.T_NONE else None
        ksc = self.tensor(st, ins.t[7]) if not ins.i[7] and ins.t[7] != pk.T_NONE else None      # e4m3 cache: per-cell scales
        if kc.dtype != BF16 and (ksc is None or kc.dtype != FP8 or hd != 128):
            raise EngineError("the sm_100a GQA kernels read a bf16 KV cache, or an e4m3 one with head dim 128 and no gated attention")
        gqa_ops.rope_kv(qkv, kc, vc, rope, self.d_in[1], self.d_in[2], self.d_page_table, nq, nkv, hd, rot=rot,
                        pair_mode=pair, qn=qn, kn=kn, eps=float(ins.f[0]), plus_one=bool(plus_one),
                        q_out=q_out.view(st.rows, nq, hd), gate_out=gate, kv_scale=ksc)

    def _op_attn(self, st, ins):
        ao, q, kc, vc = (self.tensor(st, ins.t[k]) for k in range(4))
        nq, nkv, hd, window = ins.i[0], ins.i[1], ins.i[2], ins.i[3]
        key = ("gqa_ws", nq, nkv, hd)
        if key not in st.scratch:
            st.scratch[key] = gqa_ops.AttnWorkspace(st.rows, nq, nkv, hd, self.max_ctx + PAGE, self.device)
        ksc = self.tensor(st, ins.t[4]) if ins.t[4] != pk.T_NONE else None
        gqa_ops.attention(q.view(st.rows, nq, hd), kc, vc, self.d_page_table, self.d_in[2], self.d_in[1], st.scratch[key],
                          scale=float(ins.f[0]), window=window, out=ao, kv_scale=ksc)

    # -- gated delta rule (hybrid linear-attention layers)
    def _op_gdn(self, st, ins):
        out, conv_state, ssm_state, qkvz, ba, conv_w, a_log, dt_bias = (self.tensor(st, ins.t[k]) for k in range(8))
        hk, hv, hd, conv = ins.i[0], ins.i[1], ins.i[2], ins.i[3]
        plan = self._gdn_plan
        if plan is None or plan["R"] != st.rows:
            gdn_ops.gdn(qkvz, ba, conv_w, a_log, dt_bias, conv_state, ssm_state, self.d_in[1], self.d_in[2], hk, hv, hd, conv, out=out)
            return
        # long runs of new rows: chunked (WY-form) prefill, 64 tokens at a time (ops/gdn.py::chunked_prefill); everything
        # else (decode riders, short runs, padding rows) stays on the token-by-token kernel, one call per row range
        for slot, r0, r1, fresh in plan["chunked"]:
            hist = torch.zeros_like(conv_state[slot], dtype=F32) if fresh else conv_state[slot]
            S0 = torch.zeros_like(ssm_state[slot], dtype=F32) if fresh else ssm_state[slot]
            o, h, S1 = gdn_ops.chunked_prefill(qkvz[r0:r1], ba[r0:r1], conv_w, a_log, dt_bias, hist, S0, hk, hv, hd, conv)
            out[r0:r1].copy_(o)
            conv_state[slot].copy_(h)
            ssm_state[slot].copy_(S1)
        for a, b in plan["rest"]:
            gdn_ops.gdn(qkvz[a:b], ba[a:b], conv_w, a_log, dt_bias, conv_state, ssm_state, self.d_in[1][a:b], self.d_in[2][a:b],
                        hk, hv, hd, conv, out=out[a:b])

    def _op_gated_norm(self, st, ins):
        out, o, z, gamma = (self.tensor(st, ins.t[k]) for k in range(4))
        gdn_ops.gated_norm(o, z, ins.i[2], gamma, ins.i[0], ins.i[1], float(ins.f[0]), out=out)

    def _op_sigmoid_gate(self, st, ins):
        out, a, gate = (self.tensor(st, ins.t[k]) for k in range(3))
        gdn_ops.sigmoid_gate(a, gate, out=out)

    # -- sparse-attention indexer
    SPARSE_MAX_ROWS = 256

    def _op_dsa_index(self, st, ins):
        kcache, ksc, ki, kn_w, kn_b, rope = (self.tensor(st, ins.t[k]) for k in range(6))
        dsa_ops.k_write(kcache, ksc, ki, kn_w, kn_b, rope, self.d_in[1], self.d_in[2], self.d_page_table, ins.i[1])

    def _op_dsa_topk(self, st, ins):
        sel, qi, wts, kcache, ksc, rope = (self.tensor(st, ins.t[k]) for k in range(6))
        if st.scratch.get("dsa_dense_ok", False):
            return                      # every position is below top_k: the attention of this step runs densely
        B = min(st.rows, self.SPARSE_MAX_ROWS)
        key = ("dsa_ws", B)
        if key not in st.scratch:
            st.scratch[key] = dsa_ops.SelectWorkspace(B, self.max_ctx + PAGE, self.device)
        for r0 in range(0, st.rows, B):
            r1 = min(st.rows, r0 + B)
            dsa_ops.select(qi[r0:r1], wts[r0:r1], kcache, ksc, rope, self.d_in[1][r0:r1], self.d_in[2][r0:r1], self.d_page_table,
                           ins.i[2], st.scratch[key], ins.i[3], out=sel[r0:r1])
        if self.taps is not None and not torch.cuda.is_current_stream_capturing():
            # eager steps only (run with cuda_graphs=False to tap decode): the selection and what it was computed from
            self.taps[("dsa_sel", ins.i[7])] = sel.clone()
            self.taps[("dsa_in", ins.i[7])] = (qi.clone(), wts.clone(), kcache, ksc, rope, ins.i[3])

    # -- MoE
    def _op_router_topk(self, st, ins):
        table, logits = self.tensor(st, ins.t[0]), self.tensor(st, ins.t[1])
        bias = self.tensor(st, ins.t[2]) if ins.t[2] != pk.T_NONE else None
        fused = st.route.get(id(ins))
        if fused is not None:
            g, moe = fused
            x, w = self.tensor(st, g.t[1]), self.static[g.t[2]]
            local = moe is not None and not (self.comm is not None and max(1, moe.i[4]) > 1)
            al = (None,) * 4
            e_base = e_local = shared_rows = 0
            if local:
                e_local, k, ep, sg = moe.i[1], moe.i[2], max(1, moe.i[4]), bool(moe.i[6])
                e_base = self.rank * e_local if ep > 1 else 0
                shared_rows = st.rows if sg else 0
                key = ("align", id(moe))
                if key not in st.scratch:
                    ng, n_pairs = e_local + (1 if sg else 0), st.rows * k
                    st.scratch[key] = (torch.empty(ng + 1, dtype=I32, device=self.device), torch.empty(ng + 1, dtype=I32, device=self.device),
                                       torch.empty(n_pairs, dtype=I32, device=self.device),
                                       torch.empty(n_pairs + shared_rows, dtype=I32, device=self.device))
                al = st.scratch[key]
                st.scratch[("aligned", id(moe))] = True
            if self._route_ticket is None:
                self._route_ticket = torch.zeros(1, dtype=I32, device=self.device)
            ep_fused = moe is not None and not local and getattr(self.comm, "impl", None) == "fused" and self.ep > 1
            native.call("plow_moe_route", table, None, x, x.stride(0), w, bias, st.rows, g.i[1], ins.i[0], ins.i[1], max(1, ins.i[2]),
                        max(1, ins.i[3]), ins.i[4], ins.i[5], float(ins.f[0]), int(local), e_base, e_local, al[0], al[1], al[2], al[3],
                        shared_rows, 0, self._route_ticket, self.comm.args_ptr() if ep_fused else None,
                        self.comm.cursor if ep_fused else None)
            if ep_fused:
                self.comm.dispatch(self, st, moe, counts_done=True)
                return
        else:
            native.call("plow_router_topk", table, logits, bias, st.rows, ins.i[0], ins.i[1], max(1, ins.i[2]), max(1, ins.i[3]),
                        ins.i[4], ins.i[5], float(ins.f[0]))
        if self.comm is not None and self.ep > 1:
            moe = next((m for m in st.prog.insts if m.op == Op.MOE_GEMM and m.t[2] == ins.t[0]), None)
            if moe is not None:
                self.comm.dispatch(self, st, moe)

    def _op_moe_experts(self, st, ins):
        y, h, table = (self.tensor(st, ins.t[k]) for k in range(3))
        shared = self.tensor(st, ins.t[5]) if ins.t[5] != pk.T_NONE else None
        E, e_local, k, F, ep = ins.i[0], ins.i[1], ins.i[2], ins.i[3], max(1, ins.i[4])
        sg = bool(ins.i[6])          # the shared expert is group e_local of the stacked expert weights
        T, H = st.rows, self.spec.hidden
        fp8 = self.spec.weight_quant == "fp8_block128"
        if self.comm is not None and ep > 1:
            return self.comm.moe_experts(self, st, ins)
        e_base = self.rank * e_local if ep > 1 else 0
        ng = e_local + (1 if sg else 0)
        n_rows = T * k + (T if sg else 0)
        if st.scratch.pop(("aligned", id(ins)), False):
            grp_off, tile_prefix, row_of_pair, pair_of_row = st.scratch[("align", id(ins))]      # laid out by the routing kernel
        else:
            grp_off, tile_prefix, row_of_pair, pair_of_row = rowops.moe_align(table, e_base, e_local, shared_rows=T if sg else 0)
        per = max(1, (T * k + e_local - 1) // e_local)
        swap = per <= 64
        if fp8:
            xq, sx = self._quant_of(st, ins.t[1], 0, H, h)
            xs, sxs = rowops.moe_gather(xq, sx, pair_of_row, grp_off[ng:], n_rows, k)
            w1, s1 = self.static_q[ins.t[3]]
            w2, s2 = self.static_q[ins.t[4]]
            if swap:
                bn = 32 if per <= 32 else 64
                hq, shq = gemm_ops.gemm(xs, w1, sx=sxs, sw=s1, dual=True, n_out=F, n_experts=ng, grp_off=grp_off,
                                        swap=True, bn=bn, quant_out=True, ld_syq=n_rows)
                yo = gemm_ops.gemm(hq, w2, sx=shq, sw=s2, n_out=H, n_experts=ng, grp_off=grp_off, swap=True, bn=bn)
            else:
                if gemm_ops._WIDE_DEFAULT and F % 128 == 0:
                    # 128 + 128 column SwiGLU tiles hold a token's whole 1x128 group: the e4m3 twin comes out of the epilogue
                    hq, shq = gemm_ops.gemm(xs, w1, sx=sxs, sw=s1, dual=True, n_out=F, n_experts=ng, grp_off=grp_off,
                                            tile_prefix=tile_prefix, swap=False, bn=128, quant_out=True, ld_syq=n_rows)
                else:
                    hb = gemm_ops.gemm(xs, w1, sx=sxs, sw=s1, dual=True, n_out=F, n_experts=ng, grp_off=grp_off,
                                       tile_prefix=tile_prefix, swap=False, bn=64)
                    hq, shq = rowops.quant_act(hb)
                yo = gemm_ops.gemm(hq, w2, sx=shq, sw=s2, n_out=H, n_experts=ng, grp_off=grp_off, tile_prefix=tile_prefix,
                                   swap=False, bn=128)
        else:
            w1, w2 = self._bf16_weight(ins.t[3]), self._bf16_weight(ins.t[4])
            xs = h[(pair_of_row // k).long().clamp_(0, T - 1)]
            bn = 32 if per <= 32 else 64
            hb = gemm_ops.gemm(xs, w1, dual=True, n_out=F, n_experts=ng, grp_off=grp_off, tile_prefix=tile_prefix,
                               swap=swap, bn=bn if swap else 128)
            yo = gemm_ops.gemm(hb, w2, n_out=H, n_experts=ng, grp_off=grp_off, tile_prefix=tile_prefix, swap=swap,
                               bn=bn if swap else 128)
        if sg:
            native.call("plow_moe_combine", y, yo, yo, table, row_of_pair, T, k, H, grp_off[e_local:])
        else:
            native.call("plow_moe_combine", y, yo, shared, table, row_of_pair, T, k, H, None)

    HANDLERS = {
        Op.EMBED: "_op_embed", Op.RMSNORM: "_op_rmsnorm", Op.ADD_NORM: "_op_add_norm", Op.RESIDUAL: "_op_residual",
        Op.GEMM: "_op_gemm", Op.ROW_GATHER: "_op_row_gather", Op.ARGMAX: "_op_argmax",
        Op.ROPE_KV: "_op_rope_kv", Op.ATTN: "_op_attn", Op.GLU: "_op_glu",
        Op.DSA_INDEX: "_op_dsa_index", Op.DSA_TOPK: "_op_dsa_topk",
        Op.GDN_STEP: "_op_gdn", Op.GATED_NORM: "_op_gated_norm", Op.SIGMOID_GATE: "_op_sigmoid_gate",
        Op.MLA_KV_WRITE: "_op_mla_kv_write", Op.MLA_DECODE: "_op_mla_attention", Op.MLA_PREFILL: "_op_mla_attention",
        Op.ROUTER_TOPK: "_op_router_topk", Op.MOE_GEMM: "_op_moe_experts", Op.NOP: None,
    }

    def _interp_segments(self, st: _Prog):
        """Cut the program into interpreter segments and role instructions (once per program)."""
        if st.segments is None:
            def tensor_of(h):
                t = st.t.get(h, self.static.get(h))
                return t if isinstance(t, torch.Tensor) else None

            def eligible(j):
                ins = st.prog.insts[j]
                if ins.op == Op.ARGMAX and ins.i[1]:
                    return False        # packed-key variant (vocabulary-sharded lm_head) is a role kernel
                outs = [ins.t[0]] + ([ins.t[4]] if ins.op == Op.ADD_NORM else [])
                if any(h != pk.T_NONE and self._wants_q(st, h) for h in outs):
                    return False        # the role kernel emits the e4m3 twin in the same pass
                acts = [tensor_of(h) for h in ins.t[:5] if h != pk.T_NONE]
                return all(t is not None for t in acts) and all(
                    t.dtype in (BF16, I32) or (ins.op == Op.ARGMAX and t.dtype == F32) for t in acts)
            st.interp = DeviceInterp(self.packet, st.prog, tensor_of, st.rows, st.samples, self.device)
            # a cooperative interpreter launch costs ~25 us whatever it runs (measured: one ADD_NORM of 64 rows takes
            # 26 us in it against 5.5 us as a role kernel), so runs shorter than `min_run` instructions stay role kernels
            min_run = int(os.environ.get("PLOW_INTERP_MIN_RUN", "2"))
            segs = []
            for lo, hi, on_device in DeviceInterp.segments(st.prog, eligible):
                if on_device and hi - lo < min_run:
                    segs.extend((j, j + 1, False) for j in range(lo, hi))
                else:
                    segs.append((lo, hi, on_device))
            st.segments = segs
        return st.segments

    def _run_insts(self, st: _Prog) -> None:
        st.q.clear()
        st.scratch["mla_items"] = False
        if self.profile_ops:
            # eager walk with an event pair around every instruction (diagnostic: serialises nothing, but the events
            # themselves cost a few microseconds per instruction)
            evs = []
            for ins in st.prog.insts:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                self._run_one(st, ins)
                b.record()
                evs.append((ins, a, b))
            torch.cuda.synchronize(self.device)
            self.op_times_last = [(Op(ins.op).name, tuple(int(v) for v in ins.i[:3]), a.elapsed_time(b)) for ins, a, b in evs]
            return
        if self.device_interp and self.spec.dtype == "bf16":
            for lo, hi, on_device in self._interp_segments(st):
                if on_device:
                    st.interp.run(lo, hi)
                else:
                    self._run_one(st, st.prog.insts[lo])
            return
        for ins in st.prog.insts:
            self._run_one(st, ins)

    def _run_one(self, st: _Prog, ins) -> None:
        name = self.HANDLERS.get(Op(ins.op), "missing")
        if name is None:
            return
        if name == "missing":
            fn = getattr(self, "_ext_" + Op(ins.op).name.lower(), None)
            if fn is None:
                raise EngineError(f"opcode {Op(ins.op).name} has no sm_100a body in this build")
            fn(st, ins)
        else:
            getattr(self, name)(st, ins)

    def step_multi(self, batch: TokenBatch, k: int) -> list:
        """k greedy decode steps chained on the device: after each graph replay the sampled ids become the next step's
        input ids and the positions advance by one (three small device ops), and the host reads all k rows of ids
        once at the end.  Falls back to the host loop while the rung's graph is not captured yet, under a rank group,
        or when logits are wanted."""
        rows = batch.rows
        st = self.progs.get(self.pick_program(max(rows, 1), True)) if batch.decode else None
        if (k <= 1 or not batch.decode or st is None or st.graph is None or not self.cuda_graphs or batch.want_logits
                or self.step_group is not None or self.leader_group is not None or int(batch.sample_rows.shape[0]) != rows
                or not np.array_equal(batch.sample_rows, np.arange(rows, dtype=batch.sample_rows.dtype))):
            return super().step_multi(batch, k)
        R = st.rows
        hin = self.h_in
        hin[0, :rows] = torch.from_numpy(batch.ids)
        hin[1, :rows] = torch.from_numpy(batch.pos)
        hin[2, :rows] = torch.from_numpy(batch.seq)
        hin[0, rows:R] = 0
        hin[1, rows:R] = 0
        hin[2, rows:R] = self.scratch_slot
        hin[3, :rows] = torch.from_numpy(batch.sample_rows)
        hin[3, rows:st.samples] = 0
        if self._multi_out is None or self._multi_out.shape[0] < k or self._multi_out.shape[1] < st.samples:
            self._multi_out = torch.zeros(max(k, 8), self.d_out_ids.shape[0], dtype=I32, device=self.device)
            self._h_multi_out = torch.zeros(max(k, 8), self.d_out_ids.shape[0], dtype=I32).pin_memory()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        self._upload_pages()
        self.d_in[:, :R].copy_(hin[:, :R], non_blocking=True)
        torch.add(self.d_in[1, :R], 1, out=self.d_kvlen_row[:R])
        if batch.hidden is not None and self.d_hidden_in is not None and rows:
            hid = batch.hidden if torch.is_tensor(batch.hidden) else torch.from_numpy(np.ascontiguousarray(batch.hidden))
            self.d_hidden_in[:rows].copy_(hid[:rows], non_blocking=True)
        self._mla_plan = None
        st.scratch["dsa_dense_ok"] = False
        try:
            for i in range(k):
                st.graph.replay()
                self._multi_out[i, :rows].copy_(self.d_out_ids[:rows])
                if i + 1 < k:
                    self.d_in[0, :rows].copy_(self.d_out_ids[:rows])
                    self.d_in[1, :rows].add_(1)
                    self.d_kvlen_row[:rows].add_(1)
            self._h_multi_out[:k, :rows].copy_(self._multi_out[:k, :rows], non_blocking=True)
            ev1.record()
            ev1.synchronize()
            native.check_status(self.device)
        except native.NativeLibraryError as e:
            self._recover_after_device_status()
            raise EngineError(str(e), fatal=False)
        ms = ev0.elapsed_time(ev1)
        self.step_ms_last = ms / k
        ids = self._h_multi_out[:k, :rows].numpy().copy()
        return [StepResult(ids=ids[i], logits=None, device_ms=ms / k) for i in range(k)]

    def step_launch(self, batch: TokenBatch, chain_from=None):
        """A decode rung's graph replayed without waiting for it: inputs go through one of two pinned staging blocks (the
        previous launch may not have read its block yet), a chained launch takes its ids from the previous step's output
        on the device, and the ids come back through one of two pinned result blocks that step_collect reads after the
        launch's event.  Anything the graph path does not cover (first use of a rung, logits, rank groups) runs as a
        plain step."""
        rows = batch.rows
        st = self.progs.get(self.pick_program(max(rows, 1), True)) if batch.decode else None
        plain = (not batch.decode or st is None or st.graph is None or not self.cuda_graphs or batch.want_logits or batch.want_hidden
                 or batch.hidden is not None or self.step_group is not None or self.leader_group is not None
                 or int(batch.sample_rows.shape[0]) != rows
                 or not np.array_equal(batch.sample_rows, np.arange(rows, dtype=batch.sample_rows.dtype)))
        if plain or (chain_from is not None and "event" not in chain_from):
            if chain_from is not None and "event" in chain_from:
                chain_from = dict(result=self.step_collect(chain_from))
            return super().step_launch(batch, chain_from)
        if getattr(self, "_la_in", None) is None:
            self._la_in = [torch.zeros_like(self.h_in).pin_memory() for _ in range(2)]
            self._la_out = [torch.zeros_like(self.h_out).pin_memory() for _ in range(2)]
            self._la_n = 0
        k = self._la_n & 1
        self._la_n += 1
        R = st.rows
        hin = self._la_in[k]
        hin[0, :rows] = 0 if chain_from is not None else torch.from_numpy(batch.ids)
        hin[1, :rows] = torch.from_numpy(batch.pos)
        hin[2, :rows] = torch.from_numpy(batch.seq)
        hin[0, rows:R] = 0
        hin[1, rows:R] = 0
        hin[2, rows:R] = self.scratch_slot
        hin[3, :rows] = torch.from_numpy(batch.sample_rows)
        hin[3, rows:st.samples] = 0
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        self._upload_pages()
        if chain_from is not None:
            self.d_in[1:, :R].copy_(hin[1:, :R], non_blocking=True)
            self.d_in[0, :rows].copy_(self.d_out_ids[:rows])          # the previous step's tokens, still on the device
        else:
            self.d_in[:, :R].copy_(hin[:, :R], non_blocking=True)
        torch.add(self.d_in[1, :R], 1, out=self.d_kvlen_row[:R])
        self._mla_plan = None
        st.scratch["dsa_dense_ok"] = False
        st.graph.replay()
        self._la_out[k][:rows].copy_(self.d_out_ids[:rows], non_blocking=True)
        ev1.record()
        return dict(event=(ev0, ev1), out=self._la_out[k], rows=rows)

    def step_collect(self, handle) -> StepResult:
        if "event" not in handle:
            return handle["result"]
        ev0, ev1 = handle["event"]
        try:
            ev1.synchronize()
            native.check_status(self.device)
        except native.NativeLibraryError as e:
            self._recover_after_device_status()
            raise EngineError(str(e), fatal=False)
        self.step_ms_last = ev0.elapsed_time(ev1)
        return StepResult(ids=handle["out"][:handle["rows"]].numpy().copy(), logits=None, device_ms=self.step_ms_last)

    def kv_arrays(self) -> dict:
        out = {t.name: self.static[h] for h, t in enumerate(self.packet.tensors) if t.tclass == pk.TClass.KV}
        out.update({f"smax.{layer}": v for layer, v in self.kv_smax.items()})   # per-page scale bounds of fp8 latent caches
        return out

    def _recover_after_device_status(self) -> None:
        try:
            torch.cuda.synchronize(self.device)
            gemm_ops.reset_workspace(self.device)
            native.status_word(self.device).zero_()
            for st in self.progs.values():
                st.graph = None
        except Exception:
            self.health = "dead"

    def state_arrays(self) -> dict:
        return {t.name: self.static[h] for h, t in enumerate(self.packet.tensors) if t.tclass == pk.TClass.STATE}

    # ---- step ----------------------------------------------------------------------------------
    def _sync_pages(self, slot: int) -> None:
        super()._sync_pages(slot)
        self._dirty_slots.add(slot)

    def _upload_pages(self) -> None:
        if not self._dirty_slots:
            return
        if len(self._dirty_slots) * 8 >= self.h_page_table.shape[0]:
            self.d_page_table.copy_(self.h_page_table, non_blocking=True)
        else:
            for slot in self._dirty_slots:
                self.d_page_table[slot].copy_(self.h_page_table[slot], non_blocking=True)
        self._dirty_slots.clear()

    def bind_thread(self) -> None:
        # a new host thread starts on device 0: kernels launched through ctypes go to the *current* device, so a
        # dispatcher thread of a rank on another GPU must select it first
        torch.cuda.set_device(self.device)

    def set_page_row(self, slot: int, row) -> None:
        """Follower ranks: install the leader's page-table row of `slot`."""
        n = min(len(row), self.h_page_table.shape[1])
        self.page_table[slot, :n] = row[:n]
        self._dirty_slots.add(slot)

    def idle_step(self) -> bool:
        if self.step_group is None:
            return False
        e = np.zeros(0, np.int32)
        return self.step(TokenBatch(e, e, e, e, decode=True)) is not None

    def step(self, batch: TokenBatch, replay: bool = False) -> StepResult:
        rows, ns = batch.rows, int(batch.sample_rows.shape[0])
        decode = batch.decode
        if self.step_group is not None:
            # every rank launches the same program: agree on role and row count first (a rank without work joins with
            # an empty batch; when no rank has work nothing is launched)
            decode, g_rows, busy, g_samples = self.step_group.agree(batch.decode, rows, rows > 0, samples=ns)
            if not busy:
                return None
            prog_rows = g_rows
        else:
            prog_rows = rows
        if self.leader_group is not None and self.rank == 0 and not replay:
            self.leader_group.publish(dict(
                batch=dict(ids=batch.ids, pos=batch.pos, seq=batch.seq, sample_rows=batch.sample_rows, decode=batch.decode,
                           want_logits=batch.want_logits),
                pages={int(s): self.page_table[s].copy() for s in self._dirty_slots}))
        idx = self.pick_program(max(prog_rows, 1), decode)
        st = self._prepare(idx)
        st.prog = self.packet.programs[idx]
        R = st.rows
        if ns > st.samples:
            raise EngineError(f"step samples {ns} rows but the program samples {st.samples}: compile with max_seqs >= the decode width")
        hin = self.h_in
        hin[0, :rows] = torch.from_numpy(batch.ids)
        hin[1, :rows] = torch.from_numpy(batch.pos)
        hin[2, :rows] = torch.from_numpy(batch.seq)
        hin[0, rows:R] = 0
        hin[1, rows:R] = 0
        hin[2, rows:R] = self.scratch_slot
        if ns:
            hin[3, :ns] = torch.from_numpy(batch.sample_rows)
        hin[3, ns:st.samples] = 0
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        self._upload_pages()
        self.d_in[:, :R].copy_(hin[:, :R], non_blocking=True)
        torch.add(self.d_in[1, :R], 1, out=self.d_kvlen_row[:R])
        if batch.hidden is not None and self.d_hidden_in is not None and rows:
            hid = batch.hidden if torch.is_tensor(batch.hidden) else torch.from_numpy(np.ascontiguousarray(batch.hidden))
            self.d_hidden_in[:rows].copy_(hid[:rows], non_blocking=True)
        self._mla_plan = None
        self._gdn_plan = self._plan_gdn_prefill(batch, R) if (not decode and rows > 0 and self._has_gdn) else None
        # eager (prefill) steps of a sparse-attention model whose positions all lie below top_k attend densely
        st.scratch["dsa_dense_ok"] = bool(not decode and self._dsa_topk and rows > 0 and int(batch.pos.max()) < self._dsa_topk)
        if not decode and rows > 0 and self._has_mla:
            self._mla_plan = self._plan_mla_prefill(batch, R)
            self._mla_plan_rows = rows
        try:
            if self.cuda_graphs and decode:
                if st.graph is None:
                    # the first step of a rung runs eagerly (allocations, attribute sets) and IS the step; the graph is
                    # captured afterwards without being replayed, because a program with recurrent state (gated delta
                    # rule) is not idempotent: executing it twice would advance the state twice
                    self._run_insts(st)
                    torch.cuda.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        self._run_insts(st)
                    st.graph = g
                else:
                    st.graph.replay()
            else:
                self._run_insts(st)
            self.h_out[:st.samples].copy_(self.d_out_ids[:st.samples], non_blocking=True)
            ev1.record()
            ev1.synchronize()
            native.check_status(self.device)
        except native.NativeLibraryError as e:
            # a bounded wait ran out or a bounds check fired: the step failed, the context is fine.  Shared scratch
            # that kernels only re-arm on a clean finish (split-K arrival counters) is zeroed and captured graphs
            # are dropped, so the next step starts from a known state.
            self._recover_after_device_status()
            raise EngineError(str(e), fatal=False)
        self.step_ms_last = ev0.elapsed_time(ev1)
        logits = self.d_logits[:ns].float().cpu().numpy() if batch.want_logits else None
        hidden = None
        if batch.want_hidden and self.d_hidden_out is not None:
            hidden = self.d_hidden_out[:rows if self.hidden_rows == "rows" else ns].clone()      # stays on the device
        return StepResult(ids=self.h_out[:ns].numpy().copy(), logits=logits, device_ms=self.step_ms_last, hidden=hidden)
