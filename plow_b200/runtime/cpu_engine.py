"""CPU backend: the C++ counter-gated interpreter (``libplow_cpu.so``) behind the engine interface.

Everything is fp32.  Weights are read from the checkpoint by name, derived tensors built from
their recipes, RoPE tables generated; KV pools are plain host arrays indexed through the page
table.  Reference counterpart: crates/plowrt/src/exec/cpu/engine.rs and device/cpu.rs (the CPU
reference backend the hermetic API tests run on).
"""
from __future__ import annotations

import ctypes as C
import json
import os
from pathlib import Path

import numpy as np
import torch

from ..compiler import packet as pk
from ..ops import native
from ..utils.rope import rope_table
from .engine import EngineBase, EngineError, StepResult, TokenBatch
from .kv_pages import PAGE
from .weights import materialize, open_checkpoint


class StepIO(C.Structure):
    _fields_ = [("rows", C.c_int32), ("n_sample", C.c_int32), ("page_table", C.c_void_p),
                ("max_pages", C.c_int32), ("kvlen", C.c_void_p), ("n_slots", C.c_int32),
                ("pos", C.c_void_p), ("seq", C.c_void_p)]


class CpuEngine(EngineBase):
    def __init__(self, assets_dir, max_slots: int = 8, n_pages: int | None = None, max_ctx: int = 1024,
                 n_threads: int | None = None, prefix_cache: bool = True):
        assets = Path(assets_dir)
        packet = pk.read_packet(assets / "model.pkt")
        n_pages = n_pages or max_slots * ((max_ctx + PAGE - 1) // PAGE)
        super().__init__(packet, max_slots, n_pages, max_ctx, prefix_cache)
        from ..compiler.audit import audit_ops
        a = audit_ops(packet, "cpu")
        if not a["ok"]:
            raise EngineError(f"the CPU backend has no body for {a['missing'] or a['unclassified']} (used by this packet)", fatal=True)
        lib = native.cpu_lib()
        lib.plow_pkt_open.restype = C.c_void_p
        lib.plow_pkt_open.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
        lib.plow_cpu_engine_create.restype = C.c_void_p
        lib.plow_cpu_engine_create.argtypes = [C.c_void_p, C.c_int]
        lib.plow_cpu_bind.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        lib.plow_cpu_run.argtypes = [C.c_void_p, C.c_int, C.POINTER(StepIO)]
        lib.plow_cpu_engine_destroy.argtypes = [C.c_void_p]
        lib.plow_pkt_close.argtypes = [C.c_void_p]
        lib.plow_cpu_set_watchdog.argtypes = [C.c_void_p, C.c_double]
        lib.plow_cpu_set_trace.argtypes = [C.c_void_p, C.c_int]
        self.lib = lib
        err = C.create_string_buffer(256)
        self._pkt = lib.plow_pkt_open(str(assets / "model.pkt").encode(), err, 256)
        if not self._pkt:
            raise EngineError(f"packet rejected: {err.value.decode()}", fatal=True)
        n_threads = n_threads or min(packet.n_cu, os.cpu_count() or 1)
        self._eng = lib.plow_cpu_engine_create(self._pkt, n_threads)
        if not self._eng:
            lib.plow_pkt_close(self._pkt)
            raise EngineError("the CPU engine could not allocate the packet's activation arena", fatal=True)
        self._keep: dict[int, object] = {}
        self._bind_all(assets)

    # ---- binding -------------------------------------------------------------------------------
    def _bind(self, handle: int, arr) -> None:
        self._keep[handle] = arr
        ptr = arr.data_ptr() if isinstance(arr, torch.Tensor) else arr.ctypes.data
        self.lib.plow_cpu_bind(self._eng, handle, C.c_void_p(ptr))

    def _bind_all(self, assets: Path) -> None:
        pkt = self.packet
        ckpt_dir = assets / "checkpoint"
        ckpt = open_checkpoint(ckpt_dir)
        derived = pkt.section_json("derived_weights.json") or {}
        gen = pkt.section_json("gen_tensors.json") or {}
        max_rows = max(p.rows for p in pkt.programs)
        self.in_ids = np.zeros(max_rows, dtype=np.int32)
        self.in_pos = np.zeros(max_rows, dtype=np.int32)
        self.in_seq = np.zeros(max_rows, dtype=np.int32)
        self.in_sample = np.zeros(max_rows, dtype=np.int32)
        self.out_ids = np.zeros(max_rows, dtype=np.int32)
        self.out_logits = np.zeros((max_rows, self.spec.vocab), dtype=np.float32)
        self.in_hidden = np.zeros((max_rows, self.spec.hidden), dtype=np.float32)
        self.out_hidden = np.zeros((max_rows, self.spec.hidden), dtype=np.float32)
        self.hidden_rows = None        # "rows" | "samples": which rows out.hidden carries (None: the packet has none)
        for h, t in enumerate(pkt.tensors):
            tc = t.tclass
            if tc in (pk.TClass.WEIGHT, pk.TClass.DERIVED):
                w = materialize(t.name, t, derived.get(t.name), ckpt).to(torch.float32).contiguous()
                self._bind(h, w)
            elif tc == pk.TClass.GEN:
                m = gen[t.name]
                self._bind(h, np.ascontiguousarray(rope_table(min(t.dims[0], max(self.max_ctx, 64)), m["rot_dim"], m["theta"], m.get("scaling"))))
            elif tc == pk.TClass.KV:
                dims = [self.pool.n_pages if d == -3 else d for d in t.dims]
                self._bind(h, np.zeros(dims, dtype=np.float32))
            elif tc == pk.TClass.STATE:          # recurrent state: one entry per slot, zero until position 0 resets it
                dims = [self.max_slots if d == -4 else d for d in t.dims]
                self._bind(h, np.zeros(dims, dtype=np.float32))
            elif tc == pk.TClass.INPUT:
                self._bind(h, {"in.ids": self.in_ids, "in.pos": self.in_pos, "in.seq": self.in_seq,
                               "in.sample_rows": self.in_sample, "in.hidden": self.in_hidden}[t.name])
            elif tc == pk.TClass.OUTPUT:
                self._bind(h, {"out.ids": self.out_ids, "out.logits": self.out_logits, "out.hidden": self.out_hidden}[t.name])
                if t.name == "out.hidden":
                    self.hidden_rows = "rows" if t.dims[0] == -1 else "samples"

    # ---- step ----------------------------------------------------------------------------------
    def step(self, batch: TokenBatch) -> StepResult:
        rows, ns = batch.rows, int(batch.sample_rows.shape[0])
        prog = self.pick_program(rows, batch.decode)
        self.in_ids[:rows] = batch.ids
        self.in_pos[:rows] = batch.pos
        self.in_seq[:rows] = batch.seq
        self.in_sample[:ns] = batch.sample_rows
        if batch.hidden is not None:
            self.in_hidden[:rows] = batch.hidden
        io = StepIO(rows=rows, n_sample=ns, page_table=self.page_table.ctypes.data,
                    max_pages=self.max_pages_per_seq, kvlen=self.kvlen.ctypes.data, n_slots=self.max_slots,
                    pos=self.in_pos.ctypes.data, seq=self.in_seq.ctypes.data)
        rc = self.lib.plow_cpu_run(self._eng, prog, C.byref(io))
        if rc != 0:
            raise EngineError(f"cpu interpreter failed with code {rc}", fatal=rc == 2)
        return StepResult(ids=self.out_ids[:ns].copy(),
                          logits=self.out_logits[:ns].copy() if batch.want_logits else None,
                          hidden=self.out_hidden[:rows if self.hidden_rows == "rows" else ns].copy()
                          if batch.want_hidden and self.hidden_rows else None)

    def kv_arrays(self) -> dict:
        return {t.name: self._keep[h] for h, t in enumerate(self.packet.tensors) if t.tclass == pk.TClass.KV}

    def state_arrays(self) -> dict:
        return {t.name: self._keep[h] for h, t in enumerate(self.packet.tensors) if t.tclass == pk.TClass.STATE}

    def close(self) -> None:
        if getattr(self, "_eng", None):
            self.lib.plow_cpu_engine_destroy(self._eng)
            self.lib.plow_pkt_close(self._pkt)
            self._eng = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
