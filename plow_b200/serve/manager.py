"""Multi-model residency: which models are loaded on the device group, within a memory budget.

A model that is asked for and not resident is loaded; when the budget cannot hold it, the least recently used idle
models are drained and unloaded first; a model with live requests is never evicted (the load fails with
``ResidencyError`` when nothing can be evicted).  Loads are serialised.  Reference: crates/plowrt/src/serve/manager.rs:1-52
(S1 residency manager + VRAM planner), serve/cosched.rs (per-device-group turns)."""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field


class ResidencyError(RuntimeError):
    pass


@dataclass
class Resident:
    name: str
    entry: object          # whatever the loader returned (a ModelEntry in the server)
    nbytes: int
    last_used: float = field(default_factory=time.monotonic)
    loads: int = 1


class ModelManager:
    def __init__(self, budget_bytes: int, loader, sizer, live_of=lambda e: 0, unloader=lambda e: None, catalog=None,
                 clock=time.monotonic):
        """loader(name, path) -> entry; sizer(name, path) -> bytes needed; live_of(entry) -> live requests;
        unloader(entry) drains and frees; catalog: name -> path of the models that may be loaded."""
        self.budget, self.loader, self.sizer, self.live_of, self.unloader = budget_bytes, loader, sizer, live_of, unloader
        self.catalog = dict(catalog or {})
        self.clock = clock
        self.resident: dict[str, Resident] = {}
        self.lock = threading.Lock()
        self.evictions = 0

    def used(self) -> int:
        return sum(r.nbytes for r in self.resident.values())

    def available(self) -> list:
        return sorted(self.catalog)

    def status(self) -> dict:
        return {n: dict(state="resident", bytes=r.nbytes, live=self.live_of(r.entry), loads=r.loads) for n, r in self.resident.items()} | \
               {n: dict(state="available") for n in self.catalog if n not in self.resident}

    def plan(self, need: int) -> list:
        """Names to evict (LRU first, idle only) so that ``need`` more bytes fit; raises when impossible."""
        free = self.budget - self.used()
        victims = []
        for r in sorted(self.resident.values(), key=lambda r: r.last_used):
            if free >= need:
                break
            if self.live_of(r.entry) == 0:
                victims.append(r.name)
                free += r.nbytes
        if free < need:
            raise ResidencyError(f"need {need} bytes, only {free} can be freed (budget {self.budget})")
        return victims

    def acquire(self, name: str, path: str | None = None):
        """Return the resident entry of ``name``, loading (and evicting) as needed."""
        with self.lock:
            r = self.resident.get(name)
            if r is not None:
                r.last_used = self.clock()
                return r.entry
            path = path or self.catalog.get(name)
            if path is None:
                raise ResidencyError(f"model '{name}' is not in the catalog")
            need = int(self.sizer(name, path))
            if need > self.budget:
                raise ResidencyError(f"model '{name}' needs {need} bytes, budget is {self.budget}")
            for v in self.plan(need):
                self.unloader(self.resident[v].entry)
                del self.resident[v]
                self.evictions += 1
            entry = self.loader(name, path)
            self.resident[name] = Resident(name, entry, need, self.clock())
            self.catalog.setdefault(name, path)
            return entry

    def unload(self, name: str) -> None:
        with self.lock:
            r = self.resident.get(name)
            if r is None:
                raise ResidencyError(f"model '{name}' is not resident")
            if self.live_of(r.entry):
                raise ResidencyError(f"model '{name}' has live requests")
            self.unloader(r.entry)
            del self.resident[name]


def packet_bytes(assets_dir, max_slots: int, max_ctx: int) -> int:
    """Device bytes a packet needs: weights + KV pool for the requested geometry + activation arena (from build.json
    and the tensor table; the same arithmetic the engine's allocator performs)."""
    from pathlib import Path

    from ..compiler import packet as pk
    pkt = pk.read_packet(Path(assets_dir) / "model.pkt")
    pages = max_slots * ((max_ctx + 63) // 64) + 1
    total = 0
    for t in pkt.tensors:
        n = pk.DTYPE_BYTES[pk.DType(t.dtype)]
        for d in t.dims:
            n *= pages if d == -3 else (max_slots + 1 if d == -4 else (0 if d < 0 else d))
        if t.tclass in (pk.TClass.WEIGHT, pk.TClass.DERIVED, pk.TClass.GEN, pk.TClass.KV, pk.TClass.STATE):
            total += n
    return total + max(p.arena_bytes for p in pkt.programs)
