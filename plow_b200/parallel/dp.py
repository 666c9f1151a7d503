"""Data-parallel serving: N full engine copies behind a lock-free router.

Routing order: session affinity -> longest cached prefix -> least loaded; dead replicas are
skipped and `/health` reports "degraded" while at least one replica is alive (reference:
crates/plowrt/src/serve/dp.rs:1-16, docs/runtime/data-parallel.md:1-72).
"""
from __future__ import annotations

from ..runtime.engine import EngineHealth


class DpRouter:
    def __init__(self, muxes: list):
        self.muxes = muxes
        self.sessions: dict[str, int] = {}

    def alive(self) -> list:
        return [i for i, m in enumerate(self.muxes) if m.engine.health != EngineHealth.DEAD and not m.draining]

    def pick(self, ids: list, session_id: str | None = None) -> int:
        alive = self.alive()
        if not alive:
            raise RuntimeError("no data-parallel replica is alive")
        if session_id and self.sessions.get(session_id) in alive:
            return self.sessions[session_id]
        hits = {i: self.muxes[i].engine.pool.cached_prefix_len(ids) for i in alive}
        best_hit = max(hits.values())
        cands = [i for i in alive if hits[i] == best_hit] if best_hit > 0 else alive
        choice = min(cands, key=lambda i: (len(self.muxes[i].live) + len(self.muxes[i].waiting) + self.muxes[i].ingress.qsize(), i))
        if session_id:
            self.sessions[session_id] = choice
        return choice

    def route(self, _entry, ids: list, session_id: str | None = None):
        return self.muxes[self.pick(ids, session_id)]
