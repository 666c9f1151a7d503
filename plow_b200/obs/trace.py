"""Host timeline trace in Chrome ``traceEvents`` JSON (served at ``GET /trace`` when enabled;
reference: crates/plowrt/src/obs/trace.rs)."""
from __future__ import annotations

import json
import threading
import time


class Timeline:
    def __init__(self, enabled: bool = False, cap: int = 200000):
        self.enabled, self.cap = enabled, cap
        self.events: list = []
        self.lock = threading.Lock()
        self.t0 = time.perf_counter()

    def span(self, name: str, cat: str = "engine", **args):
        return _Span(self, name, cat, args)

    def add(self, name, cat, ts_us, dur_us, args):
        if not self.enabled:
            return
        with self.lock:
            if len(self.events) < self.cap:
                self.events.append(dict(name=name, cat=cat, ph="X", ts=ts_us, dur=dur_us, pid=0,
                                        tid=threading.get_ident() % 1000, args=args))

    def to_json(self) -> str:
        with self.lock:
            return json.dumps(dict(traceEvents=list(self.events)))


class _Span:
    def __init__(self, tl, name, cat, args):
        self.tl, self.name, self.cat, self.args = tl, name, cat, args

    def __enter__(self):
        self.t = time.perf_counter()
        return self

    def __exit__(self, *exc):
        now = time.perf_counter()
        self.tl.add(self.name, self.cat, (self.t - self.tl.t0) * 1e6, (now - self.t) * 1e6, self.args)
        return False
