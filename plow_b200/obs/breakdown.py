"""Breakdown logs: where a tick, a decode step and a request's time to first token go.

Three JSON-lines logs, each off unless its switch is set (environment, read once):

* ``PLOW_TICK_LOG=1``  one line per scheduler tick: kind (prefill / decode / spec / lookahead), rows, requests, the
  engine's device time, the tick's wall time and their difference (the host remainder), queue and seat counts, the
  decode rung;
* ``PLOW_DSTEP_LOG=1`` one line per decode engine call: rows, rung, steps chained in the call, device ms per step, host
  ms around the call;
* ``PLOW_TTFT_LOG=1``  one line per request at its first token: time queued before it got a slot, prefill chunks with
  their summed device time, wall time from seat to first token, cached prompt tokens.

Lines go to ``PLOW_OBS_LOG_FILE`` (appended) or standard error through a writer thread with a bounded queue: a slow
disk drops lines (counted in the ``dropped`` field of later lines) instead of stalling the dispatcher.
Reference: crates/plowrt/src/obs/{tick,dstep,ttft,logwriter}.rs.
"""
from __future__ import annotations

import json
import os
import queue
import sys
import threading
import time


class LogWriter:
    """Non-blocking line writer: ``put`` never waits."""

    def __init__(self, path: str | None = None, cap: int = 8192):
        self.path, self.q = path, queue.Queue(maxsize=cap)
        self.dropped = 0
        self._thread: threading.Thread | None = None
        self._lock = threading.Lock()

    def put(self, rec: dict) -> None:
        if self._thread is None:
            with self._lock:
                if self._thread is None:
                    self._thread = threading.Thread(target=self._run, daemon=True, name="plow-obs-log")
                    self._thread.start()
        if self.dropped:
            rec = dict(rec, dropped=self.dropped)
        try:
            self.q.put_nowait(rec)
        except queue.Full:
            self.dropped += 1

    def _run(self) -> None:
        f = open(self.path, "a", buffering=1) if self.path else sys.stderr
        while True:
            rec = self.q.get()
            if rec is None:
                break
            try:
                f.write(json.dumps(rec, separators=(",", ":")) + "\n")
            except Exception:
                self.dropped += 1
        if self.path:
            f.close()

    def flush(self, timeout_s: float = 2.0) -> None:
        t0 = time.monotonic()
        while not self.q.empty() and time.monotonic() - t0 < timeout_s:
            time.sleep(0.005)
        time.sleep(0.01)


class Breakdown:
    """The three logs behind one object; every ``*_on`` is a plain attribute read on the hot path."""

    def __init__(self, env=None, writer: LogWriter | None = None):
        env = os.environ if env is None else env
        on = lambda k: str(env.get(k, "0")).lower() in ("1", "true", "yes", "on")      # noqa: E731
        self.tick_on, self.dstep_on, self.ttft_on = on("PLOW_TICK_LOG"), on("PLOW_DSTEP_LOG"), on("PLOW_TTFT_LOG")
        self.any = self.tick_on or self.dstep_on or self.ttft_on
        self.writer = writer or (LogWriter(env.get("PLOW_OBS_LOG_FILE") or None) if self.any else None)
        self.seq = 0
        self._last_end: float | None = None

    def tick(self, kind: str, rows: int, reqs: int, device_ms: float, wall_ms: float, queued: int, live: int, rung: int = 0) -> None:
        if not self.tick_on:
            return
        now = time.perf_counter()
        gap = (now - wall_ms / 1e3 - self._last_end) * 1e3 if self._last_end is not None else 0.0
        self._last_end = now
        self.seq += 1
        self.writer.put(dict(log="TICK", seq=self.seq, kind=kind, rows=rows, reqs=reqs, device_ms=round(device_ms, 3),
                             wall_ms=round(wall_ms, 3), host_ms=round(max(0.0, wall_ms - device_ms), 3),
                             idle_before_ms=round(max(0.0, gap), 3), queued=queued, live=live, rung=rung))

    def dstep(self, rows: int, rung: int, steps: int, device_ms: float, pre_ms: float, post_ms: float) -> None:
        if not self.dstep_on:
            return
        self.writer.put(dict(log="DSTEP", rows=rows, rung=rung, steps=steps, device_ms_per_step=round(device_ms, 3),
                             host_pre_ms=round(pre_ms, 3), host_post_ms=round(post_ms, 3)))

    def ttft(self, rid: str, prompt_tokens: int, cached: int, queued_ms: float, chunks: int, prefill_device_ms: float,
             seat_to_first_ms: float, total_ms: float) -> None:
        if not self.ttft_on:
            return
        self.writer.put(dict(log="TTFT", rid=rid, prompt_tokens=prompt_tokens, cached_tokens=cached, queued_ms=round(queued_ms, 3),
                             prefill_chunks=chunks, prefill_device_ms=round(prefill_device_ms, 3),
                             seat_to_first_ms=round(seat_to_first_ms, 3), ttft_ms=round(total_ms, 3),
                             host_and_wait_ms=round(max(0.0, seat_to_first_ms - prefill_device_ms), 3)))
