"""Overload control: degrade by policy when the engine misses its deadlines, refuse new work last.

The signal is the fraction of deadlines missed over a sliding window (ten buckets).  Here a deadline is a token's
time-between-tokens objective (``tbt_target_ms``; a gap of more than 1.5 x the objective is a miss) or a request's own
``deadline_ms``.  The level moves one step at a time: up when the fraction has stayed over that level's threshold for a
dwell (half the window: a burst of misses is not overload), down when it has fallen under half the threshold below, and
at most once per dwell either way.  What each level does to a text-generation server:

1. prefill chunks are halved (decode steps of running requests wait less behind prompt work);
2. prefill chunks are quartered and speculative / lookahead extras are switched off;
3. requests that do not continue a retained session are refused with 429 and ``Retry-After`` — only once level 2 has
   held for a whole window.  Sessions already being served go on.

Off unless ``PLOW_OVERLOAD=1`` (or the scheduler is given a controller); window and thresholds:
``PLOW_OVERLOAD_WINDOW_MS`` (default 10000), ``PLOW_OVERLOAD_MISS`` (default ``0.05,0.10,0.20``).
Reference: crates/plowrt/src/serve/overload.rs:1-15.
"""
from __future__ import annotations

import os
import time

BUCKETS = 10
MIN_SAMPLES = 20


class OverloadControl:
    def __init__(self, window_s: float = 10.0, up=(0.05, 0.10, 0.20), clock=time.monotonic):
        self.window, self.up, self.clock = float(window_s), tuple(up), clock
        self.span = self.window / BUCKETS
        self.hits = [0] * BUCKETS
        self.miss = [0] * BUCKETS
        self.stamp = [-1] * BUCKETS          # which span index a bucket currently holds
        self.level = 0
        self._over_since = None              # since when the fraction has been over the current level's threshold
        self._under_since = None
        self._moved_at = -1e18
        self._level2_since = None

    @staticmethod
    def from_env(env=None):
        env = os.environ if env is None else env
        if str(env.get("PLOW_OVERLOAD", "0")).lower() not in ("1", "true", "yes", "on"):
            return None
        up = tuple(float(x) for x in str(env.get("PLOW_OVERLOAD_MISS", "0.05,0.10,0.20")).split(","))
        if len(up) != 3 or not all(0 < a < 1 for a in up) or list(up) != sorted(up):
            raise ValueError("PLOW_OVERLOAD_MISS wants three ascending fractions in (0, 1)")
        return OverloadControl(float(env.get("PLOW_OVERLOAD_WINDOW_MS", "10000")) / 1e3, up)

    # ---- signal --------------------------------------------------------------------------------
    def _bucket(self, now: float) -> int:
        idx = int(now / self.span)
        b = idx % BUCKETS
        if self.stamp[b] != idx:
            self.stamp[b], self.hits[b], self.miss[b] = idx, 0, 0
        return b

    def record(self, met: bool) -> None:
        now = self.clock()
        b = self._bucket(now)
        self.hits[b] += 1
        self.miss[b] += 0 if met else 1
        self._update(now)

    def fraction(self, now: float | None = None):
        now = self.clock() if now is None else now
        lo = int(now / self.span) - BUCKETS + 1
        n = sum(h for h, s in zip(self.hits, self.stamp) if s >= lo)
        m = sum(x for x, s in zip(self.miss, self.stamp) if s >= lo)
        return (m / n if n else 0.0), n

    def _update(self, now: float) -> None:
        frac, n = self.fraction(now)
        dwell = self.window / 2
        rise = self.level < 3 and n >= MIN_SAMPLES and frac > self.up[self.level]
        fall = self.level > 0 and frac < 0.5 * self.up[self.level - 1]
        self._over_since = (self._over_since if self._over_since is not None else now) if rise else None
        self._under_since = (self._under_since if self._under_since is not None else now) if fall else None
        if now - self._moved_at < dwell:
            return
        if rise and now - self._over_since >= dwell:
            if self.level == 2 and (self._level2_since is None or now - self._level2_since < self.window):
                return                      # refusing new work needs level 2 to have held a whole window
            self.level += 1
            self._moved_at, self._over_since = now, None
            if self.level == 2:
                self._level2_since = now
        elif fall and now - self._under_since >= dwell:
            self.level -= 1
            self._moved_at, self._under_since = now, None
            if self.level < 2:
                self._level2_since = None

    def tick(self) -> None:
        """Let time pass without samples (an idle server recovers)."""
        self._update(self.clock())

    # ---- policy --------------------------------------------------------------------------------
    def prefill_scale(self) -> float:
        return (1.0, 0.5, 0.25, 0.25)[self.level]

    def extras_allowed(self) -> bool:
        return self.level < 2

    def admit(self, continues_session: bool) -> bool:
        return self.level < 3 or continues_session

    def retry_after_s(self) -> int:
        return max(1, int(self.window / 2))
