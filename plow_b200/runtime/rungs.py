"""Decode-rung admission control and the M/D/1 service table.

A packet carries one decode program per *rung* (row count).  A step always runs the narrowest rung that covers its
rows, so how many sequences are seated decides which program every decode step pays for.  :class:`RungController`
turns that into a policy: it keeps an *admission seat* (an index into the ascending rung widths) that the scheduler
uses as its concurrency limit, widens it at once when requests queue (or when the projected wait breaks the latency
objective, or when the demanded token rate fills the seat), narrows it one rung at a time after a long quiet spell,
and — once it has timed neighbouring rungs — prefers the narrower rung when that one measures more tokens per second
(a margin keeps sampling noise from moving it; the margin is larger while requests wait, because narrowing then idles
slots somebody is queued for).  Nothing here allocates per tick.

:class:`ServiceTable` is the other half: a decode step of a compiled packet is deterministic to a fraction of a
percent, so queueing delay follows the M/D/1 form of the Pollaczek-Khinchine formula, ``Wq = rho S / (2 (1 - rho))``
— half the M/M/1 figure at the same utilisation — with the service time ``S`` read from a table (the packet's modelled
step times, replaced by measurements as they arrive) instead of being learned from scratch.

Reference: crates/plowrt/src/sched/rungs.rs:7-18 (thresholds), :265-353 (decision order), :355-449 (estimates and the
throughput seat); crates/plowrt/src/sched/mdq.rs:1-40 (M/D/1 service table and batch window).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

WIDEN_UTIL = 0.85            # demanded tokens/s over the seat's capacity above which the seat widens by one
NARROW_UTIL = 0.60           # ... and below which (on the next narrower rung) a quiet spell may narrow it
NARROW_TICKS = 128           # length of that quiet spell
MIN_DWELL_TICKS = 64         # ticks a seat is held before it may narrow for low load
MIN_SAMPLES = 4              # timed steps a rung needs before its tokens/s is believed
MARGIN_IDLE, MARGIN_BACKLOG = 1.03, 1.10
THROUGHPUT_DWELL_TICKS = 8


class Ewma:
    def __init__(self, alpha: float = 0.2):
        self.alpha, self.value, self.n = alpha, 0.0, 0

    def update(self, x: float) -> None:
        self.value = x if self.n == 0 else self.value + self.alpha * (x - self.value)
        self.n += 1


@dataclass
class RungLoad:
    occupied: int                 # sequences seated now
    queued: int                   # requests waiting for a seat
    oldest_wait_ms: float = 0.0
    arrival_rps: float = 0.0
    mean_output_tokens: float = 1.0
    slo_ms: float = 0.0


@dataclass
class RungDecision:
    actual: int                   # rung index the seated sequences need
    admission: int                # rung index admission may fill
    reason: str                   # hold | occupied | backlog | slo | utilization | throughput | low_load | single


def validate_rungs(widths, capacity: int) -> list:
    """Ascending positive widths whose widest equals the slot capacity."""
    w = [int(x) for x in widths]
    if not w:
        raise ValueError("no decode rungs")
    if any(x <= 0 for x in w):
        raise ValueError("a decode rung of zero rows")
    if any(b <= a for a, b in zip(w, w[1:])):
        raise ValueError("decode rungs must ascend")
    if w[-1] != capacity:
        raise ValueError(f"widest rung {w[-1]} != slot capacity {capacity}")
    return w


class RungController:
    def __init__(self, widths, capacity: int | None = None, min_seat: int = 0, nominal_max: int | None = None,
                 elastic_max: int | None = None, elastic_wait_ms: float = 250.0, fast_probe: bool = False,
                 throughput: bool = True):
        self.widths = validate_rungs(widths, capacity if capacity is not None else int(list(widths)[-1]))
        n = len(self.widths)
        self.service = [Ewma() for _ in range(n)]       # ms per engine call at this rung
        self.step = [Ewma() for _ in range(n)]          # ms per decode step at this rung
        self.min_seat = min(min_seat, n - 1)
        self.target = self.min_seat
        self.nominal = None if nominal_max is None else self.covering(nominal_max)
        self.elastic = None if elastic_max is None else self.covering(elastic_max)
        self.elastic_wait_ms = max(0.0, elastic_wait_ms)
        self.fast_probe, self.throughput = fast_probe, throughput
        self.dwell = MIN_DWELL_TICKS
        self.quiet = 0

    # ---- geometry ------------------------------------------------------------------------------
    def covering(self, rows: int) -> int:
        rows = max(1, rows)
        for i, w in enumerate(self.widths):
            if w >= rows:
                return i
        return len(self.widths) - 1

    def admission_limit(self) -> int:
        return self.widths[self.target]

    def ceiling(self) -> int:
        return self.widths[-1]

    def clamp_target(self, seat: int) -> None:
        """Cap the seat from outside (a rising inter-token latency, say)."""
        self.target = max(self.min_seat, min(self.target, seat))

    # ---- measurements --------------------------------------------------------------------------
    def observe_decode(self, rung: int, service_ms: float, steps: int = 1) -> None:
        if not (0 <= rung < len(self.widths)) or not math.isfinite(service_ms) or service_ms <= 0 or steps <= 0:
            return
        self.service[rung].update(service_ms)
        self.step[rung].update(service_ms / steps)

    def _estimate(self, series, rung: int) -> float:
        if series[rung].n:
            return series[rung].value
        # no sample yet: scale the nearest narrower rung's time with the width (taking it unchanged would overstate what
        # the wider rung can carry and admit a burst on evidence that does not exist)
        for i in range(rung - 1, -1, -1):
            if series[i].n:
                return series[i].value * self.widths[rung] / self.widths[i]
        return 0.0

    def step_ms(self, rung: int) -> float:
        return self._estimate(self.step, rung)

    def service_ms(self, rung: int) -> float:
        return self._estimate(self.service, rung)

    def capacity_tps(self, rung: int) -> float:
        s = self.step_ms(rung)
        return self.widths[rung] * 1000.0 / s if s > 0 else 0.0

    def utilization(self, rung: int, load: RungLoad) -> float:
        cap = self.capacity_tps(rung)
        return (max(0.0, load.arrival_rps) * max(1.0, load.mean_output_tokens)) / cap if cap > 0 else 0.0

    def projected_wait_ms(self, rung: int, load: RungLoad) -> float:
        waves = -(-load.queued // max(1, self.widths[rung]))
        return max(0.0, load.oldest_wait_ms) + waves * self.service_ms(rung)

    def _throughput_seat(self, demand: int, queued: int) -> int:
        """The seat demand asks for, unless a narrower timed rung delivers more tokens per second by a clear margin.  A
        cold controller seats the rung below the widest first and probes the widest after a few samples: a rung only
        gains samples by running."""
        if demand == 0 or not self.throughput:
            return demand
        widest = len(self.widths) - 1
        probe_after = 1 if self.fast_probe else MIN_SAMPLES
        if demand == widest and self.widths[widest] > 4 and self.step[demand].n < MIN_SAMPLES and self.step[demand - 1].n < probe_after:
            return max(demand - 1, self.min_seat)
        if self.step[demand].n < MIN_SAMPLES or self.step[demand - 1].n < MIN_SAMPLES:
            return max(demand, self.min_seat)
        timed = [r for r in range(self.min_seat, demand) if self.step[r].n >= MIN_SAMPLES]
        if not timed:
            return max(demand, self.min_seat)
        best = max(timed, key=self.capacity_tps)
        margin = MARGIN_BACKLOG if queued > 0 else MARGIN_IDLE
        return max(best if self.capacity_tps(best) > self.capacity_tps(demand) * margin else demand, self.min_seat)

    # ---- policy --------------------------------------------------------------------------------
    def decide(self, load: RungLoad) -> RungDecision:
        n = len(self.widths)
        if n == 1:
            return RungDecision(0, 0, "single")
        self.dwell += 1
        actual = self.covering(load.occupied)
        widest = n - 1
        nominal = widest if self.nominal is None else min(self.nominal, widest)
        elastic = max(nominal, widest if self.elastic is None else min(self.elastic, widest))
        burst = load.queued > 0 and (load.oldest_wait_ms >= self.elastic_wait_ms or load.queued >= 4)
        ceiling = elastic if burst else nominal
        demanded = min(load.occupied + load.queued, self.widths[ceiling])
        demand_seat = min(self.covering(demanded), ceiling)
        seat = max(min(self._throughput_seat(demand_seat, load.queued), ceiling), self.min_seat)
        reason = "occupied" if actual > self.target else "hold"

        def move(to: int, why: str) -> str:
            self.target, self.dwell, self.quiet = to, 0, 0
            return why

        if load.queued == 0 and self.target > nominal:
            reason = move(max(nominal, self.min_seat), "throughput")           # the burst is over: back under the nominal ceiling
        elif seat < demand_seat and seat < self.target and (load.queued == 0 or self.dwell >= THROUGHPUT_DWELL_TICKS):
            reason = move(seat, "throughput")                                  # a narrower rung measures faster
        elif load.queued > 0 and seat > self.target:
            wait = self.projected_wait_ms(self.target, load)
            slo = max(load.slo_ms, 8.0 * self.service_ms(self.target))
            reason = move(seat, "slo" if wait > slo else "backlog")
        elif self.target + 1 < n and self.target + 1 <= seat and self.utilization(self.target, load) >= WIDEN_UTIL:
            reason = move(self.target + 1, "utilization")
        elif (load.queued == 0 and self.target > self.min_seat and load.occupied <= self.widths[self.target] // 2
              and load.occupied <= self.widths[self.target - 1] and self.utilization(self.target - 1, load) <= NARROW_UTIL):
            self.quiet += 1
            if self.quiet >= NARROW_TICKS and self.dwell >= MIN_DWELL_TICKS:
                reason = move(max(self.target - 1, self.min_seat), "low_load")
        else:
            self.quiet = 0
        return RungDecision(actual, self.target, reason)


class ServiceTable:
    """Service time of one decode step per rung width, and what an M/D/1 queue in front of it does.

    ``modelled_ms`` comes from the compiler (``build.json`` carries the modelled time of every decode program);
    ``observe`` replaces an entry by a measurement.  All queueing results are for Poisson arrivals of *steps' worth of
    work* at rate ``lam`` per second against a deterministic server."""

    def __init__(self, widths, modelled_ms):
        self.widths = [int(w) for w in widths]
        self.ms = [float(x) for x in modelled_ms]
        self.measured = [False] * len(self.widths)
        if len(self.ms) != len(self.widths) or any(x <= 0 for x in self.ms):
            raise ValueError("one positive service time per rung")

    @staticmethod
    def from_build(build: dict) -> "ServiceTable":
        progs = [p for p in build["ranks"][0]["programs"] if p["role"] == 1]        # decode programs
        progs.sort(key=lambda p: p["rows"])
        return ServiceTable([p["rows"] for p in progs], [max(p.get("est_us", 0.0), 1.0) / 1e3 for p in progs])

    def observe(self, width: int, step_ms: float) -> None:
        i = self.widths.index(width)
        self.ms[i], self.measured[i] = float(step_ms), True

    def service_ms(self, batch: int) -> float:
        for w, s in zip(self.widths, self.ms):
            if w >= batch:
                return s
        return self.ms[-1]

    def utilization(self, lam: float, batch: int) -> float:
        return lam * self.service_ms(batch) / 1e3

    def wait_ms(self, lam: float, batch: int, cv: float = 0.0) -> float:
        """Mean time in queue (Pollaczek-Khinchine; cv = 0 is M/D/1, cv = 1 is M/M/1).  inf at or past saturation."""
        s = self.service_ms(batch)
        rho = lam * s / 1e3
        if rho >= 1.0:
            return math.inf
        return rho * s * (1.0 + cv * cv) / (2.0 * (1.0 - rho))

    def capacity_rps(self, batch: int, mean_output_tokens: float) -> float:
        """Requests per second a rung sustains when each needs ``mean_output_tokens`` steps."""
        return batch * 1000.0 / (self.service_ms(batch) * max(1.0, mean_output_tokens))

    def formation_window_ms(self, lam: float, batch: int, max_hold_ms: float = 50.0) -> float:
        """How long to hold the first request of a batch for companions (Poisson arrivals at ``lam`` per second).  A hold
        of ``w`` costs the first request ``w`` and the ``lam w`` joiners ``w / 2`` each on average; the most a joiner can
        save is one step ``S`` of its own.  The window balances the two, ``lam w^2 / 2 + w = S``, i.e.
        ``w* = (sqrt(1 + 2 lam S) - 1) / lam``: close to ``S`` when arrivals are rare against a step, ``sqrt(2 S / lam)``
        when they are dense.  Never past the step time, the cap, or the point where the batch is full."""
        if lam <= 0 or batch <= 1:
            return 0.0
        s = self.service_ms(batch) / 1e3
        w = (math.sqrt(1.0 + 2.0 * lam * s) - 1.0) / lam
        return 1e3 * min(w, s, (batch - 1) / lam, max_hold_ms / 1e3)
