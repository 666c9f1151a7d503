"""Continuous-batching scheduler: one dispatcher per model.

Per tick the dispatcher (1) drains arrivals, (2) seats queued requests while the KV budget allows
(backpressure only *before* a request starts; queued requests past their TTL are shed, live ones
never are), (3) plans the tick with a token budget — decode rows first (one per live sequence),
then mid-prefill spans packed across requests, shortest remaining prefill first with aging — and
(4) runs it on the engine, then handles produced tokens (stop ids, stop strings, limits,
streaming deltas).  When prefill work is pending, prefill chunks and decode steps alternate so
time-between-tokens stays bounded (SLO mode sizes the chunk from a TBT target).

Reference counterparts: crates/plowrt/src/serve/mux.rs:1-32 (dispatcher), sched/step.rs:1-140
(token-budget plan, SRPF with aging), sched/admission.rs:1-25 (KV-budget seating, TTL shed),
sched/rungs.rs (decode rung ladder), sched/slo.rs (TBT-budgeted prefill), serve/overload.rs.
"""
from __future__ import annotations

import queue
from collections import OrderedDict
import threading
import time
from dataclasses import dataclass, field

import numpy as np

from ..text import sample as sampling
from ..text.tokenizer import IncrementalDetok
from .engine import EngineBase, EngineError, EngineHealth, TokenBatch
from .kv_pages import PAGE, OutOfPages


@dataclass
class GenParams:
    max_tokens: int = 128
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    seed: int | None = None
    stop: list = field(default_factory=list)            # stop strings
    stop_token_ids: list = field(default_factory=list)
    ignore_eos: bool = False
    min_tokens: int = 0
    logprobs: int | None = None
    session_id: str | None = None
    session_end: bool = False             # the session's last turn: nothing is retained for it
    deadline_ms: float | None = None      # total time budget from arrival; None = no deadline
    json_mode: bool = False               # response_format json_object: tokens are filtered by a JSON recogniser
    logit_bias: dict | None = None        # token id -> value added to that token's logit before sampling (OpenAI: -100 .. 100)

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 and self.presence_penalty == 0.0 and self.frequency_penalty == 0.0 \
            and self.repetition_penalty == 1.0 and self.logprobs is None and not self.json_mode and not self.logit_bias


@dataclass
class Chunk:
    kind: str                 # token | done | error
    text: str = ""
    token_id: int | None = None
    finish_reason: str | None = None
    logprob: float | None = None
    top_logprobs: list | None = None
    usage: dict | None = None
    error: str | None = None


@dataclass
class Request:
    rid: str
    prompt: list
    params: GenParams
    out: "queue.Queue[Chunk]" = field(default_factory=queue.Queue)
    arrived: float = field(default_factory=time.monotonic)
    deadline: float | None = None
    # runtime state
    slot: int = -1
    done_prefill: int = 0            # prompt tokens whose KV is computed (incl. cached)
    cached_tokens: int = 0
    generated: list = field(default_factory=list)
    detok: IncrementalDetok | None = None
    text: str = ""
    first_token_at: float | None = None
    last_token_at: float | None = None
    rng: np.random.Generator | None = None
    waited_ticks: int = 0
    aged: bool = False               # waited longer than aging_ticks for a prefill chunk: served before newer requests
    preempted: int = 0
    cancelled: bool = False
    pf_len: int = 0                  # tokens to (re)prefill, fixed when the request is seated
    seated_at: float | None = None   # breakdown log: when it got its slot, its prefill launches and their device time
    pf_chunks: int = 0
    pf_device_ms: float = 0.0

    def all_tokens(self) -> list:
        return self.prompt + self.generated


@dataclass
class SchedConfig:
    token_budget: int = 8192          # rows per tick
    max_queue: int = 4096
    queue_ttl_s: float = 120.0
    objective: str = "auto"           # latency | throughput | auto
    tbt_target_ms: float = 0.0        # 0 = off; otherwise prefill chunks are sized to this budget
    aging_ticks: int = 32             # after this many waits a long prefill jumps the SRPF order
    reserve_tokens: int = PAGE        # KV head-room required per live sequence before seating more
    ride: bool = True                 # decode rows ride the prefill launch (mixed step) instead of waiting a tick
    spec_depth: int = 0               # > 0: speculative decoding for greedy requests (prompt-lookup drafts, span verify)
    multi_step: int = 1               # > 1: greedy decode ticks run this many steps per engine call (tokens fed back on the device)
    lookahead: bool = False           # decode step n + 1 is launched (fed on the device) before step n's tokens are read
    rung_control: bool = False        # admission follows the decode-rung controller (runtime/rungs.py) instead of the slot count
    ttft_slo_ms: float = 0.0          # latency objective the rung controller widens for (0: eight service times)
    session_ttl_s: float = 600.0      # a finished request that carried a session id keeps its slot and KV this long
    max_sessions: int = -1            # retained sessions at most (-1: half of the slots; 0: retention off)


class Metrics:
    def __init__(self):
        self.lock = threading.Lock()
        self.c = dict(requests_total=0, requests_finished=0, requests_failed=0, requests_shed=0, preemptions=0,
                      prompt_tokens=0, generation_tokens=0, cached_tokens=0, ticks=0, prefill_ticks=0, decode_ticks=0)
        self.ttft: list = []
        self.tpot: list = []
        self.e2e: list = []
        self.queue_time: list = []
        self.step_ms: list = []

    def inc(self, k, v=1):
        with self.lock:
            self.c[k] = self.c.get(k, 0) + v

    def gauge(self, k, v):
        with self.lock:
            self.c[k] = v

    def obs(self, name, v):
        with self.lock:
            lst = getattr(self, name)
            lst.append(v)
            if len(lst) > 65536:
                del lst[:32768]

    def snapshot(self) -> dict:
        with self.lock:
            def pct(a, q):
                return float(np.percentile(a, q)) if a else None
            return dict(counters=dict(self.c),
                        ttft_ms=dict(p50=pct(self.ttft, 50), p99=pct(self.ttft, 99), n=len(self.ttft)),
                        tpot_ms=dict(p50=pct(self.tpot, 50), p99=pct(self.tpot, 99), n=len(self.tpot)),
                        e2e_ms=dict(p50=pct(self.e2e, 50), p99=pct(self.e2e, 99)),
                        queue_ms=dict(p50=pct(self.queue_time, 50), p99=pct(self.queue_time, 99)),
                        step_ms=dict(p50=pct(self.step_ms, 50), p99=pct(self.step_ms, 99)))


class ModelMux:
    """Dispatcher + slot table for one engine."""

    def load_estimate(self, window_s: float = 10.0) -> dict:
        """Arrival rate (req/s over the window), service rate (finished req/s from the recent e2e times with the current
        concurrency) and utilisation rho = lambda / mu — the admission estimators of the reference (sched/admission.rs)."""
        now = time.monotonic()
        self._arrivals = [t for t in self._arrivals if now - t <= window_s]
        lam = len(self._arrivals) / window_s
        with self.metrics.lock:
            e2e = list(self.metrics.e2e[-64:])
        mean_s = (sum(e2e) / len(e2e) / 1e3) if e2e else None
        mu = (max(1, self.engine.max_slots) / mean_s) if mean_s else None
        return dict(arrival_rps=round(lam, 3), service_rps=(round(mu, 3) if mu else None), rho=(round(lam / mu, 3) if mu else None),
                    queued=len(self.waiting) + self.ingress.qsize(), live=len(self.live))

    def __init__(self, engine: EngineBase, tokenizer, cfg: SchedConfig | None = None, eos_ids=None):
        self.engine = engine
        self.tok = tokenizer
        self.cfg = cfg or SchedConfig()
        self.eos_ids = set(eos_ids if eos_ids is not None else engine.spec.eos_token_ids)
        self.ingress: "queue.Queue[Request]" = queue.Queue()
        self.waiting: list = []
        self.live: dict[int, Request] = {}
        self.free_slots = list(range(engine.max_slots - 1, -1, -1))
        self.metrics = Metrics()
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._last_was_prefill = False
        self._n = 0
        self.draining = False
        self._drain_deadline = None          # set by drain(); acted on by the dispatcher thread
        self._submit_lock = threading.Lock()
        self._arrivals: list = []          # arrival times of recent requests (rate estimator)
        # session id -> (slot, time retained): finished sequences whose KV waits for the session's next request
        # (reference: crates/plowrt/src/serve/session.rs:1-12)
        self.retained: "OrderedDict[str, tuple]" = OrderedDict()
        self.pd_target: "ModelMux | None" = None     # prefill/decode disaggregation: where finished prefills continue
        self.adopt_q: "queue.Queue" = queue.Queue()  # (request, KV image) pairs handed over by a prefill mux
        self._inflight: dict | None = None           # lookahead: the decode step launched but not yet collected
        from ..obs.breakdown import Breakdown
        self.blog = Breakdown()                       # tick / decode-step / TTFT breakdown logs (environment switches)
        self._tick_info = None                        # (kind, rows, reqs, device ms) of the tick in progress
        from ..serve.overload import OverloadControl
        self.overload = OverloadControl.from_env()    # None unless PLOW_OVERLOAD=1 (or set by the owner)
        self.rungs = None                             # decode-rung admission controller (cfg.rung_control)
        self.rung_decision = None
        self._mean_out = 1.0                          # running mean of output tokens per finished request
        if self.cfg.rung_control:
            from .rungs import RungController
            widths = sorted({w for w in engine.buckets.get("decode", []) if w < engine.max_slots} | {engine.max_slots})
            self.rungs = RungController(widths, engine.max_slots, fast_probe=self.cfg.objective == "throughput")

    # ---- public --------------------------------------------------------------------------------
    def start(self) -> "ModelMux":
        self._thread = threading.Thread(target=self._loop, name="plow-mux", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=10)
        if self._inflight is not None:
            try:
                self.engine.step_collect(self._inflight["handle"])
            except Exception:
                pass
            self._inflight = None
        grp = getattr(self.engine, "step_group", None) or getattr(self.engine, "leader_group", None)
        if grp is not None:
            grp.stop()          # releases the other ranks from their next agreement / receive

    def submit(self, prompt: list, params: GenParams, rid: str | None = None, out=None) -> Request:
        """``out``: where the request's chunks go (anything with ``put``); a fresh queue by default."""
        with self._submit_lock:             # handlers of several HTTP worker threads submit concurrently
            self._n += 1
            n = self._n
        req = Request(rid=rid or f"req-{n}", prompt=list(prompt), params=params)
        if out is not None:
            req.out = out
        if params.deadline_ms:
            req.deadline = req.arrived + params.deadline_ms / 1e3
        with self._submit_lock:
            self._arrivals.append(req.arrived)
        if self.engine.health == EngineHealth.DEAD:
            req.out.put(Chunk("error", error="engine is dead", finish_reason="error"))
            return req
        if self.draining or self.ingress.qsize() + len(self.waiting) >= self.cfg.max_queue:
            self.metrics.inc("requests_shed")
            req.out.put(Chunk("error", error="overloaded", finish_reason="overloaded"))
            return req
        if self.overload is not None and not self.overload.admit(params.session_id is not None and params.session_id in self.retained):
            self.metrics.inc("requests_shed")
            self.metrics.inc("overload_refused")
            req.out.put(Chunk("error", error="overloaded", finish_reason="overloaded", usage=dict(retry_after_s=self.overload.retry_after_s())))
            return req
        if len(prompt) + 1 > self.engine.max_ctx:
            req.out.put(Chunk("error", error="context_length_exceeded", finish_reason="error"))
            return req
        self.metrics.inc("requests_total")
        self.ingress.put(req)
        return req

    def generate(self, prompt: list, params: GenParams) -> tuple:
        """Blocking helper: returns (token ids, text, finish_reason, usage)."""
        req = self.submit(prompt, params)
        ids, text = [], []
        while True:
            ch = req.out.get()
            if ch.kind == "token":
                ids.append(ch.token_id)
                text.append(ch.text)
            elif ch.kind == "done":
                text.append(ch.text)
                return ids, "".join(text), ch.finish_reason, ch.usage
            else:
                raise EngineError(ch.error or "request failed")

    def drain(self, timeout_s: float = 30.0) -> bool:
        """Stop admitting, wait for live requests; preempt (finish as `length`) after the timeout."""
        self.draining = True
        t0 = time.monotonic()
        running = self._thread is not None and self._thread.is_alive()
        if running:
            # slots and page tables belong to the dispatcher thread: after the deadline IT finishes what is still live
            self._drain_deadline = t0 + timeout_s
            while (self.live or self.waiting or not self.ingress.empty()) and time.monotonic() - t0 < timeout_s + 5.0 \
                    and self._thread.is_alive():
                time.sleep(0.005)
            self._drain_deadline = None
            return not self.live
        while (self.live or self.waiting or not self.ingress.empty()) and time.monotonic() - t0 < timeout_s:
            if not self.tick():
                break
        for r in list(self.live.values()):
            self._finish(r, "preempted")
        return not self.live

    # ---- loop ----------------------------------------------------------------------------------
    def _loop(self) -> None:
        from ..parallel.group import GroupStopped
        lockstep = getattr(self.engine, "lockstep", False)
        self.engine.bind_thread()
        while not self._stop.is_set():
            try:
                if not self.tick():
                    if lockstep:
                        # the other ranks of the group may have work: every launch of theirs needs this rank too
                        if not self.engine.idle_step():
                            time.sleep(0.001)
                        continue
                    try:
                        self.waiting.append(self.ingress.get(timeout=0.02))
                    except queue.Empty:
                        pass
            except GroupStopped as e:
                # the rank group is gone (a member stopped or failed): nothing can run any more
                self._on_engine_error(EngineError(f"rank group stopped: {e}", fatal=True))
                return
            except EngineError as e:
                self._on_engine_error(e)
            except Exception as e:      # a scheduler bug must not leave every request hanging behind a dead thread
                self.metrics.inc("dispatcher_errors")
                self._on_engine_error(EngineError(f"dispatcher: {type(e).__name__}: {e}", fatal=False))
                if self.engine.health == EngineHealth.HEALTHY:
                    self.engine.health = EngineHealth.DEGRADED

    def tick(self) -> bool:
        """One scheduling step; returns False when there was nothing to do."""
        while True:
            try:
                self.waiting.append(self.ingress.get_nowait())
            except queue.Empty:
                break
        if self._inflight is not None:
            self._lookahead_tick()
            return True
        if self._drain_deadline is not None and time.monotonic() > self._drain_deadline:
            for r in list(self.live.values()):
                self._finish(r, "preempted")
            for r in self.waiting:
                r.out.put(Chunk("done", text="", finish_reason="preempted", usage=dict(prompt_tokens=len(r.prompt), completion_tokens=len(r.generated), total_tokens=len(r.prompt) + len(r.generated))))
            self.waiting = []
            return False
        self._shed_expired()
        self._expire_sessions()
        self._adopt()
        if self.overload is not None:
            self.overload.tick()
            self.metrics.gauge("overload_level", self.overload.level)
        if self.rungs is not None:
            from .rungs import RungLoad
            now = time.monotonic()
            self._arrivals = [t for t in self._arrivals if now - t <= 10.0]
            self.rung_decision = self.rungs.decide(RungLoad(
                occupied=len(self.live), queued=len(self.waiting),
                oldest_wait_ms=(now - min(r.arrived for r in self.waiting)) * 1e3 if self.waiting else 0.0,
                arrival_rps=len(self._arrivals) / 10.0, mean_output_tokens=self._mean_out, slo_ms=self.cfg.ttft_slo_ms))
            self.metrics.gauge("rung_admission_limit", self.rungs.admission_limit())
        self._admit()
        if not self.live:
            return False
        self.metrics.inc("ticks")
        prefilling = [r for r in self.live.values() if r.done_prefill < r.pf_len and not r.cancelled]
        decoding = [r for r in self.live.values() if r.done_prefill >= r.pf_len and not r.cancelled]
        for r in [r for r in self.live.values() if r.cancelled]:
            self._finish(r, "cancelled")
        now = time.monotonic()
        for r in [r for r in self.live.values() if r.deadline is not None and now > r.deadline]:
            # a request past its deadline stops where it is: what was generated is delivered (reference: serve/deadlines.rs)
            self.metrics.inc("deadline_exceeded")
            if self.overload is not None:
                self.overload.record(False)
            self._finish(r, "deadline")
        prefilling = [r for r in prefilling if r.slot in self.live]
        decoding = [r for r in decoding if r.slot in self.live]
        run_prefill = bool(prefilling) and (not decoding or not self._last_was_prefill or self.cfg.objective == "throughput")
        t0 = time.perf_counter()
        if run_prefill:
            riders = decoding if (self.cfg.ride and self.cfg.objective != "throughput") else []
            self._prefill_tick(prefilling, riders)
            self._last_was_prefill = True
        elif decoding:
            n_rows, ticks0 = len(decoding), self.metrics.c.get("decode_ticks", 0)
            self._decode_tick(decoding)
            self._last_was_prefill = False
            if self.rungs is not None and self._inflight is None:
                steps = self.metrics.c.get("decode_ticks", 0) - ticks0
                if steps > 0:
                    self.rungs.observe_decode(self.rungs.covering(min(n_rows, self.engine.max_rows(True))),
                                              (time.perf_counter() - t0) * 1e3, steps)
        else:
            return False
        self.metrics.obs("step_ms", (time.perf_counter() - t0) * 1e3)
        if self.blog.tick_on:
            kind, rows, nreq, dev = self._tick_info or ("decode" if not run_prefill else "prefill", 0, 0, 0.0)
            self._tick_info = None
            self.blog.tick(kind, rows, nreq, dev, (time.perf_counter() - t0) * 1e3, len(self.waiting), len(self.live),
                           self.rungs.admission_limit() if self.rungs is not None else 0)
        return True

    # ---- prefill / decode disaggregation ---------------------------------------------------------
    def _handoff(self, r: Request) -> None:
        """This mux only prefills: export the sequence's KV image, free the slot here and queue the request on the
        decode mux, which imports the image and continues (reference: serve/pd.rs:1-8)."""
        from .kv_image import export_slot
        img = export_slot(self.engine, r.slot)
        self._retire(r.slot)
        del self.live[r.slot]
        self.free_slots.append(r.slot)
        r.slot = -1
        self.metrics.inc("pd_handoffs")
        self.metrics.inc("pd_bytes", img.nbytes())
        self.pd_target.adopt_q.put((r, img))

    def _adopt(self) -> None:
        from .kv_image import import_slot
        while self.free_slots and not self.adopt_q.empty():
            r, img = self.adopt_q.queue[0]
            slot = self.free_slots.pop()
            try:
                import_slot(self.engine, slot, img)
            except OutOfPages:
                self._retire(slot)
                self.free_slots.append(slot)
                return                                   # retry when pages free up
            self.adopt_q.get_nowait()
            r.slot, r.done_prefill, r.pf_len = slot, len(r.prompt), len(r.prompt)
            self.live[slot] = r
            self.metrics.inc("pd_adopted")

    # ---- admission -----------------------------------------------------------------------------
    def _shed_expired(self) -> None:
        now = time.monotonic()
        keep = []
        for r in self.waiting:
            if (now - r.arrived > self.cfg.queue_ttl_s or (r.deadline is not None and now > r.deadline)) and r.preempted == 0:
                self.metrics.inc("requests_shed")
                r.out.put(Chunk("error", error="queue ttl exceeded", finish_reason="overloaded"))
            else:
                keep.append(r)
        self.waiting = keep

    def _admit(self) -> None:
        """Seat queued requests while slots and KV pages allow (arrival order; a request that does
        not fit blocks the ones behind it so large prompts cannot starve)."""
        eng = self.engine
        while self.waiting:
            r = self.waiting[0]
            toks = r.all_tokens()
            sid = r.params.session_id
            if sid is not None and sid in self.retained and self._resume_session(r, toks):
                continue
            if not self.free_slots:
                if self._evict_session():
                    continue
                break
            if self.rungs is not None and len(self.live) >= self.rungs.admission_limit():
                break               # the controller holds the decode steps on this rung for now
            need_pages = (len(toks) + 1 + PAGE - 1) // PAGE
            headroom = len(self.live) * ((self.cfg.reserve_tokens + PAGE - 1) // PAGE)
            # pages are reserved lazily, chunk by chunk: what seated requests have yet to reserve for the rest of their
            # prompts is spoken for, or two long prompts get admitted against the same free pages
            owed = 0
            for q in self.live.values():
                want = (q.pf_len + 1 + PAGE - 1) // PAGE
                have = len(eng.pool.seqs[q.slot].pages) if q.slot in eng.pool.seqs else 0
                owed += max(0, want - have)
            if need_pages + headroom + owed > eng.pool.available() + eng.pool.cached_prefix_len(toks) // PAGE:
                if self._evict_session():
                    continue        # a retained session gave its pages back: look again
                if not self.live and need_pages <= eng.pool.n_pages:
                    pass            # nothing else is running: the request gets the pool to itself
                else:
                    break
            self.waiting.pop(0)
            slot = self.free_slots.pop()
            try:
                cached = eng.begin_slot(slot, toks)
            except OutOfPages:
                self.free_slots.append(slot)
                self.waiting.insert(0, r)
                break
            self._seat(r, slot, cached, len(toks))

    def _seat(self, r: Request, slot: int, cached: int, n_tokens: int) -> None:
        r.slot, r.done_prefill, r.cached_tokens = slot, cached, max(r.cached_tokens, cached)
        r.pf_len = n_tokens        # a preempted request re-prefills its prompt plus what it generated
        r.seated_at = time.monotonic()
        r.detok = r.detok or IncrementalDetok(self.tok)
        r.rng = r.rng or np.random.default_rng(r.params.seed)
        self.live[slot] = r
        self.metrics.obs("queue_time", (time.monotonic() - r.arrived) * 1e3)
        self.metrics.inc("cached_tokens", cached)

    # ---- session retention -----------------------------------------------------------------------
    def _session_cap(self) -> int:
        return self.engine.max_slots // 2 if self.cfg.max_sessions < 0 else self.cfg.max_sessions

    def _retain(self, r: Request) -> bool:
        """Keep a finished request's slot for its session instead of retiring it."""
        sid = r.params.session_id
        cap = self._session_cap()
        if sid is None or cap <= 0 or self.draining or r.params.session_end:
            if sid is not None and sid in self.retained:
                self._drop_session(sid)
            return False
        if sid in self.retained:                 # the session's older sequence is superseded
            self._drop_session(sid)
        while len(self.retained) >= cap:
            self._evict_session()
        self.retained[sid] = (r.slot, time.monotonic())
        self.metrics.inc("sessions_retained")
        return True

    def _drop_session(self, sid: str) -> None:
        slot, _ = self.retained.pop(sid)
        self._retire(slot)
        self.free_slots.append(slot)

    def _evict_session(self) -> bool:
        """Give the least recently retained session's slot and pages back; False when none is retained."""
        if not self.retained:
            return False
        self._drop_session(next(iter(self.retained)))
        self.metrics.inc("sessions_evicted")
        return True

    def _expire_sessions(self) -> None:
        now = time.monotonic()
        for sid in [s for s, (_, t) in self.retained.items() if now - t > self.cfg.session_ttl_s]:
            self._drop_session(sid)
            self.metrics.inc("sessions_expired")

    def _resume_session(self, r: Request, toks: list) -> bool:
        """Seat `r` in the slot its session retained, keeping the longest identical prefix; when the slot cannot be cut
        back that far it is retired and the request takes the ordinary path."""
        sid = r.params.session_id
        slot, _ = self.retained[sid]
        eng = self.engine
        kept = eng.resume_slot(slot, toks)
        if kept < 0:
            self._drop_session(sid)
            return False
        need_pages = (len(toks) + 1 + PAGE - 1) // PAGE - len(eng.pool.seqs[slot].pages)
        while need_pages > eng.pool.available():
            other = next((s for s in self.retained if s != sid), None)
            if other is None:
                break
            self._drop_session(other)
        if need_pages > eng.pool.available() and self.live:
            return False                      # stays retained; the request waits for pages like any other
        del self.retained[sid]
        self.waiting.pop(0)
        self._seat(r, slot, kept, len(toks))
        self.metrics.inc("session_hits")
        self.metrics.inc("session_tokens_reused", kept)
        return True

    # ---- prefill -------------------------------------------------------------------------------
    def _prefill_budget(self) -> int:
        b = min(self.cfg.token_budget, self.engine.max_rows(False))
        if self.cfg.tbt_target_ms > 0 and self.metrics.step_ms:
            # crude service model: rows per ms observed on recent prefill ticks
            b = max(PAGE, min(b, int(self.cfg.tbt_target_ms * getattr(self, "_rows_per_ms", 64.0))))
        if self.overload is not None and self.overload.level:
            b = max(PAGE, int(b * self.overload.prefill_scale()))
        return b

    # ---- drafter ------------------------------------------------------------------------------
    def set_drafter(self, drafter) -> None:
        """Drafter of the speculative steps (``spec_depth`` > 0): an n-gram drafter, or a MtpDrafter over the checkpoint's
        prediction module, which the prefill, decode and verify steps then feed with the decoder's hidden states."""
        self._drafter = drafter

    def _mtp(self):
        d = getattr(self, "_drafter", None)
        return d if self.cfg.spec_depth > 0 and getattr(d, "needs_hidden", False) else None

    def _retire(self, slot: int) -> None:
        self.engine.retire_slot(slot)
        d = getattr(self, "_drafter", None)
        if getattr(d, "needs_hidden", False):
            d.retire(slot)

    def _prefill_tick(self, reqs: list, riders: list = ()) -> None:
        """One prefill launch.  ``riders`` are decoding requests whose next row is appended to the same token batch
        (a mixed step: the unified row format makes a decode row just another row), so running prompts do not
        stall token generation for a whole tick (reference: crates/plowrt/src/sched/ride.rs, mixed_step.h)."""
        eng = self.engine
        budget = self._prefill_budget()
        for r in reqs:
            r.waited_ticks += 1
            if r.waited_ticks > self.cfg.aging_ticks:
                r.aged = True
        # Shortest remaining prefill first; aged requests first of all.  Ageing is sticky: a request that waited too
        # long keeps its priority until its prompt is done.  (When it lost the priority with its first chunk, a burst of
        # long prompts aged together and then took turns, one chunk each: every one of them finished at the very end,
        # and the median time to first token of a 64-request wave was two thirds of the whole prefill phase.)
        order = sorted(reqs, key=lambda r: (0 if r.aged else 1, r.pf_len - r.done_prefill))
        ids, pos, seq, sample_rows, spans = [], [], [], [], []
        for r in order:
            if budget <= 0 or len(spans) >= eng.buckets.get("max_seqs", 64):
                break
            if r.slot < 0 or self.live.get(r.slot) is not r:
                continue            # preempted earlier in this tick to make room
            toks = r.all_tokens()[:r.pf_len]
            n = min(budget, r.pf_len - r.done_prefill)
            if n <= 0:
                continue
            try:
                eng.reserve(r.slot, r.done_prefill + n + 1)
            except OutOfPages:
                if not spans:
                    self._preempt_one(exclude=r)
                continue
            start = r.done_prefill
            ids += toks[start:start + n]
            pos += list(range(start, start + n))
            seq += [r.slot] * n
            final = start + n == len(toks)
            if final:
                sample_rows.append(len(ids) - 1)
            spans.append((r, start, n, final, toks))
            budget -= n
            r.waited_ticks = 0
        if any(sp[0].slot < 0 or self.live.get(sp[0].slot) is not sp[0] for sp in spans):
            return                  # a request already packed lost its slot to a preemption: re-plan next tick
        if not spans:
            return
        # riders: one row each, as long as sample slots and rows remain
        rode = []
        max_samples = eng.buckets.get("max_seqs", 64)
        for r in sorted(riders, key=lambda r: r.slot):
            if len(sample_rows) + 1 > max_samples - 1 or len(ids) + 1 > eng.max_rows(False):
                break
            if r.slot < 0 or self.live.get(r.slot) is not r:
                continue            # preempted earlier in this tick
            n_ctx = len(r.prompt) + len(r.generated)
            try:
                eng.reserve(r.slot, n_ctx + 1)
            except OutOfPages:
                continue
            ids.append(r.generated[-1])
            pos.append(n_ctx - 1)
            seq.append(r.slot)
            sample_rows.append(len(ids) - 1)
            rode.append(r)
        want_logits = any(not s[0].params.greedy for s in spans if s[3]) or any(not r.params.greedy for r in rode)
        if not sample_rows:
            sample_rows_arr = np.array([len(ids) - 1], dtype=np.int32)   # engines always sample >= 1 row
        else:
            sample_rows_arr = np.array(sample_rows, dtype=np.int32)
        batch = TokenBatch(np.array(ids, dtype=np.int32), np.array(pos, dtype=np.int32), np.array(seq, dtype=np.int32),
                           sample_rows_arr, decode=False, want_logits=want_logits, want_hidden=self._mtp() is not None)
        t0 = time.perf_counter()
        res = eng.step(batch)
        dt = (time.perf_counter() - t0) * 1e3
        self._rows_per_ms = 0.8 * getattr(self, "_rows_per_ms", len(ids) / max(dt, 1e-3)) + 0.2 * len(ids) / max(dt, 1e-3)
        self.metrics.inc("prefill_ticks")
        if self.blog.any:
            self._tick_info = ("prefill", len(ids), len(spans) + len(rode), res.device_ms)
            for sp in spans:
                sp[0].pf_chunks += 1
                sp[0].pf_device_ms += res.device_ms
        k = 0
        mtp = self._mtp() if res.hidden is not None else None
        seen, at = [], 0          # what the drafter's prediction module must see: (slot, start, next tokens, hidden rows)
        for (r, start, n, final, toks) in spans:
            slot = r.slot
            eng.commit(r.slot, toks[start:start + n])
            r.done_prefill = start + n
            self.metrics.inc("prompt_tokens", n)
            if final:
                lg = res.logits[k] if res.logits is not None else None
                self._produce(r, int(res.ids[k]), lg)
                k += 1
                if self.pd_target is not None and r.slot >= 0 and self.live.get(r.slot) is r:
                    self._handoff(r)
            if mtp is not None and self.live.get(slot) is r:
                allt = r.all_tokens()
                if len(allt) > start + n:           # the token behind the last row: the prompt's next one, or the one just produced
                    if start == 0:
                        mtp.begin(slot)
                    seen.append((slot, start, allt[start + 1:start + n + 1], res.hidden[at:at + n]))
            at += n
        for r in rode:
            if r.slot in self.live and self.live[r.slot] is r:
                slot, fed = r.slot, r.generated[-1]
                eng.commit(r.slot, [fed])
                self._produce(r, int(res.ids[k]), res.logits[k] if res.logits is not None else None)
                self.metrics.inc("rider_rows")
                if mtp is not None and self.live.get(slot) is r:
                    seen.append((slot, len(r.prompt) + len(r.generated) - 2, [r.generated[-1]], res.hidden[at:at + 1]))
            k += 1
            at += 1
        if seen:
            mtp.observe(seen)

    # ---- decode --------------------------------------------------------------------------------
    def _spec_tick(self, reqs: list) -> bool:
        """Speculative decode step: every greedy request contributes its pending token plus up to ``spec_depth`` drafted
        tokens as consecutive rows of one launch; the longest prefix the model agrees with is emitted.  Used while the
        rows fit the program's sample capacity (low concurrency, where latency matters); returns False to fall back."""
        from .spec import NgramDrafter
        eng = self.engine
        depth = self.cfg.spec_depth
        max_samples = eng.buckets.get("max_seqs", 64)
        if not reqs or any(not r.params.greedy for r in reqs) or len(reqs) * (depth + 1) > max_samples:
            return False
        if getattr(eng, "has_recurrent_state", False):
            return False            # rejected draft rows would already have advanced the per-slot state in place
        drafter = getattr(self, "_drafter", None) or NgramDrafter()
        self._drafter = drafter
        mtp = self._mtp()
        chained = {}
        if mtp is not None:
            chained = mtp.propose_many([r.slot for r in reqs if mtp.synced(r.slot, len(r.prompt) + len(r.generated) - 1)], depth)
        ids, pos, seq, spans = [], [], [], []
        for r in sorted(reqs, key=lambda r: r.slot):
            n_ctx = len(r.prompt) + len(r.generated)
            room = min(depth, r.params.max_tokens - len(r.generated) - 1, eng.max_ctx - n_ctx - 2)
            if r.slot in chained:
                draft = chained[r.slot][:max(0, room)]
            else:
                draft = drafter.propose(r.all_tokens(), max(0, room)) if room > 0 else []
            try:
                eng.reserve(r.slot, n_ctx + len(draft) + 1)
            except OutOfPages:
                return False
            rows = [r.generated[-1]] + draft
            spans.append((r, len(ids), draft))
            ids += rows
            pos += list(range(n_ctx - 1, n_ctx - 1 + len(rows)))
            seq += [r.slot] * len(rows)
        if len(ids) == len(spans):
            return False                      # nothing drafted: the plain decode program is cheaper
        res = eng.step(TokenBatch(np.array(ids, np.int32), np.array(pos, np.int32), np.array(seq, np.int32),
                                  np.arange(len(ids), dtype=np.int32), decode=False, want_hidden=mtp is not None))
        self.metrics.inc("spec_ticks")
        seen = []
        for (r, at, draft) in spans:
            slot, n0 = r.slot, len(r.prompt) + len(r.generated) - 1
            got = [int(x) for x in res.ids[at:at + 1 + len(draft)]]
            j = 0
            while j < len(draft) and draft[j] == got[j]:
                j += 1
            self.metrics.inc("spec_proposed", len(draft))
            self.metrics.inc("spec_accepted", j)
            pending = r.generated[-1]
            for tok_in, tok_out in zip([pending] + draft[:j], got[:j + 1]):
                if r.slot not in self.live or self.live[r.slot] is not r:
                    break                      # finished (stop / length) while emitting the accepted span
                eng.commit(r.slot, [tok_in])
                self._produce(r, tok_out, None)
            if mtp is not None and res.hidden is not None and self.live.get(slot) is r:
                new = r.all_tokens()[n0 + 1:]                  # the accepted drafts and the token behind them
                seen.append((slot, n0, new, res.hidden[at:at + len(new)]))
        if seen:
            mtp.observe(seen)
        return True

    def _decode_tick(self, reqs: list) -> None:
        eng = self.engine
        if self.cfg.spec_depth > 0 and (self.overload is None or self.overload.extras_allowed()) and self._spec_tick(reqs):
            return
        cap = eng.max_rows(True)
        reqs = sorted(reqs, key=lambda r: r.slot)[:cap]
        ready = []
        for r in reqs:
            n_ctx = len(r.prompt) + len(r.generated)
            try:
                eng.reserve(r.slot, n_ctx + 1)
                ready.append(r)
            except OutOfPages:
                self._preempt_one(exclude=None, prefer=r)
        reqs = [r for r in ready if r.slot in self.live and self.live[r.slot] is r]
        if not reqs:
            return
        ids = np.array([r.generated[-1] for r in reqs], dtype=np.int32)
        pos = np.array([len(r.prompt) + len(r.generated) - 1 for r in reqs], dtype=np.int32)
        seq = np.array([r.slot for r in reqs], dtype=np.int32)
        want_logits = any(not r.params.greedy for r in reqs)
        mtp = self._mtp()
        batch = TokenBatch(ids, pos, seq, np.arange(len(reqs), dtype=np.int32), decode=True, want_logits=want_logits,
                           want_hidden=mtp is not None)
        k = self._multi_step_depth(reqs)
        if k > 1:
            # several steps per engine call: the engine feeds each step's arg-max tokens to the next one, the host
            # sees them afterwards.  A request that stops early simply drops the tokens computed past its stop.
            results = eng.step_multi(batch, k)
            self.metrics.inc("decode_ticks", k)
            self.metrics.inc("multi_step_calls")
            fed = ids
            for res in results:
                for j, r in enumerate(reqs):
                    if r.slot in self.live and self.live[r.slot] is r:
                        eng.commit(r.slot, [int(fed[j])])
                        self._produce(r, int(res.ids[j]), None)
                fed = res.ids
            return
        if self._lookahead_ok(reqs, 1):
            # lookahead-1: leave the step running; the next tick launches its successor (fed on the device) and only
            # then reads this one's tokens, so the host's work for step n overlaps the device's step n + 1
            self._inflight = dict(handle=eng.step_launch(batch), reqs=reqs, fed=ids, pos=pos, seq=seq)
            self.metrics.inc("decode_ticks")
            return
        t_pre = time.perf_counter()
        res = eng.step(batch)
        t_run = time.perf_counter()
        self.metrics.inc("decode_ticks")
        if self.blog.any:
            self._tick_info = ("decode", len(reqs), len(reqs), res.device_ms)
        seen = []
        for k, r in enumerate(reqs):
            slot = r.slot
            eng.commit(r.slot, [int(ids[k])])
            self._produce(r, int(res.ids[k]), res.logits[k] if res.logits is not None else None)
            if mtp is not None and res.hidden is not None and self.live.get(slot) is r:
                seen.append((slot, int(pos[k]), [r.generated[-1]], res.hidden[k:k + 1]))
        if seen:
            mtp.observe(seen)
        if self.blog.dstep_on:
            rung = min((w for w in eng.buckets.get("decode", []) if w >= len(reqs)), default=len(reqs))
            self.blog.dstep(len(reqs), rung, 1, res.device_ms, (t_run - t_pre) * 1e3 - res.device_ms, (time.perf_counter() - t_run) * 1e3)

    def _lookahead_ok(self, reqs: list, ahead: int) -> bool:
        """May a decode step of these requests be left in flight (ahead = 1), or chained behind the one in flight
        (ahead = 2)?  Only plain greedy requests with at least ``ahead`` more tokens to produce, nobody waiting to be
        admitted or prefilled, no drafter, no rank group (the other ranks follow synchronous steps), no recurrent state
        (the row a chained step computes for a request that has just ended would advance a state its session keeps)."""
        eng = self.engine
        if self.overload is not None and not self.overload.extras_allowed():
            return False
        if not self.cfg.lookahead or getattr(eng, "has_recurrent_state", False) or self.cfg.spec_depth > 0 or self.waiting or not self.ingress.empty() or not self.adopt_q.empty() \
                or self.draining or getattr(eng, "step_group", None) is not None or getattr(eng, "leader_group", None) is not None:
            return False
        if any(q.done_prefill < q.pf_len for q in self.live.values()):
            return False
        now = time.monotonic()
        for r in reqs:
            p = r.params
            if self.live.get(r.slot) is not r or r.cancelled or not p.greedy or p.stop or p.json_mode \
                    or (r.deadline is not None and now > r.deadline):
                return False
            n_ctx = len(r.prompt) + len(r.generated)
            if p.max_tokens - len(r.generated) < ahead or n_ctx + ahead + 1 > eng.max_ctx:
                return False
        return True

    def _lookahead_tick(self) -> None:
        """A decode step is in flight.  If its requests can all go on, launch the next step first (its ids come from the
        in-flight step's output on the device), then collect the in-flight one and hand out its tokens.  A request that
        ends with this token simply leaves a row of the chained step unused."""
        eng, inf = self.engine, self._inflight
        reqs, pos, seq = inf["reqs"], inf["pos"], inf["seq"]
        nxt = None
        if self._lookahead_ok(reqs, 2):
            try:
                for r in reqs:
                    eng.reserve(r.slot, len(r.prompt) + len(r.generated) + 2)
                batch = TokenBatch(np.zeros(len(reqs), np.int32), pos + 1, seq, np.arange(len(reqs), dtype=np.int32), decode=True)
                nxt = eng.step_launch(batch, chain_from=inf["handle"])
                self.metrics.inc("lookahead_launches")
            except OutOfPages:
                nxt = None
        self._inflight = None
        res = eng.step_collect(inf["handle"])
        for k, r in enumerate(reqs):
            if self.live.get(r.slot) is r:
                eng.commit(r.slot, [int(inf["fed"][k])])
                self._produce(r, int(res.ids[k]), None)
        if nxt is not None:
            self._inflight = dict(handle=nxt, reqs=reqs, fed=np.asarray(res.ids[:len(reqs)], np.int32).copy(), pos=pos + 1, seq=seq)
            self.metrics.inc("decode_ticks")

    def _multi_step_depth(self, reqs: list) -> int:
        """How many decode steps the next engine call may chain: only plain greedy requests (no logprobs, penalties,
        stop strings or guided output, whose next token the host decides), nobody waiting to be admitted or prefilled
        (a chained call delays them by its whole length), and no more steps than the shortest remaining budget."""
        k = self.cfg.multi_step
        eng = self.engine
        if k <= 1 or self.waiting or not self.ingress.empty() or getattr(eng, "step_group", None) is not None \
                or getattr(eng, "leader_group", None) is not None:
            return 1
        if any(q.done_prefill < q.pf_len for q in self.live.values()):
            return 1
        for r in reqs:
            p = r.params
            if not p.greedy or p.stop or p.json_mode:
                return 1
            n_ctx = len(r.prompt) + len(r.generated)
            k = min(k, p.max_tokens - len(r.generated), eng.max_ctx - n_ctx - 1)
        if k <= 1:
            return 1
        try:
            for r in reqs:
                eng.reserve(r.slot, len(r.prompt) + len(r.generated) + k)
        except OutOfPages:
            return 1
        return k

    # ---- tokens --------------------------------------------------------------------------------
    def _produce(self, r: Request, greedy_id: int, logits) -> None:
        p = r.params
        tok, lp, top = greedy_id, None, None
        if p.json_mode and logits is not None:
            if getattr(r, "guided", None) is None:
                from ..text.guided import GuidedJson
                eos = next(iter(self.eos_ids), 0)
                r.guided = GuidedJson(lambda t: self.tok.decode([t]), eos)
            lg = sampling.apply_penalties(logits, r.generated, p.presence_penalty, p.frequency_penalty, p.repetition_penalty)
            tok = r.guided.pick(np.asarray(lg))
            if r.guided.state.complete and tok == r.guided.eos_id:
                self._finish(r, "stop")
                return
        elif not p.greedy and logits is not None:
            lg = sampling.apply_penalties(logits, r.generated, p.presence_penalty, p.frequency_penalty, p.repetition_penalty)
            if p.logit_bias:
                lg = np.array(lg, dtype=np.float32, copy=True)
                for t, b in p.logit_bias.items():
                    if 0 <= int(t) < lg.shape[0]:
                        lg[int(t)] += float(b)
            tok = sampling.sample(lg, r.rng, p.temperature, p.top_k, p.top_p, p.min_p)
            if p.logprobs is not None:
                lp, top = sampling.logprobs_of(lg, tok, p.logprobs)
        now = time.monotonic()
        if r.first_token_at is None:
            r.first_token_at = now
            self.metrics.obs("ttft", (now - r.arrived) * 1e3)
            if self.blog.ttft_on:
                seated = r.seated_at if r.seated_at is not None else r.arrived
                self.blog.ttft(r.rid, len(r.prompt), r.cached_tokens, (seated - r.arrived) * 1e3, r.pf_chunks, r.pf_device_ms,
                               (now - seated) * 1e3, (now - r.arrived) * 1e3)
        else:
            self.metrics.obs("tpot", (now - r.last_token_at) * 1e3)
            if self.overload is not None and self.cfg.tbt_target_ms > 0:
                self.overload.record((now - r.last_token_at) * 1e3 <= 1.5 * self.cfg.tbt_target_ms)
        r.last_token_at = now
        r.generated.append(tok)
        self.metrics.inc("generation_tokens")
        n_gen = len(r.generated)
        is_eos = (tok in self.eos_ids and not p.ignore_eos) or tok in p.stop_token_ids
        if is_eos and n_gen > p.min_tokens:
            r.generated.pop()          # the stop token is not part of the text
            self._finish(r, "stop")
            return
        delta = r.detok.push(tok)
        r.text += delta
        if p.stop:
            hit = min((r.text.find(s) for s in p.stop if s and s in r.text), default=-1)
            if hit >= 0 and n_gen > p.min_tokens:
                already = len(r.text) - len(delta)
                r.out.put(Chunk("token", text=r.text[already:hit] if hit > already else "", token_id=tok, logprob=lp, top_logprobs=top))
                r.text = r.text[:hit]
                self._finish(r, "stop")
                return
        r.out.put(Chunk("token", text=delta, token_id=tok, logprob=lp, top_logprobs=top))
        if n_gen >= p.max_tokens:
            self._finish(r, "length")
        elif len(r.prompt) + n_gen + 1 > self.engine.max_ctx:
            self._finish(r, "length")

    def _finish(self, r: Request, reason: str) -> None:
        tail = r.detok.flush() if r.detok else ""
        usage = dict(prompt_tokens=len(r.prompt), completion_tokens=len(r.generated),
                     total_tokens=len(r.prompt) + len(r.generated),
                     prompt_tokens_details=dict(cached_tokens=r.cached_tokens))
        r.out.put(Chunk("done", text=tail if reason != "stop" else "", finish_reason=reason, usage=usage))
        if r.slot >= 0 and self.live.get(r.slot) is r:
            del self.live[r.slot]
            if not (reason in ("stop", "length") and self._retain(r)):
                self._retire(r.slot)
                self.free_slots.append(r.slot)
        self.metrics.inc("requests_finished")
        self.metrics.obs("e2e", (time.monotonic() - r.arrived) * 1e3)
        self._mean_out += 0.1 * (max(1, len(r.generated)) - self._mean_out)

    def _preempt_one(self, exclude=None, prefer=None) -> None:
        """Free pages by sending the youngest live request back to the queue (it re-prefills its
        prompt plus what it generated; the prefix cache usually makes that cheap)."""
        cands = [r for r in self.live.values() if r is not exclude]
        if not cands:
            return
        victim = prefer or max(cands, key=lambda r: r.arrived)
        self._retire(victim.slot)
        del self.live[victim.slot]
        self.free_slots.append(victim.slot)
        victim.slot, victim.done_prefill = -1, 0
        victim.preempted += 1
        self.metrics.inc("preemptions")
        self.waiting.insert(0, victim)

    def _on_engine_error(self, e: EngineError) -> None:
        self.metrics.inc("requests_failed", len(self.live))
        if e.fatal:
            self.engine.health = EngineHealth.DEAD
        for r in list(self.live.values()):
            r.out.put(Chunk("error", error=str(e), finish_reason="error"))
            try:
                self._retire(r.slot)
            except Exception:
                pass
            self.free_slots.append(r.slot)
        self.live.clear()
        if e.fatal:
            for r in self.waiting:
                r.out.put(Chunk("error", error="engine is dead", finish_reason="error"))
            self.waiting.clear()
