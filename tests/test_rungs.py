"""Decode-rung admission controller and the M/D/1 service table (runtime/rungs.py), and the controller inside the
scheduler on the CPU engine.  Reference behaviour: crates/plowrt/src/sched/rungs.rs, sched/mdq.rs."""
import math

import numpy as np
import pytest

from plow_b200.runtime.rungs import (MIN_DWELL_TICKS, NARROW_TICKS, RungController, RungLoad, ServiceTable, validate_rungs)


def test_rung_ladder_is_validated():
    assert validate_rungs([8, 16, 64], 64) == [8, 16, 64]
    for bad, cap in (([], 8), ([0, 8], 8), ([8, 8], 8), ([16, 8], 8), ([8, 16], 32)):
        with pytest.raises(ValueError):
            validate_rungs(bad, cap)
    c = RungController([8, 16, 32, 64])
    assert c.admission_limit() == 8 and c.ceiling() == 64 and c.covering(9) == 1 and c.covering(1000) == 3
    assert RungController([4]).decide(RungLoad(2, 9)).reason == "single"


def test_backlog_widens_at_once_and_quiet_narrows_slowly():
    c = RungController([8, 16, 32, 64])
    d = c.decide(RungLoad(occupied=8, queued=1))
    assert c.admission_limit() == 16 and d.reason == "backlog"              # one waiting request: the next rung
    d = c.decide(RungLoad(occupied=16, queued=40, oldest_wait_ms=10.0))
    # a cold controller seats the rung below the widest first and probes the widest once that one has samples
    assert c.admission_limit() == 32 and d.reason in ("backlog", "slo")
    for _ in range(4):
        c.observe_decode(2, 10.0)
    d = c.decide(RungLoad(occupied=32, queued=40, oldest_wait_ms=500.0))
    assert c.admission_limit() == 64 and d.reason == "slo"                  # projected wait past eight service times
    # quiet: no queue, few sequences, low demanded rate -> one rung down only after the quiet spell and the dwell
    for _ in range(4):
        c.observe_decode(3, 12.0)
    for i in range(NARROW_TICKS + MIN_DWELL_TICKS):
        d = c.decide(RungLoad(occupied=3, queued=0, arrival_rps=0.1, mean_output_tokens=10))
        if d.reason == "low_load":
            break
    assert d.reason == "low_load" and c.admission_limit() == 32 and i + 1 >= NARROW_TICKS
    d = c.decide(RungLoad(occupied=40, queued=0))
    assert d.reason == "occupied" and d.actual == 3                         # the seated sequences need a wider rung than the seat


def test_utilisation_widens_one_rung_and_estimates_scale_with_width():
    c = RungController([8, 16, 32], throughput=False)
    c.observe_decode(0, 10.0)                                               # 8 rows in 10 ms: 800 tokens/s
    assert c.step_ms(1) == pytest.approx(20.0) and c.capacity_tps(1) == pytest.approx(800.0)      # scaled, not copied
    # the seat only follows demand: 20 seated sequences ask for the 32 rung, the rate fills the 8 rung -> one rung per tick
    d = c.decide(RungLoad(occupied=20, queued=0, arrival_rps=80.0, mean_output_tokens=9.0))
    assert d.reason == "utilization" and c.admission_limit() == 16
    d = c.decide(RungLoad(occupied=20, queued=0, arrival_rps=1.0, mean_output_tokens=9.0))
    assert d.reason == "occupied" and c.admission_limit() == 16             # low rate: the seat stays


def test_a_faster_narrower_rung_takes_the_seat_with_a_margin():
    c = RungController([8, 16, 32])
    c.target = 2
    for _ in range(4):
        c.observe_decode(1, 10.0)        # 16 rows / 10 ms = 1600 tokens/s
        c.observe_decode(2, 21.0)        # 32 rows / 21 ms = 1524 tokens/s: the narrower rung wins by 5 %
    d = c.decide(RungLoad(occupied=30, queued=0))
    assert d.reason == "throughput" and c.admission_limit() == 16
    # with requests waiting the margin is 10 %: 5 % is not enough, demand widens the seat again
    for _ in range(8):
        d = c.decide(RungLoad(occupied=16, queued=10, oldest_wait_ms=300.0))
    assert c.admission_limit() == 32


def test_md1_table_waits_half_as_long_as_mm1():
    t = ServiceTable([1, 8, 64], [5.0, 6.0, 12.0])
    assert t.service_ms(1) == 5.0 and t.service_ms(9) == 12.0 and t.service_ms(500) == 12.0
    lam = 100.0                                                             # per second against a 5 ms server: rho = 0.5
    assert t.utilization(lam, 1) == pytest.approx(0.5)
    assert t.wait_ms(lam, 1) == pytest.approx(0.5 * 5.0 / (2 * 0.5))        # 2.5 ms
    assert t.wait_ms(lam, 1, cv=1.0) == pytest.approx(2 * t.wait_ms(lam, 1))
    assert math.isinf(t.wait_ms(250.0, 1))
    assert t.capacity_rps(64, 256) == pytest.approx(64 * 1000.0 / (12.0 * 256))
    t.observe(8, 7.5)
    assert t.service_ms(8) == 7.5 and t.measured == [False, True, False]
    # the batch window: zero without arrivals or at batch 1, grows with the arrival gap, never past a step or the cap
    assert t.formation_window_ms(0.0, 8) == 0.0 and t.formation_window_ms(50.0, 1) == 0.0
    w_dense, w_sparse = t.formation_window_ms(2000.0, 8), t.formation_window_ms(20.0, 8)
    assert 0 < w_dense < w_sparse <= t.service_ms(8)
    lam_s = 2000.0 / 1e3
    assert lam_s * w_dense ** 2 / 2 + w_dense == pytest.approx(7.5, rel=1e-6)       # the balance point the docstring states
    assert t.formation_window_ms(20.0, 8, max_hold_ms=2.0) == 2.0


def test_service_table_from_a_build_report(tiny_assets):
    import json
    build = json.loads((tiny_assets / "assets" / "build.json").read_text())
    t = ServiceTable.from_build(build)
    assert t.widths == [1, 2, 4, 8] and all(ms > 0 for ms in t.ms) and t.ms == sorted(t.ms)


def test_scheduler_admission_follows_the_controller(tiny_assets):
    """Ten short requests against eight slots with rungs 1/2/4/8: the first tick seats only what the controller's seat
    allows, the backlog widens the seat to the top within a few ticks, everything finishes with the same tokens as
    without the controller, and the decode steps it ran were timed per rung."""
    from plow_b200.runtime.cpu_engine import CpuEngine
    from plow_b200.runtime.scheduler import GenParams, ModelMux, SchedConfig
    from plow_b200.text.tokenizer import ByteTokenizer
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, 32000, 20).tolist() for _ in range(10)]

    def run(ctrl):
        eng = CpuEngine(tiny_assets / "assets", max_slots=8, max_ctx=256, prefix_cache=False)
        mux = ModelMux(eng, ByteTokenizer(), SchedConfig(token_budget=256, rung_control=ctrl), eos_ids=[])
        reqs = [mux.submit(p, GenParams(max_tokens=6)) for p in prompts]
        seated = []
        for _ in range(400):
            busy = mux.tick()
            seated.append(len(mux.live))
            if not busy and not mux.live and not mux.waiting:
                break
        outs = []
        for r in reqs:
            toks = []
            while True:
                c = r.out.get(timeout=10)
                if c.kind == "token":
                    toks.append(c.token_id)
                else:
                    assert c.kind == "done", c.error
                    break
            outs.append(toks)
        ctl = mux.rungs
        eng.close()
        return outs, seated, ctl
    plain, seated0, _ = run(False)
    ctrl, seated1, ctl = run(True)
    assert plain == ctrl and all(len(t) == 6 for t in ctrl)
    assert seated0[0] == 8                         # without the controller every free slot is filled at once
    assert seated1[0] < 8 and max(seated1) >= 4     # with it the seat starts low and the backlog widens it
    assert ctl.widths == [1, 2, 4, 8] and sum(e.n for e in ctl.step) >= 5
