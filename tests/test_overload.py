"""Overload control (serve/overload.py): the sliding-window miss fraction moves a level one step per dwell; the levels
shrink prefill chunks, switch extras off and finally refuse requests that do not continue a session (429 + Retry-After)."""
import numpy as np
import pytest
from fastapi.testclient import TestClient

from plow_b200.serve.overload import MIN_SAMPLES, OverloadControl


class Clock:
    def __init__(self):
        self.t = 1000.0

    def __call__(self):
        return self.t


def _feed(oc, clk, seconds, miss_every, per_s=20):
    """`per_s` deadlines per second for `seconds`, every `miss_every`-th one missed (0: none)."""
    n = 0
    for _ in range(int(seconds * per_s)):
        clk.t += 1.0 / per_s
        n += 1
        oc.record(not (miss_every and n % miss_every == 0))


def test_levels_rise_and_fall_one_step_per_dwell():
    clk = Clock()
    oc = OverloadControl(window_s=10.0, up=(0.05, 0.10, 0.20), clock=clk)
    _feed(oc, clk, 20, 0)
    assert oc.level == 0 and oc.fraction()[0] == 0.0 and oc.prefill_scale() == 1.0 and oc.extras_allowed() and oc.admit(False)
    # a short burst of misses is not overload: four misses in a window of two hundred deadlines stay under the threshold,
    # and a heavier burst that leaves the window before a dwell has passed does not count either
    _feed(oc, clk, 0.4, 2)
    _feed(oc, clk, 10, 0)
    assert oc.level == 0
    for _ in range(30):
        clk.t += 0.01
        oc.record(False)                                   # 30 misses at once: 13 % of the window
    _feed(oc, clk, 4, 0)                                   # ... for less than a dwell
    clk.t += 20                                            # then silence: the buckets age out
    oc.tick()
    _feed(oc, clk, 6, 0)
    assert oc.level == 0
    # sustained 25 % misses: level 1 after a dwell (5 s), level 2 one dwell later, and level 3 only after level 2 held a whole window
    _feed(oc, clk, 7, 4)
    assert oc.level == 1 and oc.prefill_scale() == 0.5 and oc.extras_allowed()
    _feed(oc, clk, 6, 4)
    assert oc.level == 2 and oc.prefill_scale() == 0.25 and not oc.extras_allowed() and oc.admit(False)
    _feed(oc, clk, 6, 4)
    assert oc.level == 2                                   # a dwell has passed but not a whole window at level 2
    _feed(oc, clk, 6, 4)
    assert oc.level == 3 and not oc.admit(False) and oc.admit(True) and oc.retry_after_s() == 5
    # recovery: clean traffic brings it down one level per dwell
    _feed(oc, clk, 12, 0)
    assert oc.level < 3
    _feed(oc, clk, 20, 0)
    assert oc.level == 0
    # too few samples in the window are no evidence
    oc2 = OverloadControl(10.0, clock=clk)
    for _ in range(MIN_SAMPLES - 1):
        clk.t += 0.4
        oc2.record(False)
    clk.t += 6
    oc2.tick()
    assert oc2.level == 0
    assert OverloadControl.from_env({}) is None and OverloadControl.from_env({"PLOW_OVERLOAD": "1"}).window == 10.0
    with pytest.raises(ValueError):
        OverloadControl.from_env({"PLOW_OVERLOAD": "1", "PLOW_OVERLOAD_MISS": "0.2,0.1,0.3"})


def test_scheduler_and_api_follow_the_level(tiny_assets):
    from plow_b200.runtime.cpu_engine import CpuEngine
    from plow_b200.runtime.scheduler import GenParams, ModelMux, SchedConfig
    from plow_b200.serve.app import AppState, ModelEntry, create_app
    from plow_b200.serve.template import ChatTemplate
    from plow_b200.text.tokenizer import ByteTokenizer
    eng = CpuEngine(tiny_assets / "assets", max_slots=4, max_ctx=512)
    tok = ByteTokenizer()
    mux = ModelMux(eng, tok, SchedConfig(token_budget=256, tbt_target_ms=1e6), eos_ids=[])
    assert mux.overload is None                            # off unless asked for
    oc = mux.overload = OverloadControl(10.0)
    base = mux._prefill_budget()
    oc.level = 1
    assert mux._prefill_budget() == max(64, base // 2)
    oc.level = 2
    assert mux._prefill_budget() == max(64, base // 4) and not mux._lookahead_ok([], 1)
    oc.level = 0
    mux.start()
    state = AppState()
    state.add(ModelEntry("tiny", mux, tok, ChatTemplate()))
    try:
        with TestClient(create_app(state)) as c:
            body = dict(model="tiny", prompt="hello", max_tokens=3)
            assert c.post("/v1/completions", json=body).status_code == 200
            assert oc.fraction()[1] >= 2                   # token gaps were recorded against the (huge) objective: all met
            oc.level = 3
            r = c.post("/v1/completions", json=body)
            assert r.status_code == 429 and r.headers.get("retry-after") == "5" and r.json()["error"]["code"] == "overloaded"
            assert mux.metrics.snapshot()["counters"]["overload_refused"] == 1
            oc.level = 2
            assert c.post("/v1/completions", json=body).status_code == 200
    finally:
        mux.stop()
        eng.close()
