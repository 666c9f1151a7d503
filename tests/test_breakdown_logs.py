"""Tick / decode-step / TTFT breakdown logs (obs/breakdown.py) written by the scheduler on the CPU engine."""
import json

import numpy as np


def test_breakdown_logs_are_off_by_default_and_complete_when_on(tiny_assets, tmp_path):
    from plow_b200.obs.breakdown import Breakdown, LogWriter
    from plow_b200.runtime.cpu_engine import CpuEngine
    from plow_b200.runtime.scheduler import GenParams, ModelMux, SchedConfig
    from plow_b200.text.tokenizer import ByteTokenizer
    assert not Breakdown(env={}).any and Breakdown(env={}).writer is None
    path = tmp_path / "obs.jsonl"
    eng = CpuEngine(tiny_assets / "assets", max_slots=4, max_ctx=512, prefix_cache=False)
    mux = ModelMux(eng, ByteTokenizer(), SchedConfig(token_budget=128), eos_ids=[])
    mux.blog = Breakdown(env=dict(PLOW_TICK_LOG="1", PLOW_DSTEP_LOG="1", PLOW_TTFT_LOG="1", PLOW_OBS_LOG_FILE=str(path)))
    rng = np.random.default_rng(1)
    reqs = [mux.submit(rng.integers(0, 32000, n).tolist(), GenParams(max_tokens=5)) for n in (150, 40)]     # 150: two prefill chunks
    for _ in range(100):
        if not mux.tick() and not mux.live and not mux.waiting:
            break
    for r in reqs:
        while r.out.get(timeout=10).kind != "done":
            pass
    mux.blog.writer.flush()
    eng.close()
    recs = [json.loads(l) for l in path.read_text().splitlines()]
    ticks = [r for r in recs if r["log"] == "TICK"]
    dsteps = [r for r in recs if r["log"] == "DSTEP"]
    ttfts = {r["rid"]: r for r in recs if r["log"] == "TTFT"}
    c = mux.metrics.snapshot()["counters"]
    assert len(ticks) == c["prefill_ticks"] + c["decode_ticks"] and [t["seq"] for t in ticks] == list(range(1, len(ticks) + 1))
    assert {t["kind"] for t in ticks} == {"prefill", "decode"}
    assert all(t["wall_ms"] >= t["host_ms"] >= 0 and t["rows"] > 0 for t in ticks)
    assert len(dsteps) == c["decode_ticks"] and all(d["rows"] <= d["rung"] for d in dsteps)
    assert len(ttfts) == 2
    long, short = ttfts[reqs[0].rid], ttfts[reqs[1].rid]
    assert long["prompt_tokens"] == 150 and long["prefill_chunks"] == 2 and short["prefill_chunks"] == 1
    assert all(t["ttft_ms"] >= t["seat_to_first_ms"] >= 0 and t["queued_ms"] >= 0 for t in ttfts.values())
    # the writer never blocks: a full queue drops and counts
    w = LogWriter(str(tmp_path / "x.jsonl"), cap=1)
    w._thread = object()                  # no consumer
    w.put(dict(a=1))
    w.put(dict(a=2))
    assert w.dropped == 1
