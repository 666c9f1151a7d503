"""Randomised workloads through the scheduler on the CPU engine, every serving mode switched on in turn: whatever the
mix of prompt lengths, budgets, cancellations, deadlines and KV pressure, every request ends exactly once, slots and KV
pages all come back, and greedy outputs do not depend on the mode."""
import numpy as np
import pytest

from plow_b200.runtime.cpu_engine import CpuEngine
from plow_b200.runtime.scheduler import GenParams, ModelMux, SchedConfig
from plow_b200.text.tokenizer import ByteTokenizer

MODES = {
    "plain": {},
    "lookahead": dict(lookahead=True),
    "multi_step": dict(multi_step=3),
    "spec_ngram": dict(spec_depth=3),
    "rungs": dict(rung_control=True),
    "throughput": dict(objective="throughput", ride=False),
    "everything": dict(lookahead=True, rung_control=True, multi_step=2),
}


def _run(assets, mode, seed, n_pages, cancel):
    rng = np.random.default_rng(seed)
    eng = CpuEngine(assets, max_slots=4, max_ctx=512, n_pages=n_pages, prefix_cache=bool(seed % 2))
    mux = ModelMux(eng, ByteTokenizer(), SchedConfig(token_budget=128, reserve_tokens=0, **MODES[mode]), eos_ids=[])
    motif = rng.integers(0, 32000, 9).tolist()
    plan = []
    for i in range(9):
        n = int(rng.integers(8, 140))
        prompt = (motif * 20)[:n] if i % 3 == 0 else rng.integers(0, 32000, n).tolist()       # some repetitive: n-gram drafts exist
        plan.append((int(rng.integers(0, 25)), prompt, int(rng.integers(1, 14))))
    plan.sort(key=lambda x: x[0])
    reqs, t, ends = [], 0, {}
    pending = list(plan)
    for t in range(3000):
        while pending and pending[0][0] <= t:
            _, p, mx = pending.pop(0)
            reqs.append(mux.submit(p, GenParams(max_tokens=mx)))
        if cancel and t == 12 and reqs:
            reqs[len(reqs) // 2].cancelled = True
        busy = mux.tick()
        if not busy and not pending and not mux.live and not mux.waiting and mux._inflight is None:
            break
    outs = []
    for r in reqs:
        toks, done = [], 0
        while not r.out.empty():
            c = r.out.get_nowait()
            if c.kind == "token":
                assert not done, "a token after the end"
                toks.append(c.token_id)
            else:
                done += 1
                ends[r.rid] = (c.kind, c.finish_reason)
        assert done == 1, (mode, r.rid, done)
        outs.append(toks)
    # everything came back
    assert len(reqs) == 9 and not mux.live and not mux.waiting and mux._inflight is None
    assert sorted(mux.free_slots) == [0, 1, 2, 3]
    assert not eng.tokens and int(eng.kvlen.sum()) == 0
    held = sum(len(s.pages) for s in eng.pool.seqs.values())
    assert held == 0 and eng.pool.available() == n_pages, (eng.pool.available(), n_pages)
    eng.close()
    return plan, outs, ends, mux.metrics.snapshot()["counters"]


@pytest.mark.parametrize("seed,n_pages,cancel", [(1, 32, False), (2, 7, False), (3, 32, True)])
def test_every_mode_ends_every_request_once_and_gives_the_same_tokens(tiny_assets, seed, n_pages, cancel):
    base = None
    for mode in MODES:
        plan, outs, ends, c = _run(tiny_assets / "assets", mode, seed, n_pages, cancel)
        for (_, _, mx), toks, r in zip(plan, outs, ends.values()):
            assert r[0] == "done" and r[1] in ("length", "cancelled"), (mode, r)
            if r[1] == "length":
                assert len(toks) == mx
        if base is None:
            base = outs
        else:
            for a, b, r in zip(base, outs, ends.values()):
                if r[1] == "length":
                    assert a[:len(b)] == b[:len(a)], mode          # same greedy tokens in every mode (a cancelled one may be shorter)
        if mode == "lookahead":
            assert c.get("lookahead_launches", 0) >= 1
        if n_pages == 7:
            assert c.get("preemptions", 0) >= 0
