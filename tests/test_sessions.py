"""Session KV retention and slot snapshot / rewind / resume (reference: crates/plowrt/src/serve/session.rs:1-12,
exec/gpu.rs:8905-9149): a finished request that carried a session id keeps its slot; the session's next request resumes
from the longest identical prefix and must produce exactly what a fresh run produces."""
import numpy as np

from plow_b200.runtime.cpu_engine import CpuEngine
from plow_b200.runtime.engine import EngineError, TokenBatch
from plow_b200.runtime.scheduler import GenParams, ModelMux, SchedConfig
from plow_b200.text.tokenizer import ByteTokenizer


def _mux(tiny_assets, prefix_cache, **cfg):
    eng = CpuEngine(tiny_assets / "assets", max_slots=4, max_ctx=512, prefix_cache=prefix_cache)
    return eng, ModelMux(eng, ByteTokenizer(), SchedConfig(**cfg), eos_ids=[]).start()


def test_second_turn_resumes_from_retained_slot(tiny_assets):
    rng = np.random.default_rng(0)
    turn1 = rng.integers(0, 250, 90).tolist()
    # without the prefix cache every reused token comes from the retained slot
    eng, mux = _mux(tiny_assets, prefix_cache=False)
    try:
        t1 = mux.generate(turn1, GenParams(max_tokens=12, session_id="s1"))[0]
        assert list(mux.retained) == ["s1"] and len(mux.free_slots) == 3
        turn2 = turn1 + t1 + rng.integers(0, 250, 20).tolist()
        r = mux.submit(turn2, GenParams(max_tokens=10, session_id="s1"))
        out, usage = [], None
        while True:
            c = r.out.get(timeout=60)
            if c.kind == "token":
                out.append(c.token_id)
            elif c.kind == "done":
                usage = c.usage
                break
        # everything but the last generated token of turn 1 was already in the cache
        assert usage["prompt_tokens_details"]["cached_tokens"] == len(turn1) + len(t1) - 1
        snap = mux.metrics.snapshot()["counters"]
        assert snap["session_hits"] == 1 and snap["session_tokens_reused"] == len(turn1) + len(t1) - 1
        fresh = mux.generate(turn2, GenParams(max_tokens=10))[0]
        assert out == fresh
        # a diverging third turn keeps only the common prefix
        turn3 = turn1[:40] + rng.integers(0, 250, 30).tolist()
        t3 = mux.generate(turn3, GenParams(max_tokens=6, session_id="s1"))[0]
        fresh3 = mux.generate(turn3, GenParams(max_tokens=6))[0]
        assert t3 == fresh3
        assert mux.metrics.snapshot()["counters"]["session_tokens_reused"] == len(turn1) + len(t1) - 1 + 40
    finally:
        mux.stop()
        eng.close()


def test_retained_sessions_yield_slots_and_expire(tiny_assets):
    rng = np.random.default_rng(1)
    eng, mux = _mux(tiny_assets, prefix_cache=True, max_sessions=2, session_ttl_s=0.2)
    try:
        for i in range(3):
            mux.generate(rng.integers(0, 250, 30).tolist(), GenParams(max_tokens=3, session_id=f"s{i}"))
        assert list(mux.retained) == ["s1", "s2"]            # the cap evicts the oldest
        # four concurrent requests need all four slots: the retained ones are given back
        reqs = [mux.submit(rng.integers(0, 250, 40).tolist(), GenParams(max_tokens=4)) for _ in range(4)]
        for r in reqs:
            while r.out.get(timeout=60).kind != "done":
                pass
        assert not mux.retained and len(mux.free_slots) == 4
        mux.generate(rng.integers(0, 250, 30).tolist(), GenParams(max_tokens=3, session_id="late"))
        assert "late" in mux.retained
        import time
        time.sleep(0.3)
        mux.generate(rng.integers(0, 250, 30).tolist(), GenParams(max_tokens=3))      # any tick expires it
        assert not mux.retained and mux.metrics.snapshot()["counters"]["sessions_expired"] == 1
        eng.pool.check()
    finally:
        mux.stop()
        eng.close()


def test_snapshot_rewind_resume_on_the_engine(tiny_assets):
    eng = CpuEngine(tiny_assets / "assets", max_slots=2, max_ctx=256, prefix_cache=True)
    try:
        rng = np.random.default_rng(2)
        p = rng.integers(0, 250, 100).tolist()
        eng.begin_slot(0, p)
        eng.reserve(0, len(p) + 8)
        r = eng.step(TokenBatch(np.asarray(p, np.int32), np.arange(len(p), dtype=np.int32), np.zeros(len(p), np.int32),
                                np.asarray([len(p) - 1], np.int32), want_logits=True))
        eng.commit(0, p)
        snap = eng.snapshot_slot(0)
        assert snap["kvlen"] == 100 and snap["tokens"] == p
        # one published page (64 tokens): a cut inside it is refused, a cut past it is fine
        assert not eng.can_rewind(0, 30) and eng.can_rewind(0, 70)
        try:
            eng.rewind_slot(0, 30)
            raise AssertionError("rewind into a published page must be refused")
        except EngineError:
            pass
        eng.rewind_slot(0, 70)
        assert int(eng.kvlen[0]) == 70 and eng.tokens[0] == p[:70]
        # recompute the tail: same logits as the first pass
        tail = p[70:]
        r2 = eng.step(TokenBatch(np.asarray(tail, np.int32), np.arange(70, 100, dtype=np.int32), np.zeros(30, np.int32),
                                 np.asarray([29], np.int32), want_logits=True))
        eng.commit(0, tail)
        assert np.allclose(r2.logits[0], r.logits[0], atol=1e-4)
        assert eng.resume_slot(0, p[:80] + [1, 2, 3]) == 80
        assert eng.resume_slot(0, [9] + p[1:]) == -1          # nothing in common at position 0
        eng.pool.check()
    finally:
        eng.close()
