"""Page pool + prefix cache: scripted sequences with invariant checks after every operation
(the reference tests its KV store the same way: memory/vmm_sim_tests.rs with check_tree)."""
import random

import pytest

from plow_b200.runtime.kv_pages import PAGE, OutOfPages, PagePool


def test_prefix_share_and_release():
    pool = PagePool(16)
    a = list(range(200))
    assert pool.begin(0, a) == 0
    pool.ensure(0, 200)
    pool.publish(0, a)
    pool.check()
    b = a[:130] + [9999] * 50
    assert pool.begin(1, b) == 128          # two full pages shared
    assert pool.seqs[1].pages[:2] == pool.seqs[0].pages[:2]
    pool.ensure(1, len(b))
    pool.check()
    pool.release(0)
    pool.check()
    assert pool.begin(2, a) == 192          # (len-1)//64 full pages: the last token is always computed
    pool.release(1)
    pool.release(2)
    pool.check()
    assert pool.available() == 16


def test_no_share_on_different_tokens_and_eviction():
    pool = PagePool(4)
    a = list(range(128)) + [1]
    pool.begin(0, a); pool.ensure(0, len(a)); pool.publish(0, a); pool.release(0)
    assert pool.available() == 4 and len(pool.lru) == 2
    b = [7] * 200
    assert pool.begin(1, b) == 0
    pool.ensure(1, 200)                     # needs all 4 pages: evicts the two cached ones
    assert pool.stats["evictions"] == 2
    pool.check()
    with pytest.raises(OutOfPages):
        pool.ensure(1, 400)
    pool.release(1)
    assert pool.begin(2, a) == 0            # evicted content is gone
    pool.release(2)
    pool.check()


def test_random_walk_invariants():
    rnd = random.Random(0)
    pool = PagePool(64)
    live = {}
    prompts = [[rnd.randrange(50) for _ in range(rnd.randrange(1, 400))] for _ in range(8)]
    for step in range(400):
        if live and (rnd.random() < 0.4 or len(live) >= 6):
            s = rnd.choice(list(live))
            pool.release(s)
            del live[s]
        else:
            s = next(i for i in range(100) if i not in live)
            base = rnd.choice(prompts)
            p = base[:rnd.randrange(1, len(base) + 1)] + [rnd.randrange(50) for _ in range(rnd.randrange(0, 80))]
            try:
                cached = pool.begin(s, p)
                assert cached % PAGE == 0 and cached < len(p)
                pool.ensure(s, len(p))
                pool.publish(s, p)
                live[s] = p
            except OutOfPages:
                pool.release(s)
        pool.check()


def test_host_tier_restores_evicted_prefix_pages(tiny_assets):
    """A prefix page evicted from a tiny device pool is spilled to host memory and copied back on the next match: the
    second run of the prompt computes only its tail and produces the same tokens."""
    import numpy as np
    from plow_b200.runtime.cpu_engine import CpuEngine
    from plow_b200.runtime.engine import TokenBatch
    eng = CpuEngine(tiny_assets / "assets", max_slots=2, max_ctx=256, n_pages=4)
    eng.enable_host_kv(8)
    rng = np.random.default_rng(4)
    a = rng.integers(0, 32000, 150).tolist()
    b = rng.integers(0, 32000, 200).tolist()

    def run(slot, prompt):
        cached = eng.begin_slot(slot, prompt)
        eng.reserve(slot, len(prompt) + 1)
        part = prompt[cached:]
        r = eng.step(TokenBatch(np.asarray(part, np.int32), np.arange(cached, len(prompt), dtype=np.int32),
                                np.full(len(part), slot, np.int32), np.asarray([len(part) - 1], np.int32)))
        eng.commit(slot, part)
        eng.retire_slot(slot)
        return int(r.ids[0]), cached
    t1, c1 = run(0, a)
    assert c1 == 0
    run(1, b)                              # needs all four pages: a's two published pages are evicted (spilled)
    assert eng.pool.stats["spilled"] >= 2
    t2, c2 = run(0, a)
    assert c2 == 128 and t2 == t1 and eng.pool.stats["restored"] == 2
    eng.pool.check()
    eng.close()
