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
