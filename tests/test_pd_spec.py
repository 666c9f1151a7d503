"""KV image hand-off (prefill/decode disaggregation) and speculative decoding on the CPU engine: both must reproduce
plain greedy decoding token for token."""
import numpy as np
import pytest


def _plain(eng, slot, prompt, max_new):
    from plow_b200.runtime.engine import TokenBatch
    eng.begin_slot(slot, prompt)
    eng.reserve(slot, len(prompt) + max_new + 1)
    r = eng.step(TokenBatch(np.asarray(prompt, np.int32), np.arange(len(prompt), dtype=np.int32), np.full(len(prompt), slot, np.int32),
                            np.asarray([len(prompt) - 1], np.int32)))
    eng.commit(slot, prompt)
    out = [int(r.ids[0])]
    while len(out) < max_new:
        n = len(eng.tokens[slot])
        r = eng.step(TokenBatch(np.asarray([out[-1]], np.int32), np.asarray([n], np.int32), np.asarray([slot], np.int32),
                                np.asarray([0], np.int32), decode=True))
        eng.commit(slot, [out[-1]])
        out.append(int(r.ids[0]))
    eng.retire_slot(slot)
    return out


@pytest.fixture(scope="module")
def engines(tiny_assets):
    from plow_b200.runtime.cpu_engine import CpuEngine
    a = CpuEngine(tiny_assets / "assets", max_slots=4, max_ctx=512, prefix_cache=False)
    b = CpuEngine(tiny_assets / "assets", max_slots=4, max_ctx=512, prefix_cache=False)
    yield a, b
    a.close(); b.close()


def test_kv_image_roundtrip_and_pd_pipeline(engines):
    from plow_b200.runtime.kv_image import KvImage
    from plow_b200.serve.pd import PdPipeline
    a, b = engines
    rng = np.random.default_rng(3)
    prompt = rng.integers(0, 32000, 150).tolist()
    want = _plain(a, 0, prompt, 12)
    pd = PdPipeline(a, b, wire=True)
    first, img = pd.prefill(1, prompt, chunk=64)          # chunked prefill on engine A
    assert img.n_pages == 3 and len(img.tokens) == 150 and all(v.shape[0] == 3 for v in img.arrays.values())
    img2 = KvImage.from_bytes(img.to_bytes())
    assert img2.tokens == img.tokens and all(np.array_equal(img.arrays[k], img2.arrays[k]) for k in img.arrays)
    pd.handoff(2, img)                                     # engine B continues in a different slot
    got = pd.decode(2, first, 12)
    assert got == want
    assert pd.bytes_moved > 0
    b.retire_slot(2)


def test_kv_image_rejects_other_packet(engines):
    from plow_b200.runtime.engine import EngineError
    from plow_b200.runtime.kv_image import KvImage, import_slot
    a, _ = engines
    with pytest.raises(EngineError):
        import_slot(a, 3, KvImage("00" * 32, [1, 2, 3], {}))


def test_speculative_decoding_matches_greedy(engines):
    from plow_b200.runtime.engine import TokenBatch
    from plow_b200.runtime.spec import NgramDrafter, SpecStats, plan_depth, spec_decode
    a, _ = engines
    rng = np.random.default_rng(5)
    motif = rng.integers(0, 32000, 12).tolist()
    prompt = (motif * 8)[:90]                              # repetitive context so the n-gram drafter has material
    want = _plain(a, 0, prompt, 24)
    a.begin_slot(1, prompt)
    a.reserve(1, len(prompt) + 1)
    r = a.step(TokenBatch(np.asarray(prompt, np.int32), np.arange(len(prompt), dtype=np.int32), np.full(len(prompt), 1, np.int32),
                          np.asarray([len(prompt) - 1], np.int32)))
    a.commit(1, prompt)
    stats = SpecStats()
    got = spec_decode(a, 1, int(r.ids[0]), 24, NgramDrafter(3), depth=4, stats=stats)
    a.retire_slot(1)
    assert got == want
    assert stats.steps <= 24 and stats.emitted >= 23
    assert NgramDrafter(2).propose([1, 2, 3, 9, 1, 2], 3) == [3, 9, 1]
    assert plan_depth(0.0, 8) == 0 and plan_depth(0.9, 8) >= 3


def test_pd_disaggregation_between_two_muxes(engines):
    """A prefill mux hands every finished prompt to a decode mux through a KV image; the client sees one stream whose
    tokens equal single-engine decoding."""
    from plow_b200.runtime.scheduler import GenParams, ModelMux, SchedConfig
    from plow_b200.text.tokenizer import ByteTokenizer
    a, b = engines
    rng = np.random.default_rng(11)
    prompts = [rng.integers(0, 32000, n).tolist() for n in (90, 33)]
    want = [_plain(a, 0, p, 10) for p in prompts]
    pre = ModelMux(a, ByteTokenizer(), SchedConfig(token_budget=64), eos_ids=[])
    dec = ModelMux(b, ByteTokenizer(), SchedConfig(token_budget=64), eos_ids=[])
    pre.pd_target = dec
    reqs = [pre.submit(p, GenParams(max_tokens=10)) for p in prompts]
    for _ in range(200):
        busy = pre.tick() | dec.tick()
        if not busy and not pre.live and not dec.live and not pre.waiting and dec.adopt_q.empty():
            break
    for r, w in zip(reqs, want):
        ids = []
        while True:
            ch = r.out.get(timeout=10)
            if ch.kind == "token":
                ids.append(ch.token_id)
            else:
                assert ch.kind == "done" and ch.finish_reason == "length"
                break
        assert ids == w
    pc, dc = pre.metrics.snapshot()["counters"], dec.metrics.snapshot()["counters"]
    assert pc["pd_handoffs"] == 2 and dc["pd_adopted"] == 2 and pc.get("decode_ticks", 0) == 0 and dc["decode_ticks"] >= 9
    assert a.pool.available() == a.pool.n_pages and b.pool.available() == b.pool.n_pages
