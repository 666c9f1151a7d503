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


@pytest.mark.parametrize("family", ["gpt_oss", "kimi_linear"])
def test_new_families_serve_through_the_scheduler(tmp_path, family):
    """Three requests of different lengths batched continuously on a gpt_oss packet (sinks, sliding window, biased experts)
    and on a kimi_linear one (recurrent state per slot): every request's greedy tokens equal the fp32 reference's."""
    import glob
    import torch
    from safetensors.torch import load_file
    from plow_b200 import plowc
    from plow_b200.models import config, reference
    if family == "gpt_oss":
        cfg = dict(model_type="gpt_oss", hidden_size=128, num_attention_heads=8, num_key_value_heads=2, head_dim=32, num_hidden_layers=2,
                   layer_types=["sliding_attention", "full_attention"], sliding_window=16, num_local_experts=8, num_experts_per_tok=2,
                   intermediate_size=64, vocab_size=300, max_position_embeddings=1024, eos_token_id=299, plow_dtype="f32", plow_kv_dtype="f32")
    else:
        cfg = dict(model_type="kimi_linear", hidden_size=128, num_hidden_layers=3, num_attention_heads=4, kv_lora_rank=32, q_lora_rank=None,
                   qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                   linear_attn_config=dict(kda_layers=[1, 2], full_attn_layers=[3], num_heads=4, head_dim=32, short_conv_kernel_size=4),
                   intermediate_size=256, num_experts=8, num_experts_per_token=2, moe_intermediate_size=64, num_shared_experts=1,
                   first_k_dense_replace=1, vocab_size=300, max_position_embeddings=1024, eos_token_id=299, plow_dtype="f32", plow_kv_dtype="f32")
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=5)
    plowc.compile_dir(tmp_path / "ckpt", tmp_path / "assets", arch="cpu", n_cu=4, max_rows=128, decode_rungs=[1, 2, 4], max_seqs=4)
    state = {}
    for fn in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        state.update(load_file(fn))
    ref = reference.ReferenceModel(config.spec_from_config(cfg), {k: v.float() for k, v in state.items()})
    eng = CpuEngine(tmp_path / "assets", max_slots=4, max_ctx=256)
    mux = ModelMux(eng, ByteTokenizer(), SchedConfig(token_budget=64, reserve_tokens=0), eos_ids=[])
    rng = np.random.default_rng(8)
    prompts = [rng.integers(0, 290, n).tolist() for n in (40, 9, 75)]
    reqs = [mux.submit(p, GenParams(max_tokens=5)) for p in prompts]
    for _ in range(400):
        if not mux.tick() and not mux.live and not mux.waiting:
            break
    for p, r in zip(prompts, reqs):
        toks = []
        while not r.out.empty():
            c = r.out.get_nowait()
            if c.kind == "token":
                toks.append(c.token_id)
        want, cur = [], list(p)
        for _ in range(5):
            want.append(int(ref.forward(torch.tensor(cur))[-1].argmax()))
            cur.append(want[-1])
        assert toks == want, (family, len(p), toks, want)
    eng.close()
