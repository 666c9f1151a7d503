"""CPU plumbing: tiny dense GQA decoder, fp32, plowc -> packet -> plowrt engine ->
scheduler; logits must match the PyTorch reference to 1e-4 and greedy tokens must agree."""
import json

import numpy as np
import pytest
import torch

from plow_b200.runtime.cpu_engine import CpuEngine
from plow_b200.runtime.engine import TokenBatch
from plow_b200.runtime.scheduler import GenParams, ModelMux, SchedConfig
from plow_b200.text.tokenizer import ByteTokenizer


def _prompts(n=4, length=128, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 32000, (length,), generator=g).tolist() for _ in range(n)]


def test_prefill_and_decode_logits_match_reference(tiny_assets, tiny_reference):
    eng = CpuEngine(tiny_assets / "assets", max_slots=4, max_ctx=256)
    prompts = _prompts()
    # packed prefill of 2 prompts in one token batch, logits on each last row
    ids, pos, seq, samp = [], [], [], []
    for s, p in enumerate(prompts[:2]):
        eng.begin_slot(s, p)
        eng.reserve(s, len(p) + 2)
        ids += p
        pos += list(range(len(p)))
        seq += [s] * len(p)
        samp.append(len(ids) - 1)
    res = eng.step(TokenBatch(np.array(ids, np.int32), np.array(pos, np.int32), np.array(seq, np.int32),
                              np.array(samp, np.int32), want_logits=True))
    for s, p in enumerate(prompts[:2]):
        ref = tiny_reference.forward(torch.tensor(p))[-1]
        assert (torch.from_numpy(res.logits[s]) - ref).abs().max().item() < 1e-4
        assert int(res.ids[s]) == int(ref.argmax())
        eng.commit(s, p)
    # one decode step for both sequences
    nxt = [int(res.ids[0]), int(res.ids[1])]
    res2 = eng.step(TokenBatch(np.array(nxt, np.int32), np.array([128, 128], np.int32), np.array([0, 1], np.int32),
                               np.array([0, 1], np.int32), decode=True, want_logits=True))
    for s in range(2):
        ref = tiny_reference.forward(torch.tensor(prompts[s] + [nxt[s]]))[-1]
        assert (torch.from_numpy(res2.logits[s]) - ref).abs().max().item() < 1e-4
    eng.close()


def test_greedy_64_tokens_through_scheduler(tiny_assets, tiny_reference):
    eng = CpuEngine(tiny_assets / "assets", max_slots=4, max_ctx=256)
    mux = ModelMux(eng, ByteTokenizer(), SchedConfig(token_budget=256), eos_ids=[]).start()
    prompts = _prompts()
    reqs = [mux.submit(p, GenParams(max_tokens=64)) for p in prompts]
    outs = []
    for r in reqs:
        ids = []
        while True:
            ch = r.out.get(timeout=120)
            if ch.kind == "token":
                ids.append(ch.token_id)
            else:
                assert ch.kind == "done" and ch.finish_reason == "length"
                assert ch.usage["completion_tokens"] == 64 and ch.usage["prompt_tokens"] == 128
                break
        outs.append(ids)
    mux.stop()
    seq = list(prompts[0])
    for _ in range(64):
        seq.append(int(tiny_reference.forward(torch.tensor(seq))[-1].argmax()))
    assert outs[0] == seq[128:]
    eng.pool.check()
    assert eng.pool.available() == eng.pool.n_pages
    eng.close()


def test_prefix_cache_hit_gives_same_tokens(tiny_assets):
    eng = CpuEngine(tiny_assets / "assets", max_slots=2, max_ctx=512)
    mux = ModelMux(eng, ByteTokenizer(), eos_ids=[]).start()
    p = _prompts(1, 200, seed=3)[0]
    a = mux.generate(p, GenParams(max_tokens=8))
    b = mux.generate(p, GenParams(max_tokens=8))
    assert a[0] == b[0]
    assert a[3]["prompt_tokens_details"]["cached_tokens"] == 0
    assert b[3]["prompt_tokens_details"]["cached_tokens"] == 192
    mux.stop()
    eng.close()


def test_preemption_requeues_and_finishes(tiny_assets):
    # 6 pages only: two 130-token prompts need 3 pages each, growth forces a preemption
    eng = CpuEngine(tiny_assets / "assets", max_slots=2, max_ctx=512, n_pages=6, prefix_cache=False)
    mux = ModelMux(eng, ByteTokenizer(), SchedConfig(reserve_tokens=0), eos_ids=[]).start()
    ps = _prompts(2, 130, seed=5)
    solo = ModelMux(CpuEngine(tiny_assets / "assets", max_slots=1, max_ctx=512), ByteTokenizer(), eos_ids=[]).start()
    want = [solo.generate(p, GenParams(max_tokens=70))[0] for p in ps]
    solo.stop()
    reqs = [mux.submit(p, GenParams(max_tokens=70)) for p in ps]
    got = []
    for r in reqs:
        ids = []
        while True:
            ch = r.out.get(timeout=120)
            if ch.kind == "token":
                ids.append(ch.token_id)
            else:
                assert ch.kind == "done"
                break
        got.append(ids)
    assert mux.metrics.c["preemptions"] >= 1
    assert got == want
    mux.stop()
    eng.pool.check()


def test_stop_string_and_sampling_seed(tiny_assets):
    eng = CpuEngine(tiny_assets / "assets", max_slots=2, max_ctx=256)
    tok = ByteTokenizer()
    mux = ModelMux(eng, tok, eos_ids=[]).start()
    p = tok.encode("hello world")
    a = mux.generate(p, GenParams(max_tokens=12, temperature=0.8, top_p=0.9, seed=7))
    b = mux.generate(p, GenParams(max_tokens=12, temperature=0.8, top_p=0.9, seed=7))
    c = mux.generate(p, GenParams(max_tokens=12, temperature=0.8, top_p=0.9, seed=8))
    assert a[0] == b[0] and a[0] != c[0]
    ids, text, reason, usage = mux.generate(p, GenParams(max_tokens=5, stop_token_ids=[a[0][2]], temperature=0.8, top_p=0.9, seed=7))
    assert reason == "stop" and ids == a[0][:2] and usage["completion_tokens"] == 2
    mux.stop()
    eng.close()


def test_decode_rows_ride_prefill_launches(tiny_assets):
    """A long prompt is prefilled in small chunks while another request is decoding: with riding on, the decoder's rows
    are appended to the prefill launches (mixed steps) and both requests produce exactly the tokens they produce
    without riding."""
    def run(ride):
        eng = CpuEngine(tiny_assets / "assets", max_slots=4, max_ctx=512, prefix_cache=False)
        mux = ModelMux(eng, ByteTokenizer(), SchedConfig(token_budget=64, ride=ride), eos_ids=[])
        rng = np.random.default_rng(9)
        a = mux.submit(rng.integers(0, 32000, 20).tolist(), GenParams(max_tokens=24))
        for _ in range(4):
            mux.tick()                                   # request a is decoding by now
        b = mux.submit(rng.integers(0, 32000, 300).tolist(), GenParams(max_tokens=4))
        for _ in range(200):
            if not mux.tick() and not mux.waiting and not mux.live:
                break
        outs = []
        for r in (a, b):
            ids = []
            while True:
                ch = r.out.get(timeout=10)
                if ch.kind == "token":
                    ids.append(ch.token_id)
                else:
                    assert ch.kind == "done", ch.error
                    break
            outs.append(ids)
        riders = mux.metrics.snapshot()["counters"].get("rider_rows", 0)
        eng.close()
        return outs, riders
    plain, r0 = run(False)
    rode, r1 = run(True)
    assert plain == rode
    assert r0 == 0 and r1 >= 3


def test_mla_moe_model_on_cpu_backend_matches_reference(tmp_path):
    """The C++ interpreter's golden MLA (absorbed scores over the latent cache) and MoE (group-limited sigmoid router,
    slot-ordered combine, shared expert) ops: prefill + decode logits vs the PyTorch fp32 reference."""
    import glob
    from safetensors.torch import load_file
    from plow_b200 import plowc
    from plow_b200.models import config, reference
    from plow_b200.runtime.engine import TokenBatch
    cfg = dict(model_type="deepseek_v3", hidden_size=256, num_attention_heads=4, num_hidden_layers=2,
               q_lora_rank=64, kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
               intermediate_size=512, first_k_dense_replace=1, n_routed_experts=8, n_shared_experts=1,
               num_experts_per_tok=2, moe_intermediate_size=64, n_group=2, topk_group=1, scoring_func="sigmoid",
               norm_topk_prob=True, routed_scaling_factor=2.5, topk_method="noaux_tc", rms_norm_eps=1e-6,
               rope_theta=10000.0, vocab_size=512, tie_word_embeddings=False, max_position_embeddings=1024, eos_token_id=1,
               plow_dtype="f32", plow_kv_dtype="f32")
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=0)
    plowc.compile_dir(tmp_path / "ckpt", tmp_path / "assets", arch="cpu", n_cu=4, max_rows=128, decode_rungs=[1, 2, 4], max_seqs=4)
    eng = CpuEngine(tmp_path / "assets", max_slots=2, max_ctx=256)
    state = {}
    for f in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        state.update(load_file(f))
    ref = reference.ReferenceModel(config.spec_from_config(cfg), {k: v.float() for k, v in state.items()})
    rng = np.random.default_rng(2)
    p = rng.integers(0, 512, 70).tolist()
    eng.begin_slot(0, p)
    eng.reserve(0, len(p) + 4)
    r = eng.step(TokenBatch(np.asarray(p, np.int32), np.arange(len(p), dtype=np.int32), np.zeros(len(p), np.int32),
                            np.asarray([len(p) - 1], np.int32), want_logits=True))
    want = ref.forward(torch.tensor(p))[-1]
    assert (torch.from_numpy(r.logits[0]) - want).abs().max().item() < 2e-4 * max(1.0, want.abs().max().item())
    eng.commit(0, p)
    nxt = int(want.argmax())
    assert int(r.ids[0]) == nxt
    r = eng.step(TokenBatch(np.asarray([nxt], np.int32), np.asarray([len(p)], np.int32), np.zeros(1, np.int32), np.zeros(1, np.int32),
                            decode=True, want_logits=True))
    want = ref.forward(torch.tensor(p + [nxt]))[-1]
    assert (torch.from_numpy(r.logits[0]) - want).abs().max().item() < 2e-4 * max(1.0, want.abs().max().item())
    eng.close()


def test_deadline_stops_generation_and_load_estimate(tiny_assets):
    eng = CpuEngine(tiny_assets / "assets", max_slots=2, max_ctx=256)
    mux = ModelMux(eng, ByteTokenizer(), SchedConfig(token_budget=256), eos_ids=[])
    r = mux.submit(_prompts()[0], GenParams(max_tokens=200, deadline_ms=1.0))
    import time as _t
    mux.tick()                      # prefill + first token
    _t.sleep(0.01)
    for _ in range(5):
        mux.tick()
    got, reason = 0, None
    while True:
        ch = r.out.get(timeout=10)
        if ch.kind == "token":
            got += 1
        else:
            reason = ch.finish_reason
            break
    assert reason == "deadline" and 1 <= got < 200
    est = mux.load_estimate()
    assert est["arrival_rps"] > 0 and est["live"] == 0
    assert mux.metrics.snapshot()["counters"]["deadline_exceeded"] == 1
    eng.close()


def test_speculative_decoding_in_the_scheduler(tiny_assets):
    """spec_depth > 0: greedy requests are verified in spans; the tokens equal plain decoding and fewer launches are used."""
    def run(depth):
        eng = CpuEngine(tiny_assets / "assets", max_slots=2, max_ctx=512, prefix_cache=False)
        mux = ModelMux(eng, ByteTokenizer(), SchedConfig(token_budget=256, spec_depth=depth), eos_ids=[])
        rng = np.random.default_rng(5)
        motif = rng.integers(0, 32000, 12).tolist()
        r = mux.submit((motif * 8)[:90], GenParams(max_tokens=24))
        for _ in range(100):
            if not mux.tick() and not mux.live and not mux.waiting:
                break
        ids = []
        while True:
            ch = r.out.get(timeout=10)
            if ch.kind == "token":
                ids.append(ch.token_id)
            else:
                assert ch.kind == "done" and ch.finish_reason == "length"
                break
        c = mux.metrics.snapshot()["counters"]
        eng.close()
        return ids, c
    plain, c0 = run(0)
    spec, c1 = run(4)
    assert plain == spec and len(spec) == 24
    assert c1.get("spec_ticks", 0) >= 1 and c1.get("spec_accepted", 0) >= 1
    assert c1.get("decode_ticks", 0) + c1.get("spec_ticks", 0) < c0["decode_ticks"]


def test_multi_step_decode_gives_the_same_tokens(tiny_assets):
    """`multi_step` = 4: greedy decode ticks run four steps per engine call (the engine feeds its own arg-max tokens
    forward); the tokens, stop handling and usage must equal the step-by-step run, including a request whose budget is
    not a multiple of four and one that stops on a stop token inside a chained call."""
    prompts = _prompts(3, 60, seed=9)

    def run(multi):
        eng = CpuEngine(tiny_assets / "assets", max_slots=4, max_ctx=512)
        mux = ModelMux(eng, ByteTokenizer(), SchedConfig(multi_step=multi), eos_ids=[]).start()
        try:
            first = mux.generate(prompts[0], GenParams(max_tokens=12))
            stop_tok = first[0][6]            # a token the greedy continuation is known to produce at step 7
            reqs = [mux.submit(prompts[0], GenParams(max_tokens=12, stop_token_ids=[stop_tok])),
                    mux.submit(prompts[1], GenParams(max_tokens=10)), mux.submit(prompts[2], GenParams(max_tokens=7))]
            outs = []
            for r in reqs:
                toks = []
                while True:
                    c = r.out.get(timeout=60)
                    if c.kind == "token":
                        toks.append(c.token_id)
                    elif c.kind == "done":
                        outs.append((toks, c.finish_reason, c.usage["completion_tokens"]))
                        break
            return first[0], outs, mux.metrics.snapshot()["counters"].get("multi_step_calls", 0)
        finally:
            mux.stop()
            eng.close()
    a_first, a_outs, a_calls = run(1)
    b_first, b_outs, b_calls = run(4)
    assert a_first == b_first and a_outs == b_outs
    assert a_calls == 0 and b_calls > 0
    assert a_outs[0][1] == "stop" and len(a_outs[0][0]) <= 7


def test_lookahead_decode_gives_the_same_tokens(tiny_assets):
    """`lookahead`: decode step n + 1 is launched (its ids taken from step n's output by the engine) before the host reads
    step n.  Tokens, stop handling and usage must equal the plain run: one request stops on a stop token (the row the
    chained step computed for it is dropped), one runs out of budget, and a request that arrives in the middle drains
    the pipeline, is prefilled, and joins."""
    prompts = _prompts(4, 60, seed=9)

    def run(look):
        eng = CpuEngine(tiny_assets / "assets", max_slots=4, max_ctx=512)
        mux = ModelMux(eng, ByteTokenizer(), SchedConfig(lookahead=look), eos_ids=[])
        try:
            first = []
            r0 = mux.submit(prompts[0], GenParams(max_tokens=12))
            for _ in range(100):
                if not mux.tick() and not mux.live and not mux.waiting:
                    break
            while True:
                c = r0.out.get(timeout=10)
                if c.kind == "token":
                    first.append(c.token_id)
                else:
                    break
            stop_tok = first[6]
            reqs = [mux.submit(prompts[0], GenParams(max_tokens=12, stop_token_ids=[stop_tok])),
                    mux.submit(prompts[1], GenParams(max_tokens=10)), mux.submit(prompts[2], GenParams(max_tokens=7))]
            late = None
            for t in range(200):
                if t == 6:
                    late = mux.submit(prompts[3], GenParams(max_tokens=9))
                if not mux.tick() and not mux.live and not mux.waiting and late is not None:
                    break
            outs = []
            for r in reqs + [late]:
                toks = []
                while True:
                    c = r.out.get(timeout=10)
                    if c.kind == "token":
                        toks.append(c.token_id)
                    elif c.kind == "done":
                        outs.append((toks, c.finish_reason, c.usage["completion_tokens"]))
                        break
                    else:
                        raise AssertionError(c.error)
            assert mux._inflight is None and not mux.live
            return first, outs, mux.metrics.snapshot()["counters"].get("lookahead_launches", 0)
        finally:
            eng.close()
    a_first, a_outs, a_n = run(False)
    b_first, b_outs, b_n = run(True)
    assert a_first == b_first and a_outs == b_outs
    assert a_n == 0 and b_n >= 8
    assert a_outs[0][1] == "stop" and len(a_outs[0][0]) <= 7 and [len(o[0]) for o in a_outs[1:]] == [10, 7, 9]


@pytest.mark.parametrize("n_pages,budget,lens", [(5, 64, (144, 157, 187)), (5, 96, (144, 157, 187)), (7, 128, (144, 157, 187, 120))])
def test_prefill_time_preemption_keeps_the_dispatcher_alive(tiny_assets, n_pages, budget, lens):
    """KV pressure DURING prefill: long prompts admitted against few pages with small chunks.  A request that loses its
    slot to a preemption inside a tick must not be planned again in that tick (its slot is -1), every request still
    finishes with its full output, and the dispatcher thread survives."""
    eng = CpuEngine(tiny_assets / "assets", max_slots=4, max_ctx=512, n_pages=n_pages, prefix_cache=False)
    mux = ModelMux(eng, ByteTokenizer(), SchedConfig(token_budget=budget, reserve_tokens=0), eos_ids=[]).start()
    try:
        rng = np.random.default_rng(11)
        reqs = [mux.submit(rng.integers(3, 250, size=n).tolist(), GenParams(max_tokens=12)) for n in lens]
        for r in reqs:
            n = 0
            while True:
                ch = r.out.get(timeout=120)
                if ch.kind == "token":
                    n += 1
                else:
                    assert ch.kind == "done" and ch.finish_reason == "length", (ch.kind, ch.error)
                    break
            assert n == 12
        assert mux._thread.is_alive()
        eng.pool.check()
    finally:
        mux.stop()
        eng.close()


def test_sparse_attention_model_on_cpu_backend_matches_reference(tmp_path):
    """The interpreter's golden indexer ops (index-key cache write, weighted-ReLU scores, exact top-k with ties to the
    lower position) and sparse MLA attention: a model whose indexer keeps 64 of up to 150 visible keys, prefill + decode,
    against the fp32 reference running its own indexer.  Both sides are fp32, so the selections coincide and the logits
    agree to rounding; dense attention over all keys would not."""
    import glob
    from safetensors.torch import load_file
    from plow_b200 import plowc
    from plow_b200.compiler import packet as pk
    from plow_b200.models import config, reference
    from plow_b200.runtime.engine import TokenBatch
    cfg = dict(model_type="glm_moe_dsa", hidden_size=256, num_attention_heads=4, num_hidden_layers=2,
               q_lora_rank=64, kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
               intermediate_size=512, first_k_dense_replace=1, n_routed_experts=8, n_shared_experts=1,
               num_experts_per_tok=2, moe_intermediate_size=64, n_group=2, topk_group=1, scoring_func="sigmoid",
               norm_topk_prob=True, routed_scaling_factor=2.5, topk_method="noaux_tc", rms_norm_eps=1e-6,
               rope_theta=10000.0, vocab_size=512, tie_word_embeddings=False, max_position_embeddings=1024, eos_token_id=1,
               index_n_heads=4, index_head_dim=32, index_topk=64, plow_dtype="f32", plow_kv_dtype="f32")
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=0)
    plowc.compile_dir(tmp_path / "ckpt", tmp_path / "assets", arch="cpu", n_cu=4, max_rows=256, decode_rungs=[1, 2], max_seqs=4)
    eng = CpuEngine(tmp_path / "assets", max_slots=2, max_ctx=256)
    assert any(i.op == pk.Op.DSA_TOPK for i in eng.packet.programs[0].insts)
    state = {}
    for f in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        state.update(load_file(f))
    state = {k: v.float() for k, v in state.items()}
    spec = config.spec_from_config(cfg)
    ref = reference.ReferenceModel(spec, state)
    dense = reference.ReferenceModel(config.spec_from_config({**cfg, "index_n_heads": 0, "model_type": "deepseek_v3"}), state)
    rng = np.random.default_rng(2)
    p = rng.integers(0, 512, 150).tolist()
    eng.begin_slot(0, p)
    eng.reserve(0, len(p) + 4)
    r = eng.step(TokenBatch(np.asarray(p, np.int32), np.arange(len(p), dtype=np.int32), np.zeros(len(p), np.int32),
                            np.asarray([len(p) - 1], np.int32), want_logits=True))
    want = ref.forward(torch.tensor(p))[-1]
    err = (torch.from_numpy(r.logits[0]) - want).abs().max().item()
    assert err < 5e-4 * max(1.0, want.abs().max().item()), err
    assert (dense.forward(torch.tensor(p))[-1] - want).abs().max().item() > 50 * err      # sparse is not dense
    eng.commit(0, p)
    toks = list(p)
    nxt = int(want.argmax())
    for _ in range(2):
        r = eng.step(TokenBatch(np.asarray([nxt], np.int32), np.asarray([len(toks)], np.int32), np.zeros(1, np.int32), np.zeros(1, np.int32),
                                decode=True, want_logits=True))
        eng.commit(0, [nxt])
        toks.append(nxt)
        want = ref.forward(torch.tensor(toks))[-1]
        assert (torch.from_numpy(r.logits[0]) - want).abs().max().item() < 5e-4 * max(1.0, want.abs().max().item())
        nxt = int(want.argmax())
    eng.close()


def test_gdn_hybrid_model_on_cpu_backend_matches_reference(tmp_path):
    """Golden gated-delta-rule ops of the C++ interpreter (causal depthwise conv + SiLU, L2-normalised q / k, the state
    update, the gated per-head norm) and gated full attention ([Q | gate] query heads, partial rotary, (1 + gamma)
    norms) on a small hybrid MoE model: a prompt prefilled in two chunks with a second sequence packed beside it (the
    recurrent state is per slot and carried between steps), then decode, against the PyTorch fp32 reference."""
    import glob
    from safetensors.torch import load_file
    from plow_b200 import plowc
    from plow_b200.models import config, reference
    from plow_b200.runtime.engine import TokenBatch
    cfg = dict(model_type="qwen3_next", hidden_size=256, num_hidden_layers=4, full_attention_interval=4,
               num_attention_heads=4, num_key_value_heads=2, head_dim=64, partial_rotary_factor=0.25,
               linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=32, linear_value_head_dim=32,
               linear_conv_kernel_dim=4, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
               shared_expert_intermediate_size=64, norm_topk_prob=True, rms_norm_eps=1e-6, rope_theta=10000.0,
               vocab_size=512, tie_word_embeddings=False, max_position_embeddings=1024, eos_token_id=1,
               plow_dtype="f32", plow_kv_dtype="f32")
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=0)
    plowc.compile_dir(tmp_path / "ckpt", tmp_path / "assets", arch="cpu", n_cu=4, max_rows=128, decode_rungs=[1, 2, 4], max_seqs=4)
    eng = CpuEngine(tmp_path / "assets", max_slots=3, max_ctx=256)
    assert eng.has_recurrent_state and set(eng.state_arrays()) == {f"state.{i}.{k}" for i in (0, 1, 2) for k in ("conv", "ssm")}
    state = {}
    for f in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        state.update(load_file(f))
    ref = reference.ReferenceModel(config.spec_from_config(cfg), {k: v.float() for k, v in state.items()})
    rng = np.random.default_rng(2)
    pa, pb = rng.integers(0, 512, 90).tolist(), rng.integers(0, 512, 33).tolist()

    def close(got, want):
        return (torch.from_numpy(got) - want).abs().max().item() < 2e-4 * max(1.0, want.abs().max().item())
    # step 1: the first 50 tokens of A (slot 2) and all of B (slot 0) in one batch; step 2: the rest of A
    eng.begin_slot(2, pa)
    eng.begin_slot(0, pb)
    eng.reserve(2, len(pa) + 4)
    eng.reserve(0, len(pb) + 4)
    ids = pa[:50] + pb
    r = eng.step(TokenBatch(np.asarray(ids, np.int32), np.asarray(list(range(50)) + list(range(len(pb))), np.int32),
                            np.asarray([2] * 50 + [0] * len(pb), np.int32), np.asarray([49, len(ids) - 1], np.int32), want_logits=True))
    assert close(r.logits[0], ref.forward(torch.tensor(pa[:50]))[-1]) and close(r.logits[1], ref.forward(torch.tensor(pb))[-1])
    eng.commit(2, pa[:50])
    eng.commit(0, pb)
    r = eng.step(TokenBatch(np.asarray(pa[50:], np.int32), np.arange(50, len(pa), dtype=np.int32), np.full(len(pa) - 50, 2, np.int32),
                            np.asarray([len(pa) - 51], np.int32), want_logits=True))
    assert close(r.logits[0], ref.forward(torch.tensor(pa))[-1])
    eng.commit(2, pa[50:])
    # decode both sequences together for three steps
    cur = {2: list(pa), 0: list(pb)}
    for _ in range(3):
        nxt = {s: int(ref.forward(torch.tensor(c))[-1].argmax()) for s, c in cur.items()}
        slots = sorted(cur)
        r = eng.step(TokenBatch(np.asarray([nxt[s] for s in slots], np.int32), np.asarray([len(cur[s]) for s in slots], np.int32),
                                np.asarray(slots, np.int32), np.arange(2, dtype=np.int32), decode=True, want_logits=True))
        for k, s in enumerate(slots):
            cur[s].append(nxt[s])
            eng.commit(s, [nxt[s]])
            assert close(r.logits[k], ref.forward(torch.tensor(cur[s]))[-1])
    # a new sequence in a used slot starts from zero state (position 0 resets it)
    eng.retire_slot(0)
    eng.begin_slot(0, pa[:20])
    eng.reserve(0, 24)
    r = eng.step(TokenBatch(np.asarray(pa[:20], np.int32), np.arange(20, dtype=np.int32), np.zeros(20, np.int32),
                            np.asarray([19], np.int32), want_logits=True))
    assert close(r.logits[0], ref.forward(torch.tensor(pa[:20]))[-1])
    eng.close()


@pytest.mark.parametrize("model_type", ["qwen3_moe", "mixtral"])
def test_gqa_moe_families_on_cpu_backend_match_reference(tmp_path, model_type):
    """Grouped-query attention + routed MoE decoders: qwen3_moe (per-head q / k norm, experts under ``mlp`` named
    gate_proj / up_proj / down_proj, one dense layer through mlp_only_layers) and mixtral (experts under
    ``block_sparse_moe`` named w1 / w3 / w2, sliding window): prefill and decode logits against the fp32 reference."""
    import glob
    from safetensors.torch import load_file
    from plow_b200 import plowc
    from plow_b200.models import config, reference
    from plow_b200.runtime.engine import TokenBatch
    base = dict(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64, num_hidden_layers=3,
                num_experts_per_tok=2, rms_norm_eps=1e-6, rope_theta=10000.0, vocab_size=512, tie_word_embeddings=False,
                max_position_embeddings=1024, eos_token_id=1, plow_dtype="f32", plow_kv_dtype="f32")
    if model_type == "qwen3_moe":
        cfg = dict(base, model_type="qwen3_moe", num_experts=8, moe_intermediate_size=64, intermediate_size=384,
                   norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[1])
    else:
        cfg = dict(base, model_type="mixtral", num_local_experts=8, intermediate_size=96, sliding_window=48)
    spec = config.spec_from_config(cfg)
    assert spec.family == "gqa_moe" and [l.ffn.kind for l in spec.layers] == (["moe", "dense", "moe"] if model_type == "qwen3_moe" else ["moe"] * 3)
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=0)
    names = set(json.loads((tmp_path / "ckpt" / "model.safetensors.index.json").read_text())["weight_map"])
    assert ("model.layers.0.block_sparse_moe.experts.3.w3.weight" in names) == (model_type == "mixtral")
    assert ("model.layers.0.mlp.experts.3.up_proj.weight" in names) == (model_type == "qwen3_moe")
    plowc.compile_dir(tmp_path / "ckpt", tmp_path / "assets", arch="cpu", n_cu=4, max_rows=128, decode_rungs=[1, 2], max_seqs=4)
    eng = CpuEngine(tmp_path / "assets", max_slots=2, max_ctx=256)
    state = {}
    for f in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        state.update(load_file(f))
    ref = reference.ReferenceModel(spec, {k: v.float() for k, v in state.items()})
    rng = np.random.default_rng(4)
    p = rng.integers(0, 512, 80).tolist()                        # longer than the 48-token window
    eng.begin_slot(0, p)
    eng.reserve(0, len(p) + 4)
    r = eng.step(TokenBatch(np.asarray(p, np.int32), np.arange(len(p), dtype=np.int32), np.zeros(len(p), np.int32),
                            np.asarray([len(p) - 1], np.int32), want_logits=True))
    want = ref.forward(torch.tensor(p))[-1]
    assert (torch.from_numpy(r.logits[0]) - want).abs().max().item() < 2e-4 * max(1.0, want.abs().max().item())
    eng.commit(0, p)
    cur = list(p)
    for _ in range(2):
        nxt = int(ref.forward(torch.tensor(cur))[-1].argmax())
        r = eng.step(TokenBatch(np.asarray([nxt], np.int32), np.asarray([len(cur)], np.int32), np.zeros(1, np.int32), np.zeros(1, np.int32),
                                decode=True, want_logits=True))
        cur.append(nxt)
        eng.commit(0, [nxt])
        want = ref.forward(torch.tensor(cur))[-1]
        assert (torch.from_numpy(r.logits[0]) - want).abs().max().item() < 2e-4 * max(1.0, want.abs().max().item())
    eng.close()


def test_gelu_gated_model_runs_on_cpu_and_unsupported_shapes_are_refused(tmp_path):
    """A gemma-style decoder (GELU-tanh gate, (1 + gamma) norms, scaled embeddings, one kv head of width 128): the gate's
    activation travels as a flag of the fused GEMM (and of the GLU row op when the fusion is off) and the logits match the
    fp32 reference.  Model types whose layers this compiler would misread (gemma2, biased MLPs) and unknown activations are
    refused by name instead of being computed as something else."""
    import glob
    from safetensors.torch import load_file
    from plow_b200 import plowc
    from plow_b200.compiler import packet as pk
    from plow_b200.models import config, reference
    from plow_b200.runtime.engine import TokenBatch
    cfg = dict(model_type="gemma", hidden_size=256, num_attention_heads=4, num_key_value_heads=1, head_dim=128, num_hidden_layers=2,
               intermediate_size=512, hidden_act="gelu_pytorch_tanh", rms_norm_eps=1e-6, rope_theta=10000.0, vocab_size=512,
               tie_word_embeddings=True, max_position_embeddings=1024, eos_token_id=1, plow_dtype="f32", plow_kv_dtype="f32")
    spec = config.spec_from_config(cfg)
    assert spec.layers[0].ffn.act == "gelu_tanh" and spec.norm_plus_one and spec.embed_scale == 16.0
    for bad in (dict(cfg, model_type="gemma2"), dict(cfg, hidden_act="relu2"),
                dict(cfg, model_type="gemma", attention_bias=True), dict(cfg, model_type="llama", hidden_act="silu", mlp_bias=True),
                dict(cfg, model_type="qwen2", hidden_act="silu", use_sliding_window=True)):
        with pytest.raises(ValueError, match="not supported|unsupported"):
            config.spec_from_config(bad)
    with pytest.raises(ValueError, match="routed experts"):
        config.spec_from_config(dict(model_type="mixtral", hidden_size=64, num_attention_heads=2, num_hidden_layers=1, num_local_experts=4,
                                     num_experts_per_tok=2, intermediate_size=64, vocab_size=64, hidden_act="gelu"))
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=0)
    state = {}
    for f in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        state.update(load_file(f))
    state = {k: (v + 0.1 * torch.randn_like(v) if k.endswith("norm.weight") else v).float() for k, v in state.items()}     # (1 + gamma) with gamma != 0
    from safetensors.torch import save_file
    for f in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        save_file({k: state[k] for k in load_file(f)}, f)
    ref = reference.ReferenceModel(spec, state)
    p = np.random.default_rng(5).integers(0, 512, 60).tolist()
    want = ref.forward(torch.tensor(p))[-1]
    assert (want - reference.ReferenceModel(config.spec_from_config(dict(cfg, hidden_act="silu")), state).forward(torch.tensor(p))[-1]).abs().max() > 1e-3
    for out, kw in (("fused", {}), ("unfused", dict(disable_rules=("gated-mlp-fuse",)))):
        plowc.compile_dir(tmp_path / "ckpt", tmp_path / out, arch="cpu", n_cu=4, max_rows=128, decode_rungs=[1], max_seqs=4, **kw)
        pkt = pk.read_packet(tmp_path / out / "model.pkt")
        insts = pkt.programs[0].insts
        if out == "fused":
            assert any(i.op == pk.Op.GEMM and i.i[2] & pk.GEMM_ACT_GELU_TANH for i in insts)
        else:
            assert any(i.op == pk.Op.GLU and i.i[0] == pk.GEMM_ACT_GELU_TANH for i in insts)
        eng = CpuEngine(tmp_path / out, max_slots=2, max_ctx=256)
        eng.begin_slot(0, p)
        eng.reserve(0, 64)
        r = eng.step(TokenBatch(np.asarray(p, np.int32), np.arange(60, dtype=np.int32), np.zeros(60, np.int32), np.asarray([59], np.int32),
                                want_logits=True))
        eng.close()
        assert (torch.from_numpy(r.logits[0]) - want).abs().max().item() < 2e-4 * max(1.0, want.abs().max().item()), out


@pytest.mark.parametrize("mt", ["qwen2", "llama"])
def test_projection_biases_run_on_cpu(tmp_path, mt):
    """qwen2 (biases on q / k / v) and a llama-shaped model with attention_bias (o_proj too): the biases ride the fused qkv
    GEMM as a concatenated vector (flag + operand 7) and the output projection's GEMM; prefill and decode logits match the
    fp32 reference, which differs from the same weights without biases.  Also on the AVX-512 and AMX GEMM bodies."""
    import glob
    from safetensors.torch import load_file
    from plow_b200 import plowc
    from plow_b200.compiler import packet as pk
    from plow_b200.models import config, reference
    from plow_b200.ops import native
    from plow_b200.runtime.engine import TokenBatch
    cfg = dict(model_type=mt, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=2, intermediate_size=512,
               hidden_act="silu", rms_norm_eps=1e-6, rope_theta=10000.0, vocab_size=512, tie_word_embeddings=False,
               max_position_embeddings=1024, eos_token_id=1, plow_dtype="f32", plow_kv_dtype="f32")
    if mt == "llama":
        cfg["attention_bias"] = True
    spec = config.spec_from_config(cfg)
    assert spec.layers[0].attn.qkv_bias and spec.layers[0].attn.o_bias == (mt == "llama")
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=3)
    state = {}
    for f in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        state.update(load_file(f))
    nb = [k for k in state if k.endswith("proj.bias")]
    assert len(nb) == 2 * (4 if mt == "llama" else 3) and all(state[k].abs().max() > 0.1 for k in nb)
    ref = reference.ReferenceModel(spec, state)
    p = np.random.default_rng(7).integers(0, 512, 40).tolist()
    want = ref.forward(torch.tensor(p + [5]))
    nobias = reference.ReferenceModel(spec, {k: v for k, v in state.items() if k not in nb}).forward(torch.tensor(p))[-1]
    assert (want[len(p) - 1] - nobias).abs().max() > 1e-2
    plowc.compile_dir(tmp_path / "ckpt", tmp_path / "assets", arch="cpu", n_cu=4, max_rows=128, decode_rungs=[1], max_seqs=4)
    pkt = pk.read_packet(tmp_path / "assets" / "model.pkt")
    biased = [i for i in pkt.programs[0].insts if i.op == pk.Op.GEMM and i.i[2] & pk.GEMM_BIAS]
    assert len(biased) == 2 * (2 if mt == "llama" else 1) and all(i.t[7] != pk.T_NONE for i in biased)
    assert any(t.name.endswith("qkv_proj.bias") for t in pkt.tensors)
    lib = native.cpu_lib()
    start = lib.plow_cpu_tier()
    try:
        for tier, tol in ((0, 2e-4), (1, 2e-4), (2, 2e-4), (3, 5e-2)):
            if lib.plow_cpu_set_tier(tier) != tier:
                continue
            eng = CpuEngine(tmp_path / "assets", max_slots=2, max_ctx=256)
            eng.begin_slot(0, p)
            eng.reserve(0, 64)
            r = eng.step(TokenBatch(np.asarray(p, np.int32), np.arange(40, dtype=np.int32), np.zeros(40, np.int32), np.asarray([39], np.int32),
                                    want_logits=True))
            d = eng.step(TokenBatch(np.asarray([5], np.int32), np.asarray([40], np.int32), np.zeros(1, np.int32), np.asarray([0], np.int32),
                                    want_logits=True))
            eng.close()
            scale = max(1.0, want.abs().max().item())
            assert (torch.from_numpy(r.logits[0]) - want[39]).abs().max().item() < tol * scale, tier
            assert (torch.from_numpy(d.logits[0]) - want[40]).abs().max().item() < tol * scale, tier
    finally:
        lib.plow_cpu_set_tier(start)


@pytest.mark.parametrize("moe", [False, True])
def test_qwen3_5_hybrid_runs_on_cpu(tmp_path, moe):
    """qwen3_5 (dense MLPs) and qwen3_5_moe: the gated-delta-rule layers ship [q | k | v], z, b and a as four projections
    (stacked into the two operands of the recurrent op), the layer kinds come from layer_types, the rotary parameters are
    nested under rope_parameters.  Chunked prefill and decode match the fp32 reference; vision-tower configs are refused."""
    import glob
    from safetensors.torch import load_file
    from plow_b200 import plowc
    from plow_b200.models import config, reference
    from plow_b200.runtime.engine import TokenBatch
    cfg = dict(model_type="qwen3_5_moe" if moe else "qwen3_5", hidden_size=256, num_hidden_layers=4,
               layer_types=["linear_attention", "linear_attention", "full_attention", "linear_attention"],
               num_attention_heads=4, num_key_value_heads=2, head_dim=64, attn_output_gate=True, attention_bias=False,
               rope_parameters=dict(rope_theta=10000.0, partial_rotary_factor=0.25, rope_type="default", mrope_interleaved=False),
               linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=32, linear_value_head_dim=32,
               linear_conv_kernel_dim=4, intermediate_size=384, hidden_act="silu", rms_norm_eps=1e-6, vocab_size=512,
               tie_word_embeddings=False, max_position_embeddings=1024, eos_token_id=1, plow_dtype="f32", plow_kv_dtype="f32")
    if moe:
        cfg.update(num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, shared_expert_intermediate_size=64, norm_topk_prob=True)
    spec = config.spec_from_config(cfg)
    assert [l.attn.kind for l in spec.layers] == ["gdn", "gdn", "gqa", "gdn"] and spec.layers[0].attn.gdn_split_proj
    assert spec.layers[0].ffn.kind == ("moe" if moe else "dense") and spec.rope.rot_dim == 16 and spec.layers[2].attn.gated
    with pytest.raises(ValueError, match="vision tower"):
        config.spec_from_config(dict(cfg, vision_config={}))
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=4)
    state = {}
    for fn in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        state.update(load_file(fn))
    assert "model.layers.0.linear_attn.in_proj_qkv.weight" in state and "model.layers.0.linear_attn.in_proj_qkvz.weight" not in state
    ref = reference.ReferenceModel(spec, {k: v.float() for k, v in state.items()})
    p = np.random.default_rng(6).integers(0, 512, 70).tolist()
    want = ref.forward(torch.tensor(p + [3]))
    plowc.compile_dir(tmp_path / "ckpt", tmp_path / "assets", arch="cpu", n_cu=4, max_rows=128, decode_rungs=[1], max_seqs=4)
    eng = CpuEngine(tmp_path / "assets", max_slots=2, max_ctx=256)
    eng.begin_slot(0, p)
    eng.reserve(0, 80)
    for lo, hi in ((0, 40), (40, 70)):
        n = hi - lo
        r = eng.step(TokenBatch(np.asarray(p[lo:hi], np.int32), np.arange(lo, hi, dtype=np.int32), np.zeros(n, np.int32),
                                np.asarray([n - 1], np.int32), want_logits=True))
    d = eng.step(TokenBatch(np.asarray([3], np.int32), np.asarray([70], np.int32), np.zeros(1, np.int32), np.asarray([0], np.int32),
                            want_logits=True))
    eng.close()
    scale = max(1.0, want.abs().max().item())
    assert (torch.from_numpy(r.logits[0]) - want[69]).abs().max().item() < 3e-4 * scale
    assert (torch.from_numpy(d.logits[0]) - want[70]).abs().max().item() < 3e-4 * scale


@pytest.mark.parametrize("floor", [0.0, -5.0])
def test_kimi_linear_kda_hybrid_runs_on_cpu(tmp_path, floor):
    """kimi_linear: three Kimi Delta Attention layers (separate q / k / v short convolutions, per-channel forget gate from a
    low-rank projection — unbounded and, with gate_lower_bound, bounded —, delta-rule state, sigmoid-gated per-head norm) and
    one latent-attention layer without rotary embedding, dense first layer then a sigmoid-routed MoE with a shared expert.
    A chunked prefill (the state carries across steps) and a decode step match the fp32 reference."""
    import glob
    from safetensors.torch import load_file
    from plow_b200 import plowc
    from plow_b200.compiler import packet as pk
    from plow_b200.models import config, reference
    from plow_b200.runtime.engine import TokenBatch
    cfg = dict(model_type="kimi_linear", hidden_size=128, num_hidden_layers=4, num_attention_heads=4, kv_lora_rank=32, q_lora_rank=None,
               qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, mla_use_nope=True,
               linear_attn_config=dict(kda_layers=[1, 2, 3], full_attn_layers=[4], num_heads=4, head_dim=32, short_conv_kernel_size=4,
                                       gate_lower_bound=floor or None),
               intermediate_size=256, num_experts=8, num_experts_per_token=2, moe_intermediate_size=64, num_shared_experts=1,
               first_k_dense_replace=1, moe_router_activation_func="sigmoid", moe_renormalize=True, routed_scaling_factor=2.0,
               num_expert_group=1, topk_group=1, rms_norm_eps=1e-5, rope_theta=10000.0, vocab_size=512, tie_word_embeddings=False,
               max_position_embeddings=1024, eos_token_id=1, plow_dtype="f32", plow_kv_dtype="f32")
    spec = config.spec_from_config(cfg)
    assert [l.attn.kind for l in spec.layers] == ["kda", "kda", "kda", "mla"] and spec.layers[0].ffn.kind == "dense"
    assert spec.layers[1].ffn.block == "block_sparse_moe" and spec.rope.scaling["type"] == "nope" and spec.layers[0].attn.kda_gate_floor == floor
    with pytest.raises(ValueError, match="split the layers"):
        config.spec_from_config(dict(cfg, linear_attn_config=dict(cfg["linear_attn_config"], kda_layers=[1, 2])))
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=13)
    state = {}
    for fn in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        state.update(load_file(fn))
    assert state["model.layers.0.self_attn.A_log"].shape == (1, 1, 4, 1) and state["model.layers.0.self_attn.q_conv1d.weight"].shape == (128, 1, 4)
    ref = reference.ReferenceModel(spec, state)
    p = np.random.default_rng(3).integers(0, 512, 45).tolist()
    want = ref.forward(torch.tensor(p + [9]))
    plowc.compile_dir(tmp_path / "ckpt", tmp_path / "assets", arch="cpu", n_cu=4, max_rows=128, decode_rungs=[1], max_seqs=4)
    pkt = pk.read_packet(tmp_path / "assets" / "model.pkt")
    steps = [i for i in pkt.programs[0].insts if i.op == pk.Op.GDN_STEP]
    assert len(steps) == 3 and all(i.i[4] == 1 and i.f[0] == floor for i in steps)
    assert "recurrent_state" in pkt.sections
    eng = CpuEngine(tmp_path / "assets", max_slots=2, max_ctx=256)
    assert eng.has_recurrent_state
    eng.begin_slot(0, p)
    eng.reserve(0, 64)
    for lo, hi in ((0, 30), (30, 45)):          # two prefill chunks: conv windows and the delta-rule state carry over
        n = hi - lo
        r = eng.step(TokenBatch(np.asarray(p[lo:hi], np.int32), np.arange(lo, hi, dtype=np.int32), np.zeros(n, np.int32),
                                np.asarray([n - 1], np.int32), want_logits=True))
    d = eng.step(TokenBatch(np.asarray([9], np.int32), np.asarray([45], np.int32), np.zeros(1, np.int32), np.asarray([0], np.int32),
                            want_logits=True))
    eng.close()
    scale = max(1.0, want.abs().max().item())
    assert (torch.from_numpy(r.logits[0]) - want[44]).abs().max().item() < 3e-4 * scale
    assert (torch.from_numpy(d.logits[0]) - want[45]).abs().max().item() < 3e-4 * scale


def test_gpt_oss_runs_on_cpu(tmp_path):
    """gpt_oss: biased q / k / v / o projections, per-head attention sinks, a sliding-window layer beside a full one, YaRN
    tables without truncation, a biased router with softmax over the chosen experts, and experts stored as one tensor per
    projection (interleaved gate / up columns) with biases and the clamped GLU.  Prefill beyond the window and a decode
    step match the fp32 reference; dropping the sinks or the clamp changes the reference, so the test sees both."""
    import glob
    from safetensors.torch import load_file
    from plow_b200 import plowc
    from plow_b200.compiler import packet as pk
    from plow_b200.models import config, reference
    from plow_b200.runtime.engine import TokenBatch
    cfg = dict(model_type="gpt_oss", hidden_size=128, num_attention_heads=8, num_key_value_heads=2, head_dim=32, num_hidden_layers=2,
               layer_types=["sliding_attention", "full_attention"], sliding_window=16, num_local_experts=8, num_experts_per_tok=2,
               intermediate_size=64, swiglu_limit=1.0, rms_norm_eps=1e-5, rope_theta=150000.0, vocab_size=512, tie_word_embeddings=False,
               rope_scaling=dict(rope_type="yarn", factor=32.0, beta_fast=32.0, beta_slow=1.0, original_max_position_embeddings=64,
                                 truncate=False),
               max_position_embeddings=2048, eos_token_id=1, plow_dtype="f32", plow_kv_dtype="f32")
    spec = config.spec_from_config(cfg)
    a0, a1, f = spec.layers[0].attn, spec.layers[1].attn, spec.layers[0].ffn
    assert a0.window == 16 and a1.window == 0 and a0.sinks and a0.o_bias and f.fused_experts and f.swiglu_limit == 1.0
    with pytest.raises(ValueError, match="quantization"):
        config.spec_from_config(dict(cfg, quantization_config=dict(quant_method="awq")))
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=11)
    state = {}
    for fn in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        state.update(load_file(fn))
    # expert weights large enough that the clamp at 1.0 bites
    from safetensors.torch import save_file
    state = {k: (v * 20 if k.endswith("experts.gate_up_proj") else v) for k, v in state.items()}
    for fn in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        save_file({k: state[k].contiguous() for k in load_file(fn)}, fn)
    ref = reference.ReferenceModel(spec, state)
    p = np.random.default_rng(9).integers(0, 512, 50).tolist()
    want = ref.forward(torch.tensor(p + [7]))
    import copy
    nosink = copy.deepcopy(spec)
    for l in nosink.layers:
        l.attn.sinks = False
    noclamp = copy.deepcopy(spec)
    for l in noclamp.layers:
        l.ffn.swiglu_limit = 1e9
    for other in (nosink, noclamp):
        assert (reference.ReferenceModel(other, state).forward(torch.tensor(p))[-1] - want[49]).abs().max() > 1e-3
    plowc.compile_dir(tmp_path / "ckpt", tmp_path / "assets", arch="cpu", n_cu=4, max_rows=128, decode_rungs=[1], max_seqs=4)
    pkt = pk.read_packet(tmp_path / "assets" / "model.pkt")
    insts = pkt.programs[0].insts
    assert all(i.t[5] != pk.T_NONE for i in insts if i.op == pk.Op.ATTN)
    assert all(i.t[6] != pk.T_NONE and i.t[7] != pk.T_NONE and i.f[0] == 1.0 for i in insts if i.op == pk.Op.MOE_GEMM)
    assert sorted(i.i[3] for i in insts if i.op == pk.Op.ATTN) == [0, 16]
    eng = CpuEngine(tmp_path / "assets", max_slots=2, max_ctx=256)
    eng.begin_slot(0, p)
    eng.reserve(0, 64)
    r = eng.step(TokenBatch(np.asarray(p, np.int32), np.arange(50, dtype=np.int32), np.zeros(50, np.int32), np.asarray([49], np.int32),
                            want_logits=True))
    d = eng.step(TokenBatch(np.asarray([7], np.int32), np.asarray([50], np.int32), np.zeros(1, np.int32), np.asarray([0], np.int32),
                            want_logits=True))
    eng.close()
    scale = max(1.0, want.abs().max().item())
    assert (torch.from_numpy(r.logits[0]) - want[49]).abs().max().item() < 2e-4 * scale
    assert (torch.from_numpy(d.logits[0]) - want[50]).abs().max().item() < 2e-4 * scale


def test_gpt_oss_mxfp4_expert_blocks_are_dequantised_at_load(tmp_path):
    """The original gpt_oss release stores the experts as fp4 (e2m1) blocks of the transposed matrices with one E8M0 scale
    per 32 values.  The codec round-trips its own code points exactly; a checkpoint rewritten into that form compiles and
    the CPU engine matches the fp32 reference run on the dequantised weights."""
    import glob
    import json
    from safetensors.torch import load_file, save_file
    from plow_b200 import plowc
    from plow_b200.models import config, reference
    from plow_b200.runtime import weights
    from plow_b200.runtime.engine import TokenBatch
    g = torch.Generator().manual_seed(0)
    codes = torch.randint(0, 16, (3, 5, 64), generator=g)
    exact = torch.tensor(weights.FP4_VALUES)[codes] * torch.tensor([0.25, 1.0, 8.0])[:, None, None]
    exact[..., 0] = 6.0 * torch.tensor([0.25, 1.0, 8.0])[:, None]                    # pin each group's scale
    exact[..., 32] = 6.0 * torch.tensor([0.25, 1.0, 8.0])[:, None]
    b, s = weights.quant_mxfp4(exact)
    assert b.shape == (3, 5, 2, 16) and s.shape == (3, 5, 2) and torch.equal(weights.dequant_mxfp4(b, s, torch.float32), exact)
    cfg = dict(model_type="gpt_oss", hidden_size=128, num_attention_heads=8, num_key_value_heads=2, head_dim=32, num_hidden_layers=2,
               layer_types=["sliding_attention", "full_attention"], sliding_window=16, num_local_experts=4, num_experts_per_tok=2,
               intermediate_size=64, swiglu_limit=7.0, rms_norm_eps=1e-5, rope_theta=150000.0, vocab_size=512, tie_word_embeddings=False,
               max_position_embeddings=2048, eos_token_id=1, plow_dtype="f32", plow_kv_dtype="f32",
               quantization_config=dict(quant_method="mxfp4", modules_to_not_convert=["model.layers.*.self_attn", "model.layers.*.mlp.router"]))
    spec = config.spec_from_config(cfg)
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=21)
    state, deq = {}, {}
    for fn in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        state.update(load_file(fn))
    packed = {}
    for k, v in state.items():
        if k.endswith("experts.gate_up_proj") or k.endswith("experts.down_proj"):
            blocks, scales = weights.quant_mxfp4(v.transpose(1, 2).contiguous())      # stored transposed: [E, out, in]
            packed[k + "_blocks"], packed[k + "_scales"] = blocks, scales
            deq[k] = weights.dequant_mxfp4(blocks, scales, torch.float32).transpose(1, 2).contiguous()
            assert (deq[k] - v).abs().max() < 0.3 * v.abs().max() and not torch.equal(deq[k], v)
        else:
            packed[k] = deq[k] = v
    for fn in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        __import__("os").remove(fn)
    idx = tmp_path / "ckpt" / "model.safetensors.index.json"
    if idx.exists():
        idx.unlink()
    save_file({k: v.contiguous() for k, v in packed.items()}, str(tmp_path / "ckpt" / "model.safetensors"))
    ref = reference.ReferenceModel(spec, deq)
    p = np.random.default_rng(4).integers(0, 512, 30).tolist()
    want = ref.forward(torch.tensor(p))[-1]
    plowc.compile_dir(tmp_path / "ckpt", tmp_path / "assets", arch="cpu", n_cu=4, max_rows=128, decode_rungs=[1], max_seqs=4)
    eng = CpuEngine(tmp_path / "assets", max_slots=2, max_ctx=256)
    eng.begin_slot(0, p)
    eng.reserve(0, 40)
    r = eng.step(TokenBatch(np.asarray(p, np.int32), np.arange(30, dtype=np.int32), np.zeros(30, np.int32), np.asarray([29], np.int32),
                            want_logits=True))
    eng.close()
    assert (torch.from_numpy(r.logits[0]) - want).abs().max().item() < 2e-4 * max(1.0, want.abs().max().item())


def test_mla_under_yarn_scales_its_softmax(tmp_path):
    """A YaRN-extended MLA checkpoint multiplies the softmax scale by mscale(factor, mscale_all_dim)^2 (1.87 for factor 40):
    the compiled attention carries it and the CPU engine matches the reference, which differs from the unscaled model."""
    import glob
    import math
    from safetensors.torch import load_file
    from plow_b200 import plowc
    from plow_b200.compiler import packet as pk
    from plow_b200.models import config, reference
    from plow_b200.runtime.engine import TokenBatch
    from plow_b200.utils.rope import mla_softmax_factor
    yarn = dict(type="yarn", factor=40.0, original_max_position_embeddings=64, beta_fast=32, beta_slow=1, mscale=1.0, mscale_all_dim=1.0)
    assert mla_softmax_factor(yarn) == pytest.approx((0.1 * math.log(40.0) + 1.0) ** 2) and mla_softmax_factor(None) == 1.0
    assert mla_softmax_factor(dict(yarn, mscale_all_dim=0)) == 1.0 and mla_softmax_factor(dict(type="llama3", factor=8.0)) == 1.0
    cfg = dict(model_type="deepseek_v3", hidden_size=256, num_attention_heads=4, num_hidden_layers=2,
               q_lora_rank=64, kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
               intermediate_size=512, first_k_dense_replace=2, n_routed_experts=0, rms_norm_eps=1e-6,
               rope_theta=10000.0, rope_scaling=yarn, vocab_size=512, tie_word_embeddings=False, max_position_embeddings=1024,
               eos_token_id=1, plow_dtype="f32", plow_kv_dtype="f32")
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=0)
    plowc.compile_dir(tmp_path / "ckpt", tmp_path / "assets", arch="cpu", n_cu=4, max_rows=128, decode_rungs=[1], max_seqs=4)
    pkt = pk.read_packet(tmp_path / "assets" / "model.pkt")
    scales = {round(i.f[0], 5) for p in pkt.programs for i in p.insts if i.op in (pk.Op.MLA_PREFILL, pk.Op.MLA_DECODE)}
    assert scales == {round(24 ** -0.5 * mla_softmax_factor(yarn), 5)}
    state = {}
    for f in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        state.update(load_file(f))
    state = {k: v.float() * (8.0 if "q_b_proj" in k or "kv_b_proj" in k else 1.0) for k, v in state.items()}     # logits large enough to matter
    from safetensors.torch import save_file
    for f in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        save_file({k: state[k] for k in load_file(f)}, f)
    ref = reference.ReferenceModel(config.spec_from_config(cfg), state)
    plain = reference.ReferenceModel(config.spec_from_config({k: v for k, v in cfg.items() if k != "rope_scaling"}), state)
    p = np.random.default_rng(8).integers(0, 512, 90).tolist()
    want = ref.forward(torch.tensor(p))[-1]
    assert (want - plain.forward(torch.tensor(p))[-1]).abs().max() > 1e-4
    eng = CpuEngine(tmp_path / "assets", max_slots=2, max_ctx=256)
    eng.begin_slot(0, p)
    eng.reserve(0, 96)
    r = eng.step(TokenBatch(np.asarray(p, np.int32), np.arange(90, dtype=np.int32), np.zeros(90, np.int32), np.asarray([89], np.int32), want_logits=True))
    eng.close()
    assert (torch.from_numpy(r.logits[0]) - want).abs().max().item() < 2e-4 * max(1.0, want.abs().max().item())
    with pytest.raises(ValueError, match="topk_method"):
        config.spec_from_config(dict(cfg, n_routed_experts=8, num_experts_per_tok=2, moe_intermediate_size=32, n_group=2, topk_group=1,
                                     topk_method="group_limited_greedy", first_k_dense_replace=0))


def test_gemma3_text_model_on_cpu_backend_matches_reference(tmp_path):
    """Gemma 3 text decoder: four (1 + gamma) norms per layer, per-head q / k norms, GELU-tanh gate, scaled embeddings,
    softmax scale from query_pre_attn_scalar, two sliding-window layers with the local rotary base for every global layer
    (global base with linear scaling): a prompt longer than the window, prefill and decode, against the fp32 reference."""
    import glob
    from safetensors.torch import load_file, save_file
    from plow_b200 import plowc
    from plow_b200.compiler import packet as pk
    from plow_b200.models import config, reference
    from plow_b200.runtime.engine import TokenBatch
    cfg = dict(model_type="gemma3_text", hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64, num_hidden_layers=6,
               intermediate_size=512, hidden_activation="gelu_pytorch_tanh", rms_norm_eps=1e-6, rope_theta=1000000.0,
               rope_local_base_freq=10000.0, rope_scaling=dict(rope_type="linear", factor=8.0), sliding_window=32, sliding_window_pattern=3,
               query_pre_attn_scalar=128, vocab_size=512, max_position_embeddings=1024, eos_token_id=1, plow_dtype="f32", plow_kv_dtype="f32")
    spec = config.spec_from_config(cfg)
    assert spec.sandwich_norms and spec.norm_plus_one and spec.tie_embeddings and spec.embed_scale == 16.0
    assert [l.attn.window for l in spec.layers] == [32, 32, 0, 32, 32, 0] and spec.layers[0].attn.rope_theta == 10000.0
    assert spec.layers[2].attn.rope_theta == 0.0 and spec.layers[0].attn.scale == pytest.approx(128 ** -0.5)
    wrapped = config.spec_from_config(dict(model_type="gemma3", text_config=cfg))        # the multimodal wrapper's text part
    assert wrapped.n_layers == 6 and wrapped.sandwich_norms
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=0)
    state = {}
    for f in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        state.update(load_file(f))
    assert "model.layers.3.pre_feedforward_layernorm.weight" in state and "model.layers.3.post_feedforward_layernorm.weight" in state
    state = {k: (v + 0.1 * torch.randn_like(v) if k.endswith("norm.weight") else v).float() for k, v in state.items()}
    for f in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        save_file({k: state[k] for k in load_file(f)}, f)
    ref = reference.ReferenceModel(spec, state)
    plowc.compile_dir(tmp_path / "ckpt", tmp_path / "assets", arch="cpu", n_cu=4, max_rows=128, decode_rungs=[1], max_seqs=4)
    pkt = pk.read_packet(tmp_path / "assets" / "model.pkt")
    gens = {t.name for t in pkt.tensors if t.tclass == pk.TClass.GEN}
    assert gens == {"gen.rope", "gen.rope.local"}
    assert {i.i[3] for i in pkt.programs[0].insts if i.op == pk.Op.ATTN} == {0, 32}
    p = np.random.default_rng(6).integers(0, 512, 90).tolist()
    eng = CpuEngine(tmp_path / "assets", max_slots=2, max_ctx=256)
    eng.begin_slot(0, p)
    eng.reserve(0, 96)
    r = eng.step(TokenBatch(np.asarray(p, np.int32), np.arange(90, dtype=np.int32), np.zeros(90, np.int32), np.asarray([89], np.int32), want_logits=True))
    want = ref.forward(torch.tensor(p))[-1]
    assert (torch.from_numpy(r.logits[0]) - want).abs().max().item() < 3e-4 * max(1.0, want.abs().max().item())
    eng.commit(0, p)
    cur = list(p)
    for _ in range(2):
        nxt = int(ref.forward(torch.tensor(cur))[-1].argmax())
        r = eng.step(TokenBatch(np.asarray([nxt], np.int32), np.asarray([len(cur)], np.int32), np.zeros(1, np.int32), np.zeros(1, np.int32),
                                decode=True, want_logits=True))
        cur.append(nxt)
        eng.commit(0, [nxt])
        want = ref.forward(torch.tensor(cur))[-1]
        assert (torch.from_numpy(r.logits[0]) - want).abs().max().item() < 3e-4 * max(1.0, want.abs().max().item())
    eng.close()
