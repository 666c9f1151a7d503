"""Prediction-module (MTP) drafter on the CPU backend: the drafter packet (`plowc --mtp`) against the fp32 reference's
``mtp_forward``, the chain of drafts, and speculative decoding through it (library call and scheduler).  Reference:
crates/devgen/src/mtp.rs, crates/plowrt/src/exec/gpu/spec.rs:1-12."""
import glob

import numpy as np
import pytest
import torch

from plow_b200.runtime.cpu_engine import CpuEngine
from plow_b200.runtime.engine import TokenBatch
from plow_b200.runtime.spec import MtpDrafter, SpecStats, spec_decode

MLA_MOE = dict(model_type="deepseek_v3", hidden_size=256, num_attention_heads=4, num_hidden_layers=2,
               q_lora_rank=64, kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
               intermediate_size=512, first_k_dense_replace=1, n_routed_experts=8, n_shared_experts=1,
               num_experts_per_tok=2, moe_intermediate_size=64, n_group=2, topk_group=1, scoring_func="sigmoid",
               norm_topk_prob=True, routed_scaling_factor=2.5, topk_method="noaux_tc", rms_norm_eps=1e-6,
               rope_theta=10000.0, vocab_size=512, tie_word_embeddings=False, max_position_embeddings=1024, eos_token_id=1,
               plow_dtype="f32", plow_kv_dtype="f32", num_nextn_predict_layers=1)


def _build(tmp, cfg):
    from safetensors.torch import load_file
    from plow_b200 import plowc
    from plow_b200.models import config, reference
    reference.write_checkpoint(cfg, tmp / "ckpt", seed=0)
    rep = plowc.compile_dir(tmp / "ckpt", tmp / "assets", arch="cpu", n_cu=4, max_rows=128, decode_rungs=[1, 2, 4, 8], max_seqs=8,
                            mtp=True)
    assert rep["mtp"]["ranks"][0]["verify"]["ok"] and (tmp / "assets" / "mtp" / "model.pkt").exists()
    from plow_b200.compiler import packet as pk
    main_s = pk.read_packet(tmp / "assets" / "model.pkt").section_json("spec.json")
    draft_s = pk.read_packet(tmp / "assets" / "mtp" / "model.pkt").section_json("spec.json")
    assert main_s["kind"] == "mtp" and main_s["drafter_packet"] == "mtp/model.pkt" and main_s["hidden_rows"] == "rows"
    assert draft_s["role"] == "mtp" and draft_s["hidden_rows"] == "samples" and draft_s["module_layer"] == main_s["module_layer"] == cfg["num_hidden_layers"]
    state = {}
    for f in glob.glob(str(tmp / "ckpt" / "*.safetensors")):
        state.update(load_file(f))
    return reference.ReferenceModel(config.spec_from_config(cfg), {k: v.float() for k, v in state.items()})


def _prefill(eng, slot, prompt, hidden=None):
    n = len(prompt)
    eng.reserve(slot, n + 1)
    return eng.step(TokenBatch(np.asarray(prompt, np.int32), np.arange(n, dtype=np.int32), np.full(n, slot, np.int32),
                               np.asarray([n - 1], np.int32), want_logits=True, want_hidden=True, hidden=hidden))


def _ref_chain(ref, prompt, pending, k):
    """k drafts of the reference: the module over the decoder's hidden states, then over its own."""
    _, h = ref.forward_hidden(torch.tensor(prompt))
    nxt = torch.tensor(prompt[1:] + [pending])
    out = []
    for _ in range(k):
        lg, g = ref.mtp_forward(nxt, h)
        out.append(int(lg[-1].argmax()))
        h, nxt = torch.cat([h, g[-1:]]), torch.cat([nxt, torch.tensor([out[-1]])])
    return out


@pytest.mark.parametrize("family", ["dense", "mla_moe"])
def test_drafter_packet_matches_the_reference_module(tmp_path, family):
    from plow_b200.models import config
    cfg = dict(config.tiny_dense_config(), num_nextn_predict_layers=1) if family == "dense" else MLA_MOE
    ref = _build(tmp_path, cfg)
    main = CpuEngine(tmp_path / "assets", max_slots=2, max_ctx=256)
    dr = CpuEngine(tmp_path / "assets" / "mtp", max_slots=2, max_ctx=256, prefix_cache=False)
    assert dr.spec.role == "mtp" and dr.spec.n_layers == 1 and dr.spec.name_base == cfg["num_hidden_layers"]
    rng = np.random.default_rng(3)
    prompt = rng.integers(0, cfg["vocab_size"], 40).tolist()
    main.begin_slot(0, prompt)
    r = _prefill(main, 0, prompt)
    main.commit(0, prompt)
    lg, h = ref.forward_hidden(torch.tensor(prompt))
    assert r.hidden.shape == (40, cfg["hidden_size"])
    assert np.abs(r.hidden - h.numpy()).max() < 1e-4                     # the decoder's out.hidden: every row, after the final norm
    pending = int(r.ids[0])
    assert pending == int(lg[-1].argmax())
    # the module over the whole prompt: logits and hidden state of the last row
    dr.begin_slot(0, [])
    r2 = _prefill(dr, 0, prompt[1:] + [pending], hidden=r.hidden)
    l2, g = ref.mtp_forward(torch.tensor(prompt[1:] + [pending]), h)
    assert np.abs(r2.logits[0] - l2[-1].numpy()).max() < 2e-4 * max(1.0, float(l2[-1].abs().max()))
    assert np.abs(r2.hidden[0] - g[-1].numpy()).max() < 1e-4 and r2.hidden.shape == (1, cfg["hidden_size"])
    dr.retire_slot(0)
    # the chain drafter: first draft from the decoder's states, the next ones from the module's own
    d = MtpDrafter(dr)
    d.begin(0)
    d.observe([(0, 0, prompt[1:] + [pending], r.hidden)])
    assert d.synced(0, len(prompt))
    assert d.propose_many([0], 3)[0] == _ref_chain(ref, prompt, pending, 3)
    d.retire(0)
    # speculative decoding through it is plain greedy decoding
    plain = [pending]
    for _ in range(11):
        plain.append(int(ref.forward(torch.tensor(prompt + plain))[-1].argmax()))
    stats = SpecStats()
    got = spec_decode(main, 0, pending, 12, d, depth=3, stats=stats, prefill_hidden=r.hidden)
    assert got == plain and stats.proposed >= stats.steps          # a model drafter always has a draft
    assert 0 not in dr.tokens                                      # its slot went back
    main.close()
    dr.close()


def test_accepted_spans_keep_the_drafter_in_step(tmp_path):
    """An oracle that drafts the decoder's true continuation makes every verify step accept its whole span; the module
    then observes several rows per step (accepted drafts + the new pending token) and its next first draft must still be
    what the reference module predicts at that point."""
    from plow_b200.models import config
    cfg = dict(config.tiny_dense_config(), num_nextn_predict_layers=1)
    ref = _build(tmp_path, cfg)
    main = CpuEngine(tmp_path / "assets", max_slots=2, max_ctx=256)
    dr = CpuEngine(tmp_path / "assets" / "mtp", max_slots=2, max_ctx=256, prefix_cache=False)
    rng = np.random.default_rng(4)
    prompt = rng.integers(0, 32000, 30).tolist()
    main.begin_slot(0, prompt)
    r = _prefill(main, 0, prompt)
    main.commit(0, prompt)
    pending = int(r.ids[0])
    truth = [pending]
    for _ in range(12):
        truth.append(int(ref.forward(torch.tensor(prompt + truth))[-1].argmax()))
    firsts = []

    class Oracle(MtpDrafter):
        def propose_many(self, slots, k):
            n = len(main.tokens[0])                       # committed tokens; the pending one is truth[n - len(prompt)]
            firsts.append((n, self.first[0][0]))
            at = n - len(prompt) + 1
            return {0: truth[at:at + k]}

    d = Oracle(dr)
    stats = SpecStats()
    got = spec_decode(main, 0, pending, 10, d, depth=3, stats=stats, prefill_hidden=r.hidden)
    assert got == truth[:10]
    assert stats.accepted == stats.proposed and stats.steps <= 4     # whole spans accepted: 1 + 3 tokens per step
    for n, first in firsts:
        # the module's own first draft at that point = reference module over the n committed tokens + pending
        seq = (prompt + truth)[:n + 1]
        assert first == _ref_chain(ref, seq[:-1], seq[-1], 1)[0]
    main.close()
    dr.close()


def test_scheduler_drafts_with_the_prediction_module(tmp_path):
    """ModelMux with spec_depth > 0 and a MtpDrafter: prefill chunks, verify steps and plain decode steps feed the module
    the decoder's hidden states; the tokens equal plain decoding; a request whose prompt is found in the prefix cache
    (no hidden states for the cached part) falls back to prompt lookup instead of drafting from a cache with a hole."""
    from plow_b200.models import config
    from plow_b200.runtime.scheduler import GenParams, ModelMux, SchedConfig
    from plow_b200.text.tokenizer import ByteTokenizer
    cfg = dict(config.tiny_dense_config(), num_nextn_predict_layers=1)
    _build(tmp_path, cfg)
    rng = np.random.default_rng(6)
    prompts = [rng.integers(0, 32000, n).tolist() for n in (150, 40)]        # 150 rows: two prefill chunks of the 128-row bucket

    def run(depth, again=False):
        eng = CpuEngine(tmp_path / "assets", max_slots=2, max_ctx=512, prefix_cache=again)
        mux = ModelMux(eng, ByteTokenizer(), SchedConfig(token_budget=128, spec_depth=depth), eos_ids=[])
        dr = None
        if depth:
            dr = CpuEngine(tmp_path / "assets" / "mtp", max_slots=2, max_ctx=512, prefix_cache=False)
            mux.set_drafter(MtpDrafter(dr))
        outs = []
        for rnd in range(2 if again else 1):
            reqs = [mux.submit(p, GenParams(max_tokens=10)) for p in prompts]
            for _ in range(200):
                if not mux.tick() and not mux.live and not mux.waiting:
                    break
            for r in reqs:
                ids = []
                while True:
                    ch = r.out.get(timeout=10)
                    if ch.kind == "token":
                        ids.append(ch.token_id)
                    else:
                        assert ch.kind == "done", ch.error
                        break
                outs.append(ids)
        c = mux.metrics.snapshot()["counters"]
        left = dict(dr.tokens) if dr else {}
        eng.close()
        if dr:
            dr.close()
        return outs, c, left
    plain, c0, _ = run(0)
    spec, c1, left = run(3)
    assert plain == spec and all(len(t) == 10 for t in spec)
    assert c1["spec_ticks"] >= 1 and c1["spec_proposed"] >= 3 * c1["spec_ticks"]      # every request drafted to full depth
    assert left == {}                                                                 # finished requests gave the drafter's slots back
    twice, c2, left = run(3, again=True)
    assert twice[:2] == plain and twice[2:] == plain and left == {}


@pytest.mark.parametrize("n_pages", [48, 6])
def test_randomised_workload_with_the_drafter_keeps_every_invariant(tmp_path, n_pages):
    """Nine requests of mixed lengths against four slots (and, with 6 pages, against a KV pool that holds two long prompts at most): with the
    prediction-module drafter on, tokens equal the plain run, every request ends once, and both engines get all their
    slots and pages back."""
    from plow_b200.models import config
    from plow_b200.runtime.scheduler import GenParams, ModelMux, SchedConfig
    from plow_b200.text.tokenizer import ByteTokenizer
    cfg = dict(config.tiny_dense_config(), num_nextn_predict_layers=1)
    _build(tmp_path, cfg)
    rng = np.random.default_rng(11)
    plan = sorted(((int(rng.integers(0, 20)), rng.integers(0, 32000, int(rng.integers(8, 150))).tolist(), int(rng.integers(2, 12)))
                   for _ in range(9)), key=lambda x: x[0])

    def run(depth):
        eng = CpuEngine(tmp_path / "assets", max_slots=4, max_ctx=512, n_pages=n_pages, prefix_cache=False)
        mux = ModelMux(eng, ByteTokenizer(), SchedConfig(token_budget=128, reserve_tokens=0, spec_depth=depth), eos_ids=[])
        dr = None
        if depth:
            dr = CpuEngine(tmp_path / "assets" / "mtp", max_slots=4, max_ctx=512, n_pages=n_pages, prefix_cache=False)
            mux.set_drafter(MtpDrafter(dr))
        pending, reqs = list(plan), []
        for t in range(4000):
            while pending and pending[0][0] <= t:
                _, p, mx = pending.pop(0)
                reqs.append(mux.submit(p, GenParams(max_tokens=mx)))
            if not mux.tick() and not pending and not mux.live and not mux.waiting:
                break
        outs = []
        for r in reqs:
            toks, done = [], 0
            while not r.out.empty():
                c = r.out.get_nowait()
                if c.kind == "token":
                    toks.append(c.token_id)
                else:
                    assert c.kind == "done" and c.finish_reason == "length", (c.kind, c.error)
                    done += 1
            assert done == 1
            outs.append(toks)
        for e in (eng, dr):
            if e is not None:
                assert not e.tokens and sum(len(s.pages) for s in e.pool.seqs.values()) == 0 and e.pool.available() == n_pages
                e.close()
        return outs, mux.metrics.snapshot()["counters"]
    plain, c0 = run(0)
    spec, c1 = run(3)
    assert plain == spec and [len(t) for t in spec] == [mx for _, _, mx in plan]
    assert c1.get("spec_ticks", 0) >= 3


def test_plowrt_pairs_the_drafter_through_the_packets_spec_section(tmp_path):
    """`plowrt serve --spec-depth N` on assets compiled with `plowc --mtp`: the entry opens the drafter packet named by the
    main packet's spec.json in an engine of its own and the scheduler drafts with it; `--spec-drafter ngram` keeps prompt
    lookup, and asking for mtp without a drafter packet is an error."""
    from plow_b200 import config as cfgmod, plowrt
    from plow_b200.models import config
    from plow_b200.runtime.scheduler import GenParams
    _build(tmp_path, dict(config.tiny_dense_config(), num_nextn_predict_layers=1))
    base = dict(backend="cpu", max_slots=2, max_ctx=256, spec_depth=3)
    entry = plowrt.make_entry("tiny", tmp_path / "assets", cfgmod.RuntimeConfig.load(cli=base, env={}))
    try:
        d = entry.mux._drafter
        assert isinstance(d, MtpDrafter) and d.eng.spec.role == "mtp" and d.eng.pool.enable_prefix is False
        toks = entry.mux.generate(list(range(3, 40)), GenParams(max_tokens=6))[0]
        assert len(toks) == 6 and entry.mux.metrics.snapshot()["counters"].get("spec_ticks", 0) >= 1
    finally:
        entry.mux.stop()
    plain = plowrt.make_entry("tiny", tmp_path / "assets", cfgmod.RuntimeConfig.load(cli=dict(base, spec_drafter="ngram"), env={}))
    try:
        assert not isinstance(getattr(plain.mux, "_drafter", None), MtpDrafter)
        assert plain.mux.generate(list(range(3, 40)), GenParams(max_tokens=6))[0] == toks
    finally:
        plain.mux.stop()
    import shutil
    shutil.rmtree(tmp_path / "assets" / "mtp")
    with pytest.raises(SystemExit):
        plowrt.make_entry("tiny", tmp_path / "assets", cfgmod.RuntimeConfig.load(cli=dict(base, spec_drafter="mtp"), env={}))
