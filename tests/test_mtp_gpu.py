"""Prediction-module (MTP) drafter on the sm_100a engine: a small MLA + MoE checkpoint with one prediction module, e4m3
weights and latent cache.  The decoder's ``out.hidden`` and the drafter packet's logits are compared with the fp32
reference over the same (quantise-dequantised) weights; speculative decoding through the chain drafter must give the
engine's own greedy tokens, from the library call and from the scheduler."""
import glob

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rt(w):
    from plow_b200.ops import quant
    q, s = quant.quant_weight_128x128(w.float().cuda())
    return quant.dequant_weight_128x128(q, s).cpu()


@pytest.fixture(scope="module")
def mtp_assets(tmp_path_factory):
    from plow_b200 import plowc
    from plow_b200.models import reference
    from plow_b200.runtime.smoke import small_mla_moe_config
    d = tmp_path_factory.mktemp("mtp")
    cfg = dict(small_mla_moe_config(), num_nextn_predict_layers=1)
    reference.write_checkpoint(cfg, d / "ckpt", seed=0, dtype=torch.bfloat16)
    rep = plowc.compile_dir(d / "ckpt", d / "assets", max_rows=256, prefill_buckets=[128, 256], decode_rungs=[1, 4, 8], max_seqs=8,
                            mtp=True)
    assert rep["mtp"]["ranks"][0]["verify"]["ok"]
    return d, cfg


def _reference(d, cfg, engines):
    from safetensors.torch import load_file
    from plow_b200.models import config, reference
    fp8_src = set()
    for eng in engines:
        pkt = eng.packet
        derived = pkt.section_json("derived_weights.json")
        for n in {pkt.tensors[h].name for h in eng.static_q}:
            r = derived.get(n)
            if r is None:
                fp8_src.add(n)
            elif r["op"] == "cat":
                fp8_src.update(r["parts"])
            elif r["op"] == "cols":
                fp8_src.add(r["src"])
            else:
                for e in range(r["n"]):
                    fp8_src.update(f"{r['prefix']}.{e}.{p}.weight" for p in r["parts"])
                fp8_src.update(r.get("tail", []))
    state = {}
    for f in glob.glob(str(d / "ckpt" / "*.safetensors")):
        state.update(load_file(f))
    state = {k: (_rt(v) if k in fp8_src else v.float()) for k, v in state.items()}
    return reference.ReferenceModel(config.spec_from_config(cfg), state)


def _rel(a, b):
    return ((a - b).norm() / b.norm()).item()


def test_drafter_packet_and_chain_on_the_gpu(mtp_assets):
    from plow_b200.runtime.engine import TokenBatch
    from plow_b200.runtime.gpu_engine import GpuEngine
    from plow_b200.runtime.spec import MtpDrafter, SpecStats, spec_decode
    d, cfg = mtp_assets
    main = GpuEngine(d / "assets", max_slots=4, max_ctx=512)
    dr = GpuEngine(d / "assets" / "mtp", max_slots=4, max_ctx=512, prefix_cache=False)
    assert dr.spec.role == "mtp" and dr.d_hidden_in is not None and dr.hidden_rows == "samples" and main.hidden_rows == "rows"
    ref = _reference(d, cfg, [main, dr])
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, 1024, (100,), generator=g).tolist()
    n = len(prompt)
    main.begin_slot(0, prompt)
    main.reserve(0, n + 1)
    r = main.step(TokenBatch(np.asarray(prompt, np.int32), np.arange(n, dtype=np.int32), np.zeros(n, np.int32),
                             np.asarray([n - 1], np.int32), want_logits=True, want_hidden=True))
    main.commit(0, prompt)
    lg, h = ref.forward_hidden(torch.tensor(prompt))
    assert torch.is_tensor(r.hidden) and r.hidden.is_cuda and tuple(r.hidden.shape) == (n, cfg["hidden_size"])
    assert _rel(r.hidden.float().cpu(), h) < 0.06
    pending = int(r.ids[0])
    # the module over the prompt, fed the ENGINE's hidden states: only the module's own error is left
    nxt = prompt[1:] + [pending]
    dr.begin_slot(0, [])
    dr.reserve(0, n + 1)
    r2 = dr.step(TokenBatch(np.asarray(nxt, np.int32), np.arange(n, dtype=np.int32), np.zeros(n, np.int32),
                            np.asarray([n - 1], np.int32), want_logits=True, want_hidden=True, hidden=r.hidden))
    l2, g2 = ref.mtp_forward(torch.tensor(nxt), r.hidden.float().cpu())
    assert _rel(torch.from_numpy(r2.logits[0]), l2[-1]) < 0.06
    assert _rel(r2.hidden[0].float().cpu(), g2[-1]) < 0.06
    top2 = l2[-1].topk(2).values
    if float(top2[0] - top2[1]) > 0.05 * float(l2[-1].abs().max()):
        assert int(r2.ids[0]) == int(l2[-1].argmax())
    dr.retire_slot(0)
    # chain of three drafts: one multi-row step over the prompt, then two single-row steps through the decode graph
    drafter = MtpDrafter(dr)
    drafter.begin(0)
    drafter.observe([(0, 0, nxt, r.hidden)])
    drafts = drafter.propose_many([0], 3)[0]
    assert len(drafts) == 3 and drafts[0] == int(r2.ids[0]) and all(0 <= t < 1024 for t in drafts)
    again = drafter.propose_many([0], 3)[0]                # speculative rows are not committed: asking twice changes nothing
    assert again == drafts
    drafter.retire(0)
    # plain greedy continuation of the same engine (decode graph), then the speculative one
    main.begin_slot(1, prompt)
    main.reserve(1, n + 14)
    main.step(TokenBatch(np.asarray(prompt, np.int32), np.arange(n, dtype=np.int32), np.ones(n, np.int32), np.asarray([n - 1], np.int32)))
    main.commit(1, prompt)
    plain, tok = [pending], pending
    for i in range(11):
        rr = main.step(TokenBatch(np.asarray([tok], np.int32), np.asarray([n + i], np.int32), np.ones(1, np.int32),
                                  np.zeros(1, np.int32), decode=True))
        main.commit(1, [tok])
        tok = int(rr.ids[0])
        plain.append(tok)
    main.retire_slot(1)
    stats = SpecStats()
    got = spec_decode(main, 0, pending, 12, drafter, depth=3, stats=stats, prefill_hidden=r.hidden)
    # verify spans run through the prefill program, plain decoding through the decode graph: near-ties of a random-weight
    # model may flip late tokens, the first ones must agree
    assert len(got) == 12 and got[:3] == plain[:3]
    assert sum(int(a == b) for a, b in zip(got, plain)) >= 8
    assert stats.proposed >= stats.steps and 0 not in dr.tokens
    from plow_b200.ops import native
    assert int(native.status_word(main.device)[0]) == 0


def test_scheduler_with_the_prediction_module_on_the_gpu(mtp_assets):
    from plow_b200.runtime.gpu_engine import GpuEngine
    from plow_b200.runtime.scheduler import GenParams, ModelMux, SchedConfig
    from plow_b200.runtime.spec import MtpDrafter
    from plow_b200.text.tokenizer import ByteTokenizer
    d, cfg = mtp_assets
    rng = np.random.default_rng(7)
    prompts = [rng.integers(3, 1000, size=k).tolist() for k in (300, 60)]          # 300 rows: two chunks of the 256-row bucket

    def run(depth):
        eng = GpuEngine(d / "assets", max_slots=4, max_ctx=1024, prefix_cache=False)
        mux = ModelMux(eng, ByteTokenizer(), SchedConfig(token_budget=256, spec_depth=depth), eos_ids=[])
        dr = None
        if depth:
            dr = GpuEngine(d / "assets" / "mtp", max_slots=4, max_ctx=1024, prefix_cache=False)
            mux.set_drafter(MtpDrafter(dr))
        mux.start()
        try:
            reqs = [mux.submit(p, GenParams(max_tokens=12)) for p in prompts]
            outs = []
            for r in reqs:
                toks = []
                while True:
                    c = r.out.get(timeout=120)
                    if c.kind == "token":
                        toks.append(c.token_id)
                    elif c.kind == "done":
                        break
                    else:
                        raise AssertionError(c.error)
                outs.append(toks)
            return outs, mux.metrics.snapshot()["counters"], (dict(dr.tokens) if dr else {})
        finally:
            mux.stop()
    plain, c0, _ = run(0)
    spec, c1, left = run(3)
    for a, b in zip(plain, spec):
        assert len(a) == 12 and len(b) == 12 and a[:2] == b[:2]
        assert sum(int(x == y) for x, y in zip(a, b)) >= 8
    assert c1["spec_ticks"] >= 1 and c1["spec_proposed"] >= 2 * c1["spec_ticks"] and left == {}
