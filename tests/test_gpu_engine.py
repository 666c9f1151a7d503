"""sm_100a engine end to end on a small MLA + MoE model (e4m3 weights and latent cache) vs the
fp32 PyTorch reference evaluated on the same (quantise-dequantised) weights."""
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
def mla_assets(tmp_path_factory):
    from plow_b200 import plowc
    from plow_b200.models import reference
    from plow_b200.runtime.smoke import small_mla_moe_config
    d = tmp_path_factory.mktemp("mla")
    cfg = small_mla_moe_config()
    reference.write_checkpoint(cfg, d / "ckpt", seed=0, dtype=torch.bfloat16)
    plowc.compile_dir(d / "ckpt", d / "assets", max_rows=256, prefill_buckets=[128, 256], decode_rungs=[4, 8], max_seqs=8)
    return d, cfg


def test_engine_matches_reference(mla_assets):
    from safetensors.torch import load_file
    from plow_b200.compiler import packet as pk
    from plow_b200.models import config, reference
    from plow_b200.runtime.engine import TokenBatch
    from plow_b200.runtime.gpu_engine import GpuEngine
    d, cfg = mla_assets
    eng = GpuEngine(d / "assets", max_slots=4, max_ctx=512)
    pkt = eng.packet
    fp8_names = {pkt.tensors[h].name for h in eng.static_q}
    derived = pkt.section_json("derived_weights.json")
    fp8_src = set()
    for n in fp8_names:
        r = derived.get(n)
        if r is None:
            fp8_src.add(n)
        elif r["op"] == "cat":
            fp8_src.update(r["parts"])
        else:
            for e in range(r["n"]):
                fp8_src.update(f"{r['prefix']}.{e}.{p}.weight" for p in r["parts"])
    state = {}
    for f in glob.glob(str(d / "ckpt" / "*.safetensors")):
        state.update(load_file(f))
    state = {k: (_rt(v) if k in fp8_src else v.float()) for k, v in state.items()}
    ref = reference.ReferenceModel(config.spec_from_config(cfg), state)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (100, 37)]
    ids, pos, seq, samp = [], [], [], []
    for s, p in enumerate(prompts):
        eng.begin_slot(s, p)
        eng.reserve(s, len(p) + 8)
        ids += p
        pos += list(range(len(p)))
        seq += [s] * len(p)
        samp.append(len(ids) - 1)
    res = eng.step(TokenBatch(np.array(ids, np.int32), np.array(pos, np.int32), np.array(seq, np.int32),
                              np.array(samp, np.int32), want_logits=True))
    for s, p in enumerate(prompts):
        want = ref.forward(torch.tensor(p))[-1]
        got = torch.from_numpy(res.logits[s])
        rel = ((got - want).norm() / want.norm()).item()
        assert rel < 0.12, (s, rel)
        eng.commit(s, p)
    # decode two steps for both sequences (CUDA graph path), feeding the reference's greedy tokens
    cur = [list(p) for p in prompts]
    for step in range(2):
        nxt = [int(ref.forward(torch.tensor(c))[-1].argmax()) for c in cur]
        for s in range(2):
            eng.reserve(s, len(cur[s]) + 2)
        r = eng.step(TokenBatch(np.array(nxt, np.int32), np.array([len(c) for c in cur], np.int32), np.array([0, 1], np.int32),
                                np.array([0, 1], np.int32), decode=True, want_logits=True))
        for s in range(2):
            cur[s].append(nxt[s])
            eng.commit(s, [nxt[s]])
            want = ref.forward(torch.tensor(cur[s]))[-1]
            got = torch.from_numpy(r.logits[s])
            assert ((got - want).norm() / want.norm()).item() < 0.12


def test_dsa_model_identity_selection_matches_dense_reference(tmp_path):
    """MLA-MoE with a sparse-attention indexer whose top-k covers the whole context: the indexer cache write, the
    score / select kernels, the gather and the decode over the compact cache all run, and the result must equal dense
    attention (the fp32 reference has no indexer)."""
    from safetensors.torch import load_file
    from plow_b200 import plowc
    from plow_b200.compiler.packet import Op
    from plow_b200.models import config, reference
    from plow_b200.runtime.engine import TokenBatch
    from plow_b200.runtime.gpu_engine import GpuEngine
    from plow_b200.runtime.smoke import small_mla_moe_config
    cfg = small_mla_moe_config()
    cfg.update(model_type="glm_moe_dsa", index_n_heads=64, index_head_dim=128, index_topk=128)
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=0, dtype=torch.bfloat16)
    plowc.compile_dir(tmp_path / "ckpt", tmp_path / "assets", max_rows=256, prefill_buckets=[128, 256], decode_rungs=[4, 8], max_seqs=8)
    eng = GpuEngine(tmp_path / "assets", max_slots=4, max_ctx=512)
    assert any(i.op == Op.DSA_TOPK for i in eng.packet.programs[0].insts)
    pkt = eng.packet
    fp8_names = {pkt.tensors[h].name for h in eng.static_q}
    derived = pkt.section_json("derived_weights.json")
    fp8_src = set()
    for n in fp8_names:
        r = derived.get(n)
        if r is None:
            fp8_src.add(n)
        elif r["op"] == "cat":
            fp8_src.update(r["parts"])
        else:
            for e in range(r["n"]):
                fp8_src.update(f"{r['prefix']}.{e}.{p}.weight" for p in r["parts"])
    state = {}
    for f in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        state.update(load_file(f))
    state = {k: (_rt(v) if k in fp8_src else v.float()) for k, v in state.items()}
    ref = reference.ReferenceModel(config.spec_from_config(cfg), state)
    g = torch.Generator().manual_seed(1)
    p = torch.randint(0, 1024, (100,), generator=g).tolist()
    eng.begin_slot(0, p)
    eng.reserve(0, len(p) + 8)
    res = eng.step(TokenBatch(np.array(p, np.int32), np.arange(len(p), dtype=np.int32), np.zeros(len(p), np.int32),
                              np.array([len(p) - 1], np.int32), want_logits=True))
    want = ref.forward(torch.tensor(p))[-1]
    assert ((torch.from_numpy(res.logits[0]) - want).norm() / want.norm()).item() < 0.12
    eng.commit(0, p)
    nxt = int(want.argmax())
    r = eng.step(TokenBatch(np.array([nxt], np.int32), np.array([len(p)], np.int32), np.array([0], np.int32), np.array([0], np.int32),
                            decode=True, want_logits=True))
    want = ref.forward(torch.tensor(p + [nxt]))[-1]
    assert ((torch.from_numpy(r.logits[0]) - want).norm() / want.norm()).item() < 0.12
    sel = next(st for st in eng.progs.values() if st.role == 1)
    assert any(k[0] == "dsa_cc" for k in sel.scratch)


def test_smoke_runs():
    from plow_b200.runtime import smoke
    smoke.run()
