"""sm_100a engine end to end on a small dense GQA model (bf16 weights, paged bf16 KV cache) vs the fp32
PyTorch reference: packed two-prompt prefill through the tcgen05 flash kernel, then graph-captured decode."""
import glob

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

CFG = dict(model_type="llama", hidden_size=512, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
           num_hidden_layers=2, intermediate_size=1024, rms_norm_eps=1e-5, rope_theta=10000.0, vocab_size=1024,
           tie_word_embeddings=False, max_position_embeddings=2048, eos_token_id=2, plow_kv_dtype="bf16")


@pytest.fixture(scope="module")
def dense_assets(tmp_path_factory):
    from plow_b200 import plowc
    from plow_b200.models import reference
    d = tmp_path_factory.mktemp("dense")
    reference.write_checkpoint(CFG, d / "ckpt", seed=0, dtype=torch.bfloat16)
    plowc.compile_dir(d / "ckpt", d / "assets", max_rows=256, prefill_buckets=[128, 256], decode_rungs=[4, 8], max_seqs=8)
    # second build with the row fusions off: RESIDUAL -> RMSNORM and GLU stay separate instructions, so the
    # on-device interpreter gets multi-instruction segments whose units wait on one another's counters
    plowc.compile_dir(d / "ckpt", d / "assets_unfused", max_rows=256, prefill_buckets=[128, 256], decode_rungs=[4, 8],
                      max_seqs=8, disable_rules=("residual-rmsnorm-fuse", "gated-mlp-fuse"))
    return d


def test_interpreter_segments_cover_row_ops(dense_assets):
    from plow_b200.compiler import packet as pk
    from plow_b200.compiler.packet import Op
    from plow_b200.runtime.device_interp import DeviceInterp
    pkt = pk.read_packet(dense_assets / "assets_unfused" / "model.pkt")
    segs = DeviceInterp.segments(pkt.programs[0])
    assert sum(hi - lo for lo, hi, _ in segs) == len(pkt.programs[0].insts)
    assert any(dev and hi - lo >= 2 for lo, hi, dev in segs)
    assert all(Op(pkt.programs[0].insts[lo].op) in (Op.GEMM, Op.ROPE_KV, Op.ATTN) for lo, hi, dev in segs if not dev)


@pytest.mark.parametrize("assets,interp", [("assets", True), ("assets", False), ("assets_unfused", True), ("assets_unfused", False)])
def test_dense_engine_matches_reference(dense_assets, assets, interp):
    from safetensors.torch import load_file
    from plow_b200.models import config, reference
    from plow_b200.runtime.engine import TokenBatch
    from plow_b200.runtime.gpu_engine import GpuEngine
    d = dense_assets
    eng = GpuEngine(d / assets, max_slots=4, max_ctx=512, device_interp=interp)
    state = {}
    for f in glob.glob(str(d / "ckpt" / "*.safetensors")):
        state.update(load_file(f))
    ref = reference.ReferenceModel(config.spec_from_config(CFG), {k: v.float() for k, v in state.items()})
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (150, 37)]
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
        assert rel < 0.05, (s, rel)
        eng.commit(s, p)
    cur = [list(p) for p in prompts]
    for step in range(3):
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
            assert ((got - want).norm() / want.norm()).item() < 0.05
    if interp:
        assert all(st.interp is not None and st.interp.launches > 0 for st in eng.progs.values())


def test_dense_engine_with_e4m3_kv_cache(tmp_path):
    """plow_kv_dtype=fp8 on a GQA model: the writer stores e4m3 cells + per-cell scales, prefill and decode attention read
    them through the converter warps; logits against the fp32 reference, and half the KV bytes per token (+ scales)."""
    from safetensors.torch import load_file
    from plow_b200 import plowc
    from plow_b200.compiler import packet as pk
    from plow_b200.models import config, reference
    from plow_b200.runtime.engine import TokenBatch
    from plow_b200.runtime.gpu_engine import GpuEngine
    cfg = dict(CFG, plow_kv_dtype="fp8")
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=0, dtype=torch.bfloat16)
    plowc.compile_dir(tmp_path / "ckpt", tmp_path / "assets", max_rows=256, prefill_buckets=[128, 256], decode_rungs=[4, 8], max_seqs=8)
    spec = config.spec_from_config(cfg)
    assert spec.kv_bytes_per_token() == 2 * (2 * 2 * 128 + 8 * 2) and config.spec_from_config(CFG).kv_bytes_per_token() == 2 * 2 * 2 * 128 * 2
    eng = GpuEngine(tmp_path / "assets", max_slots=4, max_ctx=512)
    kinds = {t.name: pk.DType(t.dtype) for t in eng.packet.tensors if t.tclass == pk.TClass.KV}
    assert kinds["kv.0.k"] == pk.DType.E4M3 and kinds["kv.0.s"] == pk.DType.F32
    state = {}
    for f in glob.glob(str(tmp_path / "ckpt" / "*.safetensors")):
        state.update(load_file(f))
    ref = reference.ReferenceModel(spec, {k: v.float() for k, v in state.items()})
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (150, 37)]
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
        rel = ((torch.from_numpy(res.logits[s]) - want).norm() / want.norm()).item()
        assert rel < 0.06, (s, rel)
        eng.commit(s, p)
    cur = [list(p) for p in prompts]
    for step in range(3):
        nxt = [int(ref.forward(torch.tensor(c))[-1].argmax()) for c in cur]
        for s in range(2):
            eng.reserve(s, len(cur[s]) + 2)
        r = eng.step(TokenBatch(np.array(nxt, np.int32), np.array([len(c) for c in cur], np.int32), np.array([0, 1], np.int32),
                                np.array([0, 1], np.int32), decode=True, want_logits=True))
        for s in range(2):
            cur[s].append(nxt[s])
            eng.commit(s, [nxt[s]])
            want = ref.forward(torch.tensor(cur[s]))[-1]
            rel = ((torch.from_numpy(r.logits[s]) - want).norm() / want.norm()).item()
            assert rel < 0.06, (step, s, rel)
    from plow_b200.ops import native
    assert int(native.status_word(eng.device)[0]) == 0
