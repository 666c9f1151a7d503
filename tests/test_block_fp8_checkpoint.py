"""Checkpoints that are already block-quantised (e4m3 codes under ``<name>.weight`` + one f32 ``<name>.weight_scale_inv``
per 128 x 128 block, the layout fp8 MLA-MoE checkpoints ship in): dequantised where bf16 / f32 is wanted, handed to the
e4m3 GEMMs as they are where codes are wanted."""
import glob

import numpy as np
import torch


def _quantise_checkpoint(src, dst):
    """bf16 safetensors checkpoint -> block-fp8 one (projections with both dims a multiple of 128; norms, router, embeddings stay)."""
    import json
    import shutil
    from safetensors.torch import load_file, save_file
    from plow_b200.ops import quant
    dst.mkdir()
    shutil.copy(src / "config.json", dst / "config.json")
    out, n_q = {}, 0
    for f in glob.glob(str(src / "*.safetensors")):
        for k, v in load_file(f).items():
            if v.dim() == 2 and v.shape[0] % 128 == 0 and v.shape[1] % 128 == 0 and "embed" not in k and "lm_head" not in k and ".gate.weight" not in k:
                q, s = quant.quant_weight_128x128(v)
                out[k], out[k + "_scale_inv"] = q, s
                n_q += 1
            else:
                out[k] = v
    save_file(out, str(dst / "model.safetensors"))
    return n_q


def test_block_fp8_checkpoint_is_read_faithfully(tmp_path):
    from plow_b200 import plowc
    from plow_b200.compiler import packet as pk
    from plow_b200.models import config, reference
    from plow_b200.ops import quant
    from plow_b200.runtime.cpu_engine import CpuEngine
    from plow_b200.runtime.engine import TokenBatch
    from plow_b200.runtime.fp8_dir import fp8_weight_handles
    from plow_b200.runtime.smoke import small_mla_moe_config
    from plow_b200.runtime.weights import fp8_codes, is_block_fp8, materialize, open_checkpoint
    cfg = dict(small_mla_moe_config(hidden=512, experts=8), plow_kv_dtype="f32")
    reference.write_checkpoint(cfg, tmp_path / "bf16", seed=0, dtype=torch.bfloat16)
    n_q = _quantise_checkpoint(tmp_path / "bf16", tmp_path / "fp8")
    assert n_q > 20
    ck8, ck16 = open_checkpoint(tmp_path / "fp8"), open_checkpoint(tmp_path / "bf16")
    name = "model.layers.0.self_attn.o_proj.weight"
    assert is_block_fp8(ck8, name) and not is_block_fp8(ck16, name) and ck8.get(name).dtype == torch.float8_e4m3fn
    # the sm_100a packet: which tensors its GEMMs read as e4m3, and what the loader hands them
    plowc.compile_dir(tmp_path / "fp8", tmp_path / "gpu_assets", max_rows=128, prefill_buckets=[128], decode_rungs=[8], max_seqs=8)
    pkt = pk.read_packet(tmp_path / "gpu_assets" / "model.pkt")
    derived = pkt.section_json("derived_weights.json")
    kinds = set()
    for h in sorted(fp8_weight_handles(pkt, "fp8_block128")):
        ent = pkt.tensors[h]
        rec = derived.get(ent.name)
        got = fp8_codes(ent.name, ent, rec, ck8)
        assert got is not None, ent.name
        q, s = got
        # the same codes and scales as quantising the bf16 original (the checkpoint WAS made that way): nothing was rounded twice
        q2, s2 = quant.quant_weight_128x128(materialize(ent.name, ent, rec, ck16).to(torch.bfloat16))
        assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s, s2), ent.name
        # and the dequantised view the bf16 / CPU paths get is codes x scales
        w = materialize(ent.name, ent, rec, ck8)
        assert w.dtype == torch.bfloat16 and torch.equal(w, quant.dequant_weight_128x128(q, s).to(torch.bfloat16))
        kinds.add(rec["op"] if rec else "plain")
    assert kinds >= {"plain", "cat", "stack_experts"}
    assert fp8_codes(name, pkt.tensors[pkt.tensor_index(name)], None, ck16) is None          # an unquantised checkpoint: the caller quantises
    # the CPU backend serves the quantised checkpoint: its logits are those of the reference over the dequantised weights
    cpu_cfg = dict(cfg, plow_dtype="f32")
    import json
    (tmp_path / "fp8" / "config.json").write_text(json.dumps(cpu_cfg))
    plowc.compile_dir(tmp_path / "fp8", tmp_path / "cpu_assets", arch="cpu", n_cu=4, max_rows=128, decode_rungs=[1], max_seqs=4)
    spec = config.spec_from_config(cpu_cfg)
    state = {}
    for n in ck8.names():
        if n.endswith("_scale_inv"):
            continue
        state[n] = (quant.dequant_weight_128x128(ck8.get(n), ck8.get(n + "_scale_inv")).to(torch.bfloat16) if is_block_fp8(ck8, n) else ck8.get(n)).float()
    ref = reference.ReferenceModel(spec, state)
    p = np.random.default_rng(1).integers(0, 1024, 70).tolist()
    eng = CpuEngine(tmp_path / "cpu_assets", max_slots=2, max_ctx=256)
    eng.begin_slot(0, p)
    eng.reserve(0, 80)
    r = eng.step(TokenBatch(np.asarray(p, np.int32), np.arange(70, dtype=np.int32), np.zeros(70, np.int32), np.asarray([69], np.int32), want_logits=True))
    eng.close()
    want = ref.forward(torch.tensor(p))[-1]
    assert (torch.from_numpy(r.logits[0]) - want).abs().max().item() < 2e-4 * max(1.0, want.abs().max().item())
