"""Pre-quantised e4m3 weight twins (runtime/fp8_dir.py): written by ``plowc --fp8-dir``, trusted only for the packet they
were written for, equal to quantising at load."""
import json

import torch


def test_fp8_twins_round_trip_and_are_bound_to_their_packet(tmp_path):
    from plow_b200 import plowc
    from plow_b200.compiler import packet as pk
    from plow_b200.models import reference
    from plow_b200.ops import quant
    from plow_b200.runtime.fp8_dir import Fp8Dir, fp8_weight_handles
    from plow_b200.runtime.smoke import small_mla_moe_config
    from plow_b200.runtime.weights import materialize, open_checkpoint
    cfg = small_mla_moe_config(hidden=512, experts=8)
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=0, dtype=torch.bfloat16)
    rep = plowc.compile_dir(tmp_path / "ckpt", tmp_path / "assets", max_rows=128, prefill_buckets=[128], decode_rungs=[8], max_seqs=8,
                            fp8_dir=True)
    assert rep["fp8_dir"][0]["tensors"] >= 8
    pkt = pk.read_packet(tmp_path / "assets" / "model.pkt")
    handles = fp8_weight_handles(pkt, "fp8_block128")
    names = {pkt.tensors[h].name for h in handles}
    assert any(n.startswith("cat/") for n in names) and not any("gate.weight" in n and "experts" not in n and "gate_up" not in n for n in names)
    twins = Fp8Dir(tmp_path / "assets", pkt)
    assert twins and set(twins.map) == names | {n + ".scale" for n in names}
    derived = pkt.section_json("derived_weights.json")
    ckpt = open_checkpoint(tmp_path / "assets" / "checkpoint")
    for h in sorted(handles)[:6]:
        ent = pkt.tensors[h]
        q, s = twins.get(ent.name, "cpu")
        w = materialize(ent.name, ent, derived.get(ent.name), ckpt).to(torch.bfloat16)
        q2, s2 = quant.quant_weight_128x128(w)
        assert q.dtype == torch.float8_e4m3fn and tuple(q.shape) == tuple(w.shape)
        assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s, s2)
    assert twins.get("model.norm.weight", "cpu") is None
    # the index names the packet it belongs to: another build of the packet does not pick the twins up
    idx_file = tmp_path / "assets" / "fp8" / "fp8_index.json"
    idx = json.loads(idx_file.read_text())
    idx["packet_sha256"] = "00" * 32
    idx_file.write_text(json.dumps(idx))
    assert not Fp8Dir(tmp_path / "assets", pkt)


def test_plowc_cli_writes_twins_for_the_decoder_and_its_drafter(tmp_path, capsys):
    from plow_b200 import plowc
    from plow_b200.models import reference
    from plow_b200.runtime.smoke import small_mla_moe_config
    cfg = dict(small_mla_moe_config(hidden=512, experts=8), num_nextn_predict_layers=1)
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=0, dtype=torch.bfloat16)
    rc = plowc.main(["--hf-dir", str(tmp_path / "ckpt"), "--out", str(tmp_path / "out"), "--max-rows", "128", "--prefill-buckets", "128",
                     "--decode-rungs", "8", "--max-seqs", "8", "--fp8-dir", "--mtp"])
    assert rc == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["ranks"] == 1
    for d in (tmp_path / "out", tmp_path / "out" / "mtp"):
        idx = json.loads((d / "fp8" / "fp8_index.json").read_text())
        assert idx["weight_map"] and (d / "model.pkt").exists()
    build = json.loads((tmp_path / "out" / "build.json").read_text())
    assert build["fp8_dir"][0]["tensors"] >= 8 and build["mtp"]["fp8_dir"][0]["tensors"] >= 4
    # the drafter's eh_proj halves are e4m3 twins too (column ranges of one checkpoint matrix)
    names = set(json.loads((tmp_path / "out" / "mtp" / "fp8" / "fp8_index.json").read_text())["weight_map"])
    assert any(n.startswith("cols/") and n.endswith(".e") for n in names)
    # a checkpoint without prediction modules refuses --mtp
    reference.write_checkpoint(small_mla_moe_config(hidden=512, experts=8), tmp_path / "plain", seed=0, dtype=torch.bfloat16)
    assert plowc.main(["--hf-dir", str(tmp_path / "plain"), "--out", str(tmp_path / "o2"), "--max-rows", "128", "--mtp"]) == 2
