"""Opcode audit and counter report (compiler/audit.py)."""
import re
from pathlib import Path

import pytest

from plow_b200.compiler import audit, emit, graph, hwspec, packet as pk, rewrite
from plow_b200.compiler.packet import Op
from plow_b200.models import config

ROOT = Path(__file__).resolve().parent.parent


def test_cpu_table_is_the_interpreters_own_dispatch():
    src = (ROOT / "csrc" / "cpu" / "interp.cpp").read_text()
    cases = set(re.findall(r"case PLOW_OP_([A-Z0-9_]+):", src))
    assert {o.name for o in audit.CPU_OPS} == cases
    # every opcode of the ABI belongs to exactly one class
    for o in Op:
        assert sum(o in ops for ops in audit.CLASSES.values()) == 1, o.name
    assert audit.op_class(Op.GEMM) == "gemm" and audit.op_class(Op.XA2A_COMBINE) == "collective" and audit.op_class(200) is None


def test_audit_and_counter_report_on_real_packets(tiny_assets, capsys):
    from plow_b200 import plowrt
    from plow_b200.runtime.cpu_engine import CpuEngine
    from plow_b200.runtime.engine import EngineError
    pkt = pk.read_packet(tiny_assets / "assets" / "model.pkt")
    a = audit.audit_ops(pkt, "cpu")
    assert a["ok"] and a["used"]["GEMM"] > 0 and a["by_class"]["attention"] == ["ATTN"] and a["by_class"]["collective"] == []
    g = audit.audit_ops(pkt, "cuda")
    assert g["ok"], g["missing"]
    # a tensor-parallel packet: its collectives have sm_100a bodies and no CPU ones
    spec = config.spec_from_config(config.dense_8b_config())
    gr = graph.build_graph(spec, tp=2)
    rewrite.fuse(gr)
    tp = emit.emit_packet(gr, [], hwspec.lookup("b200"), 148, dict(prefill=[128], decode=[8], max_seqs=8))
    assert audit.audit_ops(tp, "cuda")["ok"]
    c = audit.audit_ops(tp, "cpu")
    assert not c["ok"] and set(c["missing"]) <= {"XREDUCE", "XREDUCE_ADD_NORM", "GEMM_XREDUCE", "XARGMAX_FIN", "XGATHER"} and c["missing"]
    # an opcode nobody classifies is refused, and the CPU engine refuses such a packet at load instead of mid-step
    p0 = pkt.programs[0]
    old = p0.insts[3].op
    p0.insts[3].op = 200
    assert audit.audit_ops(pkt, "cpu")["unclassified"] == [200]
    p0.insts[3].op = old
    # counter report: one counter per instruction that ran, most of them waited on, depth about the layer chain
    r = audit.counter_report(p0)
    assert r["counters"] == len(p0.insts) and r["waited"] >= r["counters"] - 1 - len(r["dead"]) and r["dependency_depth"] >= 10
    assert all(0 <= d < len(p0.insts) - 1 for d in r["dead"])
    assert plowrt.main(["inventory", str(tiny_assets / "assets")]) == 0
    out = capsys.readouterr().out
    assert '"missing"' in out and '"dependency_depth"' in out


def test_audit_names_operand_variants_only_the_cpu_backend_runs(tmp_path, tiny_assets):
    """A qwen2 packet (biased q / k / v GEMM) is fine for the CPU backend and flagged for the sm_100a one, by the variant's
    name; the plain llama packet is fine for both.  The list mirrors what the sm_100a engine refuses when it loads a packet."""
    from plow_b200 import plowc
    from plow_b200.compiler import audit, packet as pk
    from plow_b200.models import reference
    cfg = dict(model_type="qwen2", hidden_size=128, num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=1, intermediate_size=256,
               hidden_act="silu", rms_norm_eps=1e-6, rope_theta=10000.0, vocab_size=256, max_position_embeddings=512, eos_token_id=1,
               plow_dtype="f32", plow_kv_dtype="f32")
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=0)
    plowc.compile_dir(tmp_path / "ckpt", tmp_path / "assets", arch="cpu", n_cu=4, max_rows=128, decode_rungs=[1], max_seqs=2)
    pkt = pk.read_packet(tmp_path / "assets" / "model.pkt")
    assert audit.audit_ops(pkt, "cpu")["ok"]
    cuda = audit.audit_ops(pkt, "cuda")
    assert not cuda["ok"] and cuda["cpu_only_variants"] == ["GEMM bias"] and not cuda["missing"]
    import json
    assert json.loads((tmp_path / "assets" / "build.json").read_text())["runtime_requires"] == dict(backend="cpu", cpu_only_variants=["GEMM bias"])
    assert json.loads((tiny_assets / "assets" / "build.json").read_text())["runtime_requires"]["backend"] == "any"
    plain = pk.read_packet(tiny_assets / "assets" / "model.pkt")
    assert audit.audit_ops(plain, "cuda")["ok"] and audit.cpu_only_variants(plain) == []
    # the engine's load-time refusals name the same instructions
    src = (ROOT / "plow_b200" / "runtime" / "gpu_engine.py").read_text()
    for needle in ("pk.GEMM_BIAS", "GEMM_ACT_GELU_TANH", "ins.t[5] != pk.T_NONE", "ins.t[6] != pk.T_NONE", "ins.i[4] == 1"):
        assert needle in src, needle
