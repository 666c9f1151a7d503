"""Graph builders, fusion rules (positive and negative), scheduler, verifier."""
import pytest

from plow_b200.compiler import emit, graph, hwspec, packet as pk, rewrite, schedule, verify
from plow_b200.models import config


def _fused(cfg, **kw):
    spec = config.spec_from_config(cfg)
    g = graph.build_graph(spec, **kw)
    sites = rewrite.fuse(g)
    return g, sites


def test_dense_fusion_coverage():
    g, sites = _fused(config.tiny_dense_config())
    cov = rewrite.coverage(sites)
    assert cov == {"qkv-fuse": 4, "rope-kv-fuse": 4, "gated-mlp-fuse": 4, "residual-rmsnorm-fuse": 8}
    ops = [n.op for n in g.nodes]
    assert "silu_mul" not in ops and "rope" not in ops and "kv_write" not in ops
    assert ops.count("add_norm") == 8 and ops.count("linear_glu") == 4


def test_qwen3_headnorm_is_swallowed_by_rope_kv():
    cfg = dict(config.tiny_dense_config(), model_type="qwen3")
    g, sites = _fused(cfg)
    assert rewrite.coverage(sites)["rope-kv-fuse"] == 4
    rk = next(n for n in g.nodes if n.op == "rope_kv")
    assert rk.inputs[1] is not None and rk.inputs[2] is not None and rk.attrs["eps"] > 0
    assert not any(n.op == "headnorm" for n in g.nodes)


def test_negative_fusions():
    spec = config.spec_from_config(config.tiny_dense_config())
    g = graph.build_graph(spec)
    # a second consumer of the gate projection must block gated-mlp-fuse on that layer
    sm = next(n for n in g.nodes if n.op == "silu_mul")
    extra = g.tmp("probe", g.values[sm.inputs[0]].shape)
    g.add("add", [sm.inputs[0], sm.inputs[0]], [extra], layer=sm.layer)
    sites = rewrite.fuse(g)
    assert rewrite.coverage(sites)["gated-mlp-fuse"] == 3
    # a disabled rule does not fire
    g2 = graph.build_graph(spec)
    sites2 = rewrite.fuse(g2, disable={"qkv-fuse"})
    assert "qkv-fuse" not in rewrite.coverage(sites2) and "rope-kv-fuse" not in rewrite.coverage(sites2)


def test_tp_graph_has_fused_collectives():
    g, sites = _fused(config.dense_8b_config(), tp=8)
    cov = rewrite.coverage(sites)
    # every row-parallel projection's reduction (o_proj and down_proj of 32 layers) folds into the all-reduce + add + norm
    # kernel that follows it; with that rule off the reductions fuse into the GEMM epilogues instead
    assert cov["xreduce-add-norm-fuse"] + cov.get("gemm-xreduce-fuse", 0) == 64 and cov["xreduce-add-norm-fuse"] >= 63
    g2 = graph.build_graph(config.spec_from_config(config.dense_8b_config()), tp=8)
    assert rewrite.coverage(rewrite.fuse(g2, disable={"xreduce-add-norm-fuse"}))["gemm-xreduce-fuse"] == 64
    q = next(n for n in g.nodes if n.op == "linear" and n.site == "qkv-fuse")
    assert g.values[q.inputs[1]].shape == ((32 + 16) * 128 // 8, 4096)


@pytest.mark.parametrize("cfg_fn,kw", [(lambda: config.mla_moe_671b_config(n_layers=5), dict(ep=8)),
                                       (lambda: config.mla_moe_671b_config(n_layers=4, dsa=True), dict(ep=8)),
                                       (config.gdn_hybrid_80b_config, dict(tp=2, ep=4)),
                                       (config.qwen3_moe_30b_config, dict(ep=8)),
                                       (config.mixtral_8x7b_config, dict(ep=2)),
                                       (config.gpt_oss_120b_config, dict(ep=8)),
                                       (config.kimi_linear_48b_config, dict(ep=8))])
def test_big_families_build_and_verify(cfg_fn, kw):
    cfg = cfg_fn()
    if "num_hidden_layers" in cfg and cfg["num_hidden_layers"] > 8:
        cfg["num_hidden_layers"] = 8
        if "layer_types" in cfg:
            cfg["layer_types"] = cfg["layer_types"][:8]
        if "linear_attn_config" in cfg:
            lac = cfg["linear_attn_config"]
            cfg["linear_attn_config"] = dict(lac, kda_layers=[i for i in lac["kda_layers"] if i <= 8],
                                             full_attn_layers=[i for i in lac["full_attn_layers"] if i <= 8])
    spec = config.spec_from_config(cfg)
    g = graph.build_graph(spec, **kw)
    rewrite.fuse(g)
    pkt = emit.emit_packet(g, [], hwspec.lookup("b200"), 148, dict(prefill=[128], decode=[8, 64], max_seqs=8))
    res = verify.verify_packet(pkt)
    assert res["ok"], res["failures"]
    ops = {pk.Op(i.op).name for p in pkt.programs for i in p.insts}
    assert "ROUTER_TOPK" in ops and "MOE_GEMM" in ops


def test_schedule_protocol_and_arena(tiny_assets):
    pkt = pk.read_packet(tiny_assets / "assets" / "model.pkt")
    assert verify.verify_packet(pkt)["ok"]
    for p in pkt.programs:
        sim = schedule.simulate(p)
        assert sim["completed"]
        # op-major completion: an instruction's entries never complete before its producers'
        done_at = {}
        for step, (_c, inst) in enumerate(sim["order"]):
            done_at[inst] = step
        for e in p.stream:
            for (ctr, _t) in p.waits[e.wait_ofs:e.wait_ofs + e.n_wait]:
                assert done_at[ctr] < done_at[e.inst] or ctr == e.inst


def test_verifier_refuses_broken_protocol(tiny_assets):
    pkt = pk.read_packet(tiny_assets / "assets" / "model.pkt")
    p = pkt.programs[0]
    c, t = p.waits[0]
    p.waits[0] = (c, t + 1)          # a wait no producer can satisfy
    res = verify.verify_packet(pkt)
    assert not res["ok"]


def test_arch_refusal():
    with pytest.raises(ValueError, match="sm_100a"):
        hwspec.check_arch("sm_90a")
    hw = hwspec.lookup("b200")
    assert hw.sm_count == 148 and hw.isa.tcgen05 and not hw.isa.wgmma


def test_rope_tables_scaling():
    import numpy as np
    from plow_b200.utils.rope import rope_table
    t = rope_table(64, 64, 10000.0)
    assert t.dtype == np.float32 and t.shape == (64, 64)
    assert np.allclose(t[0, :32], 1.0) and np.allclose(t[0, 32:], 0.0)
    l3 = rope_table(64, 64, 500000.0, dict(type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                          original_max_position_embeddings=8192))
    ya = rope_table(64, 64, 10000.0, dict(type="yarn", factor=40.0, original_max_position_embeddings=4096,
                                          beta_fast=32, beta_slow=1, mscale=1.0, mscale_all_dim=1.0))
    assert np.isfinite(l3).all() and np.isfinite(ya).all()
    assert not np.allclose(l3[5], rope_table(64, 64, 500000.0)[5])
    # gpt_oss: YaRN whose ramp ends are not rounded (truncate = false), attention factor 0.1 ln(32) + 1 on cos and sin
    import math
    sc = dict(type="yarn", factor=32.0, beta_fast=32.0, beta_slow=1.0, original_max_position_embeddings=4096, truncate=False)
    got = rope_table(8, 64, 150000.0, sc)
    half, att = 32, 0.1 * math.log(32.0) + 1.0
    base = 1.0 / 150000.0 ** (np.arange(half) * 2.0 / 64)
    lo, hi = (64 * math.log(4096 / (b * 2 * math.pi)) / (2 * math.log(150000.0)) for b in (32.0, 1.0))
    ramp = np.clip((np.arange(half) - lo) / (hi - lo), 0, 1)
    f = base / 32.0 * ramp + base * (1 - ramp)
    assert np.allclose(got[5, :half], np.cos(5 * f) * att, atol=1e-6) and np.allclose(got[5, half:], np.sin(5 * f) * att, atol=1e-6)
    assert not np.allclose(got, rope_table(8, 64, 150000.0, dict(sc, truncate=True)))


def test_device_interp_tables_build_on_cpu(tiny_assets):
    """The on-device interpreter's host side: packet tables serialise to the ABI strides and every program is cut
    into row segments + role instructions that cover it exactly (no device needed to build them)."""
    import torch
    from plow_b200.compiler import packet as pk
    from plow_b200.compiler.packet import Op
    from plow_b200.runtime.device_interp import DeviceInterp, ROW_OPS
    pkt = pk.read_packet(tiny_assets / "assets" / "model.pkt")
    prog = pkt.programs[0]
    bound = {h: torch.zeros(4) for h in range(len(pkt.tensors))}
    di = DeviceInterp(pkt, prog, lambda h: bound.get(h), rows=prog.rows, samples=4, device="cpu")
    assert di.insts.numel() == 64 * len(prog.insts) and di.stream.numel() == 24 * len(prog.stream)
    assert di.aux.shape == (len(prog.insts), 2) and int(di.aux[0, 0]) == prog.rows
    segs = DeviceInterp.segments(prog)
    assert [lo for lo, _, _ in segs] == sorted(lo for lo, _, _ in segs) and segs[0][0] == 0 and segs[-1][1] == len(prog.insts)
    assert all(segs[k][1] == segs[k + 1][0] for k in range(len(segs) - 1))
    for lo, hi, dev in segs:
        assert all((Op(prog.insts[j].op) in ROW_OPS) == dev for j in range(lo, hi))


def test_emitted_instructions_have_all_operand_slots():
    """An engine may be handed the emitter's packet object directly (no file in between): every instruction then has
    the eight operand and eight immediate slots of the packed form, unused ones empty."""
    spec = config.spec_from_config(dict(config.tiny_dense_config(), head_dim=128, hidden_size=1024))
    g = graph.build_graph(spec)
    rewrite.fuse(g)
    pkt = emit.emit_packet(g, [], hwspec.lookup("b200"), 148, dict(prefill=[128], decode=[8], max_seqs=8))
    for p in pkt.programs:
        for ins in p.insts:
            assert len(ins.t) == 8 and len(ins.i) == 8
    attn = next(i for i in pkt.programs[0].insts if i.op == pk.Op.ATTN)
    assert attn.t[4] == pk.T_NONE                    # no scale tensor: a bf16 cache


def test_emission_is_deterministic_and_keyed_by_its_inputs(tmp_path):
    """The same checkpoint configuration and knobs give the same packet bytes (content hash) on every run — a packet is
    an artefact a store can address by hash — and any knob that changes the programs changes the hash."""
    from plow_b200 import plowc
    from plow_b200.models import reference
    cfg = config.tiny_dense_config()
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=0)
    kw = dict(arch="cpu", n_cu=8, max_rows=256, decode_rungs=[1, 2, 4, 8], max_seqs=8)
    a = plowc.compile_dir(tmp_path / "ckpt", tmp_path / "a", **kw)["ranks"][0]["sha256"]
    b = plowc.compile_dir(tmp_path / "ckpt", tmp_path / "b", **kw)["ranks"][0]["sha256"]
    assert a == b and (tmp_path / "a" / "model.pkt").read_bytes() == (tmp_path / "b" / "model.pkt").read_bytes()
    c = plowc.compile_dir(tmp_path / "ckpt", tmp_path / "c", **dict(kw, decode_rungs=[1, 2, 4]))["ranks"][0]["sha256"]
    d = plowc.compile_dir(tmp_path / "ckpt", tmp_path / "d", **dict(kw, disable_rules=("gated-mlp-fuse",)))["ranks"][0]["sha256"]
    e = plowc.compile_dir(tmp_path / "ckpt", tmp_path / "e", **dict(kw, n_cu=4))["ranks"][0]["sha256"]
    assert len({a, c, d, e}) == 4
    # weights are not part of the packet: another seed of the same shape compiles to the same bytes
    reference.write_checkpoint(cfg, tmp_path / "ckpt2", seed=9)
    assert plowc.compile_dir(tmp_path / "ckpt2", tmp_path / "f", **kw)["ranks"][0]["sha256"] == a
