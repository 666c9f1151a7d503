"""Device-memory budget of a packet (runtime/budget.py, `plowrt budget`)."""
import json

import torch


def test_memory_plan_counts_what_the_packet_holds(tiny_assets, tmp_path, capsys):
    from plow_b200 import plowc, plowrt
    from plow_b200.compiler import emit, graph, hwspec, packet as pk, rewrite
    from plow_b200.models import config
    from plow_b200.runtime.budget import plan_memory
    pkt = pk.read_packet(tiny_assets / "assets" / "model.pkt")
    plan = plan_memory(pkt, 8 << 30, max_slots=8, max_ctx=512, kv_fraction=0.5, reserve_bytes=1 << 30)
    cfg = config.tiny_dense_config()
    # f32 model: 4 layers x (k, v) x 64 tokens x 2 kv heads x 64 dims x 4 bytes per page
    assert plan.page_bytes == 4 * 2 * 64 * 2 * 64 * 4 and plan.fp8_weight_bytes == 0
    n_params = config.spec_from_config(cfg).param_count()
    assert 0.95 * 4 * n_params < plan.weights_bytes < 1.25 * 4 * n_params          # + rope table, fused copies of q/k/v and gate/up
    assert plan.arena_bytes_max > 0 and plan.arena_bytes_sum >= plan.arena_bytes_max and plan.state_bytes == 0
    assert plan.n_pages == plan.budget_bytes // plan.page_bytes and plan.kv_tokens == plan.n_pages * 64
    assert plan.full_sequences == plan.n_pages // 8 and plan.pages_wanted == 64 and plan.fits
    assert not plan_memory(pkt, 1 << 20, 8, 512).fits                               # a megabyte of device memory: nothing fits
    # the headline shape at EP8: one rank's packet against a 180 GB device
    spec = config.spec_from_config(config.mla_moe_671b_config())
    g = graph.build_graph(spec, ep=8, rank=0)
    sites = rewrite.fuse(g)
    big = emit.emit_packet(g, sites, hwspec.lookup("b200"), 148, dict(prefill=[2048], decode=[64], max_seqs=64), rank=0)
    p8 = plan_memory(big, 180 << 30, max_slots=64, max_ctx=8768)
    assert 80 << 30 < p8.weights_bytes < 110 << 30 and p8.fp8_weight_bytes > 0.9 * p8.weights_bytes      # ~1/8 of the experts + the dense parts, e4m3
    assert p8.page_bytes == 61 * 64 * (512 + 64 + 4) and p8.fits and p8.full_sequences >= 64              # e4m3 latent + rope + scale per token
    # the hybrid carries recurrent state per slot
    hy = config.gdn_hybrid_80b_config()
    hy["num_hidden_layers"] = 8
    gh = graph.build_graph(config.spec_from_config(hy))
    rewrite.fuse(gh)
    ph = plan_memory(emit.emit_packet(gh, [], hwspec.lookup("b200"), 148, dict(prefill=[128], decode=[8], max_seqs=8)), 180 << 30, 8, 4096)
    assert ph.state_bytes > 0
    # CLI
    assert plowrt.main(["budget", "--assets", str(tiny_assets / "assets"), "--device-gb", "8", "--max-slots", "8", "--max-ctx", "512"]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["fits"] and out["gib"]["weights"] > 0 and out["n_pages"] > 0
    assert plowrt.main(["budget", "--assets", str(tiny_assets / "assets"), "--device-gb", "0.01"]) == 1
