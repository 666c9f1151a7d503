"""Decode-context-parallel layout + merge oracle, pipeline stage planning and the p2p pipeline runner (gloo)."""
import os
import subprocess
import sys

import torch


def test_dcp_layout_and_merge_equals_unsharded_attention():
    from plow_b200.parallel import dcp
    assert dcp.shard_lengths(200, 4) == [64, 64, 64, 8] and sum(dcp.shard_lengths(1000, 3)) == 1000
    assert dcp.owner_of_token(0, 4) == 0 and dcp.owner_of_token(64, 4) == 1 and dcp.owner_of_token(64 * 4 + 3, 4) == 0
    assert dcp.local_index(64 * 4 + 3, 4) == 64 + 3
    assert dcp.pages_needed(200, 4) == 1 and dcp.pages_needed(64 * 9, 4) == 3 and dcp.kv_budget_tokens(10, 8) == 5120
    torch.manual_seed(0)
    T, H, D = 333, 4, 32
    q, k, v = torch.randn(H, D), torch.randn(T, H, D), torch.randn(T, H, D)
    s = torch.einsum("hd,thd->ht", q, k) / D ** 0.5
    want = torch.einsum("ht,thd->hd", torch.softmax(s, -1), v)
    for d in (1, 2, 4, 8):
        got = dcp.reference_attention_sharded(q, k, v, d)
        assert torch.allclose(got, want, atol=1e-5), d


def test_stage_plan_balances_layers():
    from plow_b200.compiler import stage_plan
    from plow_b200.models.config import mla_moe_671b_config, spec_from_config
    p = stage_plan.plan_stages([1, 1, 1, 1, 4, 1, 1, 1, 1], 3)
    assert p["cuts"][0] == 0 and p["cuts"][-1] == 9 and p["beat_us"] == 4.0
    spec = spec_from_config(mla_moe_671b_config())
    costs = stage_plan.layer_costs_us(spec, batch=64, ctx=4096)
    assert len(costs) == 61 and all(c > 0 for c in costs)
    plan = stage_plan.plan_stages(costs, 4, head_us=5.0, tail_us=300.0)
    assert len(plan["stage_us"]) == 4 and plan["balance"] > 0.85 and plan["cuts"] == sorted(plan["cuts"])


WORKER = r'''
import os, sys, datetime
import torch, torch.distributed as dist
sys.path.insert(0, os.environ["PLOW_ROOT"])
from plow_b200.parallel.pp import PipelineRunner
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{os.environ['PORT']}", rank=rank, world_size=world,
                        timeout=datetime.timedelta(seconds=120))
torch.manual_seed(0)
ws = [torch.randn(16, 16) for _ in range(world)]          # every rank builds all stage weights, uses its own
stage = lambda x: torch.tanh(x @ ws[rank])
xs = [torch.randn(4, 16) for _ in range(5)]
runner = PipelineRunner(stage, rank, world, (4, 16))
outs = runner.run(xs if rank == 0 else None, 5)
if rank == world - 1:
    ok = True
    for x, y in zip(xs, outs):
        r = x
        for w in ws:
            r = torch.tanh(r @ w)
        ok = ok and torch.allclose(r, y, atol=1e-6)
    print("PIPELINE_OK" if ok else "PIPELINE_MISMATCH")
dist.destroy_process_group()
'''


def test_pipeline_runner_three_stages_gloo(tmp_path):
    f = tmp_path / "w.py"
    f.write_text(WORKER)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    port = 29800 + os.getpid() % 100
    procs = [subprocess.Popen([sys.executable, str(f)], env=dict(os.environ, PLOW_ROOT=root, RANK=str(r), WORLD_SIZE="3", PORT=str(port)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(3)]
    outs = [p.communicate(timeout=120)[0] for p in procs]
    assert "PIPELINE_OK" in outs[2], outs
