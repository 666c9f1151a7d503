"""Expert-parallel MoE on 2+ GPUs: fused peer-memory dispatch/combine and the NCCL arm must both
reproduce the single-GPU engine (all experts local) on the same synthetic weights."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys, json
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["PLOW_ROOT"])
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
from plow_b200.compiler import emit, graph, hwspec, rewrite
from plow_b200.models.config import spec_from_config
from plow_b200.parallel.ep import EpComm
from plow_b200.runtime.engine import TokenBatch
from plow_b200.runtime.gpu_engine import GpuEngine, SyntheticWeights
from plow_b200.runtime.smoke import small_mla_moe_config
from plow_b200.compiler import packet as pk

cfg = small_mla_moe_config(experts=16)
spec = spec_from_config(cfg)

class SharedSeedWeights(SyntheticWeights):
    """Every tensor seeded by its name so ranks agree on replicated weights and experts can be cut out."""
    def __init__(self, dev, ep, rank, n_experts):
        super().__init__(dev)
        self.ep, self.rank, self.n_experts = ep, rank, n_experts
    def _full(self, ent, fp8):
        import zlib
        dims = [int(d) for d in ent.dims]
        # stacked expert matrices: "<...>.experts.<part>" holds e_local experts, "<...>.experts_shared.<part>" holds
        # e_local experts followed by the (replicated) shared expert
        shared = ent.name.startswith("cat/") and ".experts_shared." in ent.name
        stacked = shared or (ent.name.startswith("cat/") and ".experts." in ent.name)
        e_local = self.n_experts // self.ep
        blk = dims[0] // (e_local + (1 if shared else 0)) if stacked else 0
        if stacked:
            dims[0] = blk * (self.n_experts + (1 if shared else 0))      # the whole model's stack, same on every rank
        self.gen.manual_seed(zlib.crc32(ent.name.encode()))
        e = pk.TensorEnt(ent.name, ent.dtype, ent.tclass, tuple(dims))
        out = SyntheticWeights.fp8(self, e, None) if fp8 else SyntheticWeights.bf16(self, e, None)
        if stacked:
            rows = list(range(self.rank * e_local * blk, (self.rank + 1) * e_local * blk))
            if shared:
                rows += list(range(self.n_experts * blk, (self.n_experts + 1) * blk))
            idx = torch.tensor(rows, device=self.device)
            if fp8:
                sidx = torch.tensor(sorted({r // 128 for r in rows}), device=self.device)
                return out[0].view(torch.uint8)[idx].view(torch.float8_e4m3fn).contiguous(), out[1][sidx].contiguous()
            return out[idx].contiguous()
        return out
    def bf16(self, ent, recipe): return self._full(ent, False)
    def fp8(self, ent, recipe): return self._full(ent, True)

def build(ep, r, comm):
    g = graph.build_graph(spec, ep=ep, rank=r)
    sites = rewrite.fuse(g)
    pkt = emit.emit_packet(g, sites, hwspec.lookup("b200"), 148, dict(prefill=[128], decode=[8], max_seqs=8), rank=r)
    dev = torch.device("cuda", rank)
    return GpuEngine(packet=pkt, weights=SharedSeedWeights(dev, ep, r, 16), max_slots=8, max_ctx=512, rank=r, comm=comm, prefix_cache=False)

impl = os.environ["PLOW_IMPL"]
rng = np.random.default_rng(5 + rank)
prompt = rng.integers(0, 1024, size=90).astype(np.int32)
def run(eng):
    eng.begin_slot(0, prompt.tolist()); eng.reserve(0, 100)
    r = eng.step(TokenBatch(prompt, np.arange(90, dtype=np.int32), np.zeros(90, np.int32), np.array([89], np.int32), want_logits=True))
    eng.commit(0, prompt.tolist())
    outs = [r.logits[0].copy()]
    tok = int(r.ids[0])
    for i in range(3):
        r = eng.step(TokenBatch(np.array([tok], np.int32), np.array([90 + i], np.int32), np.zeros(1, np.int32), np.array([0], np.int32), decode=True, want_logits=True))
        eng.commit(0, [tok]); outs.append(r.logits[0].copy()); tok = int(r.ids[0])
    return outs
ref = run(build(1, 0, None))                 # every rank: all 16 experts local
comm = EpComm(rank, world, spec, max_rows=128, impl=impl)
got = run(build(world, rank, comm))
err = max(float(np.linalg.norm(a - b) / np.linalg.norm(b)) for a, b in zip(got, ref))
from plow_b200.ops import native
native.check_status()
t = torch.tensor([err], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX)
if rank == 0: print(json.dumps({"impl": impl, "max_rel_err": float(t)}))
dist.destroy_process_group()
'''


@pytest.mark.parametrize("impl", ["fused", "nccl"])
def test_ep_matches_single_gpu(impl, tmp_path):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    f = tmp_path / "worker.py"
    f.write_text(WORKER)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PLOW_ROOT=root, PLOW_IMPL=impl)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", "29611", str(f)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    import json
    line = [l for l in r.stdout.splitlines() if l.startswith("{")][-1]
    assert json.loads(line)["max_rel_err"] < 2e-2, line
