"""Fused GEMM -> all-reduce over peer memory on 2 GPUs vs an fp32 reference of the same sum, plus the
NCCL arm and a device-timed comparison (printed, not asserted)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys, json
import torch, torch.distributed as dist
sys.path.insert(0, os.environ["PLOW_ROOT"])
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
from plow_b200.ops import native, quant
from plow_b200.parallel.tp import TpComm
fused = TpComm(rank, world, impl="fused")
nccl = TpComm(rank, world, impl="nccl")
out = {}
for (M, N, K, fp8) in [(64, 7168, 8192, True), (17, 1024, 2048, False), (64, 4096, 7168, False)]:
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    x = torch.randn(M, K, device="cuda", generator=g)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.05
    if fp8:
        xq, sx = quant.quant_act_1x128(x); wq, sw = quant.quant_weight_128x128(w)
        xr, wr = quant.dequant_act_1x128(xq, sx), quant.dequant_weight_128x128(wq, sw)
    else:
        xq, wq, sx, sw = x.bfloat16(), w.bfloat16(), None, None
        xr, wr = xq.float(), wq.float()
    part = (xr @ wr.t()).bfloat16().float()
    ref = part.clone(); dist.all_reduce(ref)
    for call in range(2):
        y = fused.gemm_allreduce(xq, wq, N, sx=sx, sw=sw).clone()
        torch.cuda.synchronize(); native.check_status()
        err = ((y.float() - ref).norm() / ref.norm()).item()
        gathered = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(gathered, y)
        same = all(torch.equal(gathered[0], t) for t in gathered)
        out[f"{M}x{N}x{K}{'fp8' if fp8 else 'bf16'}#{call}"] = dict(err=err, identical=same)
    yn = nccl.gemm_allreduce(xq, wq, N, sx=sx, sw=sw)
    out[f"{M}x{N}x{K}nccl"] = dict(err=((yn.float() - ref).norm() / ref.norm()).item(), identical=True)
    def timeit(f, n=20):
        for _ in range(3): f()
        dist.barrier(); torch.cuda.synchronize()
        s = torch.cuda.Event(enable_timing=True); e = torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(n): f()
        e.record(); torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) * 1000 / n], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)
    out[f"{M}x{N}x{K}us"] = dict(fused=timeit(lambda: fused.gemm_allreduce(xq, wq, N, sx=sx, sw=sw)),
                                 nccl=timeit(lambda: nccl.gemm_allreduce(xq, wq, N, sx=sx, sw=sw)))
if rank == 0: print(json.dumps(out))
dist.destroy_process_group()
'''


def test_fused_gemm_allreduce(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    f = tmp_path / "worker.py"
    f.write_text(WORKER)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PLOW_ROOT=root, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29621", str(f)], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    print(json.dumps({k: v for k, v in res.items() if k.endswith("us")}))
    for k, v in res.items():
        if not k.endswith("us"):
            assert v["err"] < 1e-2 and v["identical"], (k, v)
