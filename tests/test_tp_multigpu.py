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
fused = TpComm(rank, world, impl="fused", form="oneshot")        # push partials to every rank, reduce locally
fused2 = TpComm(rank, world, impl="fused", form="twoshot")       # owner reduces from peer memory, stores to every rank
fused3 = TpComm(rank, world, impl="fused", form="nvls") if fused.mc_ptr and os.environ.get("PLOW_TEST_NVLS", "1") == "1" else None
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
    for form, comm in (("oneshot", fused), ("twoshot", fused2)) + ((("nvls", fused3),) if fused3 else ()):
        for call in range(3):
            y = comm.gemm_allreduce(xq, wq, N, sx=sx, sw=sw).clone()
            torch.cuda.synchronize(); native.check_status()
            err = ((y.float() - ref).norm() / ref.norm()).item()
            gathered = [torch.empty_like(y) for _ in range(world)]
            dist.all_gather(gathered, y)
            same = all(torch.equal(gathered[0], t) for t in gathered)
            out[f"{M}x{N}x{K}{'fp8' if fp8 else 'bf16'}/{form}#{call}"] = dict(err=err, identical=same)
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
                                 twoshot=timeit(lambda: fused2.gemm_allreduce(xq, wq, N, sx=sx, sw=sw)),
                                 nvls=(timeit(lambda: fused3.gemm_allreduce(xq, wq, N, sx=sx, sw=sw)) if fused3 else None),
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
    env = dict(os.environ, PLOW_ROOT=root)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29621", str(f)], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    print(json.dumps({k: v for k, v in res.items() if k.endswith("us")}))
    for k, v in res.items():
        if not k.endswith("us"):
            assert v["err"] < 1e-2 and v["identical"], (k, v)


ARN_WORKER = r'''
import os, sys, json
import torch, torch.distributed as dist
sys.path.insert(0, os.environ["PLOW_ROOT"])
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
from plow_b200.ops import native
from plow_b200.parallel.tp import TpComm
tp = TpComm(rank, world, impl="fused", ar_rows=2048, ar_width=8192)    # rows above the serving default, to cover the multi-row loop
out = {}
def rms(x, g, eps, plus_one):
    x = x.float()
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * ((1.0 + g.float()) if plus_one else g.float())
for (M, H, plus_one) in [(64, 4096, False), (5, 7168, True), (1500, 4096, False)]:
    g = torch.Generator(device="cuda").manual_seed(11 + rank)
    part = torch.randn(M, H, device="cuda", generator=g).bfloat16()
    gs = torch.Generator(device="cuda").manual_seed(5)               # same residual and weight on every rank
    x_in = torch.randn(M, H, device="cuda", generator=gs).bfloat16()
    gamma = (torch.randn(H, device="cuda", generator=gs) * 0.1 + (0.0 if plus_one else 1.0)).bfloat16()
    total = part.float().clone(); dist.all_reduce(total)
    want_sum = (x_in.float() + total.bfloat16().float()).bfloat16()
    want_norm = rms(want_sum, gamma, 1e-6, plus_one)
    for call in range(3):
        x_out = torch.empty(M, H, dtype=torch.bfloat16, device="cuda"); h_out = torch.empty_like(x_out)
        tp.allreduce_add_norm(part, x_in, gamma, x_out, h_out, 1e-6, plus_one)
        torch.cuda.synchronize(); native.check_status()
        gathered = [torch.empty_like(h_out) for _ in range(world)]
        dist.all_gather(gathered, h_out)
        out[f"{M}x{H}#{call}"] = dict(sum_err=((x_out.float() - want_sum.float()).norm() / want_sum.float().norm()).item(),
                                      norm_err=((h_out.float() - want_norm).norm() / want_norm.norm()).item(),
                                      identical=all(torch.equal(gathered[0], t) for t in gathered))
    # plain in-place all-reduce through the same kernel
    y = part.clone(); tp.all_reduce(y)
    torch.cuda.synchronize(); native.check_status()
    out[f"{M}x{H}ar"] = dict(sum_err=((y.float() - total).norm() / total.norm()).item(), norm_err=0.0, identical=True)
    def timeit(f, n=20):
        for _ in range(3): f()
        dist.barrier(); torch.cuda.synchronize()
        s = torch.cuda.Event(enable_timing=True); e = torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(n): f()
        e.record(); torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) * 1000 / n], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)
    x_out = torch.empty(M, H, dtype=torch.bfloat16, device="cuda"); h_out = torch.empty_like(x_out)
    from plow_b200.ops import rowops
    def nccl_arm():
        y = part.clone(); dist.all_reduce(y)
        native.call("plow_add_norm", h_out, None, None, M, x_out, x_in, y, gamma, M, H, 1e-6, int(plus_one))
    out[f"{M}x{H}us"] = dict(fused=timeit(lambda: tp.allreduce_add_norm(part, x_in, gamma, x_out, h_out, 1e-6, plus_one)), nccl=timeit(nccl_arm))
if rank == 0: print(json.dumps(out))
dist.destroy_process_group()
'''


def test_allreduce_add_norm_kernel(tmp_path):
    """All-reduce + residual + RMSNorm as one peer-memory kernel on 2 GPUs against the fp32 statement of the same three
    steps (NCCL all-reduce for the reference sum), at decode and prefill row counts; results identical on both ranks."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    f = tmp_path / "worker.py"
    f.write_text(ARN_WORKER)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PLOW_ROOT=root)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29627", str(f)], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    print(json.dumps({k: v for k, v in res.items() if k.endswith("us")}))
    for k, v in res.items():
        if not k.endswith("us"):
            assert v["sum_err"] < 1e-2 and v["norm_err"] < 1e-2 and v["identical"], (k, v)


AG_WORKER = r'''
import os, sys, json
import torch, torch.distributed as dist
sys.path.insert(0, os.environ["PLOW_ROOT"])
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
from plow_b200.ops import native
from plow_b200.parallel.tp import TpComm
fused = TpComm(rank, world, impl="fused", max_rows=128, max_k=8192)
nccl = TpComm(rank, world, impl="nccl")
out = {}
for (M, N, K) in [(64, 2048, 4096), (16, 1024, 512), (128, 3584, 8192)]:
    band = M // world
    g = torch.Generator(device="cuda").manual_seed(7 + rank)
    xb = torch.randn(band, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
    xs = [torch.empty_like(xb) for _ in range(world)]
    dist.all_gather(xs, xb)
    ref = torch.cat(xs).float() @ w.float().t()
    for call in range(3):
        y = fused.allgather_gemm(xb, w, N)
        torch.cuda.synchronize(); native.check_status()
        out[f"{M}x{N}x{K}#{call}"] = ((y.float() - ref).norm() / ref.norm()).item()
    def timeit(f, n=20):
        for _ in range(3): f()
        dist.barrier(); torch.cuda.synchronize()
        s = torch.cuda.Event(enable_timing=True); e = torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(n): f()
        e.record(); torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) * 1000 / n], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)
    out[f"{M}x{N}x{K}us"] = dict(fused=timeit(lambda: fused.allgather_gemm(xb, w, N)), nccl=timeit(lambda: nccl.allgather_gemm(xb, w, N)))
if rank == 0: print(json.dumps(out))
dist.destroy_process_group()
'''


ENGINE_WORKER = r'''
import os, sys, json, glob
import numpy as np
import torch, torch.distributed as dist
sys.path.insert(0, os.environ["PLOW_ROOT"])
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
from safetensors.torch import load_file
from plow_b200.models import config, reference
from plow_b200.parallel.tp import TpComm
from plow_b200.runtime.engine import TokenBatch
from plow_b200.runtime.gpu_engine import GpuEngine
d = os.environ["PLOW_ASSETS"]
cfg = json.load(open(os.path.join(d, "checkpoint", "config.json")))
out = {}
for impl in ("fused", "nccl"):
    tp = TpComm(rank, world, impl=impl, max_rows=64, max_n=4096, max_k=4096)
    eng = GpuEngine(d, max_slots=4, max_ctx=512, rank=rank, tp_comm=tp)
    state = {}
    for f in glob.glob(os.path.join(d, "checkpoint", "*.safetensors")):
        state.update(load_file(f))
    ref = reference.ReferenceModel(config.spec_from_config(cfg), {k: v.float() for k, v in state.items()})
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (90, 37)]
    ids, pos, seq, samp = [], [], [], []
    for s, p in enumerate(prompts):
        eng.begin_slot(s, p); eng.reserve(s, len(p) + 8)
        ids += p; pos += list(range(len(p))); seq += [s] * len(p); samp.append(len(ids) - 1)
    res = eng.step(TokenBatch(np.array(ids, np.int32), np.array(pos, np.int32), np.array(seq, np.int32), np.array(samp, np.int32), want_logits=True))
    errs = []
    for s, p in enumerate(prompts):
        want = ref.forward(torch.tensor(p))[-1]
        errs.append(((torch.from_numpy(res.logits[s]) - want).norm() / want.norm()).item())
        eng.commit(s, p)
    cur = [list(p) for p in prompts]
    toks = []
    for step in range(3):
        nxt = [int(ref.forward(torch.tensor(c))[-1].argmax()) for c in cur]
        for s in range(2): eng.reserve(s, len(cur[s]) + 2)
        r = eng.step(TokenBatch(np.array(nxt, np.int32), np.array([len(c) for c in cur], np.int32), np.array([0, 1], np.int32),
                                np.array([0, 1], np.int32), decode=True, want_logits=True))
        for s in range(2):
            cur[s].append(nxt[s]); eng.commit(s, [nxt[s]])
            want = ref.forward(torch.tensor(cur[s]))[-1]
            errs.append(((torch.from_numpy(r.logits[s]) - want).norm() / want.norm()).item())
        toks.append([int(t) for t in r.ids])
    t = torch.tensor(toks, device="cuda"); ts = [torch.empty_like(t) for _ in range(world)]; dist.all_gather(ts, t)
    out[impl] = dict(max_err=max(errs), same_tokens=all(torch.equal(ts[0], x) for x in ts))
    del eng, tp
if rank == 0: print(json.dumps(out))
dist.destroy_process_group()
'''


def _run(worker_src, tmp_path, port, extra_env=None, nproc=2, timeout=420):
    f = tmp_path / "worker.py"
    f.write_text(worker_src)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PLOW_ROOT=root, **(extra_env or {}))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), str(f)], env=env, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    return json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])


def test_fused_allgather_gemm(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    res = _run(AG_WORKER, tmp_path, 29622)
    print(json.dumps({k: v for k, v in res.items() if k.endswith("us")}))
    for k, v in res.items():
        if not k.endswith("us"):
            assert v < 1e-2, (k, v)


def test_dense_engine_tp2(tmp_path):
    """Dense GQA model compiled for TP=2: one engine per rank, row-parallel projections through the fused
    GEMM->all-reduce kernel (and the NCCL arm), logits vs the fp32 reference, identical greedy tokens on both ranks."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from plow_b200 import plowc
    from plow_b200.models import reference
    cfg = dict(model_type="llama", hidden_size=512, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
               num_hidden_layers=2, intermediate_size=1024, rms_norm_eps=1e-5, rope_theta=10000.0, vocab_size=1024,
               tie_word_embeddings=False, max_position_embeddings=2048, eos_token_id=2, plow_kv_dtype="bf16")
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=0, dtype=torch.bfloat16)
    plowc.compile_dir(tmp_path / "ckpt", tmp_path / "assets", max_rows=256, prefill_buckets=[128, 256], decode_rungs=[4, 8],
                      max_seqs=8, num_gpus=2, parallel="tp")
    res = _run(ENGINE_WORKER, tmp_path, 29623, extra_env=dict(PLOW_ASSETS=str(tmp_path / "assets")))
    for impl, v in res.items():
        assert v["max_err"] < 0.05 and v["same_tokens"], (impl, v)
