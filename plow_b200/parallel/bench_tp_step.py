"""Decode step of the dense 8B model under tensor parallelism, three ways of doing the row-parallel reductions.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m plow_b200.parallel.bench_tp_step --batch 64

Compiles the Llama-3-8B-shaped model (synthetic weights) for TP = world size three times: (a) the compiler's default
(all-reduce + residual + RMSNorm as one peer-memory kernel after a plain GEMM), (b) the reduction inside the GEMM
epilogue (rule `xreduce-add-norm-fuse` off, so `gemm-xreduce-fuse` takes the reductions), (c) NCCL all-reduce + the
add/norm row kernel.  Every variant runs the same decode batch from a captured CUDA graph; prints the median step time
(MAX over ranks) of each as one JSON line.  A timing tool: nothing here is on the serving path.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--steps", type=int, default=10)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from ..compiler import emit, graph, hwspec, rewrite
    from ..models.config import dense_8b_config, spec_from_config
    from ..ops import native
    from ..runtime.engine import TokenBatch
    from ..runtime.gpu_engine import GpuEngine, SyntheticWeights
    from .tp import TpComm

    B = args.batch
    spec = spec_from_config(dense_8b_config())
    dev = torch.device("cuda", torch.cuda.current_device())
    res = {}
    for name, impl, disable in (("allreduce_add_norm_kernel", "fused", set()), ("reduction_in_gemm_epilogue", "fused", {"xreduce-add-norm-fuse"}),
                                ("nccl", "nccl", set())):
        g = graph.build_graph(spec, tp=world, rank=rank)
        sites = rewrite.fuse(g, disable=disable)
        pkt = emit.emit_packet(g, sites, hwspec.lookup("b200"), 148, dict(prefill=[512], decode=[B], max_seqs=B), rank=rank)
        tp = TpComm(rank, world, impl=impl, max_rows=128, max_n=16384, max_k=16384)
        eng = GpuEngine(packet=pkt, weights=SyntheticWeights(dev, seed=1, scaled_init_layers=len(spec.layers)), max_slots=B + 1,
                        max_ctx=2048 + 64, prefix_cache=False, rank=rank, tp_comm=tp)
        rng = np.random.default_rng(0)                 # every rank runs the same token batch
        ctx = rng.integers(512, 2000, size=B)
        for s in range(B):
            eng.pool.begin(s, [0])
            eng.tokens[s] = [0] * int(ctx[s])
            eng.kvlen[s] = int(ctx[s])
            eng.reserve(s, int(ctx[s]) + args.steps + 16)

        def one(i):
            ids = rng.integers(0, spec.vocab, size=B).astype(np.int32)
            return eng.step(TokenBatch(ids, (ctx + i).astype(np.int32), np.arange(B, dtype=np.int32), np.arange(B, dtype=np.int32),
                                       decode=True)).device_ms
        for i in range(5):
            one(i)
        dist.barrier()
        ms = [one(5 + i) for i in range(args.steps)]
        native.check_status()
        t = torch.tensor([float(np.median(ms))], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res[name] = round(float(t), 3)
        del eng, tp
        torch.cuda.empty_cache()
    if rank == 0:
        print(json.dumps(dict(model="dense 8B", tp=world, batch=B, ms_per_step=res)))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
