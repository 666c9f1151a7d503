"""Device-side phase trace of the expert-parallel MoE layer under CUDA-graph replay.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m plow_b200.parallel.ep_trace --layers 9 --batch 64

Builds the MLA-MoE model with synthetic weights on every rank (32 routed experts per rank), warms the decode program up
until its graph is captured, then replays one step with the EP kernels' trace marks on (globaltimer stamps written by
CTA 0 of the push and combine kernels: csrc/comm/ep.cu, `trace_mark`).  Prints, per MoE layer and rank, how long the
rank waited for the other ranks' counts, the push preamble / row copies / system fence, the two expert GEMMs (push end
to combine start: includes the in-kernel wait for the peers' rows), the wait for the peers' outputs and the combine.
A timing tool: nothing here is on the serving path.
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
    ap.add_argument("--layers", type=int, default=9)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--json", default="", help="also write the raw marks of every rank to <path>.<rank>.json")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from ..compiler import emit, graph, hwspec, rewrite
    from ..compiler.packet import Op
    from ..models.config import mla_moe_671b_config, spec_from_config
    from ..ops import native
    from ..runtime.engine import TokenBatch
    from ..runtime.gpu_engine import GpuEngine, SyntheticWeights
    from .ep import EpComm

    L, B = args.layers, args.batch
    spec = spec_from_config(mla_moe_671b_config(n_experts=32 * world, n_layers=L))
    g = graph.build_graph(spec, ep=world, rank=rank)
    sites = rewrite.fuse(g)
    pkt = emit.emit_packet(g, sites, hwspec.lookup("b200"), 148, dict(prefill=[512], decode=[B], max_seqs=B), rank=rank)
    comm = EpComm(rank, world, spec, max_rows=512, impl="fused")
    dev = torch.device("cuda", torch.cuda.current_device())
    eng = GpuEngine(packet=pkt, weights=SyntheticWeights(dev, seed=1 + rank, scaled_init_layers=L), max_slots=B + 1,
                    max_ctx=8192 + 64, prefix_cache=False, rank=rank, comm=comm)
    rng = np.random.default_rng(rank)
    ctx = rng.integers(1024, 8000, size=B)
    for s in range(B):
        eng.pool.begin(s, [0])
        eng.tokens[s] = [0] * int(ctx[s])
        eng.kvlen[s] = int(ctx[s])
        eng.reserve(s, int(ctx[s]) + 40)
    for ins in pkt.programs[0].insts:
        if ins.op == Op.MLA_KV_WRITE:          # synthetic cache pages need a per-page scale bound
            sm = torch.zeros(eng.static[ins.t[0]].shape[0], 4, dtype=torch.float32, device=dev)
            sm[:, 0] = 1.0
            eng.kv_smax[ins.i[7]] = sm
    comm.device_trace(True)                    # before the graph is captured: the trace pointer is a kernel argument

    def one(i):
        ids = rng.integers(0, spec.vocab, size=B).astype(np.int32)
        return eng.step(TokenBatch(ids, (ctx + i).astype(np.int32), np.arange(B, dtype=np.int32), np.arange(B, dtype=np.int32), decode=True))
    for i in range(6):
        one(i)
    torch.cuda.synchronize()
    dist.barrier()
    comm._trace.zero_()
    ms = one(6).device_ms
    torch.cuda.synchronize()
    rows = comm.device_trace_rows()
    native.check_status()
    if args.json:
        json.dump(dict(rank=rank, ms=ms, rows=rows), open(f"{args.json}.{rank}.json", "w"))
    layers, cur = [], {}
    for tag, ts in rows:
        if tag == 3 and cur:
            layers.append(cur)
            cur = {}
        cur.setdefault(tag, ts)
    layers.append(cur)

    def gap(l, a, b):
        return f"{(l[b] - l[a]) / 1000:7.1f}" if a in l and b in l else "      -"
    lines = [f"rank {rank}: step {ms:.3f} ms, {len(layers)} MoE layers (us per layer)",
             "layer  cnt_wait   counts  preamble   rows    fence    tail    gemms   y_wait  combine"]
    for i, l in enumerate(layers):
        lines.append(f"{i:5d}  " + "  ".join(gap(l, a, b) for a, b in ((3, 4), (4, 40), (40, 41), (41, 42), (42, 43), (43, 5), (5, 7), (7, 8), (8, 9))))
    for r in range(world):
        if r == rank:
            print("\n".join(lines), flush=True)
        dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
