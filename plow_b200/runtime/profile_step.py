"""Where a step's device time goes: per-instruction and per-launcher times of one eager step of the MLA-MoE model.

    python -m plow_b200.runtime.profile_step --layers 8 --rows 2048            # one prefill chunk of 2048 rows
    python -m plow_b200.runtime.profile_step --layers 8 --decode --rows 64     # one decode step of 64 requests

Builds the fp8 MLA-MoE model (32 routed experts, synthetic weights) with the given number of layers, runs the step
twice untimed, then once with an event pair around every packet instruction (`GpuEngine.profile_ops`) and once with an
event pair around every kernel-launcher call (`ops/native.py` PROFILE hook; GEMMs are labelled with their shape and
tile).  Eager launches: the times include no CUDA-graph effects and a few microseconds of event overhead per call, so
compare shares, not absolutes.  A timing tool: nothing here is on the serving path.
"""
from __future__ import annotations

import argparse
import collections

import numpy as np
import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--rows", type=int, default=2048, help="prompt rows of the prefill chunk, or requests of the decode step")
    ap.add_argument("--decode", action="store_true")
    ap.add_argument("--ctx", type=int, default=0, help="tokens already cached before the step (prefill) / per request (decode)")
    args = ap.parse_args()
    from ..compiler import emit, graph, hwspec, rewrite
    from ..compiler.packet import Op
    from ..models.config import mla_moe_671b_config, spec_from_config
    from ..ops import native
    from .engine import TokenBatch
    from .gpu_engine import GpuEngine, SyntheticWeights

    L, N = args.layers, args.rows
    spec = spec_from_config(mla_moe_671b_config(n_experts=32, n_layers=L))
    g = graph.build_graph(spec, ep=1, rank=0)
    sites = rewrite.fuse(g)
    buckets = dict(prefill=[max(128, N)], decode=[N if args.decode else 8], max_seqs=max(8, N if args.decode else 8))
    pkt = emit.emit_packet(g, sites, hwspec.lookup("b200"), 148, buckets, rank=0)
    dev = torch.device("cuda", torch.cuda.current_device())
    slots = (N if args.decode else 1) + 1
    ctx = args.ctx or (4096 if args.decode else 0)
    eng = GpuEngine(packet=pkt, weights=SyntheticWeights(dev, seed=1, scaled_init_layers=L), max_slots=slots,
                    max_ctx=max(8192, ctx + N) + 64, prefix_cache=False, cuda_graphs=False)
    rng = np.random.default_rng(0)
    if args.decode:
        for s in range(N):
            eng.pool.begin(s, [0])
            eng.tokens[s] = [0] * ctx
            eng.kvlen[s] = ctx
            eng.reserve(s, ctx + 16)
        for ins in pkt.programs[0].insts:
            if ins.op == Op.MLA_KV_WRITE:        # synthetic cache pages need a per-page scale bound
                sm = torch.zeros(eng.static[ins.t[0]].shape[0], 4, dtype=torch.float32, device=dev)
                sm[:, 0] = 1.0
                eng.kv_smax[ins.i[7]] = sm

    step_no = [0]

    def run():
        if args.decode:
            i = step_no[0]
            step_no[0] += 1
            ids = rng.integers(0, spec.vocab, size=N).astype(np.int32)
            return eng.step(TokenBatch(ids, np.full(N, ctx + i, np.int32), np.arange(N, dtype=np.int32), np.arange(N, dtype=np.int32),
                                       decode=True)).device_ms
        n = ctx + N
        prompt = rng.integers(0, spec.vocab, size=n).astype(np.int32)
        eng.begin_slot(0, prompt.tolist())
        eng.reserve(0, n + 2)
        ms = 0.0
        for a in range(0, n, N):
            b = min(n, a + N)
            ms = eng.step(TokenBatch(prompt[a:b], np.arange(a, b, dtype=np.int32), np.zeros(b - a, np.int32),
                                     np.array([b - a - 1], np.int32))).device_ms
            eng.commit(0, prompt[a:b].tolist())
        eng.retire_slot(0)
        return ms                                    # the last chunk: the one that sees the whole context

    run()
    print(f"step (eager, untimed instruments): {run():.3f} ms")
    eng.profile_ops = True
    run()
    eng.profile_ops = False
    agg: dict = collections.OrderedDict()
    for name, i3, t in eng.op_times_last:
        e = agg.setdefault((name, i3 if name in ("GEMM", "MOE_GEMM") else ()), [0, 0.0])
        e[0] += 1
        e[1] += t
    tot = sum(v[1] for v in agg.values())
    print(f"\nper instruction (sum {tot:.3f} ms)")
    for k, (c, t) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
        print(f"  {k[0]:16s} {str(k[1]):24s} n={c:3d}  total {t:8.3f} ms  each {t / c * 1e3:8.1f} us  {100 * t / tot:5.1f} %")
    native.PROFILE = []
    run()
    rows = native.profile_summary()
    native.PROFILE = None
    tot = sum(t for _, _, t in rows)
    print(f"\nper launcher call (sum {tot:.3f} ms)")
    for k, c, t in rows:
        print(f"  {k:58s} n={c:3d}  total {t:8.3f} ms  each {t / c * 1e3:8.1f} us  {100 * t / tot:5.1f} %")
    native.check_status()


if __name__ == "__main__":
    main()
