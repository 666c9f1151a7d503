"""Closed-loop serving benchmark of a named model shape with synthetic weights, through the scheduler the server uses.

    python -m plow_b200.serve.bench_synth --config dense8b --requests 256 --concurrency 64 \\
        --prompt-min 512 --prompt-max 4096 --output 256                                  # one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m plow_b200.serve.bench_synth --config dense8b --requests 256 --concurrency 64   # tensor parallel over the ranks

Shapes: `dense8b` (32-layer GQA decoder, bf16), `gdn80b` (gated-delta-rule / gated-attention hybrid MoE; `--layers`
cuts it down, the full shape needs several GPUs), `mla_moe` (fp8 MLA-MoE, 32 routed experts), `mla_moe_dsa` (the same
with a sparse-attention indexer per layer, top-2048).  `--arrival-rate R` switches from the closed loop to Poisson
arrivals at R requests per second (open loop: requests queue when all slots are busy); `--shared-prefix-frac F
--shared-prefix-len N` gives a fraction F of the prompts one common N-token prefix (exercises the prefix cache).  Weights are random
(`SyntheticWeights`), prompts are uniform random token ids, EOS is ignored.  With more than one rank the model is
compiled for tensor parallelism: rank 0 owns the scheduler and broadcasts every step, the other ranks replay it
(`parallel/group.py`, LeaderGroup).  At most `--concurrency` requests are in flight; a finished request is replaced by
the next one.  Prints one JSON line: output tok/s, total tok/s, p50 / p99 TTFT and TPOT from the scheduler's metrics.
"""
from __future__ import annotations

import argparse
import json
import os
import threading
import time

import numpy as np
import torch
import torch.distributed as dist


def _teardown() -> None:
    """Leave the process group without waiting on it for ever: on this stack `destroy_process_group` has been seen to
    block in both ranks after a serving run that used symmetric memory from a second host thread; the results are
    already printed, so the teardown gets 20 s and the process exits either way."""
    import sys
    torch.cuda.synchronize()
    t = threading.Thread(target=dist.destroy_process_group, daemon=True)
    t.start()
    t.join(20.0)
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="dense8b", choices=["dense8b", "gdn80b", "mla_moe", "mla_moe_dsa"])
    ap.add_argument("--arrival-rate", type=float, default=0.0, help="Poisson arrivals per second (0: closed loop at --concurrency)")
    ap.add_argument("--shared-prefix-frac", type=float, default=0.0)
    ap.add_argument("--shared-prefix-len", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0: the shape's own)")
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--concurrency", type=int, default=64)
    ap.add_argument("--prompt-min", type=int, default=512)
    ap.add_argument("--prompt-max", type=int, default=4096)
    ap.add_argument("--output", type=int, default=256)
    ap.add_argument("--chunk", type=int, default=2048, help="largest prefill bucket / rows per scheduler tick")
    ap.add_argument("--multi-step", type=int, default=1)
    ap.add_argument("--lookahead", action="store_true", help="lookahead-1 decode pipeline")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if os.environ.get("PLOW_DUMP_STACKS_AFTER_S"):
        # diagnostic: print every thread's stack if the run is still going after this many seconds
        import faulthandler
        faulthandler.dump_traceback_later(float(os.environ["PLOW_DUMP_STACKS_AFTER_S"]), exit=True)
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from ..compiler import emit, graph, hwspec, rewrite
    from ..models import config as cfgs
    from ..ops import native
    from ..parallel.group import LeaderGroup, follower_loop
    from ..runtime.gpu_engine import GpuEngine, SyntheticWeights
    from ..runtime.scheduler import GenParams, ModelMux, SchedConfig
    from ..text.tokenizer import ByteTokenizer

    cfg = {"dense8b": cfgs.dense_8b_config, "gdn80b": cfgs.gdn_hybrid_80b_config,
           "mla_moe": lambda: cfgs.mla_moe_671b_config(n_experts=32),
           "mla_moe_dsa": lambda: cfgs.mla_moe_671b_config(n_experts=32, dsa=True)}[args.config]()
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    spec = cfgs.spec_from_config(cfg)
    C = args.concurrency
    g = graph.build_graph(spec, tp=world, rank=rank)
    sites = rewrite.fuse(g)
    rungs = sorted({r for r in (1, 2, 4, 8, 16, 32, 64, 128, 256) if r < C} | {C})
    pkt = emit.emit_packet(g, sites, hwspec.lookup("b200"), 148, dict(prefill=sorted({512, args.chunk}), decode=rungs, max_seqs=max(8, C)),
                           rank=rank)
    dev = torch.device("cuda", torch.cuda.current_device())
    tp = lg = None
    if world > 1:
        from ..parallel.tp import TpComm
        tp = TpComm(rank, world, impl="fused", max_rows=128, max_n=max(16384, spec.hidden), max_k=16384, ar_width=max(8192, spec.hidden))
        lg = LeaderGroup(rank, world, timeout_s=600.0)
    eng = GpuEngine(packet=pkt, weights=SyntheticWeights(dev, seed=1, scaled_init_layers=len(spec.layers)), max_slots=C,
                    max_ctx=args.prompt_max + args.output + 64, prefix_cache=args.shared_prefix_frac > 0, rank=rank, tp_comm=tp,
                    leader_group=lg)
    if world > 1 and rank != 0:
        follower_loop(eng, lg)
        native.check_status()
        _teardown()
        return
    rng = np.random.default_rng(7)
    prompts = [rng.integers(3, spec.vocab, size=int(n)).tolist() for n in rng.integers(args.prompt_min, args.prompt_max + 1, size=args.requests)]
    if args.shared_prefix_frac > 0 and args.shared_prefix_len > 0:
        common = rng.integers(3, spec.vocab, size=args.shared_prefix_len).tolist()
        for i in range(len(prompts)):
            if rng.random() < args.shared_prefix_frac and len(prompts[i]) > args.shared_prefix_len:
                prompts[i][:args.shared_prefix_len] = common
    mux = ModelMux(eng, ByteTokenizer(), SchedConfig(token_budget=args.chunk, objective="auto", queue_ttl_s=36000.0, multi_step=args.multi_step, lookahead=args.lookahead),
                   eos_ids=[]).start()
    lock, state = threading.Lock(), dict(next=0, out=0, failed=0)

    def client():
        while True:
            with lock:
                i = state["next"]
                state["next"] += 1
            if i >= len(prompts):
                return
            r = mux.submit(prompts[i], GenParams(max_tokens=args.output, ignore_eos=True))
            n = 0
            while True:
                ch = r.out.get(timeout=3600)
                if ch.kind == "token":
                    n += 1
                elif ch.kind == "done":
                    break
                else:
                    with lock:
                        state["failed"] += 1
                        state.setdefault("first_error", ch.error)
                    break
            with lock:
                state["out"] += n

    def drain(r):
        n = 0
        while True:
            ch = r.out.get(timeout=3600)
            if ch.kind == "token":
                n += 1
            elif ch.kind == "done":
                break
            else:
                with lock:
                    state["failed"] += 1
                    state.setdefault("first_error", ch.error)
                break
        with lock:
            state["out"] += n

    torch.cuda.synchronize()
    t0 = time.perf_counter()
    if args.arrival_rate > 0:
        # open loop: exponential gaps between submissions, one collector thread per request
        threads = []
        for p in prompts:
            r = mux.submit(p, GenParams(max_tokens=args.output, ignore_eos=True))
            th = threading.Thread(target=drain, args=(r,), daemon=True)
            th.start()
            threads.append(th)
            time.sleep(float(rng.exponential(1.0 / args.arrival_rate)))
    else:
        threads = [threading.Thread(target=client, daemon=True) for _ in range(C)]
        for t in threads:
            t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    snap = mux.metrics.snapshot()
    mux.stop()
    if lg is not None:
        lg.stop()
    native.check_status()
    n_prompt = sum(len(p) for p in prompts)
    print(json.dumps(dict(config=args.config, layers=len(spec.layers), tp=world, requests=args.requests, concurrency=C,
                          prompt_tokens=n_prompt, output_tokens=state["out"], failed=state["failed"], first_error=state.get("first_error"), wall_s=round(wall, 2),
                          output_tok_s=round(state["out"] / wall, 1), total_tok_s=round((state["out"] + n_prompt) / wall, 1),
                          ttft_ms=snap["ttft_ms"], tpot_ms=snap["tpot_ms"],
                          arrival_rate=args.arrival_rate or None,
                          counters={k: snap["counters"].get(k) for k in ("prefill_ticks", "decode_ticks", "preemptions", "rider_rows", "multi_step_calls", "lookahead_launches", "cached_tokens")},
                          data="synthetic: random token ids, random-init weights")), flush=True)
    if world > 1:
        _teardown()


if __name__ == "__main__":
    main()
