#!/usr/bin/env python
"""Headline benchmark: decode output tok/s per box (+ p50 TTFT / TPOT) of the fp8 MLA-MoE decoder
(671B-total shape at 8 GPUs) with expert parallelism over the GPUs of one node and data-parallel
attention.

    python bench.py --gpus 1 --steps 20 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 20 --warmup 3

Weak scaling: every GPU holds 32 routed experts per MoE layer and serves 64 concurrent requests, so
at 8 GPUs the model is exactly the named configuration (256 routed experts, 512 concurrent requests);
at fewer GPUs the expert count shrinks with the GPU count (256 experts do not fit below 8 x 180 GB).
Weights are random-init (block-scaled e4m3, 128x128 fp32 scales), prompts are synthetic: each request
has a context drawn uniformly from [1024, 8192] plus the tokens decoded so far; its latent cache is
filled with random e4m3 rows.  One step = one decode token for every live request.

Printed JSON: `value` is device-timed (CUDA events, max over ranks) aggregate tok/s; `e2e` is the same
metric through `GpuEngine.step()` — host token batch -> pinned H2D -> graph -> D2H ids — by wall clock.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

METRIC = "decode output tok/s per box (fp8 MLA-MoE, EP over the box, attention data-parallel)"


def reference_arm() -> int:
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference is a Rust/Nix workspace with no Python package (pip: 'neither setup.py nor "
                      "pyproject.toml found'), no cargo/rustc/nix on this image, and its compiler refuses --arch sm_100a"}))
    return 0


class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.mark_at = index, [], None, 0

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def mark(self):
        """Start of the timed region: the sampler is started earlier (nvidia-smi takes a moment to come up), only the
        samples taken from here on are reported."""
        self.mark_at = len(self.rows)
        return self

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        rows = self.rows[self.mark_at:] or self.rows[-1:]      # a very short region: the sample that straddles it
        self.rows = rows
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = max([int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()] or [0])
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 7 for i in range(4) if r[3 + i].lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": reasons, "samples": len(sm)}


def serving_phase(eng, spec, world, rank, n_req, n_out, chunk, slots, dev) -> dict:
    """One wave of `n_req` requests per GPU through ModelMux (the scheduler the HTTP server uses)."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from plow_b200.runtime.scheduler import GenParams, ModelMux, SchedConfig
    from plow_b200.text.tokenizer import ByteTokenizer
    for s in list(eng.pool.seqs):
        eng.retire_slot(s)
    if world > 1:
        from plow_b200.parallel.group import StepGroup
        eng.step_group = StepGroup(rank, world, timeout_s=120.0)
        eng.lockstep = True
        stats_pg = dist.new_group(backend="gloo")
    eng.max_slots = slots
    mux = ModelMux(eng, ByteTokenizer(), SchedConfig(token_budget=chunk, objective="auto", queue_ttl_s=3600.0))
    rng = np.random.default_rng(1000 + rank)
    prompts = [rng.integers(3, spec.vocab, size=int(n)).tolist() for n in rng.integers(1024, 8193, size=n_req)]
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    mux.start()
    reqs = [mux.submit(p, GenParams(max_tokens=n_out, ignore_eos=True)) for p in prompts]
    n_tok, failed = 0, 0
    for r in reqs:
        while True:
            ch = r.out.get(timeout=1800)
            if ch.kind == "token":
                n_tok += 1
            elif ch.kind == "done":
                break
            else:
                failed += 1
                break
    wall = time.perf_counter() - t0
    # The dispatcher thread keeps joining the other ranks' steps while this thread waits for the slowest rank.  The
    # totals travel over a CPU (gloo) group: a device collective issued from this thread would sit in the stream between
    # two steps of this rank and wait for ranks that are still stepping.
    snap = mux.metrics.snapshot()
    ttft, tpot = snap["ttft_ms"], snap["tpot_ms"]
    t = torch.tensor([float(n_tok), float(failed), float(sum(len(p) for p in prompts)), ttft["p50"] or 0.0, tpot["p50"] or 0.0,
                      ttft["p99"] or 0.0, tpot["p99"] or 0.0], dtype=torch.float64)
    w = torch.tensor([wall], dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=stats_pg)
        dist.all_reduce(w, op=dist.ReduceOp.MAX, group=stats_pg)
    mux.stop()
    eng.step_group, eng.lockstep = None, False
    tot_tok, tot_failed, tot_prompt, max_wall = float(t[0]), float(t[1]), float(t[2]), float(w[0])
    pair = t[3:] / world
    return {"requests": n_req * world, "output_tokens": int(tot_tok), "prompt_tokens": int(tot_prompt), "failed": int(tot_failed),
            "wall_s": round(max_wall, 2), "output_tok_s": round(tot_tok / max_wall, 1),
            "p50_ttft_ms": round(float(pair[0]), 1), "p50_tpot_ms": round(float(pair[1]), 3),
            "p99_ttft_ms": round(float(pair[2]), 1), "p99_tpot_ms": round(float(pair[3]), 3),
            "note": "one wave: every request arrives at t = 0, so TTFT includes the queue behind the other prompts' prefill; "
                    "percentiles are per rank, averaged over ranks",
            "counters": {k: snap["counters"].get(k) for k in ("prefill_ticks", "decode_ticks", "preemptions", "rider_rows")}}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="fused", choices=["fused", "nccl", "reference"])
    ap.add_argument("--layers", type=int, default=61, help="debug only: anything but 61 is not the named config")
    ap.add_argument("--batch-per-gpu", type=int, default=64)
    ap.add_argument("--ttft-prompts", type=int, default=2)
    ap.add_argument("--prefill-chunk", type=int, default=2048, help="rows of the prefill program used for the TTFT prompts")
    ap.add_argument("--serve-requests", type=int, default=-1,
                    help="requests per GPU of the serving phase that measures TTFT / TPOT under load through the scheduler "
                         "(-1: as many as decode slots; 0: skip the phase)")
    ap.add_argument("--serve-output", type=int, default=512, help="output tokens per request in the serving phase")
    ap.add_argument("--no-baseline", action="store_true", help="skip the NCCL-arm run that follows the timed region at N > 1")
    ap.add_argument("--init", default="scaled", choices=["scaled", "plain"],
                    help="scaled: depth-scaled random init (balanced routing, like a trained checkpoint); plain: N(0,0.02) everywhere")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()

    import numpy as np
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if world != args.gpus:
        print(f"bench.py: WORLD_SIZE={world} but --gpus {args.gpus}", file=sys.stderr)
        return 2
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from plow_b200.compiler import emit, graph, hwspec, rewrite
    from plow_b200.models.config import mla_moe_671b_config, spec_from_config
    from plow_b200.ops import native
    from plow_b200.runtime.engine import TokenBatch
    from plow_b200.runtime.gpu_engine import FP8, GpuEngine, SyntheticWeights

    B = args.batch_per_gpu
    W = max(3, args.warmup)
    cfg = mla_moe_671b_config(n_experts=32 * world, n_layers=args.layers)
    spec = spec_from_config(cfg)
    g = graph.build_graph(spec, ep=world, rank=rank)
    sites = rewrite.fuse(g)
    max_ctx = 8192 + 512 + 64
    pkt = emit.emit_packet(g, sites, hwspec.lookup("b200"), 148, dict(prefill=sorted({512, args.prefill_chunk}), decode=[B], max_seqs=max(8, B)), rank=rank)
    comm = None
    if world > 1:
        from plow_b200.parallel.ep import EpComm
        comm = EpComm(rank, world, spec, max_rows=max(512, args.prefill_chunk), impl=args.impl)
    dev = torch.device("cuda", local)
    t_load = time.time()
    eng = GpuEngine(packet=pkt, weights=SyntheticWeights(dev, seed=1234 + rank, scaled_init_layers=(args.layers if args.init == "scaled" else 0)), max_slots=B + 1, max_ctx=max_ctx,
                    prefix_cache=False, rank=rank, comm=comm)
    load_s = time.time() - t_load

    # ---- synthetic live requests: contexts uniform in [1024, 8192], random e4m3 latent rows ----
    rng = np.random.default_rng(7 + rank)
    ctx = rng.integers(1024, 8193, size=B)
    total_steps = 3 * W + 2 * args.steps + 2
    for s in range(B):
        eng.pool.begin(s, [0])
        eng.tokens[s] = [0] * int(ctx[s])
        eng.kvlen[s] = int(ctx[s])
        eng.reserve(s, int(ctx[s]) + total_steps + 2)
    gen = torch.Generator(device=dev).manual_seed(99 + rank)
    for h, t in enumerate(pkt.tensors):
        if t.name.endswith(".latent"):
            flat = eng.static[h].view(-1)
            for i in range(0, flat.numel(), 1 << 28):
                m = min(1 << 28, flat.numel() - i)
                flat[i:i + m] = (torch.randn(m, device=dev, generator=gen) * 64.0).to(FP8)
        elif t.name.endswith(".latent_scale"):
            eng.static[h].fill_(1.0 / 64.0)
    # the cache writer keeps a per-page upper bound of the scales; the synthetic pages need one too
    from plow_b200.compiler.packet import Op as _Op
    for ins in pkt.programs[0].insts:
        if ins.op == _Op.MLA_KV_WRITE:
            sm = torch.zeros(eng.static[ins.t[0]].shape[0], 4, dtype=torch.float32, device=dev)
            sm[:, 0] = 1.0 / 64.0
            eng.kv_smax[ins.i[7]] = sm
    eng_prefill_ttft = []

    # ---- TTFT: real chunked prefill of fresh prompts in the spare slot (512-row ticks) ----
    def prefill_once(n_tokens: int) -> float:
        slot = B
        prompt = rng.integers(0, spec.vocab, size=n_tokens).astype(np.int32)
        eng.begin_slot(slot, prompt.tolist())
        eng.reserve(slot, n_tokens + 2)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for a in range(0, n_tokens, args.prefill_chunk):
            b = min(n_tokens, a + args.prefill_chunk)
            eng.step(TokenBatch(prompt[a:b], np.arange(a, b, dtype=np.int32), np.full(b - a, slot, np.int32),
                                np.array([b - a - 1], np.int32)))
        dt = (time.perf_counter() - t0) * 1e3
        eng.retire_slot(slot)
        return dt

    ids = rng.integers(0, spec.vocab, size=B).astype(np.int32)
    seq = np.arange(B, dtype=np.int32)
    samp = np.arange(B, dtype=np.int32)

    def one_step(k: int):
        pos = (ctx + k).astype(np.int32)
        r = eng.step(TokenBatch(ids, pos, seq, samp, decode=True))
        for s in range(B):
            eng.kvlen[s] += 1
        return r

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local).start()        # started before the warm-up; mark() opens the reported window
    for k in range(W):
        one_step(k)
    n0 = native.LAUNCHES["n"]
    launches_per_step = None
    # kernels per decode step: count one eager walk of the program (the graph replays the same launches)
    st = eng.progs[eng.pick_program(B, True)]
    n0 = native.LAUNCHES["n"]
    eng._run_insts(st)
    torch.cuda.synchronize()
    launches_per_step = native.LAUNCHES["n"] - n0

    barrier()
    sampler.mark()
    t0 = time.perf_counter()
    dev_ms = []
    for k in range(args.steps):
        r = one_step(W + k)
        dev_ms.append(r.device_ms)
    barrier()
    wall = time.perf_counter() - t0
    clocks = sampler.stop()

    # ---- same-box baseline: the NCCL arm of the same model (all-gather + local experts + reduce-scatter, NCCL at its
    # defaults), same engine, weights, requests, warm-up and step count; only the expert-parallel layer differs ----
    base = None
    if comm is not None and args.impl == "fused" and not args.no_baseline:
        comm.impl = "nccl"
        st.graph = None
        for k in range(W):
            one_step(W + args.steps + k)
        barrier()
        b_ms = [one_step(2 * W + args.steps + k).device_ms for k in range(args.steps)]
        barrier()
        comm.impl = "fused"
        st.graph = None
        bt = torch.tensor([float(np.sum(b_ms))], dtype=torch.float64, device=dev)
        dist.all_reduce(bt, op=dist.ReduceOp.MAX)
        base = float(bt.item())
    route = None
    if comm is not None and getattr(comm, "grp_off", None) is not None:
        go = comm.grp_off.cpu().numpy().astype(np.int64)       # rows per local expert in the last MoE layer
        per = np.diff(go)
        rs = torch.tensor([float(go[-1]), float(per.max())], dtype=torch.float64, device=dev)
        mx = rs.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        route = {"rows_rank0": int(go[-1]), "max_rows_any_rank": int(mx[0]), "max_rows_one_expert": int(mx[1]),
                 "mean_rows_per_rank": B * 8}
    ttfts, ttft_lens = [], []
    # every rank prefills a prompt of the same length at the same time (EP layers are collective); one untimed prompt
    # that touches every prefill bucket first (lazy scratch allocations are not part of a steady-state TTFT)
    if args.ttft_prompts:
        prefill_once(args.prefill_chunk + 100)
    for n in list(np.random.default_rng(11).integers(1024, 8193, size=args.ttft_prompts)):
        ttft_lens.append(int(n))
        ttfts.append(prefill_once(int(n)))
    # ---- serving phase: the named workload through the scheduler.  Every GPU gets `serve_requests` requests at once
    # (prompts uniform in [1024, 8192] random token ids, `serve_output` output tokens each, greedy, EOS ignored); the
    # continuous-batching scheduler of each rank prefills in chunks, decodes, and the ranks step in lockstep
    # (plow_b200/parallel/group.py).  TTFT / TPOT are the scheduler's own per-request measurements.
    serve = None
    n_serve = B if args.serve_requests < 0 else args.serve_requests
    if n_serve:
        try:
            serve = serving_phase(eng, spec, world, rank, n_serve, args.serve_output, args.prefill_chunk, B, dev)
        except Exception as e:          # the decode-step figures above stand on their own
            serve = {"error": f"{type(e).__name__}: {e}"[:300]}
    dev_total = float(np.sum(dev_ms))
    stats = torch.tensor([dev_total, wall, float(np.median(dev_ms))], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    dev_total, wall, tpot = [float(v) for v in stats.tolist()]
    tokens = B * world * args.steps
    value = tokens / (dev_total / 1e3)
    e2e = tokens / wall
    if rank == 0:
        hbm, src = hwspec.lookup("b200", peaks_file=os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")).hbm_peak()
        out = {
            "metric": METRIC, "value": round(value, 1), "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": W,
            "ms_per_step": round(dev_total / args.steps, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (None if base is None else {"impl": "nccl", "value": round(tokens / (base / 1e3), 1),
                                                       "ms_per_step": round(base / args.steps, 3), "ratio": round(base / dev_total, 4)}),
            "dtype": "fp8 (e4m3 block-scaled weights, e4m3 latent KV, bf16 activations)", "data": ("synthetic: random token ids, random e4m3 latent cache, random-init weights "
                     + ("(N(0,0.02); unit-variance embeddings and residual-output projections scaled by 1/(2L), which keeps "
                        "expert routing balanced as in a trained checkpoint)" if args.init == "scaled" else "(N(0,0.02) everywhere; routing collapses with depth)")),
            "impl": args.impl,
            "config": {"model": f"MLA-MoE 671B-shape ({32 * world} routed experts, {args.layers} layers)", "global_batch": B * world,
                       "seq_len": "ctx uniform 1024-8192 + decoded tokens", "parallelism": f"ep{world} + dp-attention",
                       "l2": "no flush needed: each step streams >90 GB of weights and KV per GPU (L2 is 126 MB)",
                       "named_config": bool(world == 8 and args.layers == 61)},
            "p50_tpot_ms": (serve or {}).get("p50_tpot_ms"), "p50_ttft_ms": (serve or {}).get("p50_ttft_ms"),
            "serving": serve, "decode_step_p50_ms": round(tpot, 3),
            "idle_ttft_ms": round(float(np.median(ttfts)), 1) if ttfts else None, "idle_ttft_ms_all": [round(t, 1) for t in ttfts],
            "idle_ttft_prompt_tokens": ttft_lens,
            "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": int(4 * 4 * B), "d2h_bytes_per_step": int(4 * B)},
            "gpu_launches": int(launches_per_step * args.steps), "launches_per_step": int(launches_per_step),
            "clocks": clocks, "load_s": round(load_s, 1), "ep_routing_last_layer": route,
            "hbm_peak_gbs": hbm, "hbm_peak_source": src,
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
