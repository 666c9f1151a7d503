"""``plowrt`` — load a packet directory and serve / bench / inspect it.

Subcommands: ``serve`` (OpenAI API), ``bench`` (drive the production scheduler without HTTP),
``show`` (packet summary), ``disasm`` (instruction listing), ``simulate`` (walk the counter
protocol on the host), ``devices``, ``knob-scope``, ``inventory`` (which opcodes a packet needs and
which backend bodies exist).  Reference: crates/plowrt/src/main.rs:58-940.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

from . import config as cfgmod
from .compiler import disasm as disasm_mod, packet as pk, schedule


def load_engine(assets, cfg: cfgmod.RuntimeConfig, device=None):
    backend = cfg.backend
    if backend == "auto":
        import torch
        backend = "cuda" if torch.cuda.is_available() else "cpu"
    if backend == "cpu":
        from .runtime.cpu_engine import CpuEngine
        return CpuEngine(assets, max_slots=cfg.max_slots, max_ctx=cfg.max_ctx, n_pages=cfg.n_pages or None,
                         prefix_cache=cfg.prefix_cache)
    from .runtime.gpu_engine import GpuEngine
    return GpuEngine(assets, max_slots=cfg.max_slots, max_ctx=cfg.max_ctx, n_pages=cfg.n_pages or None,
                     kv_fraction=cfg.kv_fraction, prefix_cache=cfg.prefix_cache, cuda_graphs=cfg.cuda_graphs, device=device)


def make_entry(name, assets, cfg):
    from .runtime.scheduler import ModelMux, SchedConfig
    from .serve.app import ModelEntry
    from .serve.template import ChatTemplate
    from .text.tokenizer import load_tokenizer
    build = Path(assets) / "build.json"
    if build.exists():
        for p in cfgmod.check_assets(json.loads(build.read_text()), cfg):
            print(f"plowrt: warning: {p}", file=sys.stderr)
    eng = load_engine(assets, cfg)
    tok = load_tokenizer(assets)
    sched = SchedConfig(token_budget=min(cfg.token_budget, eng.max_rows(False)), objective=cfg.objective,
                        tbt_target_ms=cfg.tbt_target_ms, queue_ttl_s=cfg.queue_ttl_s, ride=cfg.ride, spec_depth=cfg.spec_depth, multi_step=cfg.multi_step, lookahead=cfg.lookahead, rung_control=cfg.rung_control)
    mux = ModelMux(eng, tok, sched)
    mtp_dir = Path(assets) / "mtp"
    if cfg.spec_depth > 0 and cfg.spec_drafter != "ngram":
        pairing = eng.packet.section_json("spec.json") or {}
        if pairing.get("kind") == "mtp" and pairing.get("drafter_packet"):
            mtp_dir = (Path(assets) / pairing["drafter_packet"]).parent
        if (mtp_dir / "model.pkt").exists():
            # the prediction module runs in an engine of its own (own KV pages, same device) behind the chain drafter
            from .runtime.spec import MtpDrafter
            mux.set_drafter(MtpDrafter(load_engine(mtp_dir, cfg.replace(prefix_cache=False))))
        elif cfg.spec_drafter == "mtp":
            raise SystemExit(f"plowrt: --spec-drafter mtp: {mtp_dir} does not exist (compile with plowc --mtp)")
    if cfg.pd:
        # prefill / decode disaggregation: this engine only prefills; a second engine (the next GPU when there is one)
        # imports each sequence's KV image and decodes it
        import torch
        dev2 = f"cuda:{(torch.cuda.current_device() + 1) % torch.cuda.device_count()}" if torch.cuda.is_available() and cfg.backend != "cpu" else None
        mux.pd_target = ModelMux(load_engine(assets, cfg, device=dev2), tok, sched).start()
    mux.start()
    return ModelEntry(name, mux, tok, ChatTemplate.from_assets(assets))


def cmd_serve(args) -> int:
    import uvicorn
    from .obs.trace import Timeline
    from .serve.app import AppState, create_app
    cfg = cfgmod.RuntimeConfig.load(cli=dict(host=args.host, port=args.port, max_slots=args.max_slots, max_ctx=args.max_ctx,
                                             backend=args.backend, objective=args.objective, trace=args.trace or None,
                                             api_keys=args.api_key or None, dp=args.dp, spec_depth=args.spec_depth, spec_drafter=args.spec_drafter, multi_step=args.multi_step, lookahead=args.lookahead or None, rung_control=args.rung_control or None, pd=args.pd or None))
    state = AppState(api_keys=cfg.api_keys, timeline=Timeline(cfg.trace), loader=lambda n, p: make_entry(n, p, cfg))
    name = args.name or Path(args.assets).resolve().name
    n_ranks, mode = (args.ep, "ep") if args.ep else (args.tp, "tp") if args.tp else (args.dp_procs, "dp") if args.dp_procs else (0, "")
    if n_ranks:
        # one rank-worker process per GPU; this process keeps HTTP, routing and supervision (serve/rank_group.py)
        from .parallel.dp import DpRouter
        from .serve.app import ModelEntry
        from .serve.rank_group import RankGroup
        from .serve.template import ChatTemplate
        from .text.tokenizer import load_tokenizer
        wargs = []
        for flag, val in (("--max-slots", args.max_slots), ("--max-ctx", args.max_ctx), ("--backend", args.backend)):
            if val is not None:
                wargs += [flag, str(val)]
        group = RankGroup(args.assets, n_ranks, mode, worker_args=wargs)
        state.add(ModelEntry(name, group.muxes[0], load_tokenizer(args.assets), ChatTemplate.from_assets(args.assets)))
        if len(group.muxes) > 1:
            state.router = DpRouter(group.muxes)
        try:
            uvicorn.run(create_app(state), host=cfg.host, port=cfg.port, log_level="warning")
        finally:
            group.shutdown()
        return 0
    if cfg.dp > 1:
        from .parallel.dp import DpRouter
        entries = [make_entry(name, args.assets, cfg) for _ in range(cfg.dp)]
        state.add(entries[0])
        state.router = DpRouter([e.mux for e in entries])
    else:
        state.add(make_entry(name, args.assets, cfg))
    uvicorn.run(create_app(state), host=cfg.host, port=cfg.port, log_level="warning")
    return 0


def cmd_bench(args) -> int:
    import numpy as np
    from .runtime.scheduler import GenParams
    cfg = cfgmod.RuntimeConfig.load(cli=dict(max_slots=args.concurrency, max_ctx=args.input_len + args.output_len + 64,
                                             backend=args.backend))
    entry = make_entry("bench", args.assets, cfg)
    rng = np.random.default_rng(args.seed)
    V = entry.mux.engine.spec.vocab
    prompts = [rng.integers(3, V, size=args.input_len).tolist() for _ in range(args.num_prompts)]
    t0 = time.perf_counter()
    reqs = [entry.mux.submit(p, GenParams(max_tokens=args.output_len, ignore_eos=True)) for p in prompts]
    n_out = 0
    for r in reqs:
        while True:
            ch = r.out.get()
            if ch.kind == "token":
                n_out += 1
            elif ch.kind == "done":
                break
            else:
                print(f"request failed: {ch.error}", file=sys.stderr)
                break
    dt = time.perf_counter() - t0
    snap = entry.mux.metrics.snapshot()
    print(json.dumps(dict(output_tok_s=n_out / dt, total_tok_s=(n_out + args.num_prompts * args.input_len) / dt,
                          ttft_ms=snap["ttft_ms"], tpot_ms=snap["tpot_ms"], wall_s=dt, requests=args.num_prompts)))
    entry.mux.stop()
    return 0


def cmd_show(args) -> int:
    pkt = pk.read_packet(Path(args.assets) / "model.pkt" if Path(args.assets).is_dir() else args.assets)
    print(json.dumps(dict(tensors=len(pkt.tensors), programs=[dict(role=p.role, rows=p.rows, rank=p.rank, insts=len(p.insts),
                                                                    stream=len(p.stream), arena=p.arena_bytes) for p in pkt.programs],
                          sections=sorted(pkt.sections), n_cu=pkt.n_cu, sha256=pkt.content_hash.hex()), indent=1))
    return 0


def cmd_disasm(args) -> int:
    pkt = pk.read_packet(Path(args.assets) / "model.pkt" if Path(args.assets).is_dir() else args.assets)
    print(disasm_mod.disasm(pkt, args.program, limit=args.limit))
    return 0


def cmd_simulate(args) -> int:
    pkt = pk.read_packet(Path(args.assets) / "model.pkt" if Path(args.assets).is_dir() else args.assets)
    ok = True
    for i, p in enumerate(pkt.programs):
        r = schedule.simulate(p)
        ok &= r["completed"]
        print(f"program {i} role={p.role} rows={p.rows}: {'ok' if r['completed'] else 'DEADLOCK'} entries={len(r['order'])}")
    return 0 if ok else 1


def cmd_inventory(args) -> int:
    """Opcodes of a packet by class, which backend has a body for each (the audit refuses what neither classifies), and the
    counter report of every program (dead counters, redundant waits, dependency depth)."""
    from .compiler import audit
    pkt = pk.read_packet(Path(args.assets) / "model.pkt" if Path(args.assets).is_dir() else args.assets)
    ops = sorted({pk.Op(i.op).name for p in pkt.programs for i in p.insts})
    audits = {b: audit.audit_ops(pkt, b) for b in ("cpu", "cuda")}
    counters = [dict(role=p.role, rows=p.rows, **audit.counter_report(p)) for p in pkt.programs]
    for c in counters:
        c["dead"] = len(c["dead"])
    print(json.dumps(dict(opcodes=ops, must_understand=(pkt.section_json("abi.json") or {}).get("must_understand", []),
                          by_class=audits["cpu"]["by_class"], missing={b: a["missing"] for b, a in audits.items()},
                          unclassified=audits["cpu"]["unclassified"], counters=counters), indent=1))
    return 0 if not audits["cpu"]["unclassified"] else 1


def cmd_budget(args) -> int:
    """Memory plan of a packet against a device size: weights, arenas, state, KV page size, pages that fit."""
    from .runtime.budget import plan_memory
    pkt = pk.read_packet(Path(args.assets) / "model.pkt" if Path(args.assets).is_dir() else args.assets)
    plan = plan_memory(pkt, int(args.device_gb * 2 ** 30), args.max_slots, args.max_ctx, args.kv_fraction, int(args.reserve_gb * 2 ** 30))
    out = plan.to_json()
    out["gib"] = {k[:-6]: round(v / 2 ** 30, 3) for k, v in out.items() if k.endswith("_bytes")}
    print(json.dumps(out, indent=1))
    return 0 if plan.fits else 1


def cmd_devices(_args) -> int:
    import torch
    devs = []
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            devs.append(dict(index=i, name=p.name, sm=f"{p.major}{p.minor}", sms=p.multi_processor_count, mem_gb=round(p.total_memory / 2 ** 30, 1)))
    print(json.dumps(dict(cuda=devs, cpu_threads=__import__("os").cpu_count()), indent=1))
    return 0


def cmd_dist(args) -> int:
    """Asset distribution subcommands (bundles, local store with generations, directory registry)."""
    from .dist import store as d
    st = d.Store(args.store, trusted_keys=args.trust or None, require_signature=bool(args.trust))
    c = args.cmd
    if c == "keygen":
        print(json.dumps(dict(key=args.path, public_key=d.keygen(args.path))))
    elif c == "pack":
        print(d.pack(args.assets, args.out, args.name, key_path=args.key, with_weights=args.with_weights))
    elif c == "load":
        print(st.load(args.bundle))
    elif c == "ls":
        print(json.dumps(st.ls(), indent=1))
    elif c == "rollback":
        print(st.rollback(args.name))
    elif c == "rm":
        st.rm(args.name, args.generation)
    elif c == "gc":
        print(json.dumps(st.gc(args.keep)))
    elif c in ("publish", "push"):
        print(json.dumps(d.Registry(args.registry).publish(args.bundle)))
    elif c == "pull":
        pkg = d.Registry(args.registry).pull(args.name, args.out)
        print(st.load(pkg) if args.load else pkg)
    elif c == "catalog":
        print(json.dumps(d.Registry(args.registry).catalog(show_all=args.all), indent=1))
    elif c in ("unlist", "list"):
        print(json.dumps(dict(unlisted=d.Registry(args.registry).set_listed(args.name, c == "list"))))
    elif c == "unpublish":
        print(json.dumps(d.Registry(args.registry).unpublish(args.name, args.index)))
    elif c == "prepare":
        print(json.dumps(st.prepare(args.name, args.checkpoint)))
    elif c == "upgrade":
        names = [m["name"] for m in st.ls() if m["active"]] if args.all else [args.name]
        if not names or names == [None]:
            raise SystemExit("plowrt upgrade: name a model or pass --all")
        print(json.dumps([st.upgrade(n, d.Registry(args.registry), dry_run=args.dry_run) for n in names], indent=1))
    elif c == "target":
        t = d.host_target()
        print(json.dumps(t) if args.json else " ".join(f"{k}={v}" for k, v in t.items()))
    return 0


def cmd_op_audit(args) -> int:
    """Opcode classes of the whole ISA (--table) or of a packet's programs; an unclassified opcode is refused (exit 1)."""
    from .compiler import audit
    if args.table or not args.blob:
        rows = [dict(op=o.name, value=int(o), cls=audit.op_class(o), cpu=o in audit.CPU_OPS, cuda=o in audit.gpu_ops()) for o in pk.Op]
        if args.format == "json":
            print(json.dumps(rows, indent=1))
        else:
            for r in rows:
                print(f"{r['value']:3d} {r['op']:<20} {r['cls']:<10} cpu={'y' if r['cpu'] else '-'} cuda={'y' if r['cuda'] else '-'}")
        return 0
    pkt = pk.read_packet(Path(args.blob) / "model.pkt" if Path(args.blob).is_dir() else args.blob)
    if args.program is not None:
        want_role, want_rows = (pk.Role.DECODE, None) if args.program == 1 else (pk.Role.PREFILL, args.program)
        pkt.programs = [p for p in pkt.programs if p.role == want_role and (want_rows is None or p.rows == want_rows)]
        if not pkt.programs:
            raise SystemExit(f"plowrt op-audit: the packet has no such program ({args.program})")
    out = {b: audit.audit_ops(pkt, b) for b in ("cpu", "cuda")}
    if args.format == "json":
        print(json.dumps(out, indent=1))
    else:
        for b, a in out.items():
            print(f"[{b}] ok={a['ok']} missing={a['missing']} unclassified={a['unclassified']}"
                  + (f" cpu-only variants={a['cpu_only_variants']}" if a["cpu_only_variants"] else ""))
            for cls, ops in a["by_class"].items():
                print(f"  {cls:<10} {' '.join(ops)}")
    return 0 if not out["cpu"]["unclassified"] else 1


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="plowrt")
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("serve")
    s.add_argument("--assets", required=True)
    s.add_argument("--name")
    s.add_argument("--host")
    s.add_argument("--port", type=int)
    s.add_argument("--max-slots", type=int)
    s.add_argument("--max-ctx", type=int)
    s.add_argument("--backend")
    s.add_argument("--objective")
    s.add_argument("--spec-depth", type=int, dest="spec_depth")
    s.add_argument("--spec-drafter", dest="spec_drafter", choices=["auto", "ngram", "mtp"])
    s.add_argument("--rung-control", action="store_true", dest="rung_control", help="admission follows the decode-rung controller")
    s.add_argument("--lookahead", action="store_true", help="lookahead-1 decode pipeline (step n+1 launched before step n's tokens are read)")
    s.add_argument("--multi-step", type=int, dest="multi_step", help="greedy decode steps per engine call (default 1)")
    s.add_argument("--pd", action="store_true", help="prefill on one engine, decode on a second one (KV image hand-off)")
    s.add_argument("--dp", type=int)
    s.add_argument("--ep", type=int, help="expert parallelism over N GPUs (one rank-worker process each, attention data-parallel)")
    s.add_argument("--tp", type=int, help="tensor parallelism over N GPUs (one rank-worker process each)")
    s.add_argument("--dp-procs", type=int, dest="dp_procs", help="N data-parallel replicas, each in a process of its own")
    s.add_argument("--trace", action="store_true")
    s.add_argument("--api-key", action="append")
    s.set_defaults(fn=cmd_serve)
    w = sub.add_parser("rank-worker", help="one rank of a multi-GPU group (started by `serve --ep/--tp/--dp-procs`)")
    w.add_argument("--assets", required=True)
    w.add_argument("--rank", type=int, required=True)
    w.add_argument("--world", type=int, required=True)
    w.add_argument("--mode", choices=["ep", "tp", "dp"], required=True)
    w.add_argument("--master-port", type=int, required=True, dest="master_port")
    w.add_argument("--leader", required=True, help="host:port of the leader's control listener")
    w.add_argument("--max-slots", type=int, dest="max_slots")
    w.add_argument("--max-ctx", type=int, dest="max_ctx")
    w.add_argument("--backend")
    w.add_argument("--group-timeout", type=float, default=60.0, dest="group_timeout")
    w.set_defaults(fn=lambda a: __import__("plow_b200.serve.rank_group", fromlist=["worker_main"]).worker_main(a))
    b = sub.add_parser("bench")
    b.add_argument("--assets", required=True)
    b.add_argument("--input-len", type=int, default=128)
    b.add_argument("--output-len", type=int, default=64)
    b.add_argument("--num-prompts", type=int, default=8)
    b.add_argument("--concurrency", type=int, default=8)
    b.add_argument("--backend")
    b.add_argument("--seed", type=int, default=0)
    b.set_defaults(fn=cmd_bench)
    for name, fn in (("show", cmd_show), ("simulate", cmd_simulate), ("inventory", cmd_inventory)):
        p = sub.add_parser(name)
        p.add_argument("assets")
        p.set_defaults(fn=fn)
    d = sub.add_parser("disasm")
    d.add_argument("assets")
    d.add_argument("--program", type=int, default=0)
    d.add_argument("--limit", type=int, default=200)
    d.set_defaults(fn=cmd_disasm)
    sub.add_parser("devices").set_defaults(fn=cmd_devices)
    bg = sub.add_parser("budget", help="device-memory plan of a packet: weights, arenas, state, KV pages that fit")
    bg.add_argument("--assets", required=True)
    bg.add_argument("--device-gb", type=float, default=180.0, dest="device_gb")
    bg.add_argument("--max-slots", type=int, default=64, dest="max_slots")
    bg.add_argument("--max-ctx", type=int, default=8192, dest="max_ctx")
    bg.add_argument("--kv-fraction", type=float, default=0.9, dest="kv_fraction")
    bg.add_argument("--reserve-gb", type=float, default=2.0, dest="reserve_gb")
    bg.set_defaults(fn=cmd_budget)
    k = sub.add_parser("knob-scope")
    k.set_defaults(fn=lambda a: print(json.dumps(cfgmod.knob_table("runtime"), indent=1)) or 0)
    def dist_parser(cmd_name, *pos, **opts):
        p = sub.add_parser(cmd_name)
        for a in pos:
            p.add_argument(a)
        for o, kw in opts.items():
            p.add_argument("--" + o.replace("_", "-"), **kw)
        p.add_argument("--store")
        p.add_argument("--trust", action="append", help="hex ed25519 public key; when given, unsigned or foreign bundles are refused")
        p.set_defaults(fn=cmd_dist)
    dist_parser("keygen", "path")
    dist_parser("pack", "assets", name=dict(required=True), out=dict(default="."), key=dict(), with_weights=dict(action="store_true"))
    dist_parser("load", "bundle")
    dist_parser("ls")
    dist_parser("rollback", "name")
    dist_parser("rm", "name", generation=dict())
    dist_parser("gc", keep=dict(type=int, default=2))
    dist_parser("publish", "bundle", registry=dict(required=True))
    dist_parser("push", "bundle", registry=dict(required=True))
    dist_parser("pull", "name", registry=dict(required=True), out=dict(default="."), load=dict(action="store_true"))
    dist_parser("catalog", registry=dict(required=True), all=dict(action="store_true"))
    dist_parser("unlist", "name", registry=dict(required=True))
    dist_parser("list", "name", registry=dict(required=True))
    dist_parser("unpublish", "name", registry=dict(required=True), index=dict(type=int, default=-1))
    dist_parser("prepare", "name", checkpoint=dict(required=True))
    dist_parser("target", json=dict(action="store_true"))
    up = sub.add_parser("upgrade", help="move a model's pin to the newest build in the registry that this machine can run")
    up.add_argument("name", nargs="?")
    up.add_argument("--all", action="store_true")
    up.add_argument("--dry-run", action="store_true", dest="dry_run")
    up.add_argument("--registry", required=True)
    up.add_argument("--store")
    up.add_argument("--trust", action="append")
    up.set_defaults(fn=cmd_dist)
    oa = sub.add_parser("op-audit", help="opcode classes of the ISA or of a packet; unclassified opcodes are refused")
    oa.add_argument("blob", nargs="?")
    oa.add_argument("--table", action="store_true")
    oa.add_argument("--program", type=int)
    oa.add_argument("--format", default="text", choices=["text", "json"])
    oa.set_defaults(fn=cmd_op_audit)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
