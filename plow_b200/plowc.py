"""``plowc`` — compile a checkpoint directory into a packet directory.

    python -m plow_b200.plowc --hf-dir CKPT --out ASSETS --gpu b200 --arch sm_100a --num-gpus 8 --parallel ep

writes ``model.pkt`` (tensor table + one program per prefill bucket / decode rung + metadata
sections), ``weights.json`` (which checkpoint tensors the packet binds), ``build.json`` (knobs,
fusion coverage, verifier results, decode lower bound), copies ``tokenizer.json`` and links
``checkpoint/``.  Same outputs as the reference's ``plowc --emit devblob``
(crates/plowc/src/main.rs:1933-2284); ``--arch`` other than sm_100a / cpu is refused.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import sys
from pathlib import Path

from .compiler import costmodel, emit, graph, hwspec, packet as pk, rewrite, verify
from .models.config import load_spec


def compile_dir(hf_dir, out_dir, gpu="b200", arch="sm_100a", num_gpus=1, parallel="tp", n_cu=None,
                max_rows=8192, prefill_buckets=None, decode_rungs=None, max_seqs=64, disable_rules=(),
                emit_trace=False, mtp=False, fp8_dir=False, _spec=None) -> dict:
    """``mtp=True`` (the checkpoint must carry prediction modules, ``num_nextn_predict_layers``) also writes a drafter
    packet directory ``<out>/mtp`` (the first module as a one-layer model that reads a token and a hidden state per row)
    and makes the main packet return its normed hidden states (``out.hidden``) for it."""
    hwspec.check_arch(arch)
    hw = hwspec.lookup("cpu" if arch == "cpu" else gpu)
    spec = _spec or load_spec(hf_dir)
    if mtp and spec.role == "main" and not spec.mtp_layers:
        raise ValueError("--mtp: the checkpoint's config.json names no prediction module (num_nextn_predict_layers)")
    if parallel not in ("tp", "ep", "dp"):
        raise ValueError(f"--parallel {parallel}: supported strategies are tp, ep (experts over ranks, attention data-parallel) and dp")
    tp = num_gpus if parallel == "tp" else 1
    ep = num_gpus if parallel == "ep" else 1
    n_cu = n_cu or hw.sm_count
    buckets = emit.default_buckets(max_rows)
    if prefill_buckets:
        buckets["prefill"] = sorted(prefill_buckets)
    if decode_rungs:
        buckets["decode"] = sorted(decode_rungs)
    buckets["max_seqs"] = max_seqs
    if not buckets["prefill"] or not buckets["decode"]:
        raise ValueError(f"no {'prefill bucket' if not buckets['prefill'] else 'decode rung'} fits max_rows={max_rows}: the smallest "
                         "prefill bucket is 128 rows (or name the buckets)")
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    report = dict(model_type=spec.model_type, family=spec.family, arch=arch, gpu=hw.name, n_cu=n_cu, tp=tp, ep=ep,
                  parallel=parallel, buckets=buckets, ranks=[])
    n_ranks = num_gpus if parallel in ("tp", "ep") else 1
    for rank in range(n_ranks):
        g = graph.build_graph(spec, tp=tp, ep=ep, rank=rank, emit_hidden=bool(mtp))
        n_prim = len(g.nodes)
        sites = rewrite.fuse(g, disable=set(disable_rules))
        extra = None
        if mtp or spec.role == "mtp":
            # spec.json: what a runtime needs to pair a decoder packet with its drafter (reference: crates/plow-asset/src/spec_draft.rs)
            extra = {"spec.json": json.dumps(dict(
                kind="mtp", role=spec.role, hidden=spec.hidden, drafter_packet="mtp/model.pkt" if spec.role == "main" else None,
                module_layer=(spec.n_layers if spec.role == "main" else spec.name_base), modules=spec.mtp_layers if spec.role == "main" else 1,
                hidden_output="out.hidden", hidden_rows="rows" if spec.role == "main" else "samples", default_depth=3)).encode()}
        pkt = emit.emit_packet(g, sites, hw, n_cu, buckets, extra_sections=extra, rank=rank)
        checks = verify.verify_packet(pkt)
        if not checks["ok"]:
            raise RuntimeError(f"verifier refused the packet: {checks['failures']}")   # nothing is written
        name = "model.pkt" if rank == 0 else f"model.rank{rank}.pkt"
        digest = pk.write_packet(pkt, out / name)
        report["ranks"].append(dict(rank=rank, packet=name, sha256=digest.hex(), primitive_nodes=n_prim,
                                    fused_nodes=len(g.nodes), fusion_coverage=rewrite.coverage(sites),
                                    programs=[dict(role=p.role, rows=p.rows, insts=len(p.insts), stream=len(p.stream),
                                                   waits=len(p.waits), arena_bytes=p.arena_bytes,
                                                   est_us=round(getattr(p, "est_us", 0.0), 2)) for p in pkt.programs],
                                    verify=checks))
        if rank == 0:
            # operand variants that only the CPU interpreter runs: recorded, and said aloud when the target is a GPU
            from .compiler.audit import cpu_only_variants
            report["runtime_requires"] = dict(backend="cpu" if cpu_only_variants(pkt) else "any", cpu_only_variants=cpu_only_variants(pkt))
            if arch != "cpu" and report["runtime_requires"]["cpu_only_variants"]:
                import sys
                print(f"plowc: warning: {spec.model_type} uses {', '.join(report['runtime_requires']['cpu_only_variants'])}; the {arch} engine "
                      "refuses this packet at load, the CPU backend runs it", file=sys.stderr)
            weights = sorted(t.name for t in pkt.tensors if t.tclass == pk.TClass.WEIGHT)
            derived = pkt.section_json("derived_weights.json")
            (out / "weights.json").write_text(json.dumps(dict(weights=weights, derived=derived), indent=1))
    report["decode_floor_us"] = {str(b): round(costmodel.decode_step_floor_us(spec, hw, b, 2048, ep=ep, tp=tp), 1)
                                 for b in (1, 8, 64)}
    (out / "build.json").write_text(json.dumps(report, indent=1))
    src = Path(hf_dir).resolve()
    link = out / "checkpoint"
    if link.is_symlink() or link.exists():
        link.unlink() if link.is_symlink() else shutil.rmtree(link)
    os.symlink(src, link, target_is_directory=True)
    for fn in ("tokenizer.json", "tokenizer_config.json", "chat_template.jinja", "generation_config.json"):
        if (src / fn).exists():
            shutil.copy(src / fn, out / fn)
    if fp8_dir and spec.weight_quant == "fp8_block128":
        # pre-quantised e4m3 twins of every projection the programs read as e4m3 (runtime/fp8_dir.py): loaded instead of
        # quantising the checkpoint at every start
        from .runtime.fp8_dir import write_fp8_dir
        report["fp8_dir"] = [dict(rank=r, tensors=len(write_fp8_dir(out, "model.pkt" if r == 0 else f"model.rank{r}.pkt", r, tp)["weight_map"]) // 2)
                             for r in range(n_ranks)]
        (out / "build.json").write_text(json.dumps(report, indent=1))
    if mtp and spec.role == "main":
        report["mtp"] = compile_dir(hf_dir, out / "mtp", gpu=gpu, arch=arch, num_gpus=num_gpus, parallel=parallel, n_cu=n_cu,
                                    max_rows=max_rows, prefill_buckets=prefill_buckets, decode_rungs=decode_rungs,
                                    max_seqs=max_seqs, disable_rules=disable_rules, fp8_dir=fp8_dir, _spec=spec.drafter_spec())
        (out / "build.json").write_text(json.dumps(report, indent=1))
    return report


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="plowc", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd")
    ap.add_argument("--hf-dir", "--model", dest="hf_dir")
    ap.add_argument("--out", default="assets")
    ap.add_argument("--emit", default="devblob", choices=["devblob", "packets"])
    ap.add_argument("--gpu", default="b200")
    ap.add_argument("--arch", default="sm_100a")
    ap.add_argument("--num-gpus", type=int, default=1)
    ap.add_argument("--parallel", default="tp")
    ap.add_argument("--n-cu", type=int)
    ap.add_argument("--max-rows", type=int, default=8192)
    ap.add_argument("--max-seqs", type=int, default=64)
    ap.add_argument("--prefill-buckets", type=lambda s: [int(x) for x in s.split(",")])
    ap.add_argument("--decode-rungs", type=lambda s: [int(x) for x in s.split(",")])
    ap.add_argument("--disable-rule", action="append", default=[])
    ap.add_argument("--fp8-dir", action="store_true", dest="fp8_dir", help="write pre-quantised e4m3 weight twins next to the packet (<out>/fp8)")
    ap.add_argument("--mtp", action="store_true", help="also compile the checkpoint's prediction module as a drafter (<out>/mtp)")
    v = sub.add_parser("viz", help="write an HTML view of the fused graph")
    v.add_argument("hf_dir")
    v.add_argument("--out", default="graph.html")
    sp = sub.add_parser("stage-plan", help="cut the layers into pipeline stages of balanced modelled time")
    sp.add_argument("hf_dir")
    sp.add_argument("--stages", type=int, default=2)
    sp.add_argument("--batch", type=int, default=64)
    sp.add_argument("--ctx", type=int, default=2048)
    tn = sub.add_parser("tune", help="measure decode GEMM tiles on this GPU and write the tuning store")
    tn.add_argument("hf_dir")
    tn.add_argument("--rows", type=lambda s: [int(x) for x in s.split(",")], default=[8, 64])
    tn.add_argument("--db")
    k = sub.add_parser("knob-scope", help="list compile knobs and the programs they affect")
    args = ap.parse_args(argv)
    if args.cmd == "viz":
        from .compiler import viz
        spec = load_spec(args.hf_dir)
        g = graph.build_graph(spec)
        rewrite.fuse(g)
        Path(args.out).write_text(viz.to_html(g))
        return 0
    if args.cmd == "stage-plan":
        from .compiler import stage_plan
        spec = load_spec(args.hf_dir)
        costs = stage_plan.layer_costs_us(spec, hwspec.lookup(args.gpu), args.batch, args.ctx)
        print(json.dumps(stage_plan.plan_stages(costs, args.stages), indent=1))
        return 0
    if args.cmd == "tune":
        from .compiler import tunedb
        spec = load_spec(args.hf_dir)
        g = graph.build_graph(spec)
        rewrite.fuse(g)
        fp8 = spec.weight_quant == "fp8_block128"
        shapes = set()
        for n in g.nodes:
            if n.op in ("linear", "linear_glu"):
                w = g.values[n.inputs[1]]
                if len(w.shape) == 2 and w.shape[0] % 128 == 0 and w.shape[1] % 128 == 0:
                    dual = n.op == "linear_glu"
                    for m in args.rows:
                        shapes.add((m, w.shape[0] // (2 if dual else 1), w.shape[1], fp8, dual))
        db = tunedb.TuneDb(args.db, tunedb.device_fingerprint())
        for key, (cfg, us) in tunedb.tune_gemm(db, sorted(shapes)):
            print(f"{key}: {cfg} {us:.1f} us")
        return 0
    if args.cmd == "knob-scope":
        from . import config as knobs
        print(json.dumps(knobs.knob_table("emit"), indent=1))
        return 0
    if not args.hf_dir:
        ap.error("--hf-dir is required")
    try:
        rep = compile_dir(args.hf_dir, args.out, args.gpu, args.arch, args.num_gpus, args.parallel, args.n_cu,
                          args.max_rows, args.prefill_buckets, args.decode_rungs, args.max_seqs, args.disable_rule, mtp=args.mtp, fp8_dir=args.fp8_dir)
    except (ValueError, KeyError, RuntimeError) as e:
        print(f"plowc: error: {e}", file=sys.stderr)
        return 2
    print(json.dumps(dict(out=args.out, ranks=len(rep["ranks"]), programs=len(rep["ranks"][0]["programs"]),
                          fusion=rep["ranks"][0]["fusion_coverage"])))
    return 0


if __name__ == "__main__":
    sys.exit(main())
