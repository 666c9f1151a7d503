"""``campaign`` — recipes and the build / gate / bench / compare / report loop around them.

    python -m plow_b200.campaign build   recipes/tiny-cpu.toml --work runs/tiny
    python -m plow_b200.campaign gate    recipes/tiny-cpu.toml --work runs/tiny
    python -m plow_b200.campaign bench   recipes/tiny-cpu.toml --work runs/tiny
    python -m plow_b200.campaign compare runs/base/bench.json runs/tiny/bench.json --tolerance 0.05
    python -m plow_b200.campaign report  runs/

A *recipe* (TOML, schema ``plow.recipe.v1``) names a checkpoint, the target, the compile and serve knobs, a workload and
the quality thresholds; every step reads the recipe and writes one JSON file into the work directory, so a campaign is
reproducible from the recipe alone.  ``gate`` comes before ``bench``: a build whose logits do not agree with the fp32
reference has no performance number.  The gate compares next-token distributions of the compiled engine with the
PyTorch fp32 reference over sampled prompts (KL divergence, top-1 agreement, relative logit error) and probes the cache
paths (a prompt prefilled in chunks and through a prefix-cache hit must reproduce the one-shot logits).  ``compare``
sets two bench results side by side and fails on a regression past the tolerance.

Reference: scripts/campaign/campaign.py (build / bench / gate / compare / report), recipes/infervisor/*/*.toml
(``plow.recipe.v1``), tools/bench-api/compare.py.
"""
from __future__ import annotations

import argparse
import glob
import json
import sys
import time
import tomllib
from pathlib import Path

import numpy as np

SCHEMA = "plow.recipe.v1"
_SECTIONS = {
    "model": dict(required=["checkpoint"], optional=["name", "seed", "synthetic_config"]),
    "target": dict(required=[], optional=["gpu", "arch", "num_gpus", "parallel", "backend"]),
    "compile": dict(required=[], optional=["max_rows", "prefill_buckets", "decode_rungs", "max_seqs", "disable_rules", "mtp", "n_cu"]),
    "serve": dict(required=[], optional=["max_slots", "max_ctx", "token_budget", "spec_depth", "multi_step", "lookahead", "rung_control",
                                          "prefix_cache", "objective"]),
    "bench": dict(required=[], optional=["requests", "concurrency", "prompt_min", "prompt_max", "output", "seed"]),
    "gate": dict(required=[], optional=["prompts", "prompt_len", "kl_max", "top1_min", "rel_err_max", "decode_steps"]),
}
# which direction is better, for compare
_HIGHER = {"output_tok_s", "total_tok_s"}
_LOWER = {"ttft_ms_p50", "ttft_ms_p99", "tpot_ms_p50", "tpot_ms_p99", "wall_s"}


class RecipeError(ValueError):
    pass


def load_recipe(path) -> dict:
    r = tomllib.loads(Path(path).read_text())
    if r.get("schema") != SCHEMA:
        raise RecipeError(f"{path}: schema must be '{SCHEMA}' (got {r.get('schema')!r})")
    for sec, body in r.items():
        if sec == "schema":
            continue
        if sec not in _SECTIONS:
            raise RecipeError(f"{path}: unknown section [{sec}]")
        known = set(_SECTIONS[sec]["required"]) | set(_SECTIONS[sec]["optional"])
        for k in body:
            if k not in known:
                raise RecipeError(f"{path}: [{sec}] has no key '{k}' (known: {sorted(known)})")
    for sec, spec in _SECTIONS.items():
        for k in spec["required"]:
            if k not in r.get(sec, {}):
                raise RecipeError(f"{path}: [{sec}] {k} is required")
    r["_path"] = str(path)
    r["_dir"] = str(Path(path).resolve().parent)
    return r


def _checkpoint(recipe: dict, work: Path) -> Path:
    """The recipe's checkpoint directory; ``synthetic:<name>`` writes a random-init checkpoint of a built-in
    configuration (or of [model] synthetic_config) into the work directory once."""
    ck = recipe["model"]["checkpoint"]
    if not ck.startswith("synthetic:"):
        p = Path(ck)
        return p if p.is_absolute() else Path(recipe["_dir"]) / p
    from .models import config, reference
    out = work / "checkpoint"
    if not (out / "config.json").exists():
        name = ck.split(":", 1)[1]
        cfg = dict(recipe["model"].get("synthetic_config") or getattr(config, f"{name}_config")())
        import torch
        dt = torch.float32 if cfg.get("plow_dtype") == "f32" else torch.bfloat16
        reference.write_checkpoint(cfg, out, seed=int(recipe["model"].get("seed", 0)), dtype=dt)
    return out


def _engine(recipe: dict, work: Path):
    t, s = recipe.get("target", {}), recipe.get("serve", {})
    backend = t.get("backend", "cpu" if t.get("arch") == "cpu" else "cuda")
    kw = dict(max_slots=int(s.get("max_slots", 8)), max_ctx=int(s.get("max_ctx", 1024)), prefix_cache=bool(s.get("prefix_cache", True)))
    if backend == "cpu":
        from .runtime.cpu_engine import CpuEngine
        return CpuEngine(work / "assets", **kw)
    from .runtime.gpu_engine import GpuEngine
    return GpuEngine(work / "assets", **kw)


# ---- steps ------------------------------------------------------------------------------------------------------
def step_build(recipe: dict, work: Path) -> dict:
    from . import plowc
    t, c = recipe.get("target", {}), recipe.get("compile", {})
    ck = _checkpoint(recipe, work)
    t0 = time.perf_counter()
    rep = plowc.compile_dir(ck, work / "assets", gpu=t.get("gpu", "b200"), arch=t.get("arch", "sm_100a"), num_gpus=int(t.get("num_gpus", 1)),
                            parallel=t.get("parallel", "tp"), n_cu=c.get("n_cu"), max_rows=int(c.get("max_rows", 8192)),
                            prefill_buckets=c.get("prefill_buckets"), decode_rungs=c.get("decode_rungs"),
                            max_seqs=int(c.get("max_seqs", 64)), disable_rules=tuple(c.get("disable_rules", ())), mtp=bool(c.get("mtp", False)))
    out = dict(step="build", recipe=recipe["_path"], seconds=round(time.perf_counter() - t0, 2), family=rep["family"],
               ranks=len(rep["ranks"]), programs=len(rep["ranks"][0]["programs"]), fusion=rep["ranks"][0]["fusion_coverage"],
               verify_ok=all(r["verify"]["ok"] for r in rep["ranks"]), sha256=rep["ranks"][0]["sha256"])
    (work / "build_step.json").write_text(json.dumps(out, indent=1))
    return out


def step_gate(recipe: dict, work: Path) -> dict:
    """Quality gate against the fp32 reference.  Passing means: mean KL(reference || engine) of the next-token
    distribution <= kl_max, top-1 agreement >= top1_min, relative logit error <= rel_err_max, over prefill and a few
    decode steps, and the chunked / prefix-cached prefill reproduces the one-shot logits."""
    import torch
    from .models import config, reference
    from .runtime.engine import TokenBatch
    from .runtime.weights import SCALE_SUFFIX, open_checkpoint, shard_slice
    g = recipe.get("gate", {})
    n_prompts, plen, steps = int(g.get("prompts", 4)), int(g.get("prompt_len", 48)), int(g.get("decode_steps", 2))
    kl_max, top1_min, rel_max = float(g.get("kl_max", 1e-3)), float(g.get("top1_min", 0.99)), float(g.get("rel_err_max", 0.02))
    ck = _checkpoint(recipe, work)
    spec = config.load_spec(ck)
    ckpt = open_checkpoint(ck)
    # the reference sees what the engine sees: block-quantised tensors dequantised through their scales
    state = {n: shard_slice(ckpt, n, None, 1, 0).float() for n in ckpt.names() if not n.endswith(SCALE_SUFFIX)}
    ref = reference.ReferenceModel(spec, state)
    eng = _engine(recipe, work)
    rng = np.random.default_rng(int(recipe.get("bench", {}).get("seed", 0)) + 17)
    kls, agree, rels = [], [], []

    def score(got, want):
        lw, lg = torch.log_softmax(want.float(), -1), torch.log_softmax(torch.from_numpy(np.asarray(got)).float(), -1)
        kls.append(float((lw.exp() * (lw - lg)).sum()))
        agree.append(int(int(lw.argmax()) == int(lg.argmax())))
        rels.append(float((torch.from_numpy(np.asarray(got)).float() - want.float()).norm() / want.float().norm()))
    try:
        for i in range(n_prompts):
            p = rng.integers(3, spec.vocab, size=plen).tolist()
            slot = i % eng.max_slots
            eng.begin_slot(slot, p)
            eng.reserve(slot, plen + steps + 2)
            r = eng.step(TokenBatch(np.asarray(p, np.int32), np.arange(plen, dtype=np.int32), np.full(plen, slot, np.int32),
                                    np.asarray([plen - 1], np.int32), want_logits=True))
            eng.commit(slot, p)
            score(r.logits[0], ref.forward(torch.tensor(p))[-1])
            cur = list(p)
            for _ in range(steps):
                nxt = int(ref.forward(torch.tensor(cur))[-1].argmax())
                r = eng.step(TokenBatch(np.asarray([nxt], np.int32), np.asarray([len(cur)], np.int32), np.asarray([slot], np.int32),
                                        np.zeros(1, np.int32), decode=True, want_logits=True))
                eng.commit(slot, [nxt])
                cur.append(nxt)
                score(r.logits[0], ref.forward(torch.tensor(cur))[-1])
            eng.retire_slot(slot)
        # cache probe: the same long prompt one-shot, in two chunks, and again (prefix-cache hit when the engine has one)
        probe = rng.integers(3, spec.vocab, size=max(plen, 80)).tolist()
        want = None
        probe_err = 0.0
        for mode in ("oneshot", "chunked", "again"):
            cached = eng.begin_slot(0, probe)
            eng.reserve(0, len(probe) + 2)
            cuts = [cached, len(probe)] if mode != "chunked" else [cached, max(cached + 1, len(probe) // 2), len(probe)]
            for a, b in zip(cuts, cuts[1:]):
                if b <= a:
                    continue
                r = eng.step(TokenBatch(np.asarray(probe[a:b], np.int32), np.arange(a, b, dtype=np.int32), np.zeros(b - a, np.int32),
                                        np.asarray([b - a - 1], np.int32), want_logits=True))
                eng.commit(0, probe[a:b])
            got = np.asarray(r.logits[0], np.float64)
            if want is None:
                want = got
            else:
                probe_err = max(probe_err, float(np.linalg.norm(got - want) / np.linalg.norm(want)))
            eng.retire_slot(0)
    finally:
        if hasattr(eng, "close"):
            eng.close()
    out = dict(step="gate", recipe=recipe["_path"], samples=len(kls), kl_mean=float(np.mean(kls)), kl_max_seen=float(np.max(kls)),
               top1_agreement=float(np.mean(agree)), rel_err_mean=float(np.mean(rels)), cache_probe_rel_err=probe_err,
               thresholds=dict(kl_max=kl_max, top1_min=top1_min, rel_err_max=rel_max))
    out["passed"] = bool(out["kl_mean"] <= kl_max and out["top1_agreement"] >= top1_min and out["rel_err_mean"] <= rel_max
                         and probe_err <= max(rel_max, 1e-6))
    (work / "gate.json").write_text(json.dumps(out, indent=1))
    return out


def step_bench(recipe: dict, work: Path) -> dict:
    """The recipe's workload through the scheduler (closed loop at the recipe's concurrency), in process."""
    gate = work / "gate.json"
    if gate.exists() and not json.loads(gate.read_text()).get("passed"):
        raise RecipeError(f"{gate} did not pass: a build that fails its quality gate has no performance number")
    from .runtime.scheduler import GenParams, ModelMux, SchedConfig
    from .text.tokenizer import ByteTokenizer
    b, s = recipe.get("bench", {}), recipe.get("serve", {})
    eng = _engine(recipe, work)
    cfg = SchedConfig(token_budget=int(s.get("token_budget", min(8192, eng.max_rows(False)))), objective=s.get("objective", "auto"),
                      spec_depth=int(s.get("spec_depth", 0)), multi_step=int(s.get("multi_step", 1)), lookahead=bool(s.get("lookahead", False)),
                      rung_control=bool(s.get("rung_control", False)), queue_ttl_s=36000.0)
    mux = ModelMux(eng, ByteTokenizer(), cfg, eos_ids=[]).start()
    rng = np.random.default_rng(int(b.get("seed", 0)))
    n, conc, out_len = int(b.get("requests", 16)), int(b.get("concurrency", 4)), int(b.get("output", 16))
    lens = rng.integers(int(b.get("prompt_min", 16)), int(b.get("prompt_max", 64)) + 1, size=n)
    prompts = [rng.integers(3, eng.spec.vocab, size=int(k)).tolist() for k in lens]
    import threading
    lock, st = threading.Lock(), dict(next=0, out=0, failed=0)

    def client():
        while True:
            with lock:
                i = st["next"]
                st["next"] += 1
            if i >= n:
                return
            r = mux.submit(prompts[i], GenParams(max_tokens=out_len, ignore_eos=True))
            k = 0
            while True:
                ch = r.out.get(timeout=3600)
                if ch.kind == "token":
                    k += 1
                elif ch.kind == "done":
                    break
                else:
                    with lock:
                        st["failed"] += 1
                    break
            with lock:
                st["out"] += k
    t0 = time.perf_counter()
    threads = [threading.Thread(target=client, daemon=True) for _ in range(conc)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    snap = mux.metrics.snapshot()
    mux.stop()
    if hasattr(eng, "close"):
        eng.close()
    out = dict(step="bench", recipe=recipe["_path"], requests=n, concurrency=conc, failed=st["failed"], wall_s=round(wall, 3),
               prompt_tokens=int(lens.sum()), output_tokens=st["out"], output_tok_s=round(st["out"] / wall, 2),
               total_tok_s=round((int(lens.sum()) + st["out"]) / wall, 2),
               ttft_ms_p50=snap["ttft_ms"]["p50"], ttft_ms_p99=snap["ttft_ms"]["p99"], tpot_ms_p50=snap["tpot_ms"]["p50"],
               tpot_ms_p99=snap["tpot_ms"]["p99"], counters={k: v for k, v in snap["counters"].items() if isinstance(v, (int, float))})
    (work / "bench.json").write_text(json.dumps(out, indent=1))
    return out


def compare(base: dict, cand: dict, tolerance: float = 0.05) -> dict:
    """Metric by metric: ratio candidate / baseline and whether it regressed past the tolerance."""
    rows, worst = [], None
    for k in sorted(_HIGHER | _LOWER):
        a, b = base.get(k), cand.get(k)
        if not isinstance(a, (int, float)) or not isinstance(b, (int, float)) or a == 0:
            continue
        ratio = b / a
        regressed = ratio < 1.0 - tolerance if k in _HIGHER else ratio > 1.0 + tolerance
        improved = ratio > 1.0 + tolerance if k in _HIGHER else ratio < 1.0 - tolerance
        rows.append(dict(metric=k, baseline=a, candidate=b, ratio=round(ratio, 4),
                         verdict="regressed" if regressed else "improved" if improved else "same"))
        if regressed:
            worst = k if worst is None else worst
    if cand.get("failed", 0) > base.get("failed", 0):
        rows.append(dict(metric="failed", baseline=base.get("failed", 0), candidate=cand.get("failed", 0), ratio=None, verdict="regressed"))
        worst = worst or "failed"
    return dict(step="compare", tolerance=tolerance, rows=rows, regressed=worst is not None, first_regression=worst)


def report(root: Path) -> str:
    """Markdown table over every work directory under ``root`` that holds step results."""
    lines = ["| run | family | gate | KL mean | top-1 | out tok/s | p50 TTFT ms | p50 TPOT ms | failed |", "|---|---|---|---|---|---|---|---|---|"]
    for d in sorted({Path(p).parent for p in glob.glob(str(root / "**" / "*.json"), recursive=True)}):
        def rd(name):
            f = d / name
            return json.loads(f.read_text()) if f.exists() else {}
        bu, ga, be = rd("build_step.json"), rd("gate.json"), rd("bench.json")
        if not (bu or ga or be):
            continue
        f = lambda v, fmt="{:.4g}": fmt.format(v) if isinstance(v, (int, float)) else "—"      # noqa: E731
        lines.append(f"| {d.relative_to(root) if d != root else '.'} | {bu.get('family', '—')} | "
                     f"{'pass' if ga.get('passed') else 'FAIL' if ga else '—'} | {f(ga.get('kl_mean'))} | {f(ga.get('top1_agreement'))} | "
                     f"{f(be.get('output_tok_s'))} | {f(be.get('ttft_ms_p50'))} | {f(be.get('tpot_ms_p50'))} | {be.get('failed', '—')} |")
    return "\n".join(lines) + "\n"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="campaign", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("build", "gate", "bench", "all"):
        p = sub.add_parser(name)
        p.add_argument("recipe")
        p.add_argument("--work", required=True)
    c = sub.add_parser("compare")
    c.add_argument("baseline")
    c.add_argument("candidate")
    c.add_argument("--tolerance", type=float, default=0.05)
    r = sub.add_parser("report")
    r.add_argument("root")
    v = sub.add_parser("check", help="validate recipe files")
    v.add_argument("recipes", nargs="+")
    a = ap.parse_args(argv)
    try:
        if a.cmd == "check":
            for p in a.recipes:
                load_recipe(p)
                print(f"{p}: ok")
            return 0
        if a.cmd == "compare":
            res = compare(json.loads(Path(a.baseline).read_text()), json.loads(Path(a.candidate).read_text()), a.tolerance)
            print(json.dumps(res, indent=1))
            return 1 if res["regressed"] else 0
        if a.cmd == "report":
            sys.stdout.write(report(Path(a.root)))
            return 0
        recipe, work = load_recipe(a.recipe), Path(a.work)
        work.mkdir(parents=True, exist_ok=True)
        steps = dict(build=[step_build], gate=[step_gate], bench=[step_bench], all=[step_build, step_gate, step_bench])[a.cmd]
        for fn in steps:
            out = fn(recipe, work)
            print(json.dumps(out))
            if out.get("step") == "gate" and not out["passed"]:
                return 1
        return 0
    except (RecipeError, FileNotFoundError) as e:
        print(f"campaign: error: {e}", file=sys.stderr)
        return 2


if __name__ == "__main__":
    sys.exit(main())
