"""Recipes and the build / gate / bench / compare / report loop (plow_b200/campaign.py) on the CPU backend."""
import json
from pathlib import Path

import pytest

from plow_b200 import campaign

ROOT = Path(__file__).resolve().parent.parent


def test_shipped_recipes_validate_and_bad_ones_are_refused(tmp_path):
    shipped = sorted((ROOT / "recipes").glob("*.toml"))
    assert len(shipped) >= 3
    for p in shipped:
        r = campaign.load_recipe(p)
        assert r["schema"] == campaign.SCHEMA and "checkpoint" in r["model"]
    assert campaign.main(["check"] + [str(p) for p in shipped]) == 0
    for body, why in (('schema = "other"\n[model]\ncheckpoint = "x"\n', "schema"),
                      ('schema = "plow.recipe.v1"\n[model]\nname = "x"\n', "required"),
                      ('schema = "plow.recipe.v1"\n[model]\ncheckpoint = "x"\n[serve]\nturbo = true\n', "no key"),
                      ('schema = "plow.recipe.v1"\n[model]\ncheckpoint = "x"\n[extras]\na = 1\n', "unknown section")):
        f = tmp_path / "bad.toml"
        f.write_text(body)
        with pytest.raises(campaign.RecipeError, match=why):
            campaign.load_recipe(f)
    assert campaign.main(["check", str(f)]) == 2


def test_campaign_runs_end_to_end_on_the_cpu_backend(tmp_path, capsys):
    recipe = ROOT / "recipes" / "tiny-dense-cpu.toml"
    work = tmp_path / "runs" / "a"
    assert campaign.main(["all", str(recipe), "--work", str(work)]) == 0
    build, gate, bench = (json.loads((work / n).read_text()) for n in ("build_step.json", "gate.json", "bench.json"))
    assert build["verify_ok"] and build["family"] == "dense_gqa" and build["programs"] >= 5
    assert gate["passed"] and gate["samples"] == 9 and gate["top1_agreement"] == 1.0 and gate["kl_mean"] < 1e-6
    assert gate["cache_probe_rel_err"] < 1e-5                # chunked and prefix-cached prefill reproduce the one-shot logits
    assert bench["failed"] == 0 and bench["output_tokens"] == 12 * 8 and bench["output_tok_s"] > 0 and bench["ttft_ms_p50"] > 0
    # compare: against itself nothing moves; a slower candidate regresses and the exit code says so
    assert campaign.main(["compare", str(work / "bench.json"), str(work / "bench.json")]) == 0
    slow = dict(bench, output_tok_s=bench["output_tok_s"] * 0.8, tpot_ms_p50=(bench["tpot_ms_p50"] or 1.0) * 1.3)
    (tmp_path / "slow.json").write_text(json.dumps(slow))
    assert campaign.main(["compare", str(work / "bench.json"), str(tmp_path / "slow.json"), "--tolerance", "0.05"]) == 1
    res = campaign.compare(bench, slow, 0.05)
    verdicts = {r["metric"]: r["verdict"] for r in res["rows"]}
    assert verdicts["output_tok_s"] == "regressed" and verdicts["tpot_ms_p50"] == "regressed" and verdicts["wall_s"] == "same"
    assert campaign.compare(slow, bench, 0.05)["regressed"] is False
    capsys.readouterr()
    assert campaign.main(["report", str(tmp_path / "runs")]) == 0
    table = capsys.readouterr().out
    assert "| a | dense_gqa | pass |" in table
    # a failed gate blocks the bench
    (work / "gate.json").write_text(json.dumps(dict(gate, passed=False)))
    assert campaign.main(["bench", str(recipe), "--work", str(work)]) == 2
