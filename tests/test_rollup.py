"""Roll-up of sweep timings over a model's uses: parity with the reference's pricing
(scripts/model_graph_accounting.py:413-535) through golden cases, and the per-model projection."""
import json
from pathlib import Path

import pytest

from better_benchmark_b200 import rollup, sweep

CASES = json.loads((Path(__file__).parent / "golden" / "rollup_cases.json").read_text())


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_price_uses_matches_reference(case):
    got = rollup.price_uses(case["entry"], case["shape_hashes"])
    assert got == case["expected"]
    assert got["matched_occ"] + got["fallback_occ"] + got["unpriced_occ"] == got["total_occ"]


def _pt(us, compile_us=None, status="OK"):
    d = {"oracle_us": us, "status": status, "dispatch": {"fallback": False}}
    if compile_us is not None:
        d["compile_us"] = compile_us
    return d


def test_project_models_from_a_sweep_file(tmp_path):
    results = {"/r/ln_a": {"bert_h1": _pt(10.0, 20.0), "gpt_h2": _pt(40.0, 50.0)},
               "/r/sm_b": {"bert_h3": _pt(5.0, 5.0)}}
    path = tmp_path / "timings.json"
    sweep.write_oracle_timings(path, results, metadata={"note": "t"})
    timings = rollup.load_timings(path)
    assert set(timings) == {"ln_a", "sm_b"}        # bookkeeping keys dropped

    uses = [rollup.Use("bert", "ln_a", "h1")] * 12 + [rollup.Use("bert", "sm_b", "h3")] * 6 \
        + [rollup.Use("bert", None, "zz")] \
        + [rollup.Use("gpt", "ln_a", "h2"), rollup.Use("gpt", "ln_a", "h9"), rollup.Use("gpt", "nope", "h1")]
    rep = rollup.project_models(timings, uses)
    bert, gpt = rep["bert"], rep["gpt"]
    assert bert["oracle_us_total"] == 12 * 10.0 + 6 * 5.0 and bert["compile_us_total"] == 12 * 20.0 + 6 * 5.0
    assert (bert["matched_occ"], bert["fallback_occ"], bert["unpriced_occ"], bert["total_occ"]) == (18, 0, 1, 19)
    assert bert["speedup"] == round(270.0 / 150.0, 4)
    assert bert["directories"]["<unmatched>"]["mode"] == "untimed"
    # gpt: one use at its own shape, one at the directory's representative time, one unpriced
    assert (gpt["matched_occ"], gpt["fallback_occ"], gpt["unpriced_occ"]) == (1, 1, 1)
    assert gpt["oracle_us_total"] == 40.0 + timings["ln_a"]["oracle_us"]
    assert 0 < gpt["priced_fraction"] < 1


def test_load_timings_unreadable(tmp_path):
    assert rollup.load_timings(tmp_path / "missing.json") == {}
    bad = tmp_path / "bad.json"
    bad.write_text("{not json")
    assert rollup.load_timings(bad) == {}


def test_cli(tmp_path, capsys):
    t = tmp_path / "t.json"
    t.write_text(json.dumps({"_meta": {}, "d": {"oracle_us": 2.0, "compile_us": 3.0,
                                                "points_by_shape": {"h": {"oracle_us": 1.0, "compile_us": 4.0}}}}))
    u = tmp_path / "u.json"
    u.write_text(json.dumps([{"model": "m", "directory": "d", "shape_hash": "h"},
                             {"model": "m", "directory": "d", "shape_hash": "other"}]))
    assert rollup.main([str(t), str(u)]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["m"]["oracle_us_total"] == 3.0 and out["m"]["compile_us_total"] == 7.0
    assert out["m"]["speedup"] == round(7.0 / 3.0, 4)
