"""Writes rollup_cases.json: timings entries and use lists priced by the reference's own roll-up
(scripts/model_graph_accounting.py ``_rollup_occurrence_timings``), for the parity test of
``better_benchmark_b200.rollup.price_uses``.

    python tests/golden/make_rollup_golden.py <path to the reference checkout>

Times are dyadic fractions so that sums are exact whatever the order of addition.
"""
import importlib.util
import json
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))


def reference_module(root: Path):
    spec = importlib.util.spec_from_file_location("ref_model_graph_accounting",
                                                  root / "scripts" / "model_graph_accounting.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def sweep_entry():
    """An entry as this repo's sweep writes it, so the pinned cases include the real schema."""
    from better_benchmark_b200 import sweep

    def pt(us, status="OK", compile_us=None, **extra):
        d = {"oracle_us": us, "status": status, "dispatch": {"fallback": False}}
        if compile_us is not None:
            d["compile_us"] = compile_us
        d.update(extra)
        return d

    res = {"/r/var_mean_x": {"bert_aaaa1111": pt(12.5, compile_us=20.25),
                             "gpt_bbbb2222": pt(48.75, compile_us=51.5, region_bytes=1 << 20,
                                                oracle_gbps=21.5, sol_frac=0.25),
                             "t5_cccc3333": pt(7.0, status="BAD_ORACLE")}}
    return sweep.aggregate_oracle_timings(res)["var_mean_x"]


def cases():
    table = {"s1": {"oracle_us": 10.5, "compile_us": 16.25}, "s2": {"oracle_us": 3.25},
             "s3": {"status": "BAD_ORACLE"}, "s4": "not a record"}
    full = {"oracle_us": 6.75, "compile_us": 9.5, "points_by_shape": table}
    return [
        ("no entry", None, ["s1", "s2"]),
        ("empty entry", {}, ["s1"]),
        ("no uses", full, []),
        ("legacy priced", {"oracle_us": 4.5, "compile_us": 8.25}, ["a", "b", "c"]),
        ("legacy oracle only", {"oracle_us": 4.5}, ["a", "b"]),
        ("legacy unpriced", {"compile_us": 8.25}, ["a", "b"]),
        ("per shape", full, ["s1", "s2", "s1", "s1"]),
        ("partial", full, ["s1", "zz", "s3", "s2", "s4"]),
        ("fallback only", full, ["zz", "yy", "s3"]),
        ("no representative", {"points_by_shape": table}, ["s1", "zz", "s3"]),
        ("nothing priced", {"points_by_shape": table}, ["zz", "s3", "s4"]),
        ("compile from representative only", {"oracle_us": 2.5, "compile_us": 5.0,
                                              "points_by_shape": {"s2": {"oracle_us": 3.25}}},
         ["s2", "s2", "qq"]),
        ("no compile anywhere", {"oracle_us": 2.5, "points_by_shape": {"s2": {"oracle_us": 3.25}}},
         ["s2", "qq"]),
        ("sweep entry", sweep_entry(), ["aaaa1111", "bbbb2222", "cccc3333", "dddd4444", "aaaa1111"]),
    ]


def main():
    root = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_ROOT", ""))
    if not (root / "scripts" / "model_graph_accounting.py").is_file():
        raise SystemExit("usage: make_rollup_golden.py <reference checkout>")
    ref = reference_module(root)
    out = []
    for name, entry, hashes in cases():
        occs = [ref.PartitionOccurrence(graph_name="g", pattern_hash="p", shape_hash=h, n_ops=1,
                                        op_counts={}, origin_ops=[], input_shapes=[],
                                        max_output_shape=None, has_reduction=True) for h in hashes]
        out.append({"name": name, "entry": entry, "shape_hashes": hashes,
                    "expected": ref._rollup_occurrence_timings(entry, occs)})
    (HERE / "rollup_cases.json").write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")
    print(f"wrote {len(out)} cases")


if __name__ == "__main__":
    main()
