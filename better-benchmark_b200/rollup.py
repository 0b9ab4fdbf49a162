"""Model-level roll-up of a sweep's timings file.

The sweep (``sweep.py``) writes one entry per canonical directory with a representative
``oracle_us`` / ``compile_us`` and a ``points_by_shape`` table. A model uses a directory's region
many times, each use at its own shape; the projected time of the model is the sum, over uses, of
the time measured at that use's shape. This module does that pricing with the same three-way
classification the reference's accounting uses
(scripts/model_graph_accounting.py:413-535 ``_rollup_occurrence_timings``):

  matched   the use's shape hash has a measured point of its own
  fallback  the directory is timed, this shape is not: the directory's representative time is used
  unpriced  nothing usable: the use is counted but contributes no time

``matched + fallback + unpriced == total`` always holds, and a projection is only as good as its
unpriced count is small; ``project_models`` reports the counts beside every total.

The reference needs its captured graphs to know which model uses which (directory, shape); here
the uses are passed in as plain records, so the arithmetic can be checked without the graphs.
"""
from __future__ import annotations

import json
from collections import Counter
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable, Mapping, Optional, Sequence


def _number(v) -> bool:
    return isinstance(v, (int, float))


def load_timings(path) -> dict:
    """Directory name -> entry, without the ``_``-prefixed bookkeeping keys; {} if unreadable
    (scripts/model_graph_accounting.py:398-406)."""
    try:
        data = json.loads(Path(path).read_text())
    except (OSError, json.JSONDecodeError):
        return {}
    return {k: v for k, v in data.items() if not k.startswith("_")}


def price_uses(entry: Optional[Mapping], shape_hashes: Sequence[str]) -> dict:
    """Price every use of one directory. ``entry`` is that directory's record from the timings file
    (or None when the sweep has none), ``shape_hashes`` one hash per use.

    Returns ``{oracle_us_total, compile_us_total, matched_occ, fallback_occ, unpriced_occ,
    total_occ, mode}`` with the reference's field names; totals are rounded to 0.01 us and are
    None when no use could be priced. ``mode`` is one of ``untimed``, ``legacy`` (an entry without
    ``points_by_shape``: every use is booked at the representative time), ``per_shape``,
    ``partial``, ``fallback_only``."""
    total = len(shape_hashes)
    if not entry:
        return dict(oracle_us_total=None, compile_us_total=None, matched_occ=0, fallback_occ=0,
                    unpriced_occ=total, total_occ=total, mode="untimed")
    rep_o, rep_c = entry.get("oracle_us"), entry.get("compile_us")
    table = entry.get("points_by_shape")

    if not isinstance(table, dict):
        priced = _number(rep_o)
        return dict(oracle_us_total=round(rep_o * total, 2) if priced else None,
                    compile_us_total=round(rep_c * total, 2) if _number(rep_c) else None,
                    matched_occ=0, fallback_occ=total if priced else 0,
                    unpriced_occ=0 if priced else total, total_occ=total, mode="legacy")

    sums = {"o": 0.0, "c": 0.0}
    seen = {"o": False, "c": False}
    counts = Counter()
    for h in shape_hashes:          # one addition per use, in order: the rounding of the total
        point = table.get(h)        # then depends only on the sequence the caller gives
        o = point.get("oracle_us") if isinstance(point, dict) else None
        c = point.get("compile_us") if isinstance(point, dict) else None
        if _number(o):
            counts["matched"] += 1
        elif _number(rep_o):
            o = rep_o
            counts["fallback"] += 1
        else:
            counts["unpriced"] += 1
        if not _number(c) and _number(rep_c):
            c = rep_c
        for key, v in (("o", o), ("c", c)):
            if _number(v):
                sums[key] += v
                seen[key] = True

    if counts["unpriced"] == total:
        mode = "untimed"
    elif counts["matched"] == total:
        mode = "per_shape"
    elif counts["matched"]:
        mode = "partial"
    else:
        mode = "fallback_only"
    return dict(oracle_us_total=round(sums["o"], 2) if seen["o"] else None,
                compile_us_total=round(sums["c"], 2) if seen["c"] else None,
                matched_occ=counts["matched"], fallback_occ=counts["fallback"],
                unpriced_occ=counts["unpriced"], total_occ=total, mode=mode)


@dataclass(frozen=True)
class Use:
    """One use of a canonical region by a model."""
    model: str
    directory: Optional[str]      # canonical directory name, None when the region has no directory
    shape_hash: str


def project_models(timings: Mapping[str, Mapping], uses: Iterable[Use]) -> dict:
    """Per model: the priced totals of all its uses, the counts behind them and, where both arms
    are priced for the same uses, ``speedup`` = compile time / oracle time of those uses.

    A use contributes to ``speedup`` only when BOTH its oracle and its compile time are known, so
    the ratio never mixes a numerator and a denominator taken over different sets of regions."""
    grouped: dict[str, dict[Optional[str], list[str]]] = {}
    for u in uses:
        grouped.setdefault(u.model, {}).setdefault(u.directory, []).append(u.shape_hash)

    report = {}
    for model in sorted(grouped):
        row = dict(oracle_us_total=0.0, compile_us_total=0.0, matched_occ=0, fallback_occ=0,
                   unpriced_occ=0, total_occ=0, directories={})
        paired_o = paired_c = 0.0
        for directory in sorted(grouped[model], key=lambda d: (d is None, d or "")):
            hashes = grouped[model][directory]
            entry = timings.get(directory) if directory else None
            priced = price_uses(entry, hashes)
            row["directories"][directory or "<unmatched>"] = priced
            for k in ("matched_occ", "fallback_occ", "unpriced_occ", "total_occ"):
                row[k] += priced[k]
            for k in ("oracle_us_total", "compile_us_total"):
                if priced[k] is not None:
                    row[k] += priced[k]
            if priced["oracle_us_total"] is not None and priced["compile_us_total"] is not None \
                    and priced["unpriced_occ"] == 0:
                paired_o += priced["oracle_us_total"]
                paired_c += priced["compile_us_total"]
        row["oracle_us_total"] = round(row["oracle_us_total"], 2)
        row["compile_us_total"] = round(row["compile_us_total"], 2)
        row["priced_fraction"] = ((row["matched_occ"] + row["fallback_occ"]) / row["total_occ"]
                                  if row["total_occ"] else 0.0)
        row["speedup"] = round(paired_c / paired_o, 4) if paired_o > 0 and paired_c > 0 else None
        report[model] = row
    return report


def main(argv=None) -> int:
    """``python -m better_benchmark_b200.rollup TIMINGS.json USES.json``: USES.json is a list of
    ``{"model", "directory", "shape_hash"}`` records; prints the per-model report as JSON."""
    import argparse
    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("timings")
    ap.add_argument("uses")
    args = ap.parse_args(argv)
    timings = load_timings(args.timings)
    records = json.loads(Path(args.uses).read_text())
    uses = [Use(r["model"], r.get("directory"), r["shape_hash"]) for r in records]
    print(json.dumps(project_models(timings, uses), indent=1, sort_keys=True))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
