"""Run this backend's oracles beside the reference's own, through the reference's UNMODIFIED harness.

The reference is a Python project; nothing of it is part of this repository. ``stage`` copies the
few files this comparison needs from a checkout of it into ``baseline/_ref/`` (kept out of version
control), so that they travel to the machine with the GPU:

    oracle_harness.py repro_harness.py byte_accounting.py input_codec.py scripts/gpu_lock.py
    repros/canonical/<id>/{repro.py, oracle.py, shapes.json, meta.json}   for the compared directories

``check`` and ``compare`` then import ``oracle_harness`` from there and use its public functions
as they are (``check_oracle_all_shapes`` oracle_harness.py:972-1050, ``bench_oracle`` :1057-1287):

    check    every shape point of every staged directory this backend has a stub for, through
             ``check_oracle_all_shapes``; records PASS/FAIL, the dispatch tier and the kernel that ran
    compare  per chosen point: the reference's Triton ``oracle.py`` and this backend's stub, each
             checked and then timed by ``bench_oracle`` (which also times ``torch.compile`` of the
             eager module): ``triton_us``, ``b200_us``, ``compile_us`` and the ratios

For both, a directory of this backend is assembled next to the staged one: the reference's
``repro.py`` / ``shapes.json`` / ``meta.json`` plus this repository's ``canonical/<id>/oracle.py`` in
the place of the Triton file, exactly what a maintainer would do by hand.

Work is done in a child process that appends one JSON line per finished task; the parent restarts
it after a crash or a time-out and goes on with the next task, so one bad point costs one line.

    python -m better_benchmark_b200.reference_arm stage --reference /path/to/better-benchmark
    python -m better_benchmark_b200.reference_arm check   --out results.jsonl
    python -m better_benchmark_b200.reference_arm compare --out results.jsonl --max-points 2
    python -m better_benchmark_b200.reference_arm report  results.jsonl > table.md
    python -m better_benchmark_b200.reference_arm tree --workdir /tmp/tree     # directories for the sweep
"""
from __future__ import annotations

import argparse
import json
import math
import os
import shutil
import subprocess
import sys
import time
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
REPO_ROOT = PACKAGE_DIR.parent
DEFAULT_REF = REPO_ROOT / "baseline" / "_ref"
STUB_ROOT = PACKAGE_DIR / "canonical"
OWN_REPRO_ROOT = REPO_ROOT / "oracle" / "canonical"  # the five benchmark configurations' eager modules

HARNESS_FILES = ("oracle_harness.py", "repro_harness.py", "byte_accounting.py", "input_codec.py",
                 "scripts/gpu_lock.py", "scripts/bench_parallel.py", "scripts/model_graph_accounting.py")
DIR_FILES = ("repro.py", "oracle.py", "shapes.json", "shapes.txt", "meta.json")

# Directories without a stub here that are still worth timing: the nearest corpus points of the
# benchmark configurations (the reference's Triton oracle and torch.compile only).
EXTRA_REFERENCE_DIRS = ()


def stub_ids() -> list:
    return sorted(p.parent.name for p in STUB_ROOT.glob("*/oracle.py"))


# ---------------------------------------------------------------------------------------------
# stage: copy the needed reference files (run where the reference checkout is)
# ---------------------------------------------------------------------------------------------
def stage(reference: Path, dest: Path, extra=()) -> dict:
    reference, dest = Path(reference), Path(dest)
    if not (reference / "oracle_harness.py").is_file():
        raise FileNotFoundError(f"{reference} is not a checkout of the reference (no oracle_harness.py)")
    copied = {"harness": [], "dirs": [], "missing": []}
    for rel in HARNESS_FILES:
        target = dest / rel
        target.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(reference / rel, target)
        copied["harness"].append(rel)
    for name in sorted(set(stub_ids()) | set(EXTRA_REFERENCE_DIRS) | set(extra)):
        src = reference / "repros" / "canonical" / name
        if not src.is_dir():
            if not (OWN_REPRO_ROOT / name).is_dir():
                copied["missing"].append(name)
            continue
        out = dest / "repros" / "canonical" / name
        out.mkdir(parents=True, exist_ok=True)
        for f in DIR_FILES:
            if (src / f).is_file():
                shutil.copyfile(src / f, out / f)
        copied["dirs"].append(name)
    return copied


# ---------------------------------------------------------------------------------------------
# Assembling this backend's directories beside the staged ones
# ---------------------------------------------------------------------------------------------
def assemble_b200_dirs(ref_root: Path, out_root: Path) -> dict:
    """``out_root/<id>_b200/`` = the eager module and shape points of the directory + this backend's
    stub as ``oracle.py``. Returns {id: path}. Directories whose eager module is neither staged nor
    one of the five benchmark configurations are left out. (The directory name differs from the
    staged one on purpose: the reference names an oracle module after its directory and keeps the
    registrations per module name, so two directories of one name would share a registry and the
    file loaded first would answer for both.)"""
    out_root.mkdir(parents=True, exist_ok=True)
    made = {}
    for name in stub_ids():
        staged = ref_root / "repros" / "canonical" / name
        own = OWN_REPRO_ROOT / name
        if staged.is_dir():
            sources = {f: staged / f for f in DIR_FILES if f != "oracle.py" and (staged / f).is_file()}
        elif own.is_dir():
            sources = {"repro.py": own / "repro.py"}
        else:
            continue
        d = out_root / f"{name}_b200"
        d.mkdir(exist_ok=True)
        for f, src in sources.items():
            shutil.copyfile(src, d / f)
        for f in (STUB_ROOT / name).iterdir():
            if f.is_file() and (f.name == "oracle.py" or f.name not in sources):
                shutil.copyfile(f, d / f.name)
        made[name] = d
    return made


def build_sweep_tree(ref_root: Path, out_root: Path) -> dict:
    """A directory tree for ``python -m better_benchmark_b200.sweep``: this backend's directories
    (see assemble_b200_dirs) under ``out_root/canonical`` and, under ``out_root/support``, links to
    the three reference modules a staged ``repro.py`` imports (repro_harness, byte_accounting,
    input_codec) - but not to oracle_harness, so that the stubs register with this package's
    harness, which is the one the sweep's workers dispatch through. Put ``support`` on PYTHONPATH."""
    dirs = assemble_b200_dirs(ref_root, out_root / "canonical")
    support = out_root / "support"
    support.mkdir(parents=True, exist_ok=True)
    for name in ("repro_harness.py", "byte_accounting.py", "input_codec.py"):
        target = support / name
        if target.exists() or target.is_symlink():
            target.unlink()
        shutil.copyfile(ref_root / name, target)
    return {"canonical": str(out_root / "canonical"), "pythonpath": str(support), "directories": len(dirs)}


def _import_reference(ref_root: Path):
    for p in (str(ref_root / "scripts"), str(ref_root)):
        if p not in sys.path:
            sys.path.insert(0, p)
    if str(REPO_ROOT) not in sys.path:
        sys.path.insert(0, str(REPO_ROOT))
    import oracle_harness  # noqa: F401  (the reference's file, found on the path just set)
    import repro_harness  # noqa: F401
    here = Path(oracle_harness.__file__).resolve()
    if ref_root.resolve() not in here.parents:
        raise RuntimeError(f"oracle_harness came from {here}, not from {ref_root}")
    return oracle_harness, repro_harness


def _input_bytes(config) -> int:
    total = 0
    for spec in config.get("inputs", []):
        if isinstance(spec, dict) and spec.get("kind", "tensor") == "tensor" and "shape" in spec:
            n = 1
            for s in spec["shape"]:
                n *= max(int(s), 1) if isinstance(s, int) else 1
            total += n * {"f32": 4, "i32": 4, "i64": 8, "f64": 8}.get(str(spec.get("dtype", "")), 2)
    return total


def pick_points(configs: dict, max_points: int) -> list:
    """Labels to time: all of them when few, else the largest, the median and the smallest by
    input bytes (then evenly spaced ones), so that both ends of the size range are seen."""
    labels = list(configs)
    if max_points <= 0 or len(labels) <= max_points:
        return labels
    by_size = sorted(labels, key=lambda k: -_input_bytes(configs[k]))
    if max_points == 1:
        return [by_size[0]]
    idx = sorted({round(i * (len(by_size) - 1) / (max_points - 1)) for i in range(max_points)})
    return [by_size[i] for i in idx]


def list_tasks(ref_root: Path, mode: str, only=None, max_points: int = 0) -> list:
    """Task strings ``<id>::<label>`` for ``mode`` in {"check", "compare"}."""
    sys.path.insert(0, str(ref_root))
    from repro_harness import load_shape_configs  # the reference's loader

    names = stub_ids() + ([d for d in EXTRA_REFERENCE_DIRS] if mode == "compare" else [])
    tasks = []
    for name in names:
        if only and name not in only:
            continue
        staged = ref_root / "repros" / "canonical" / name
        repro = staged / "repro.py" if staged.is_dir() else OWN_REPRO_ROOT / name / "repro.py"
        if not repro.is_file():
            continue
        shapes_dir = staged if staged.is_dir() else STUB_ROOT / name
        configs = load_shape_configs(str(shapes_dir / "repro.py"))
        labels = pick_points(configs, max_points) if mode == "compare" else list(configs)
        for label in labels or ["default"]:
            tasks.append(f"{name}::{label}")
    return tasks


# ---------------------------------------------------------------------------------------------
# Child side
# ---------------------------------------------------------------------------------------------
def _last_kernel() -> str:
    from . import native

    lib = native.load()
    name = lib.b200_last_kernel()
    return name.decode() if name else ""


def _check_one(oh, fn, d, repro_id, label):
    """The reference's own check at one point; True/False, plus what it printed at the end."""
    point = None if label == "default" else label
    verdicts = oh.check_oracle_all_shapes(fn, d, repro_id, skip_stochastic=True, point=point)
    return all(v not in ("fail", False) for v in verdicts.values()) and bool(verdicts)


def _dispatch_of(oh, fn, config, rh):
    if config is None:
        return None
    oh._seed_input_generation(1)
    inputs = rh.make_inputs_from_config(config)
    _, info = oh.resolve_oracle(fn, inputs)
    if info is None:
        return None
    return {"matched": info["matched"], "fallback": info["fallback"]}


def child_main(args) -> int:
    import torch

    ref_root = Path(args.ref)
    oh, rh = _import_reference(ref_root)
    from .byte_model import count_bytes_effective

    b200_dirs = assemble_b200_dirs(ref_root, Path(args.workdir))
    tasks = [t for t in args.tasks.split(",") if t]
    out = open(args.out, "a", buffering=1)
    loaded = {}

    def load(kind, name):
        key = (kind, name)
        if key not in loaded:
            d = b200_dirs[name] if kind == "b200" else ref_root / "repros" / "canonical" / name
            loaded[key] = oh._load_oracle_module(d)
        return loaded[key]

    for task in tasks:
        name, label = task.split("::", 1)
        row = {"task": task, "dir": name, "label": label, "mode": args.mode}
        print(f"=== {task}", flush=True)
        out.write(json.dumps({"task": task, "started": True}) + "\n")
        t0 = time.time()
        try:
            has_stub = name in b200_dirs
            ref_dir = ref_root / "repros" / "canonical" / name
            shapes_dir = b200_dirs[name] if has_stub else ref_dir
            configs = rh.load_shape_configs(str(shapes_dir / "repro.py"))
            config = configs.get(label)
            if has_stub:
                _, b200_fn, b200_dir = load("b200", name)
                row["b200_check"] = _check_one(oh, b200_fn, b200_dir, name, label)
                row["b200_kernel"] = _last_kernel()
                row["b200_dispatch"] = _dispatch_of(oh, b200_fn, config, rh)
            if args.mode == "compare":
                instance = oh.get_repro_instance(shapes_dir)
                if config is not None:
                    inputs = rh.make_inputs_from_config(config)
                else:
                    inputs = oh.get_inputs(shapes_dir)
                try:
                    row["region_bytes"] = int(count_bytes_effective(instance, inputs))
                except Exception as e:  # noqa: BLE001 - an annotation only
                    row["region_bytes_error"] = str(e)[:200]
                point_id = f"{name}_{label}"
                kw = dict(warmup=args.warmup, rep=args.rep, rounds=args.rounds,
                          numerics_optout=oh.load_numerics_optout(shapes_dir))
                if (ref_dir / "oracle.py").is_file():
                    _, triton_fn, _ = load("triton", name)
                    row["triton_check"] = _check_one(oh, triton_fn, ref_dir, name, label)
                    row["triton"] = oh.bench_oracle(triton_fn, oh.get_repro_instance(ref_dir), inputs,
                                                    point_id + ":triton", **kw)
                if has_stub and row.get("b200_check"):
                    if config is not None:
                        inputs = rh.make_inputs_from_config(config)
                    row["b200"] = oh.bench_oracle(b200_fn, instance, inputs, point_id + ":b200", **kw)
        except Exception as e:  # noqa: BLE001 - one line per failure, then the next task
            row["error"] = f"{type(e).__name__}: {str(e)[:500]}"
            if "CUDA" in str(e) or "device-side assert" in str(e):
                row["elapsed_s"] = round(time.time() - t0, 2)
                out.write(json.dumps(row, default=str) + "\n")
                return 3  # the context cannot be trusted: the parent starts a new child
        row["elapsed_s"] = round(time.time() - t0, 2)
        out.write(json.dumps(row, default=str) + "\n")
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
    return 0


# ---------------------------------------------------------------------------------------------
# Parent side
# ---------------------------------------------------------------------------------------------
def _finished_tasks(out_path: Path):
    done, started = set(), []
    if out_path.is_file():
        for line in out_path.read_text().splitlines():
            try:
                row = json.loads(line)
            except json.JSONDecodeError:
                continue
            if row.get("started"):
                started.append(row["task"])
            else:
                done.add(row["task"])
    return done, started


def run_parent(args) -> int:
    ref_root = Path(args.ref)
    out_path = Path(args.out)
    out_path.parent.mkdir(parents=True, exist_ok=True)
    only = set(args.dirs.split(",")) if args.dirs else None
    tasks = list_tasks(ref_root, args.mode, only, args.max_points)
    if args.tasks:  # an explicit list: any point of the staged directories, not only the sampled ones
        wanted = [t for t in args.tasks.split(",") if t]
        every = set(list_tasks(ref_root, "check", only, 0))
        unknown = [t for t in wanted if t not in every]
        if unknown:
            raise SystemExit(f"unknown task(s): {unknown}")
        tasks = wanted
    deadline = time.time() + args.budget_s if args.budget_s else None
    env = os.environ.copy()
    env["PYTHONPATH"] = os.pathsep.join(
        [str(REPO_ROOT), str(ref_root), str(ref_root / "scripts")] + ([env["PYTHONPATH"]] if env.get("PYTHONPATH") else []))
    attempts = 0
    while True:
        done, started = _finished_tasks(out_path)
        crashed = [t for t in started if t not in done]
        remaining = [t for t in tasks if t not in done and t not in crashed]
        if crashed:
            with open(out_path, "a") as f:
                for t in crashed:
                    f.write(json.dumps({"task": t, "dir": t.split("::")[0], "label": t.split("::")[1],
                                        "mode": args.mode, "error": "child process died or timed out on this task"}) + "\n")
        if not remaining or attempts > args.max_restarts:
            break
        if deadline and time.time() > deadline:
            print(f"time budget used up with {len(remaining)} tasks left", file=sys.stderr)
            break
        attempts += 1
        cmd = [sys.executable, "-u", "-m", "better_benchmark_b200.reference_arm", "--child", args.mode,
               "--ref", str(ref_root), "--out", str(out_path), "--workdir", args.workdir,
               "--tasks", ",".join(remaining), "--warmup", str(args.warmup), "--rep", str(args.rep),
               "--rounds", str(args.rounds)]
        left = max(30.0, deadline - time.time()) if deadline else None
        try:
            rc = subprocess.run(cmd, env=env, cwd=str(REPO_ROOT), timeout=left).returncode
        except subprocess.TimeoutExpired:
            rc = -1
        print(f"child ended with {rc}", file=sys.stderr)
    done, _ = _finished_tasks(out_path)
    print(json.dumps({"tasks": len(tasks), "finished": len([t for t in tasks if t in done])}))
    return 0


# ---------------------------------------------------------------------------------------------
# report: a markdown table from the result lines
# ---------------------------------------------------------------------------------------------
def _geomean(values):
    values = [v for v in values if v and v > 0]
    return math.exp(sum(math.log(v) for v in values) / len(values)) if values else float("nan")


def report(paths, peak_gbps=None) -> str:
    rows = {}
    for path in paths:
        for line in Path(path).read_text().splitlines():
            try:
                r = json.loads(line)
            except json.JSONDecodeError:
                continue
            if not r.get("started"):
                rows[(r.get("mode"), r["task"])] = r
    lines = []
    cmp_rows = [r for (m, _), r in rows.items() if m == "compare"]
    if cmp_rows:
        lines += ["| directory | point | bytes | triton us | b200 us | compile us | triton/b200 | compile/b200 | b200 GB/s | b200 status |",
                  "|---|---|---|---|---|---|---|---|---|---|"]
        r_t, r_c = [], []
        for r in sorted(cmp_rows, key=lambda r: r["task"]):
            t, b = r.get("triton") or {}, r.get("b200") or {}
            tu, bu = t.get("oracle_us"), b.get("oracle_us")
            cu = b.get("compile_us") or t.get("compile_us")
            rt = tu / bu if tu and bu else None
            rc = cu / bu if cu and bu else None
            if rt:
                r_t.append(rt)
            if rc:
                r_c.append(rc)
            nbytes = r.get("region_bytes")
            gbps = nbytes / bu / 1e3 if nbytes and bu else None
            status = b.get("status") or r.get("error") or ("check failed" if r.get("b200_check") is False else "-")
            fmt = lambda v, p=2: "-" if v is None else f"{v:.{p}f}"  # noqa: E731
            lines.append(f"| {r['dir']} | {r['label'].rsplit('_', 1)[-1]} | {nbytes or '-'} | {fmt(tu)} "
                         f"({t.get('status', '-')}) | {fmt(bu)} | {fmt(cu)} | {fmt(rt, 3)} | {fmt(rc, 3)} | "
                         f"{fmt(gbps, 0)} | {status} |")
        lines += ["", f"geomean triton_us / b200_us over {len(r_t)} points: **{_geomean(r_t):.3f}**; "
                      f"geomean compile_us / b200_us over {len(r_c)} points: **{_geomean(r_c):.3f}**", ""]
    chk_rows = [r for (m, _), r in rows.items() if m == "check"]
    if chk_rows:
        per_dir = {}
        for r in chk_rows:
            d = per_dir.setdefault(r["dir"], {"pass": 0, "fail": [], "kernels": {}, "tiers": {}})
            if r.get("b200_check"):
                d["pass"] += 1
            else:
                d["fail"].append(r["label"].rsplit("_", 1)[-1] + (": " + r["error"][:80] if r.get("error") else ""))
            k = r.get("b200_kernel") or "?"
            d["kernels"][k] = d["kernels"].get(k, 0) + 1
            tier = (r.get("b200_dispatch") or {}).get("matched", "?")
            d["tiers"][tier] = d["tiers"].get(tier, 0) + 1
        lines += ["| directory | points | pass | dispatch tier | kernel that ran (count) | failures |", "|---|---|---|---|---|---|"]
        tot = ok = 0
        for name in sorted(per_dir):
            d = per_dir[name]
            n = d["pass"] + len(d["fail"])
            tot, ok = tot + n, ok + d["pass"]
            lines.append(f"| {name} | {n} | {d['pass']} | {', '.join(f'{k} {v}' for k, v in d['tiers'].items())} | "
                         f"{'; '.join(f'{k} ({v})' for k, v in sorted(d['kernels'].items()))} | {'; '.join(d['fail']) or '-'} |")
        lines += ["", f"total: {ok} of {tot} points pass `check_oracle_all_shapes`", ""]
    return "\n".join(lines)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m better_benchmark_b200.reference_arm")
    ap.add_argument("mode", choices=["stage", "check", "compare", "report", "tasks", "tree"])
    ap.add_argument("inputs", nargs="*", help="report: result files")
    ap.add_argument("--child", action="store_true", help="internal: run the tasks in this process")
    ap.add_argument("--reference", default=os.environ.get("REFERENCE_ROOT", ""),
                    help="stage: the reference checkout (default: $REFERENCE_ROOT)")
    ap.add_argument("--ref", default=str(DEFAULT_REF), help="the staged copy")
    ap.add_argument("--out", default="reference_arm.jsonl")
    ap.add_argument("--workdir", default="/tmp/b200_reference_arm")
    ap.add_argument("--dirs", default="", help="comma-separated directory names (default: all)")
    ap.add_argument("--tasks", default="", help="comma-separated <directory>::<label> tasks instead of the sampled ones")
    ap.add_argument("--max-points", type=int, default=2, help="compare: points per directory (0 = all)")
    ap.add_argument("--warmup", type=int, default=25)
    ap.add_argument("--rep", type=int, default=100)
    ap.add_argument("--rounds", type=int, default=3)
    ap.add_argument("--budget-s", type=float, default=0.0, help="stop starting new children after this long")
    ap.add_argument("--max-restarts", type=int, default=12)
    args = ap.parse_args(argv)
    if args.mode == "stage":
        if not args.reference:
            ap.error("stage needs --reference <checkout of the reference> (or $REFERENCE_ROOT)")
        print(json.dumps(stage(Path(args.reference), Path(args.ref)), indent=1))
        return 0
    if args.mode == "tree":
        print(json.dumps(build_sweep_tree(Path(args.ref), Path(args.workdir))))
        return 0
    if args.mode == "report":
        print(report(args.inputs))
        return 0
    if args.mode == "tasks":
        print("\n".join(list_tasks(Path(args.ref), "compare" if args.max_points else "check", None, args.max_points)))
        return 0
    if args.child:
        return child_main(args)
    return run_parent(args)


if __name__ == "__main__":
    raise SystemExit(main())
