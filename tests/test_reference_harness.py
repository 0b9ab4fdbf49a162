"""This backend's stubs under the reference's OWN harness file (not the mirror in the package).

``python -m better_benchmark_b200.reference_arm stage`` copies the reference's harness modules and
the compared canonical directories into ``baseline/_ref`` (not under version control). When that
copy is present these tests load every shipped stub through the reference's ``_load_oracle_module``
(oracle_harness.py:1760-1779), resolve its dispatch at every shape point of its directory
(``resolve_oracle`` :557-577, ``oracle_impl(point=)`` :468-549) and, on a GPU, run the
reference's ``check_oracle_all_shapes`` (:972-1050) on it. Without the copy they are skipped.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"

pytestmark = pytest.mark.skipif(not (REF / "oracle_harness.py").is_file(),
                                reason="no staged copy of the reference under baseline/_ref")

# The reference's module names (oracle_harness, repro_harness, ...) must not leak into the other
# tests' import state, so everything that imports them runs in a child interpreter.
_DISPATCH_SCRIPT = r"""
import json, sys
from pathlib import Path
sys.path[:0] = [sys.argv[1], sys.argv[2] + "/scripts", sys.argv[2]]
from better_benchmark_b200 import reference_arm as arm
oh, rh = arm._import_reference(Path(sys.argv[2]))
import torch
dirs = arm.assemble_b200_dirs(Path(sys.argv[2]), Path(sys.argv[3]))
out = {}
for name, d in sorted(dirs.items()):
    mod, fn, _ = oh._load_oracle_module(d)
    assert "baseline/_ref" in oh.oracle_impl.__code__.co_filename.replace("\\", "/")
    configs = rh.load_shape_configs(str(d / "repro.py"))
    tiers = {}
    for label, cfg in configs.items():
        for spec in cfg["inputs"]:
            if isinstance(spec, dict) and spec.get("kind", "tensor") == "tensor":
                spec["device"] = "meta"
        inputs = rh.make_inputs_from_config(cfg)
        _, info = oh.resolve_oracle(fn, inputs)
        tiers[info["matched"]] = tiers.get(info["matched"], 0) + 1
    out[name] = {"points": len(configs), "tiers": tiers}
print("RESULT " + json.dumps(out))
"""


def _run(script, *args, timeout=900):
    env = os.environ.copy()
    env["PYTHONPATH"] = os.pathsep.join([str(ROOT), env.get("PYTHONPATH", "")])
    res = subprocess.run([sys.executable, "-c", script, str(ROOT), str(REF), *args], capture_output=True,
                         text=True, timeout=timeout, env=env, cwd=str(ROOT))
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    return res.stdout


def test_every_stub_registers_each_shape_point_under_the_reference_harness(tmp_path):
    import json

    out = _run(_DISPATCH_SCRIPT, str(tmp_path))
    line = next(l for l in out.splitlines() if l.startswith("RESULT "))
    per_dir = json.loads(line[len("RESULT "):])
    assert len(per_dir) >= 19
    total = 0
    for name, info in per_dir.items():
        assert info["points"] >= 1, name
        total += info["points"]
        # no GPU here, so the hardware half cannot match: every point must still hit its own
        # registration by shape ("shape"), never the shape-general entry ("hardware" / "any")
        assert set(info["tiers"]) <= {"shape", "hardware+shape"}, (name, info)
    assert total >= 226


_MIRROR_SCRIPT = r"""
import contextlib, io, json, random, sys
from pathlib import Path
sys.path[:0] = [sys.argv[1], sys.argv[2] + "/scripts", sys.argv[2]]
from better_benchmark_b200 import reference_arm as arm, harness as mirror
oh, rh = arm._import_reference(Path(sys.argv[2]))
import torch
rnd = random.Random(5)
g = torch.Generator().manual_seed(5)
FLOATS = [torch.float32, torch.bfloat16, torch.float16]
compare_cases = gate_cases = 0
verdicts = {"compare": [0, 0], "gate": [0, 0]}
bad = []

def quiet(f, *a, **k):
    with contextlib.redirect_stdout(io.StringIO()):
        return f(*a, **k)

for trial in range(300):
    n_out = rnd.randint(1, 3)
    eager, oracle = [], []
    for _ in range(n_out):
        shape = [rnd.randint(1, 9), rnd.randint(1, 33)]
        kind = rnd.choice(["float", "float", "float", "int", "bool"])
        if kind == "float":
            dt = rnd.choice(FLOATS)
            e = (torch.randn(shape, generator=g) * rnd.choice([0.01, 1.0, 30.0])).to(dt)
            o = e.clone()
            mode = rnd.choice(["same", "rel", "abs", "nan_same", "nan_diff", "dtype"])
            if mode == "rel":
                o = (e.float() * (1 + rnd.choice([1e-3, 5e-3, 2e-2, 1e-1]))).to(dt)
            elif mode == "abs":
                o = (e.float() + rnd.choice([1e-3, 5e-3, 2e-2, 1e-1])).to(dt)
            elif mode == "nan_same":
                e[0, 0] = float("nan"); o = e.clone()
            elif mode == "nan_diff":
                o = e.clone(); o[0, 0] = float("nan")
            elif mode == "dtype":
                o = e.float()
        elif kind == "int":
            e = torch.randint(-5, 5, shape, generator=g)
            o = e.clone()
            if rnd.random() < 0.3: o[0, 0] += 1
        else:
            e = torch.rand(shape, generator=g) > 0.5
            o = e.clone()
            if rnd.random() < 0.3: o[0, 0] = ~o[0, 0]
        if rnd.random() < 0.05:
            o = o[:, : max(1, o.shape[1] - 1)]          # shape mismatch
        eager.append(e); oracle.append(o)
    if rnd.random() < 0.05:
        oracle = oracle[:-1] if len(oracle) > 1 else oracle + [oracle[0]]   # count mismatch
    stochastic = {0} if rnd.random() < 0.15 else set()
    a = quiet(oh._compare_oracle_outputs, eager, oracle, stochastic, atol=1e-2, rtol=1e-2)
    b = quiet(mirror._compare_oracle_outputs, eager, oracle, stochastic, atol=1e-2, rtol=1e-2)
    compare_cases += 1
    verdicts["compare"][int(bool(a))] += 1
    if bool(a) != bool(b):
        bad.append(("compare", trial, bool(a), bool(b)))

for trial in range(300):
    n_out = rnd.randint(1, 3)
    ref, comp, orc = [], [], []
    for _ in range(n_out):
        shape = [rnd.randint(1, 9), rnd.randint(1, 33)]
        if rnd.random() < 0.15:
            t = torch.randint(0, 9, shape, generator=g)
            ref.append(t); comp.append(t.clone()); orc.append(t.clone()); continue
        base = torch.randn(shape, generator=g, dtype=torch.float64) * rnd.choice([1e-3, 1.0, 100.0])
        dt = rnd.choice(FLOATS)
        ec, eo = rnd.choice([0.0, 1e-7, 1e-4, 1e-2]), rnd.choice([0.0, 1e-7, 2e-7, 1e-4, 2.9e-4, 3.1e-4, 1e-1])
        c = (base * (1 + ec)).to(dt); o = (base * (1 + eo)).to(dt)
        if rnd.random() < 0.1: o[0, 0] = float("nan")
        if rnd.random() < 0.05: c[0, 0] = float("inf")
        ref.append(base); comp.append(c); orc.append(o)
    stochastic = {0} if rnd.random() < 0.15 else set()
    a = oh._anchored_numerics_gate(orc, comp, ref, stochastic)
    b = mirror._anchored_numerics_gate(orc, comp, ref, stochastic)
    gate_cases += 1
    verdicts["gate"][int(bool(a["pass"]))] += 1
    same = a["pass"] == b["pass"] and a["worst_output_idx"] == b["worst_output_idx"] and len(a["per_output"]) == len(b["per_output"])
    for x, y in zip(a["per_output"], b["per_output"]):
        for key in ("skip", "pass"):
            same = same and x.get(key) == y.get(key)
        for key in ("err_oracle", "err_compiled", "threshold"):
            if key in x or key in y:
                u, v = x.get(key), y.get(key)
                same = same and u is not None and v is not None and (u == v or (u != u and v != v) or abs(u - v) <= 1e-12 * max(abs(u), abs(v), 1e-300))
    if not same:
        bad.append(("gate", trial, a, b))
# the reviewed opt-out: which annotations load, and which failing gates it may accept
optout_cases = 0
verdicts["optout"] = [0, 0]
tmp = Path(sys.argv[3])
METAS = [None, "not json", {}, {"numerics_optout": None}, {"numerics_optout": {"verified": True}},
         {"numerics_optout": {"verified": True, "reason": "  "}}, {"numerics_optout": {"verified": "yes", "reason": "r"}},
         {"numerics_optout": {"verified": True, "reason": "reviewed: rounding of the intermediate"}},
         {"numerics_optout": {"verified": False, "reason": "r"}}, ["list"]]
for i, meta in enumerate(METAS):
    d = tmp / f"meta_{i}"
    d.mkdir()
    if meta is not None:
        (d / "meta.json").write_text(meta if isinstance(meta, str) else json.dumps(meta))
    with contextlib.redirect_stderr(io.StringIO()):
        a, b = oh.load_numerics_optout(d), mirror.load_numerics_optout(d)
    if a != b:
        bad.append(("load_optout", i, a, b))
opt = {"verified": True, "reason": "reviewed"}
for trial in range(300):
    entries = []
    for idx in range(rnd.randint(0, 4)):
        e = {"idx": idx, "pass": rnd.choice([True, False, False])}
        if rnd.random() < 0.1:
            e["skip"] = "non_float"; e.pop("pass")
        else:
            e["err_oracle"] = rnd.choice([None, float("nan"), float("inf"), 10 ** rnd.uniform(-9, 3)])
            e["ref_absmax"] = rnd.choice([0.0, None, 10 ** rnd.uniform(-6, 4)])
        entries.append(e)
    result = rnd.choice([None, {"pass": False, "per_output": entries}, {"pass": False, "per_output": entries}])
    use = rnd.choice([opt, opt, None, {}])
    a, b = oh.numerics_optout_applies(result, use), mirror.numerics_optout_applies(result, use)
    optout_cases += 1
    verdicts["optout"][int(bool(a["accept"]))] += 1
    wa, wb = a.get("worst_offender") or {}, b.get("worst_offender") or {}
    if a["accept"] != b["accept"] or a.get("n_failing") != b.get("n_failing") or wa.get("idx") != wb.get("idx") \
            or bool(wa.get("non_finite")) != bool(wb.get("non_finite")):
        bad.append(("optout", trial, a, b))
print("RESULT " + json.dumps({"compare_cases": compare_cases, "gate_cases": gate_cases, "optout_cases": optout_cases, "verdicts": verdicts,
                              "mismatches": [str(m)[:600] for m in bad[:5]], "n_mismatches": len(bad)}))
"""


def test_mirror_comparison_and_gate_agree_with_the_reference_harness(tmp_path):
    """The package's mirror of `_compare_oracle_outputs` (oracle_harness.py:865-923) and
    `_anchored_numerics_gate` (:1479-1548), `load_numerics_optout` (:695-723) and
    `numerics_optout_applies` (:726-806) against the reference's own functions on 900 seeded
    random cases: matching and perturbed floats of three dtypes, NaNs in the same and in different
    places, dtype, shape and count mismatches, integer and boolean outputs, stochastic indices."""
    import json

    out = _run(_MIRROR_SCRIPT, str(tmp_path))
    res = json.loads(next(l for l in out.splitlines() if l.startswith("RESULT "))[len("RESULT "):])
    assert res["compare_cases"] == 300 and res["gate_cases"] == 300 and res["optout_cases"] == 300
    for kind in ("compare", "gate", "optout"):   # the cases must exercise both verdicts
        assert min(res["verdicts"][kind]) >= 30, res["verdicts"]
    assert res["n_mismatches"] == 0, res["mismatches"]


_INPUTS_SCRIPT = r"""
import json, sys
from pathlib import Path
sys.path[:0] = [sys.argv[1], sys.argv[2] + "/scripts", sys.argv[2]]
from better_benchmark_b200 import reference_arm as arm, inputs as mirror, byte_model
oh, rh = arm._import_reference(Path(sys.argv[2]))
import byte_accounting
import torch
LIMIT = 48 << 20     # bytes of tensor inputs per point: generation runs on the CPU here
dirs = sorted(p for p in (Path(sys.argv[2]) / "repros" / "canonical").iterdir() if (p / "shapes.json").is_file())
points = compared = bytes_compared = 0
bad = []

def total_bytes(cfg):
    n = 0
    for spec in cfg["inputs"]:
        if isinstance(spec, dict) and spec.get("kind", "tensor") == "tensor":
            size = 1
            for d, st in zip(spec["shape"], spec.get("stride") or mirror.contiguous_stride(spec["shape"])):
                size += (d - 1) * st if d > 0 else 0
            n += size * 4
    return n

def on_cpu(cfg):
    for spec in cfg["inputs"]:
        if isinstance(spec, dict) and spec.get("kind", "tensor") == "tensor":
            spec["device"] = "cpu"
    return cfg

def same(a, b):
    if isinstance(a, torch.Tensor) or isinstance(b, torch.Tensor):
        return (isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor) and a.dtype == b.dtype and a.shape == b.shape
                and a.stride() == b.stride() and a.storage_offset() == b.storage_offset()
                and torch.equal(torch.nan_to_num(a.float()), torch.nan_to_num(b.float())))
    return type(a) == type(b) and a == b

for d in dirs:
    ref_cfgs = rh.load_shape_configs(str(d / "repro.py"))
    my_cfgs = mirror.load_shape_configs(d / "repro.py")
    if list(ref_cfgs) != list(my_cfgs):
        bad.append((d.name, "labels differ")); continue
    instance = None
    for label in sorted(ref_cfgs, key=lambda k: total_bytes(ref_cfgs[k]))[:4]:   # the smallest points of the directory
        points += 1
        if total_bytes(ref_cfgs[label]) > LIMIT:
            continue
        oh._seed_input_generation(1)
        a = rh.make_inputs_from_config(on_cpu(ref_cfgs[label]))
        oh._seed_input_generation(1)
        b = mirror.make_inputs_from_config(on_cpu(my_cfgs[label]))
        compared += 1
        if len(a) != len(b) or not all(same(x, y) for x, y in zip(a, b)):
            bad.append((d.name, label, "inputs differ")); continue
        # alias groups: inputs that share storage in one list must share it in the other
        pa = [x.untyped_storage().data_ptr() if isinstance(x, torch.Tensor) else None for x in a]
        pb = [x.untyped_storage().data_ptr() if isinstance(x, torch.Tensor) else None for x in b]
        if [pa.index(v) for v in pa] != [pb.index(v) for v in pb]:
            bad.append((d.name, label, "aliasing differs")); continue
        if bytes_compared < 40:          # the byte model on the same inputs (an eager CPU run under dispatch)
            try:
                if instance is None:
                    instance = oh.get_repro_instance(d)
                want = int(byte_accounting.count_bytes_effective(instance, [x.clone() if isinstance(x, torch.Tensor) else x for x in a]))
                got = int(byte_model.count_bytes_effective(instance, [x.clone() if isinstance(x, torch.Tensor) else x for x in b]))
            except Exception as e:   # a graph that does not run on the CPU (device-specific ops): skipped
                continue
            bytes_compared += 1
            if want != got:
                bad.append((d.name, label, f"bytes {want} != {got}"))
print("RESULT " + json.dumps({"dirs": len(dirs), "points": points, "compared": compared, "bytes_compared": bytes_compared,
                              "n_bad": len(bad), "bad": [str(x) for x in bad[:8]]}))
"""


def test_mirror_shape_decoding_inputs_and_byte_model_agree_with_the_reference(tmp_path):
    """`inputs.load_shape_configs` / `make_inputs_from_config` against `repro_harness.py:56-157`,
    `:430-569` and `byte_model.count_bytes_effective` against `byte_accounting.py:54-66` on the staged
    directories: same labels in the same order; with the same seed the same values, dtypes, strides,
    storage offsets and alias groups (the four smallest points per directory, inputs up to 48 MB);
    the same effective byte count on up to 40 of them."""
    import json

    out = _run(_INPUTS_SCRIPT, str(tmp_path), timeout=1500)
    res = json.loads(next(l for l in out.splitlines() if l.startswith("RESULT "))[len("RESULT "):])
    assert res["dirs"] >= 19 and res["compared"] >= 60 and res["bytes_compared"] >= 20, res
    assert res["n_bad"] == 0, res["bad"]


_SWEEP_SCRIPT = r"""
import json, random, sys
from pathlib import Path
sys.path[:0] = [sys.argv[1], sys.argv[2] + "/scripts", sys.argv[2]]
from better_benchmark_b200 import reference_arm as arm, sweep as mirror
oh, rh = arm._import_reference(Path(sys.argv[2]))
import bench_parallel as bp
rnd = random.Random(11)
out_dir = Path(sys.argv[3])
bad = []

# task keys and their expansion over the staged directories (the mirror orders directories with the
# most points first; the set of keys is what has to agree)
dirs = sorted(p for p in (Path(sys.argv[2]) / "repros" / "canonical").iterdir() if (p / "repro.py").is_file())
ref_tasks = bp._expand_oracle_shape_tasks(dirs)
my_tasks = mirror.expand_shape_tasks(dirs)
if sorted(ref_tasks) != sorted(my_tasks):
    bad.append("task keys differ")
if any(bp._oracle_dir_name(t) != mirror.oracle_dir_name(t) for t in ref_tasks):
    bad.append("directory names of task keys differ")

STATUSES = ["GOOD", "AT_FLOOR", "BAD_ORACLE"] + sorted(oh._INVALID_STATUSES)
REF_POINT = ("oracle_us", "compile_us", "ratio", "status")

def point():
    status = rnd.choice(STATUSES + ["GOOD", "GOOD", "AT_FLOOR"])
    us = rnd.choice([None, round(rnd.uniform(4, 900), 2), round(rnd.uniform(4, 900), 2)])
    p = {"status": status, "oracle_us": us, "compile_us": rnd.choice([None, round(rnd.uniform(4, 900), 2)]),
         "ratio": rnd.choice([None, round(rnd.uniform(0.3, 3), 3)])}
    if rnd.random() < 0.7:
        p["dispatch"] = {"fallback": rnd.random() < 0.2, "matched": "hardware+shape"}
    if rnd.random() < 0.5:
        p.update(region_bytes=rnd.randint(1, 1 << 30), oracle_gbps=rnd.uniform(1, 6000), sol_frac=rnd.random())
    return p

def subset_equal(ref, mine, where):
    # everything the reference writes must be in the mirror's output with the same value; the mirror
    # may add fields (its GB/s columns)
    if isinstance(ref, dict):
        if not isinstance(mine, dict):
            bad.append(f"{where}: not a dict"); return
        for k, v in ref.items():
            if k not in mine:
                bad.append(f"{where}: key {k!r} missing")
            else:
                subset_equal(v, mine[k], f"{where}.{k}")
        if where.count(".") == 0 and set(mine) - set(ref):
            bad.append(f"{where}: extra top-level keys {sorted(set(mine) - set(ref))}")
    elif ref != mine:
        bad.append(f"{where}: {ref!r} != {mine!r}")

trials = 0
for trial in range(60):
    all_results, failures = {}, {}
    for d in range(rnd.randint(1, 8)):
        dname = f"/x/canonical/dir_{trial}_{d:02d}abcdef"
        hashes = [f"{rnd.getrandbits(32):08x}" for _ in range(rnd.randint(0, 5))]
        sharded = rnd.random() < 0.7
        whole = {}
        for h in hashes:
            labels = [f"model{m}_{h}" for m in range(rnd.choice([1, 1, 2]))]   # two labels can share a hash
            for label in labels:
                if rnd.random() < 0.15:
                    failures[mirror.make_task_key(dname, label)] = {"error": f"RuntimeError: boom {label}", "gpu": "0"}
                    continue
                if sharded:
                    all_results[bp._make_shape_task_key(dname, label)] = {label: point()}
                else:
                    whole[label] = point()
        if not sharded:
            all_results[dname] = whole
        if rnd.random() < 0.1:
            all_results[mirror.make_task_key(dname, "__default__")] = {"default": point()}
    a = bp._aggregate_oracle_timings(all_results)
    b = mirror.aggregate_oracle_timings(all_results)
    subset_equal(a, b, f"aggregate[{trial}]")
    wa = bp._write_oracle_timings_output(out_dir / f"ref_{trial}.json", all_results, failures or None)
    wb = mirror.write_oracle_timings(out_dir / f"mine_{trial}.json", all_results, failures or None)
    subset_equal(wa, wb, f"write[{trial}]")
    subset_equal(json.loads((out_dir / f"ref_{trial}.json").read_text()), json.loads((out_dir / f"mine_{trial}.json").read_text()),
                 f"file[{trial}]")
    trials += 1
print("RESULT " + json.dumps({"tasks": len(ref_tasks), "trials": trials, "n_bad": len(bad), "bad": bad[:8]}))
"""


def test_mirror_sweep_tasks_and_timings_file_agree_with_the_reference(tmp_path):
    """`sweep.expand_shape_tasks`, `aggregate_oracle_timings` and `write_oracle_timings` against
    `scripts/bench_parallel.py:145-168`, `:1263-1384` and `:1407-1453` of the staged reference: the
    same task keys for the staged directories, and on 60 seeded random result sets (sharded and whole
    directories, shared shape hashes, invalid statuses, missing times, failed tasks) every field the
    reference writes into the timings file with the same value; the mirror only adds fields."""
    import json

    if not (REF / "scripts" / "bench_parallel.py").is_file():
        pytest.skip("the staged copy predates the sweep script: stage again")
    out = _run(_SWEEP_SCRIPT, str(tmp_path))
    res = json.loads(next(l for l in out.splitlines() if l.startswith("RESULT "))[len("RESULT "):])
    assert res["tasks"] >= 226 and res["trials"] == 60
    assert res["n_bad"] == 0, res["bad"]


_LOCK_SCRIPT = r"""
import json, os, subprocess, sys, time
from pathlib import Path
sys.path[:0] = [sys.argv[1], sys.argv[2] + "/scripts", sys.argv[2]]
lock_dir = sys.argv[3]
os.environ["COMPILE_UTILS_GPU_LOCK_DIR"] = lock_dir
os.environ["CUDA_VISIBLE_DEVICES"] = "3"
for k in ("INDUCTOR_GPU_BENCH_LOCK_DIR", "TORCHINDUCTOR_GPU_BENCH_LOCK_DIR"):
    os.environ.pop(k, None)

HOLD_REFERENCE = (
    "import sys, time; sys.path[:0] = [%r + '/scripts', %r]\n"
    "import oracle_harness as oh\n"
    "with oh._gpu_exclusive_lock('holder'):\n"
    "    print('HELD', flush=True); time.sleep(float(sys.argv[1]))\n"
    "print('RELEASED', flush=True)\n" % (sys.argv[2], sys.argv[2]))
HOLD_MIRROR = (
    "import sys, time; sys.path[:0] = [%r]\n"
    "from better_benchmark_b200 import gpu_lock\n"
    "with gpu_lock.gpu_exclusive_lock('holder'):\n"
    "    print('HELD', flush=True); time.sleep(float(sys.argv[1]))\n"
    "print('RELEASED', flush=True)\n" % (sys.argv[1],))

def holder(code, seconds):
    p = subprocess.Popen([sys.executable, "-c", code, str(seconds)], stdout=subprocess.PIPE, text=True, env=os.environ.copy())
    assert p.stdout.readline().strip() == "HELD"
    return p

out = {}
# 1. the reference holds: the mirror must wait (time out while held, get through after the release)
from better_benchmark_b200 import gpu_lock
import oracle_harness as oh          # imported before any holder starts: the waits below time the locks only
p = holder(HOLD_REFERENCE, 2.0)
try:
    with gpu_lock.gpu_exclusive_lock("waiter", timeout_s=0.4):
        out["mirror_entered_while_reference_held"] = True
except TimeoutError:
    out["mirror_entered_while_reference_held"] = False
meta = gpu_lock.read_lock_metadata(os.path.join(lock_dir, "gpu_3.lock"))
out["mirror_reads_reference_metadata"] = {k: meta.get(k) for k in ("label", "mode", "gpu")}
p.wait(timeout=20)
t0 = time.time()
with gpu_lock.gpu_exclusive_lock("waiter", timeout_s=5):
    out["mirror_entered_after_release"] = True
# 2. the mirror holds: the reference's lock (which has no timeout) must block until the release
p = holder(HOLD_MIRROR, 1.5)
t0 = time.time()
with oh._gpu_exclusive_lock("waiter"):
    out["reference_waited_s"] = round(time.time() - t0, 2)
p.wait(timeout=20)
out["files"] = sorted(os.listdir(lock_dir))
print("RESULT " + json.dumps(out))
"""


def test_mirror_gpu_lock_and_the_reference_lock_exclude_each_other(tmp_path):
    """A sweep of this backend and a sweep of the reference on one box must not time at once: the
    mirror's lock (`gpu_lock.py`) and `oracle_harness._gpu_exclusive_lock` (:1614-1692) use the same
    gate and lock files under the same directory rule and the same flock protocol. Checked with
    holder processes on both sides."""
    import json

    out = _run(_LOCK_SCRIPT, str(tmp_path / "locks"), timeout=120)
    res = json.loads(next(l for l in out.splitlines() if l.startswith("RESULT "))[len("RESULT "):])
    assert res["mirror_entered_while_reference_held"] is False
    assert res["mirror_entered_after_release"] is True
    assert res["mirror_reads_reference_metadata"]["label"] == "holder"
    assert res["mirror_reads_reference_metadata"]["mode"] == "exclusive"
    assert res["reference_waited_s"] >= 1.0, res          # it blocked for most of the holder's 1.5 s
    assert res["files"] == ["gpu_3.gate", "gpu_3.lock"]


_REGISTRY_SCRIPT = r"""
import json, random, sys, types
from pathlib import Path
sys.path[:0] = [sys.argv[1], sys.argv[2] + "/scripts", sys.argv[2]]
from better_benchmark_b200 import reference_arm as arm, harness as mirror
oh, rh = arm._import_reference(Path(sys.argv[2]))
import torch
rnd = random.Random(23)
SHAPES = [(8, 16), (4, 4, 4), (128,), (2, 3), (1, 1, 7, 7)]
SIGS = [((8, 16),), ((8, 16), (128,)), ((4, 4, 4), (2, 3)), ((128,), (128,), (2, 3)), ((1, 1, 7, 7),)]
STRINGS = {((8, 16),): "T([8, 16], bf16)", ((8, 16), (128,)): "T([8, 16], f32), T([128], f32), S([8, 16])",
           ((4, 4, 4), (2, 3)): "T([4, 4, 4], f16), T([2, 3], i64)"}
KEYS = ("matched", "fallback", "fn_name", "description", "tuned_hardware", "registered_shape", "configs",
        "current_hardware", "actual_shapes", "dtype_mismatch")
bad, outcomes = [], {"raise": 0}
cases = 0

def build(H, name, regs):
    mod = types.ModuleType(name)
    sys.modules[name] = mod
    fns = []
    for i, (hw, sig, cfg, as_string) in enumerate(regs):
        src = f"def impl_{i}(inputs, **kw):\n    return ({i}, tuple(sorted(kw.items())))\n"
        exec(compile(src, name, "exec"), mod.__dict__)
        fn = mod.__dict__[f"impl_{i}"]
        fn.__module__ = name
        shapes = STRINGS[sig] if (as_string and sig in STRINGS) else sig
        H.oracle_impl(hardware=hw, shapes=shapes, description=f"reg {i}", **cfg)(fn)
        fns.append(fn)
    return fns

for trial in range(120):
    regs = []
    for _ in range(rnd.randint(1, 6)):
        hw = rnd.choice([None, "B200", "B200", "H100"])
        sig = rnd.choice([None, None] + SIGS)
        cfg = rnd.choice([{}, {"BLOCK": rnd.choice([128, 256])}, {"num_warps": 4, "BLOCK": 64}])
        regs.append((hw, sig, cfg, rnd.random() < 0.5))
    fa = build(oh, f"_oracle_synth_ref_{trial}", regs)
    fb = build(mirror, f"_oracle_synth_mine_{trial}", regs)
    for kind in ("B200", "H100", "unknown"):
        oh.get_gpu_kind._cached = kind
        mirror.get_gpu_kind._cached = kind
        for _ in range(4):
            sig = rnd.choice(SIGS + [((3, 3),)])
            dt = rnd.choice([torch.float32, torch.bfloat16, torch.float16])
            inputs = [torch.empty(sh, dtype=dt, device="meta") for sh in sig]
            if rnd.random() < 0.5:
                inputs.insert(rnd.randint(0, len(inputs)), [8, -1])      # a lifted shape parameter
            if rnd.random() < 0.3:
                inputs.append(7)
            res = []
            for H, fns in ((oh, fa), (mirror, fb)):
                try:
                    fn, info = H.resolve_oracle(fns[0], inputs)
                    res.append(("ok", fn(inputs), {k: info.get(k) for k in KEYS}))
                except H.OracleDispatchError:
                    res.append(("raise", None, None))
            cases += 1
            a, b = res
            if a[0] == "raise":
                outcomes["raise"] += 1
            else:
                outcomes[a[2]["matched"]] = outcomes.get(a[2]["matched"], 0) + 1
            if a[0] != b[0] or a[1] != b[1]:
                bad.append((trial, kind, str(a)[:200], str(b)[:200])); continue
            if a[0] == "ok":
                for k in KEYS:
                    if a[2][k] != b[2][k]:
                        bad.append((trial, kind, k, str(a[2][k])[:120], str(b[2][k])[:120]))
print("RESULT " + json.dumps({"cases": cases, "outcomes": outcomes, "n_bad": len(bad), "bad": [str(x) for x in bad[:6]]}))
"""


def test_mirror_registration_and_dispatch_agree_with_the_reference(tmp_path):
    """`oracle_impl` / `OracleRegistry.select` / `resolve_oracle` of the mirror against
    oracle_harness.py:468-549, :251-340, :557-577 on 120 seeded random registries (hardware or none,
    signature as tuples or as the repro's T()/S() string or none, bound launch arguments), resolved
    on three GPU kinds with matching and foreign input signatures: the same entry is chosen (or the
    same refusal raised), with the same dispatch record."""
    import json

    out = _run(_REGISTRY_SCRIPT, str(tmp_path))
    res = json.loads(next(l for l in out.splitlines() if l.startswith("RESULT "))[len("RESULT "):])
    assert res["cases"] == 120 * 3 * 4
    for tier in ("hardware+shape", "shape", "hardware", "any", "raise"):
        assert res["outcomes"].get(tier, 0) >= 20, res["outcomes"]
    assert res["n_bad"] == 0, res["bad"]


_ROLLUP_SCRIPT = r"""
import contextlib, io, json, random, sys
from pathlib import Path
sys.path[:0] = [sys.argv[1], sys.argv[2] + "/scripts", sys.argv[2]]
from better_benchmark_b200 import rollup
import model_graph_accounting as mga
rnd = random.Random(31)
bad, modes = [], {}

def occurrence(h):
    return mga.PartitionOccurrence(graph_name="g", pattern_hash="p", shape_hash=h, n_ops=1, op_counts={}, origin_ops=[],
                                   input_shapes=[], max_output_shape=None, has_reduction=False)

def number():
    return rnd.choice([None, "n/a", round(rnd.uniform(4, 900), 2), round(rnd.uniform(4, 900), 2)])

for trial in range(400):
    hashes = [f"{rnd.getrandbits(32):08x}" for _ in range(rnd.randint(0, 6))]
    kind = rnd.random()
    if kind < 0.1:
        timing = None
    elif kind < 0.25:
        timing = {"oracle_us": number(), "compile_us": number()}                     # a file without per-shape data
    else:
        timing = {"oracle_us": number(), "compile_us": number(),
                  "points_by_shape": {h: rnd.choice([{"oracle_us": number(), "compile_us": number(), "status": "GOOD"},
                                                     "junk"]) for h in hashes if rnd.random() < 0.7}}
        if rnd.random() < 0.1:
            timing = {}
    uses = [rnd.choice(hashes + ["ffffffff"]) for _ in range(rnd.randint(0, 12))] if hashes else ["ffffffff"] * rnd.randint(0, 3)
    if hashes and rnd.random() < 0.25:                                                  # every use has a point of its own
        timing = {"oracle_us": number(), "compile_us": number(),
                  "points_by_shape": {h: {"oracle_us": round(rnd.uniform(4, 900), 2), "compile_us": number()} for h in hashes}}
        uses = [rnd.choice(hashes) for _ in range(rnd.randint(1, 12))]
    with contextlib.redirect_stderr(io.StringIO()):
        a = mga._rollup_occurrence_timings(timing, [occurrence(h) for h in uses])
    b = rollup.price_uses(timing, uses)
    modes[a["mode"]] = modes.get(a["mode"], 0) + 1
    if a != b:
        bad.append((trial, a, b))
print("RESULT " + json.dumps({"cases": 400, "modes": modes, "n_bad": len(bad), "bad": [str(x)[:500] for x in bad[:5]]}))
"""


def test_rollup_pricing_agrees_with_the_reference_accounting(tmp_path):
    """`rollup.price_uses` against `_rollup_occurrence_timings`
    (scripts/model_graph_accounting.py:413-535) on 400 seeded random directory records and use
    lists: per-shape points, missing and non-numeric times, records without per-shape data, untimed
    directories. Same totals, same matched / fallback / unpriced counts, same mode."""
    import json

    if not (REF / "scripts" / "model_graph_accounting.py").is_file():
        pytest.skip("the staged copy predates the accounting script: stage again")
    out = _run(_ROLLUP_SCRIPT, str(tmp_path))
    res = json.loads(next(l for l in out.splitlines() if l.startswith("RESULT "))[len("RESULT "):])
    for mode in ("untimed", "legacy", "per_shape", "partial", "fallback_only"):
        assert res["modes"].get(mode, 0) >= 10, res["modes"]
    assert res["n_bad"] == 0, res["bad"]


_CHECK_SCRIPT = r"""
import json, sys
from pathlib import Path
sys.path[:0] = [sys.argv[1], sys.argv[2] + "/scripts", sys.argv[2]]
from better_benchmark_b200 import reference_arm as arm, native
oh, rh = arm._import_reference(Path(sys.argv[2]))
dirs = arm.assemble_b200_dirs(Path(sys.argv[2]), Path(sys.argv[3]))
before = native.load().b200_launch_count()
out = {}
for name in sys.argv[4].split(","):
    mod, fn, d = oh._load_oracle_module(dirs[name])
    verdicts = oh.check_oracle_all_shapes(fn, d, name, skip_stochastic=True)
    out[name] = {k: bool(v) for k, v in verdicts.items()}
out["_launches"] = native.load().b200_launch_count() - before
print("RESULT " + json.dumps(out))
"""


@pytest.mark.gpu
def test_reference_check_oracle_all_shapes_passes_on_shipped_stubs(tmp_path):
    import json

    names = ["var_mean_f8ec553e339e", "amax_sum_20ccc18dda60", "sum_eb86a17deab9", "pointwise_c0d19d490a2f",
             "var_mean_b200c2a00002"]
    out = _run(_CHECK_SCRIPT, str(tmp_path), ",".join(names))
    line = next(l for l in out.splitlines() if l.startswith("RESULT "))
    res = json.loads(line[len("RESULT "):])
    assert res.pop("_launches") > 0, "the reference's check ran, but this library launched nothing"
    for name in names:
        assert res[name] and all(res[name].values()), (name, res[name])
