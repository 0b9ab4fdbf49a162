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
