"""The timing side of the harness and the sweep on a real GPU: graph capture, the flushed-L2 timer,
the fp64-anchored gate inside bench_oracle, the comparison arm, the exclusive lock, and one sweep of
the five benchmark directories through persistent worker processes."""
import json
import os

import pytest
import torch

from conftest import assemble_canonical_dir

pytestmark = pytest.mark.gpu


def _load(tmp_path, name):
    from better_benchmark_b200 import harness
    from better_benchmark_b200.inputs import load_shape_configs, make_inputs_from_config
    from better_benchmark_b200.workloads import WORKLOADS
    wl = WORKLOADS[name]
    d = assemble_canonical_dir(wl.canonical_id, tmp_path)
    harness.reset_oracle_registry()
    harness.get_gpu_kind._cached = "B200"
    _, fn, d = harness._load_oracle_module(d)
    (label, config), = load_shape_configs(d / "repro.py").items()
    return wl, d, fn, harness, label, make_inputs_from_config(config, "cuda")


def test_do_bench_times_a_known_copy_and_flushes_l2():
    from better_benchmark_b200 import harness
    src = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    dst = torch.empty_like(src)
    us = harness.do_bench(lambda: dst.copy_(src), warmup=5, rep=20) * 1000
    gbps = 2 * src.numel() / (us * 1e-6) / 1e9
    assert 1000 < gbps < 9000, f"a 256 MiB device copy at {gbps:.0f} GB/s is not a B200 number"
    small = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    assert harness.do_bench(lambda: small.add_(1), warmup=2, rep=5) * 1000 < 100


def test_bench_oracle_without_comparison_arm(tmp_path):
    wl, d, fn, harness, label, inputs = _load(tmp_path, "c2_layer_norm_fwd")
    r = harness.bench_oracle(fn, harness.get_repro_instance(d), inputs, f"{d.name}_{label}", warmup=5, rep=50,
                             compile_reference=False, region_bytes=wl.algorithmic_bytes, peak_gbps=6552.0)
    assert r["status"] == "TIMED" and "compile_us" not in r
    assert 10 < r["oracle_us"] < 200
    assert r["region_bytes"] == wl.algorithmic_bytes and 0.05 < r["sol_frac"] < 1.3
    assert r["dispatch"]["matched"] == "hardware+shape" and r["dispatch"]["fallback"] is False
    gate = r["numerics_gate"]
    assert gate["pass"] is True


def test_bench_oracle_with_comparison_arm_and_lock(tmp_path, monkeypatch):
    monkeypatch.setenv("INDUCTOR_GPU_BENCH_LOCK", "1")
    monkeypatch.setenv("INDUCTOR_GPU_BENCH_LOCK_DIR", str(tmp_path / "locks"))
    wl, d, fn, harness, label, inputs = _load(tmp_path, "c1_row_mean")
    r = harness.bench_oracle(fn, harness.get_repro_instance(d), inputs, f"{d.name}_{label}", warmup=5, rep=50)
    assert r["status"] in ("GOOD", "AT_FLOOR", "BAD_ORACLE"), r
    assert r["compile_us"] > 0 and abs(r["ratio"] - r["compile_us"] / r["oracle_us"]) < 0.02
    assert (tmp_path / "locks").exists() and any((tmp_path / "locks").iterdir())


def test_bench_oracle_reports_no_oracle_for_an_unregistered_shape(tmp_path):
    wl, d, fn, harness, label, inputs = _load(tmp_path, "c1_row_mean")
    other = [torch.randn(64, 96, device="cuda")]
    r = harness.bench_oracle(fn, harness.get_repro_instance(d), other, "x", compile_reference=False)
    assert r["status"] == "NO_ORACLE_FOR_SHAPE"


def test_gate_rejects_a_sloppy_oracle(tmp_path):
    wl, d, fn, harness, label, inputs = _load(tmp_path, "c2_layer_norm_fwd")
    selected, _ = harness.resolve_oracle(fn, inputs)

    def sloppy(inp):
        y, mean, rstd = selected(inp)
        return (y * 1.05).to(y.dtype), mean, rstd

    r = harness.bench_oracle(sloppy, harness.get_repro_instance(d), inputs, "sloppy", warmup=2, rep=5)
    assert r["status"] == "NUMERICS_WORSE_THAN_COMPILED" and "oracle_us" not in r


def test_sweep_of_the_five_directories_on_one_gpu(tmp_path):
    from better_benchmark_b200 import sweep
    from better_benchmark_b200.workloads import WORKLOADS
    for wl in WORKLOADS.values():
        assemble_canonical_dir(wl.canonical_id, tmp_path)
    dirs = sweep.find_oracle_dirs([tmp_path])
    assert len(dirs) == 5
    tasks = sweep.expand_shape_tasks(dirs)
    assert len(tasks) == 5
    gpu = (os.environ.get("CUDA_VISIBLE_DEVICES") or "0").split(",")[0]
    out = tmp_path / "timings.json"
    results, failures, summary = sweep.run_sweep(
        tasks, [gpu], options=dict(warmup=3, rep=30, task_timeout=600, workers_per_gpu=2, peak_gbps=6552.0),
        output=out, log=print)
    assert not failures, failures
    timed = sweep.write_oracle_timings(out, results, failures, sweep.sweep_metadata(summary))
    on_disk = json.loads(out.read_text())
    assert "__failures__" not in on_disk
    for wl in WORKLOADS.values():
        entry = on_disk[wl.canonical_id]
        assert entry["n_points"] == 1 and 5 < entry["oracle_us"] < 500
        (point,) = entry["points_by_shape"].values()
        assert point["status"] == "TIMED" and point["fallback"] is False
        assert point["region_bytes"] == wl.algorithmic_bytes, (wl.name, point["region_bytes"])
        assert 0.05 < point["sol_frac"] < 1.3
    assert summary["n_workers"] == 2 and summary["n_ok"] == 5


def test_memcpy_sol_yardstick_and_gap_column(tmp_path):
    from better_benchmark_b200 import harness
    us = harness.memcpy_sol_us(200 << 20)
    assert 20 < us < 80, f"a 200 MiB read+write at {us:.1f} us is not a B200 number"
    wl, d, fn, harness, label, inputs = _load(tmp_path, "c3_masked_softmax")
    r = harness.bench_oracle(fn, harness.get_repro_instance(d), inputs, "sol", warmup=3, rep=20,
                             compile_reference=False, region_bytes=wl.algorithmic_bytes, memcpy_sol=True)
    assert r["status"] == "TIMED" and r["sol_us"] > 0 and 0.5 < r["gap"] < 3.0
