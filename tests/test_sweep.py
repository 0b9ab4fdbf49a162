"""Host logic of the corpus sweep: task keys, worker count, the parent/worker line protocol with
fake workers (misaligned answers, crashes, CUDA errors, timeouts), aggregation and the output file.
CPU only; the model for these cases is the reference's tests/test_oracle_sharding.py,
tests/test_bench_recovery.py and tests/test_bench_accounting.py."""
import json
import queue
import sys
import textwrap

import pytest

from better_benchmark_b200 import sweep


# ------------------------------------------------------------------------------------------ tasks
def test_task_key_roundtrip_and_default_token():
    key = sweep.make_task_key("/a/b/var_mean_123", "bert_c2a00002")
    assert key == "/a/b/var_mean_123::SHAPE::bert_c2a00002"
    assert sweep.split_task_key(key) == ("/a/b/var_mean_123", "bert_c2a00002")
    assert sweep.split_task_key(sweep.make_task_key("/d", sweep.DEFAULT_SHAPE_TOKEN)) == ("/d", "__default__")
    assert sweep.result_label("__default__") == "default" and sweep.result_label("x") == "x"


def test_split_bare_path_and_last_separator():
    assert sweep.split_task_key("/plain/dir") == ("/plain/dir", None)
    odd = "/p::SHAPE::q::SHAPE::label"
    assert sweep.split_task_key(odd) == ("/p::SHAPE::q", "label")
    assert sweep.oracle_dir_name("/x/y/sum_abc::SHAPE::l1") == "sum_abc"
    assert sweep.oracle_dir_name("/x/y/sum_abc") == "sum_abc"


def _make_dir(root, name, labels):
    d = root / name
    d.mkdir(parents=True)
    (d / "repro.py").write_text("class Repro: pass\n")
    (d / "oracle.py").write_text("def oracle_forward(inputs): return inputs\n")
    if labels is not None:
        (d / "shapes.json").write_text(json.dumps({"points": [
            {"shape_hash": l.rsplit("_", 1)[-1], "models": {f"suite/{l.rsplit('_', 1)[0]}": {"occurrences": 1}},
             "inputs": [[[2], "f32"]]} for l in labels]}))
    return d


def test_find_and_expand_sorts_big_dirs_first(tmp_path):
    _make_dir(tmp_path, "small_1", ["m_aaaa0001"])
    _make_dir(tmp_path, "big_3", ["m_bbbb0001", "m_bbbb0002", "m_bbbb0003"])
    _make_dir(tmp_path, "none_0", None)
    (tmp_path / "not_canonical").mkdir()
    (tmp_path / "not_canonical" / "oracle.py").write_text("")
    dirs = sweep.find_oracle_dirs([tmp_path])
    assert [d.name for d in dirs] == ["big_3", "none_0", "small_1"]
    tasks = sweep.expand_shape_tasks(dirs)
    assert [sweep.oracle_dir_name(t) for t in tasks[:3]] == ["big_3"] * 3
    assert any(t.endswith("::SHAPE::__default__") and "none_0" in t for t in tasks)
    assert len(tasks) == 5
    # a single canonical directory given directly
    assert [d.name for d in sweep.find_oracle_dirs([tmp_path / "small_1"])] == ["small_1"]


def test_expand_falls_back_to_default_when_shapes_cannot_be_read(tmp_path):
    d = _make_dir(tmp_path, "broken_1", None)
    (d / "shapes.json").write_text("{ not json")
    assert sweep.expand_shape_tasks([d]) == [f"{d}::SHAPE::__default__"]


# ----------------------------------------------------------------------------------- worker count
def test_worker_count_defaults_and_caps(monkeypatch):
    monkeypatch.setattr(sweep.os, "sched_getaffinity", lambda _: set(range(64)), raising=False)
    assert sweep.compute_worker_count(num_tasks=100, num_gpus=8) == (32, 4)
    monkeypatch.setattr(sweep.os, "sched_getaffinity", lambda _: set(range(8)), raising=False)
    assert sweep.compute_worker_count(num_tasks=100, num_gpus=4) == (8, 2)
    assert sweep.compute_worker_count(num_tasks=3, num_gpus=4) == (3, 2)
    assert sweep.compute_worker_count(num_tasks=100, num_gpus=2, max_workers=6) == (6, 3)
    assert sweep.compute_worker_count(num_tasks=100, num_gpus=2, max_workers=9, workers_per_gpu=2) == (4, 2)
    assert sweep.compute_worker_count(num_tasks=0, num_gpus=2) == (0, 1)
    with pytest.raises(ValueError):
        sweep.compute_worker_count(num_tasks=1, num_gpus=0)
    with pytest.raises(ValueError):
        sweep.compute_worker_count(num_tasks=1, num_gpus=1, max_workers=0)
    with pytest.raises(ValueError):
        sweep.compute_worker_count(num_tasks=1, num_gpus=1, workers_per_gpu=0)


# ------------------------------------------------------------------------- parent <-> fake worker
def _fake_worker(body: str):
    """A worker command whose per-task behaviour is the given Python snippet (sees ``task`` and
    ``n``, the 1-based count of tasks this process has served; must print one line or exit)."""
    head = textwrap.dedent("""
        import json, os, sys, time
        n = 0
        for raw in sys.stdin:
            task = raw.strip()
            if not task or task == "EXIT":
                break
            if task.startswith("PREFETCH:"):
                continue
            n += 1
    """)
    script = head + textwrap.indent(textwrap.dedent(body), "    ")
    return lambda options: [sys.executable, "-u", "-c", script]


GOOD = """
print(json.dumps({"lbl": {"oracle_us": 10.0 + n, "status": "TIMED", "pid": os.getpid(),
                          "gpu": os.environ["CUDA_VISIBLE_DEVICES"],
                          "lock": os.environ.get("INDUCTOR_GPU_BENCH_LOCK")}, "_repro": task}), flush=True)
"""


def _serve(tasks, factory, **opts):
    tq, rq = queue.Queue(), queue.Queue()
    for t in tasks:
        tq.put(t)
    sweep.serve_gpu("3", tq, rq, dict(worker_command_factory=factory, task_timeout=20, **opts))
    out = []
    while not rq.empty():
        out.append(rq.get())
    return out


def test_one_persistent_worker_serves_all_tasks_pinned_and_locked():
    res = _serve(["/d/a::SHAPE::x", "/d/b::SHAPE::y", "/d/c::SHAPE::z"], _fake_worker(GOOD))
    assert [r["status"] for r in res] == ["ok"] * 3
    assert [r["repro"] for r in res] == ["/d/a::SHAPE::x", "/d/b::SHAPE::y", "/d/c::SHAPE::z"]
    points = [r["results"]["lbl"] for r in res]
    assert len({p["pid"] for p in points}) == 1, "the worker must persist across tasks"
    assert {p["gpu"] for p in points} == {"3"} and {p["lock"] for p in points} == {"1"}
    assert all("_repro" not in r["results"] for r in res)


def test_misaligned_answer_is_rejected_and_worker_restarted():
    body = """
    echoed = "/d/other::SHAPE::q" if (n == 1 and "first" in task) else task
    print(json.dumps({"lbl": {"oracle_us": 1.0, "status": "TIMED", "pid": os.getpid()}, "_repro": echoed}), flush=True)
    """
    res = _serve(["/d/first::SHAPE::x", "/d/second::SHAPE::y"], _fake_worker(body))
    assert res[0]["status"] == "failed" and "misalignment" in res[0]["error"]
    assert res[1]["status"] == "ok"


def test_worker_crash_cuda_error_and_python_error_are_survived():
    body = """
    if "crash" in task:
        sys.stderr.write("boom from native code\\n"); sys.stderr.flush(); os._exit(7)
    if "cuda" in task:
        print("CUDA_ERROR: an illegal memory access was encountered", flush=True); sys.exit(1)
    if "pyerr" in task:
        print(json.dumps({"_repro": task, "__error__": {"error": "bad shape", "category": "runtime_error",
              "exception_type": "ValueError", "reason": "r", "hint": "h"}}), flush=True); continue
    if "garbage" in task:
        print("something unexpected", flush=True); continue
    print(json.dumps({"lbl": {"oracle_us": 2.0, "status": "TIMED", "pid": os.getpid()}, "_repro": task}), flush=True)
    """
    tasks = ["/d/ok1::SHAPE::a", "/d/crash::SHAPE::a", "/d/ok2::SHAPE::a", "/d/cuda::SHAPE::a",
             "/d/ok3::SHAPE::a", "/d/pyerr::SHAPE::a", "/d/garbage::SHAPE::a", "/d/ok4::SHAPE::a"]
    res = {sweep.oracle_dir_name(r["repro"]): r for r in _serve(tasks, _fake_worker(body))}
    assert len(res) == len(tasks), "every task must be answered exactly once"
    for name in ("ok1", "ok2", "ok3", "ok4"):
        assert res[name]["status"] == "ok"
    assert "returncode=7" in res["crash"]["error"] and "boom from native code" in res["crash"]["error"]
    assert "CUDA_ERROR" in res["cuda"]["error"]
    assert res["pyerr"]["exception_type"] == "ValueError" and res["pyerr"]["error"] == "bad shape"
    assert "something unexpected" in res["garbage"]["error"]
    pids = [res[n]["results"]["lbl"]["pid"] for n in ("ok1", "ok2", "ok3", "ok4")]
    assert pids[0] != pids[1] and pids[1] != pids[2], "a crash and a CUDA error each cost the worker"
    assert pids[2] == pids[3], "a Python error or a stray line does not"


def test_unanswered_task_times_out_and_the_sweep_goes_on():
    body = """
    if "hang" in task:
        time.sleep(600)
    print(json.dumps({"lbl": {"oracle_us": 2.0, "status": "TIMED"}, "_repro": task}), flush=True)
    """
    tq, rq = queue.Queue(), queue.Queue()
    for t in ["/d/hang::SHAPE::a", "/d/fine::SHAPE::a"]:
        tq.put(t)
    sweep.serve_gpu("0", tq, rq, dict(worker_command_factory=_fake_worker(body), task_timeout=1.5))
    first, second = rq.get_nowait(), rq.get_nowait()
    assert first["status"] == "failed" and first["category"] == "timeout"
    assert second["status"] == "ok"


def test_worker_stdout_pollution_does_not_reach_the_result_pipe(tmp_path):
    """The real worker loop re-points fd 1 at stderr; a task that raises is reported as __error__."""
    tq, rq = queue.Queue(), queue.Queue()
    missing = tmp_path / "nowhere_1"
    tq.put(f"{missing}::SHAPE::lbl")
    sweep.serve_gpu("0", tq, rq, dict(task_timeout=120, warmup=1, rep=1))
    r = rq.get_nowait()
    assert r["status"] == "failed" and r["exception_type"] == "FileNotFoundError"


def test_run_sweep_shards_tasks_over_gpus_and_accounts_for_all():
    tasks = [f"/d/dir{i}::SHAPE::m_{i:08x}" for i in range(12)]
    results, failures, summary = sweep.run_sweep(
        tasks, ["0", "1"], options=dict(worker_command_factory=_fake_worker(GOOD), workers_per_gpu=2,
                                        task_timeout=30), log=lambda *_: None)
    assert not failures and set(results) == set(tasks)
    assert summary["n_workers"] == 4 and summary["n_ok"] == 12
    gpus = {results[t]["lbl"]["gpu"] for t in tasks}
    assert gpus <= {"0", "1"} and len({results[t]["lbl"]["pid"] for t in tasks}) <= 4


# ------------------------------------------------------------------------------------ aggregation
def _pt(us, status="GOOD", compile_us=None, **kw):
    p = {"oracle_us": us, "status": status}
    if compile_us is not None:
        p.update(compile_us=compile_us, ratio=round(compile_us / us, 3))
    p.update(kw)
    return p


SHARDED = {
    "/r/sum_aaa::SHAPE::bert_11111111": {"bert_11111111": _pt(10.0, compile_us=20.0)},
    "/r/sum_aaa::SHAPE::gpt_22222222": {"gpt_22222222": _pt(30.0, compile_us=33.0, status="AT_FLOOR")},
    "/r/sum_aaa::SHAPE::t5_33333333": {"t5_33333333": _pt(50.0, compile_us=40.0, status="BAD_ORACLE")},
    "/r/mean_bbb::SHAPE::x_44444444": {"x_44444444": {"status": "UNVERIFIED_NUMERICS"}},
}
UNSHARDED = {
    "/r/sum_aaa": {"bert_11111111": _pt(10.0, compile_us=20.0),
                   "gpt_22222222": _pt(30.0, compile_us=33.0, status="AT_FLOOR"),
                   "t5_33333333": _pt(50.0, compile_us=40.0, status="BAD_ORACLE")},
    "/r/mean_bbb": {"x_44444444": {"status": "UNVERIFIED_NUMERICS"}},
}


def test_aggregate_sharded_equals_unsharded_and_contents():
    a, b = sweep.aggregate_oracle_timings(SHARDED), sweep.aggregate_oracle_timings(UNSHARDED)
    assert a == b
    entry = a["sum_aaa"]
    assert entry["oracle_us"] == 20.0 and entry["n_points"] == 2 and entry["compile_us"] == 26.5
    assert set(entry["points"]) == {"bert_11111111", "gpt_22222222", "t5_33333333"}
    assert set(entry["points_by_shape"]) == {"11111111", "22222222", "33333333"}
    assert entry["points_by_shape"]["33333333"]["status"] == "BAD_ORACLE"
    assert a["__failures__"]["mean_bbb"]["reason"] == "no_valid_point"


def test_aggregate_reasons_shape_collisions_and_extras():
    res = {
        "/r/only_bad": {"a_1": _pt(5.0, status="BAD_ORACLE", compile_us=4.0)},
        "/r/empty": {},
        "/r/dup": {"m1_abcd": _pt(9.0, status="NUMERICS_WORSE_THAN_COMPILED"), "m2_abcd": _pt(7.0),
                   "m3_abcd": _pt(8.0, dispatch={"fallback": True}, region_bytes=100, oracle_gbps=1.0, sol_frac=0.5)},
    }
    out = sweep.aggregate_oracle_timings(res)
    assert out["__failures__"]["only_bad"]["reason"] == "all_bad_oracle"
    assert out["__failures__"]["empty"]["reason"] == "no_points"
    assert out["dup"]["points_by_shape"]["abcd"]["oracle_us"] == 7.0
    assert out["dup"]["points"]["m3_abcd"]["sol_frac"] == 0.5
    assert out["dup"]["oracle_us"] == 7.5 and out["dup"]["n_points"] == 2


def test_status_timed_counts_as_a_usable_point():
    out = sweep.aggregate_oracle_timings({"/r/d::SHAPE::a_1": {"a_1": _pt(4.0, status="TIMED")}})
    assert out["d"]["oracle_us"] == 4.0 and "compile_us" not in out["d"]


def test_regroup_task_failures():
    g = sweep.regroup_task_failures({
        "/r/sum_aaa::SHAPE::l1": {"error": "e1"}, "/r/sum_aaa::SHAPE::__default__": {"error": "e2"},
        "/r/other": {"error": "e3"}})
    assert g["sum_aaa"] == {"n_failed_shapes": 2, "failed_shapes": ["l1", "default"], "example_error": "e1"}
    assert g["other"]["failed_shapes"] == ["default"]


def test_write_accounts_for_every_failed_task(tmp_path):
    out = tmp_path / "nested" / "timings.json"
    failures = {
        "/r/sum_aaa::SHAPE::lost_99999999": {"error": "worker died"},           # dir still priced
        "/r/mean_bbb::SHAPE::y_55555555": {"error": "raised"},                  # dir has an aggregator failure
        "/r/gone_ccc::SHAPE::z_66666666": {"error": "raised too"},              # dir has nothing at all
    }
    timed = sweep.write_oracle_timings(out, SHARDED, failures, metadata={"tool": "t"})
    on_disk = json.loads(out.read_text())
    assert on_disk == json.loads(json.dumps(timed))
    assert on_disk["_metadata"] == {"tool": "t"}
    assert on_disk["sum_aaa"]["shape_failures"]["failed_shapes"] == ["lost_99999999"]
    f = on_disk["__failures__"]
    assert f["mean_bbb"]["reason"] == "no_valid_point" and f["mean_bbb"]["shape_failures"]["n_failed_shapes"] == 1
    assert f["gone_ccc"]["reason"] == "all_shapes_failed" and f["gone_ccc"]["example_error"] == "raised too"
    assert not list(out.parent.glob("*.tmp")), "the temporary file must not be left behind"


def test_write_without_failures_equals_pure_aggregate(tmp_path):
    out = tmp_path / "t.json"
    timed = sweep.write_oracle_timings(out, SHARDED)
    assert timed == sweep.aggregate_oracle_timings(SHARDED)
    assert json.loads(out.read_text()) == json.loads(json.dumps(timed))
