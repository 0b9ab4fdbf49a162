"""Corpus sweep: shard (canonical dir, shape point) tasks over GPUs, check + time each point in
persistent worker processes, regroup per directory and write the timings file.

This is the ``--oracles`` path of the reference's sweep runner (scripts/bench_parallel.py):
task expansion ``:145-168``, worker count ``:824-869``, the per-worker parent loop ``:2688-2940``,
the worker's point routine ``:2943-3131`` and the aggregation ``:1263-1453``. What is kept is the
*protocol and the output schema*, so that the file this module writes can be consumed by the same
downstream tools:

  parent -> worker (one line each):  ``PREFETCH:<task>`` (hint, ignored), ``<task>``, ``EXIT``
  worker -> parent (one line per task):
      ``{"<label>": {...point...}, "_repro": "<task>"}``                     a result
      ``{"_repro": "<task>", "__error__": {...}}``                           a Python failure
      ``CUDA_ERROR: <text>``  then the worker exits                           a lost CUDA context
  task key: ``<dir>::SHAPE::<label>``; ``__default__`` for a directory without shape points.

Differences from the reference, all additive:
  * every wait for a worker's answer has a time limit (``--task-timeout``); a worker that does not
    answer in time is killed by PID and respawned, the task is recorded as failed;
  * points carry ``region_bytes`` / ``oracle_gbps`` / ``sol_frac`` when a peak is given;
  * the worker is this module (``python -m better_benchmark_b200.sweep --worker``), not a generated
    script, and GPU clocks are never touched (the reference locks them; clocks here are only read
    by the caller that wants them).

There is no cross-GPU data: results are merged on the host. One process per worker, pinned to its
GPU with CUDA_VISIBLE_DEVICES; timing windows on one GPU are serialised by the file lock
(``gpu_lock.py``), which the parent forces on through INDUCTOR_GPU_BENCH_LOCK=1.
"""
from __future__ import annotations

import argparse
import collections
import json
import os
import queue
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

SHAPE_TASK_SEP = "::SHAPE::"
DEFAULT_SHAPE_TOKEN = "__default__"
RESERVED_KEYS = frozenset({"_metadata", "__failures__", "__summary__"})
SAVE_EVERY = 50
HEARTBEAT_S = 30.0


# ---------------------------------------------------------------------------------------------
# Tasks
# ---------------------------------------------------------------------------------------------
def make_task_key(dir_path, label: str) -> str:
    return f"{dir_path}{SHAPE_TASK_SEP}{label}"


def split_task_key(task: str):
    """(dir, label) of a task key; (task, None) for a bare directory."""
    if SHAPE_TASK_SEP in task:
        d, label = task.rsplit(SHAPE_TASK_SEP, 1)
        return d, label
    return task, None


def result_label(label: str) -> str:
    return "default" if label == DEFAULT_SHAPE_TOKEN else label


def find_oracle_dirs(paths) -> list:
    """Canonical directories (holding both repro.py and oracle.py) under the given paths, sorted."""
    found = {}
    for p in map(Path, paths):
        if (p / "oracle.py").is_file() and (p / "repro.py").is_file():
            found[str(p.resolve())] = p
            continue
        if p.is_dir():
            for oracle in p.rglob("oracle.py"):
                if (oracle.parent / "repro.py").is_file():
                    found[str(oracle.parent.resolve())] = oracle.parent
    return [found[k] for k in sorted(found)]


def expand_shape_tasks(dirs) -> list:
    """One task per (directory, shape point); directories with the most points first, so that the
    long ones start early and the tail of the sweep is made of short ones."""
    from .inputs import load_shape_configs

    per_dir = []
    for d in dirs:
        try:
            configs = load_shape_configs(Path(d) / "repro.py")
        except Exception:
            configs = None
        labels = list(configs) if configs else [DEFAULT_SHAPE_TOKEN]
        per_dir.append((d, labels))
    per_dir.sort(key=lambda item: -len(item[1]))
    return [make_task_key(d, label) for d, labels in per_dir for label in labels]


def compute_worker_count(*, num_tasks: int, num_gpus: int, max_workers=None, workers_per_gpu=None):
    """(workers, workers per GPU). Default: up to 4 workers per GPU, bounded by host cores per GPU;
    never more workers than tasks."""
    if num_gpus <= 0:
        raise ValueError("No matching GPUs found")
    if max_workers is not None and max_workers < 1:
        raise ValueError("--max-workers must be >= 1")
    if workers_per_gpu is not None and workers_per_gpu < 1:
        raise ValueError("--workers-per-gpu must be >= 1")
    if num_tasks <= 0:
        return 0, workers_per_gpu or 1
    if workers_per_gpu is None:
        if max_workers is None:
            try:
                cores = len(os.sched_getaffinity(0))
            except AttributeError:
                cores = os.cpu_count() or num_gpus
            workers_per_gpu = max(1, min(4, cores // num_gpus))
        else:
            workers_per_gpu = max(1, -(-max_workers // num_gpus))
    capacity = num_gpus * workers_per_gpu
    wanted = capacity if max_workers is None else max_workers
    return min(wanted, capacity, num_tasks), workers_per_gpu


# ---------------------------------------------------------------------------------------------
# Worker process (child side)
# ---------------------------------------------------------------------------------------------
def bench_point(canonical_dir: str, label: str, *, warmup: int, rep: int, skip_check: bool,
                compile_reference: bool, peak_gbps, dtype_tolerance: bool = False, rounds: int = 5,
                fixed_rep: bool = False) -> dict:
    """Check, then time, ONE shape point of one canonical directory. Returns {label: point}."""
    from . import harness
    from .byte_model import count_bytes_effective
    from .inputs import load_shape_configs, make_inputs_from_config

    _, fn, d = harness._load_oracle_module(canonical_dir)
    repro_id = d.name
    configs = load_shape_configs(d / "repro.py")
    default = label == DEFAULT_SHAPE_TOKEN or not configs
    if not default and label not in configs:
        return {label: {"repro_id": f"{repro_id}_{label}", "status": "NO_ORACLE_FOR_SHAPE"}}
    out_label = "default" if default else label
    point_id = repro_id if default else f"{repro_id}_{label}"
    if not skip_check:
        # dtype_tolerance: this backend's per-dtype acceptance (fp32 1.3e-6 / 1e-5, 16-bit 1.6e-2 / 1e-2)
        # instead of the reference's blanket 1e-2. Outputs that draw random numbers are skipped by the
        # check either way; those regions are verified by the Philox restatement in the test-suite.
        tol = dict(atol=None, rtol=None) if dtype_tolerance else {}
        verdicts = harness.check_oracle_all_shapes(fn, d, repro_id, skip_stochastic=True,
                                                   point=None if default else label, device="cuda", **tol)
        if not all(v not in ("fail", False) for v in verdicts.values()):
            return {out_label: {"repro_id": point_id, "status": "UNVERIFIED_NUMERICS"}}
    inputs = harness.get_inputs(d) if default else make_inputs_from_config(configs[label], "cuda")
    instance = harness.get_repro_instance(d)
    region_bytes = None
    try:
        region_bytes = count_bytes_effective(instance, inputs)
    except Exception:
        pass  # the byte count is an annotation; the timing stands without it
    return {out_label: harness.bench_oracle(fn, instance, inputs, point_id, warmup=warmup, rep=rep,
                                            numerics_optout=harness.load_numerics_optout(d),
                                            compile_reference=compile_reference, rounds=rounds,
                                            adaptive_rep=not fixed_rep,
                                            region_bytes=region_bytes, peak_gbps=peak_gbps)}


def bench_dir(canonical_dir: str, **kw) -> dict:
    """All points of a directory (a bare directory task)."""
    from .inputs import load_shape_configs

    configs = load_shape_configs(Path(canonical_dir) / "repro.py")
    results = {}
    for label in (list(configs) if configs else [DEFAULT_SHAPE_TOKEN]):
        results.update(bench_point(canonical_dir, label, **kw))
    return results


def worker_main(args) -> int:
    """Serve tasks from stdin until EXIT / end of input. Only result lines reach the parent's
    pipe: file descriptor 1 is pointed at stderr and results go to a private duplicate."""
    result_pipe = os.fdopen(os.dup(1), "w", buffering=1)
    os.dup2(2, 1)
    sys.stdout = sys.stderr
    kw = dict(warmup=args.warmup, rep=args.rep, skip_check=args.skip_check,
              compile_reference=args.compile_reference, peak_gbps=args.peak_gbps,
              dtype_tolerance=args.dtype_tolerance, rounds=args.rounds, fixed_rep=args.fixed_rep)

    def send(text: str) -> None:
        result_pipe.write(text + "\n")
        result_pipe.flush()

    for raw in sys.stdin:
        task = raw.strip()
        if not task or task == "EXIT":
            break
        if task.startswith("PREFETCH:"):
            continue  # loading a module is cheap next to timing it: nothing to overlap
        try:
            d, label = split_task_key(task)
            results = bench_point(d, label, **kw) if label is not None else bench_dir(d, **kw)
            results["_repro"] = task
            send(json.dumps(results, default=str))
        except Exception as e:  # noqa: BLE001 - every failure must become a line for the parent
            text = str(e)
            if "CUDA" in text or "device-side assert" in text:
                # the context is not to be trusted any more: say so and leave; the parent respawns
                send(f"CUDA_ERROR: {text[:1000]}")
                return 1
            send(json.dumps({"_repro": task, "__error__": {
                "status": "failed", "category": "runtime_error", "exception_type": type(e).__name__,
                "error": text[:1000], "reason": "oracle worker failed while benchmarking dir/point",
                "hint": "Run `python -m better_benchmark_b200.harness <dir> --bench` directly."}}))
    return 0


# ---------------------------------------------------------------------------------------------
# Worker process (parent side)
# ---------------------------------------------------------------------------------------------
class WorkerGone(RuntimeError):
    """The worker closed its result pipe."""


class WorkerChannel:
    """One persistent worker subprocess and its three pipes.

    A reader thread moves result lines into a queue, so that the parent can wait for an answer
    with a time limit; another keeps the last lines of stderr for error reports."""

    def __init__(self, command, env, cwd):
        self.proc = subprocess.Popen(command, stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                                     stderr=subprocess.PIPE, text=True, bufsize=1, env=env, cwd=cwd)
        self._lines: queue.Queue = queue.Queue()
        self._stderr_tail = collections.deque(maxlen=20)
        threading.Thread(target=self._pump_stdout, daemon=True).start()
        threading.Thread(target=self._pump_stderr, daemon=True).start()

    def _pump_stdout(self):
        try:
            for line in self.proc.stdout:
                self._lines.put(line)
        except ValueError:
            pass  # pipe closed under us by close()
        self._lines.put(None)

    def _pump_stderr(self):
        try:
            for line in self.proc.stderr:
                line = line.rstrip()
                if line:
                    self._stderr_tail.append(line)
        except ValueError:
            pass

    def alive(self) -> bool:
        return self.proc.poll() is None

    def send(self, line: str) -> None:
        self.proc.stdin.write(line + "\n")
        self.proc.stdin.flush()

    def read_line(self, timeout):
        """Next result line; raises queue.Empty on timeout, WorkerGone at end of stream."""
        line = self._lines.get(timeout=timeout)
        if line is None:
            raise WorkerGone(f"worker exited without a result (returncode={self.proc.poll()})")
        return line.strip()

    def stderr_summary(self) -> str:
        lines = list(self._stderr_tail)[-3:]
        return ("stderr: " + " | ".join(lines))[:300] if lines else ""

    def close(self) -> None:
        """Ask the worker to leave, then terminate, then kill: this process only, by its PID."""
        p = self.proc
        if p.poll() is None:
            try:
                self.send("EXIT")
            except Exception:
                pass
            for action, wait_s in ((None, 2), (p.terminate, 5), (p.kill, 5)):
                if action is not None:
                    action()
                try:
                    p.wait(timeout=wait_s)
                    break
                except subprocess.TimeoutExpired:
                    continue
        for stream in (p.stdin, p.stdout, p.stderr):
            try:
                if stream is not None:
                    stream.close()
            except Exception:
                pass


def default_worker_command(options: dict) -> list:
    cmd = [sys.executable, "-u", "-m", "better_benchmark_b200.sweep", "--worker",
           "--warmup", str(options.get("warmup", 25)), "--rep", str(options.get("rep", 200))]
    if options.get("skip_check"):
        cmd.append("--skip-check")
    if options.get("compile_reference"):
        cmd.append("--compile-reference")
    if options.get("peak_gbps"):
        cmd += ["--peak-gbps", str(options["peak_gbps"])]
    if options.get("dtype_tolerance"):
        cmd.append("--dtype-tolerance")
    if options.get("fixed_rep"):
        cmd.append("--fixed-rep")
    cmd += ["--rounds", str(options.get("rounds", 5))]
    return cmd


def _worker_env(gpu_index: str) -> dict:
    env = os.environ.copy()
    env["CUDA_VISIBLE_DEVICES"] = str(gpu_index)
    env["INDUCTOR_GPU_BENCH_LOCK"] = "1"  # timing windows of co-located workers must not overlap
    repo_root = str(Path(__file__).resolve().parent.parent)
    env["PYTHONPATH"] = repo_root + (os.pathsep + env["PYTHONPATH"] if env.get("PYTHONPATH") else "")
    return env


def _failure(task, gpu, elapsed, error, **extra) -> dict:
    return {"repro": task, "gpu": gpu, "status": "failed", "elapsed": elapsed, "error": error[:1000], **extra}


def serve_gpu(gpu_index: str, tasks: "queue.Queue", results: "queue.Queue", options: dict) -> None:
    """Body of one parent-side thread: owns one worker process on ``gpu_index``, feeds it tasks from
    the shared queue, validates each answer and respawns the worker after any sign of trouble."""
    command_factory = options.get("worker_command_factory") or default_worker_command
    timeout = options.get("task_timeout")
    cwd = options.get("root") or os.getcwd()
    channel = None
    pending = []

    def top_up(limit, leave_for_peers=0):
        while len(pending) < limit:
            if leave_for_peers and tasks.qsize() <= leave_for_peers:
                return
            try:
                pending.append(tasks.get_nowait())
            except queue.Empty:
                return

    def drop_worker():
        nonlocal channel
        if channel is not None:
            channel.close()
            channel = None

    peers = max(0, int(options.get("n_workers", 1)) - 1)
    while True:
        if not pending:
            top_up(1)
            if not pending:
                break
        task = pending.pop(0)
        top_up(2, leave_for_peers=peers)  # at most one task held back as the prefetch hint
        if channel is None or not channel.alive():
            drop_worker()
            channel = WorkerChannel(command_factory(options), _worker_env(gpu_index), cwd)
        start = time.time()
        try:
            if pending:
                channel.send(f"PREFETCH:{pending[0]}")
            channel.send(str(task))
            try:
                line = channel.read_line(timeout)
            except queue.Empty:
                err = f"no answer within {timeout} s; worker killed"
                drop_worker()
                results.put(_failure(task, gpu_index, time.time() - start, err, category="timeout"))
                continue
            except WorkerGone as gone:
                err = "; ".join(x for x in (str(gone), channel.stderr_summary()) if x)
                drop_worker()
                results.put(_failure(task, gpu_index, time.time() - start, err))
                continue
            elapsed = time.time() - start
            if line.startswith("{"):
                payload = json.loads(line)
                echoed = payload.pop("_repro", None)
                if echoed is not None and echoed != str(task):
                    # an answer to another question: the pipe is out of step, start over
                    drop_worker()
                    results.put(_failure(task, gpu_index, elapsed,
                                         f"result misalignment: expected '{task}' but worker returned "
                                         f"result for '{echoed}'. Killed worker to reset stdout pipe."))
                    continue
                err = payload.pop("__error__", None)
                if err is not None:
                    results.put(_failure(task, gpu_index, elapsed, str(err.get("error", "")),
                                         category=err.get("category", "runtime_error"),
                                         reason=err.get("reason"), hint=err.get("hint"),
                                         exception_type=err.get("exception_type")))
                    continue
                results.put({"repro": str(task), "gpu": gpu_index, "status": "ok", "elapsed": elapsed,
                             "results": payload})
                continue
            text = "; ".join(x for x in (line[:200], channel.stderr_summary()) if x)
            if "CUDA_ERROR" in line:
                drop_worker()  # it is exiting anyway; the next task gets a fresh context
            results.put(_failure(task, gpu_index, elapsed, text))
        except Exception as e:  # noqa: BLE001 - a broken pipe, bad JSON: report, respawn, go on
            drop_worker()
            results.put(_failure(task, gpu_index, time.time() - start, str(e),
                                 category="worker_parent_error", exception_type=type(e).__name__))
    drop_worker()


# ---------------------------------------------------------------------------------------------
# Aggregation
# ---------------------------------------------------------------------------------------------
def oracle_dir_name(task: str) -> str:
    return Path(split_task_key(str(task))[0]).name


def _usable(point: dict, excluded) -> bool:
    return point.get("status") not in excluded and isinstance(point.get("oracle_us"), (int, float))


def _better_point(new: dict, old: dict, excluded) -> bool:
    """For two labels that share a shape hash: a usable point beats an unusable one, the faster of
    two usable ones wins, and among unusable ones a point with a number beats one without."""
    nu, ou = _usable(new, excluded), _usable(old, excluded)
    if nu != ou:
        return nu
    if nu:
        return new["oracle_us"] < old["oracle_us"]
    return isinstance(new.get("oracle_us"), (int, float)) and not isinstance(old.get("oracle_us"), (int, float))


_POINT_FIELDS = ("oracle_us", "compile_us", "ratio", "status")
_EXTRA_FIELDS = ("region_bytes", "oracle_gbps", "sol_frac")


def aggregate_oracle_timings(all_results: dict) -> dict:
    """{task or dir -> {label -> point}}  ->  {dir name -> entry} in the timings-file schema:

    entry = {oracle_us (median of the usable points), n_points, points{label -> ...},
             points_by_shape{shape hash -> ... + fallback}, [compile_us]}; a directory without a usable
    point goes to ``__failures__`` with a reason (no_points / all_bad_oracle / no_valid_point).
    A point is usable when its status is neither invalid nor BAD_ORACLE and it has a time."""
    from .harness import _INVALID_STATUSES

    excluded = _INVALID_STATUSES | {"BAD_ORACLE"}
    by_dir: dict = {}
    for task, results in all_results.items():
        bucket = by_dir.setdefault(oracle_dir_name(task), {})
        if isinstance(results, dict):
            bucket.update({label: p for label, p in results.items() if isinstance(p, dict)})

    out, failures = {}, {}
    for name, labelled in by_dir.items():
        points, by_shape, usable_us, usable_compile = {}, {}, [], []
        bad = 0
        for label, p in labelled.items():
            slim = {k: p.get(k) for k in _POINT_FIELDS}
            slim.update({k: p[k] for k in _EXTRA_FIELDS if k in p})
            points[label] = slim
            dispatch = p.get("dispatch")
            shaped = dict(slim, fallback=dispatch.get("fallback") if isinstance(dispatch, dict) else None)
            shape_hash = label.rsplit("_", 1)[-1]
            if shape_hash not in by_shape or _better_point(shaped, by_shape[shape_hash], excluded):
                by_shape[shape_hash] = shaped
            bad += p.get("status") == "BAD_ORACLE"
            if _usable(p, excluded):
                usable_us.append(p["oracle_us"])
                if isinstance(p.get("compile_us"), (int, float)):
                    usable_compile.append(p["compile_us"])
        if not usable_us:
            reason = "no_points" if not labelled else ("all_bad_oracle" if bad == len(labelled) else "no_valid_point")
            failures[name] = {"reason": reason, "n_points": len(labelled), "n_bad_oracle": bad, "points": points}
            continue
        entry = {"oracle_us": round(statistics.median(usable_us), 2), "n_points": len(usable_us),
                 "points": points, "points_by_shape": by_shape}
        if usable_compile:
            entry["compile_us"] = round(statistics.median(usable_compile), 2)
        out[name] = entry
    if failures:
        out["__failures__"] = failures
    return out


def regroup_task_failures(failures: dict) -> dict:
    """{task key -> failure record} -> {dir name -> {n_failed_shapes, failed_shapes, example_error}}."""
    grouped: dict = {}
    for task, record in failures.items():
        d, label = split_task_key(str(task))
        entry = grouped.setdefault(Path(d).name, {"n_failed_shapes": 0, "failed_shapes": [], "example_error": None})
        entry["n_failed_shapes"] += 1
        entry["failed_shapes"].append(result_label(label) if label is not None else "default")
        if entry["example_error"] is None:
            entry["example_error"] = (record or {}).get("error")
    return grouped


def atomic_write_json(path, payload) -> None:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    fd, tmp = tempfile.mkstemp(prefix=path.name + ".", suffix=".tmp", dir=str(path.parent))
    try:
        with os.fdopen(fd, "w") as f:
            json.dump(payload, f, indent=2, default=str)
        os.replace(tmp, path)
    except BaseException:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise


def write_oracle_timings(output_path, all_results: dict, failures=None, metadata=None) -> dict:
    """Aggregate and write the timings file. Tasks that failed in the worker are accounted per
    directory: as a ``shape_failures`` note on a directory that still has a usable point, else
    under ``__failures__`` (reason all_shapes_failed, or folded into the aggregator's record)."""
    timed = aggregate_oracle_timings(all_results)
    if failures:
        agg = timed.setdefault("__failures__", {})
        for name, note in regroup_task_failures(failures).items():
            if name in timed and name not in RESERVED_KEYS:
                timed[name]["shape_failures"] = note
            elif name in agg:
                agg[name].setdefault("shape_failures", note)
            else:
                agg[name] = {"reason": "all_shapes_failed", **note}
        if not agg:
            timed.pop("__failures__", None)
    if metadata:
        timed = {"_metadata": metadata, **timed}
    atomic_write_json(output_path, timed)
    return timed


# ---------------------------------------------------------------------------------------------
# Driver
# ---------------------------------------------------------------------------------------------
def run_sweep(tasks, gpus, *, options=None, output=None, log=print) -> tuple:
    """Run every task on the given GPUs. Returns (all_results {task -> {label -> point}},
    failures {task -> record}, summary). ``options``: warmup, rep, skip_check, compile_reference,
    peak_gbps, task_timeout, workers_per_gpu, max_workers, root, worker_command_factory."""
    options = dict(options or {})
    gpus = [str(g) for g in gpus]
    n_workers, per_gpu = compute_worker_count(num_tasks=len(tasks), num_gpus=len(gpus),
                                              max_workers=options.get("max_workers"),
                                              workers_per_gpu=options.get("workers_per_gpu"))
    options["n_workers"] = n_workers
    task_q: queue.Queue = queue.Queue()
    for t in tasks:
        task_q.put(t)
    result_q: queue.Queue = queue.Queue()
    threads = []
    for w in range(n_workers):
        th = threading.Thread(target=serve_gpu, args=(gpus[w % len(gpus)], task_q, result_q, options),
                              name=f"sweep-worker-{w}", daemon=True)
        th.start()
        threads.append(th)

    all_results, failures = {}, {}
    started = last_beat = time.time()
    done = 0
    while done < len(tasks):
        try:
            r = result_q.get(timeout=1.0)
        except queue.Empty:
            if not any(t.is_alive() for t in threads) and result_q.empty():
                break  # every worker thread is gone: whatever is missing will never come
            if time.time() - last_beat > HEARTBEAT_S:
                last_beat = time.time()
                log(f"[sweep] {done}/{len(tasks)} done, {len(failures)} failed, {last_beat - started:.0f} s")
            continue
        done += 1
        if r["status"] == "ok":
            all_results[r["repro"]] = r["results"]
        else:
            failures[r["repro"]] = {k: v for k, v in r.items() if k not in ("repro", "status")}
            log(f"[sweep] FAILED {r['repro']} on gpu {r['gpu']}: {r['error'][:200]}")
        if output and done % SAVE_EVERY == 0:
            write_oracle_timings(output, all_results, failures)
    for th in threads:
        th.join(timeout=30)
    for t in tasks:  # a task nobody reported (its thread died) is a failure, not a silence
        if t not in all_results and t not in failures:
            failures[t] = {"error": "no result was reported for this task", "category": "lost"}
    summary = {"n_tasks": len(tasks), "n_ok": len(all_results), "n_failed": len(failures), "n_workers": n_workers,
               "workers_per_gpu": per_gpu, "gpus": gpus, "wall_s": round(time.time() - started, 2)}
    return all_results, failures, summary


def sweep_metadata(summary: dict) -> dict:
    meta = {"tool": "better_benchmark_b200.sweep", "summary": summary,
            "started_utc": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())}
    try:
        import torch
        meta["torch"] = torch.__version__
        if torch.cuda.is_available():
            meta["gpu"] = torch.cuda.get_device_name(0)
    except Exception:
        pass
    return meta


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m better_benchmark_b200.sweep",
                                 description="check + time every shape point of the canonical directories under PATHS")
    ap.add_argument("paths", nargs="*")
    ap.add_argument("--gpus", default="0", help="comma-separated GPU indices")
    ap.add_argument("--output", default=None)
    ap.add_argument("--warmup", type=int, default=25)
    ap.add_argument("--rep", type=int, default=200)
    ap.add_argument("--skip-check", action="store_true")
    ap.add_argument("--compile-reference", action="store_true",
                    help="also time torch.compile of the eager module (adds compile_us and ratio)")
    ap.add_argument("--peak-gbps", type=float, default=None, help="HBM peak for the sol_frac column")
    ap.add_argument("--rounds", type=int, default=5, help="interleaved timing rounds per point (min over them)")
    ap.add_argument("--fixed-rep", action="store_true",
                    help="keep --rep as given instead of lengthening the window of fast kernels (quick sweeps)")
    ap.add_argument("--dtype-tolerance", action="store_true",
                    help="check with this backend's per-dtype tolerances instead of the reference's 1e-2")
    ap.add_argument("--task-timeout", type=float, default=600.0)
    ap.add_argument("--workers-per-gpu", type=int, default=None)
    ap.add_argument("--max-workers", type=int, default=None)
    ap.add_argument("--worker", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args(argv)
    if args.worker:
        return worker_main(args)
    dirs = find_oracle_dirs(args.paths)
    if not dirs:
        print("no canonical directory with repro.py and oracle.py found", file=sys.stderr)
        return 2
    tasks = expand_shape_tasks(dirs)
    options = dict(warmup=args.warmup, rep=args.rep, skip_check=args.skip_check,
                   compile_reference=args.compile_reference, peak_gbps=args.peak_gbps,
                   task_timeout=args.task_timeout, workers_per_gpu=args.workers_per_gpu,
                   max_workers=args.max_workers, dtype_tolerance=args.dtype_tolerance, rounds=args.rounds,
                   fixed_rep=args.fixed_rep)
    gpus = [g.strip() for g in args.gpus.split(",") if g.strip()]
    print(f"[sweep] {len(tasks)} points in {len(dirs)} directories on GPUs {gpus}")
    all_results, failures, summary = run_sweep(tasks, gpus, options=options, output=args.output)
    timed = write_oracle_timings(args.output, all_results, failures, sweep_metadata(summary)) if args.output \
        else aggregate_oracle_timings(all_results)
    n_dirs = sum(1 for k in timed if k not in RESERVED_KEYS)
    print(f"[sweep] {summary['n_ok']}/{summary['n_tasks']} points timed, {n_dirs} directories priced, "
          f"{summary['wall_s']} s")
    return 0 if not failures and "__failures__" not in timed else 1


if __name__ == "__main__":
    sys.exit(main())
