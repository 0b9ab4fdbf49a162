#!/usr/bin/env python
"""Benchmark of the B200 oracle backend.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

A step is one pass of one fused region (by default the LayerNorm-forward configuration, the
second of the baseline's list) over one batch of seeded synthetic input that is already resident
in HBM. Inputs rotate over several buffer sets whose total footprint exceeds the L2 cache, so no
step finds its input there. The metric is achieved HBM bandwidth: the region's minimum bytes
(every input once plus every output once) divided by the time per step. One JSON line is printed
by rank 0.

  value      K timed steps (captured into one CUDA graph) between CUDA events on the launching
             stream, barrier + synchronize on both sides. The graph is replayed several times, each
             replay timed by its own event pair; value is the MEDIAN replay (min and max are
             reported beside it). Outputs of the last steps stay alive during the capture, so the
             output blocks rotate over more than 4x the L2 as the inputs do and every step's
             results really go to DRAM. With N > 1 every rank runs the same configuration on its
             own GPU (independent replicas, no collective in the data path) and the time is the
             maximum over ranks, so value is the aggregate over the N GPUs.
  roofline   the dominant (here: only) kernel of the step against the measured HBM peak; its
             ``per_config`` map holds all five configurations: back-to-back microseconds and
             fraction (``us``, ``frac``) and one replay from a flushed L2 as the reference's
             ``bench_oracle`` times it (``cold_us``, ``cold_frac``).
  e2e        the same metric through the public entry point with HOST buffers: every step copies
             the inputs from pinned host memory, runs ``oracle_forward`` and copies every output
             back to pinned host memory. Upload, kernel and download of neighbouring steps overlap
             (three streams, two buffer sets); every step's copies are inside the timed region.
  cpu_baseline  the eager module of the same region on the host cores (rank 0, N = 1).
  families   one case per kernel family outside the five configurations (``family_cases.py``).

``--sweep`` runs the corpus sweep (persistent worker processes, tasks sharded over the first N
visible GPUs) on the five configuration directories and reports its wall time instead.

``--impl reference`` times only the eager module on the host cores (the reference's own CPU
path for this region) and prints the same metric with ``"impl": "reference"``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0  # used only when MEASURED_PEAKS.json is absent
L2_BYTES_ASSUMED = 126 * 1024 * 1024


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (6.65 TB/s, no MEASURED_PEAKS.json)"


def recorded_traffic(workload):
    """The committed ncu capture of this workload's kernel (one launch from a flushed L2):
    {"traffic": read + write DRAM bytes, "traffic_read", "traffic_write", "input_bytes",
    "output_bytes"}, or {} without a capture. A capture ends with the kernel, when part of the
    output is still dirty in L2, so only the read side can be compared with the algorithmic bytes
    (traffic_read against input_bytes); the write side is bounded below by what was seen."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            rec = json.load(f).get(workload, {})
    except Exception:
        return {}
    if not rec:
        return {}
    out = {"traffic": rec.get("dram_bytes_per_launch"), "traffic_read": rec.get("dram_read_bytes"),
           "traffic_write": rec.get("dram_write_bytes")}
    if rec.get("input_bytes") is not None:
        out["input_bytes"] = rec["input_bytes"]
        out["output_bytes"] = rec.get("output_bytes")
        if rec.get("dram_read_bytes"):
            out["read_over_input"] = round(rec["dram_read_bytes"] / rec["input_bytes"], 3)
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu_index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._drain, daemon=True)
        self.thread.start()

    def _drain(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def dist_env():
    from better_benchmark_b200.replicas import dist_env as env
    return env()


# ---------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the eager module on the host cores
# ---------------------------------------------------------------------------------------------
def time_eager_cpu(workload, steps, warmup, budget_s=None):
    """Seconds per call of the eager module (oracle/canonical/<id>/repro.py) on the CPU."""
    import torch
    from better_benchmark_b200.harness import load_repro_module
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(cores)
    module = load_repro_module(os.path.join(ROOT, "oracle", "canonical", workload.canonical_id))
    instance = module.Repro()
    inputs = workload.make_inputs("cpu", 1)

    def run():
        args = [i.clone() if (workload.mutates_inputs and isinstance(i, torch.Tensor)) else i for i in inputs]
        with torch.no_grad():
            return instance(*args)

    for _ in range(max(1, warmup)):
        run()
    times = []
    t_start = time.perf_counter()
    for _ in range(max(1, steps)):
        t0 = time.perf_counter()
        run()
        times.append(time.perf_counter() - t0)
        if budget_s is not None and time.perf_counter() - t_start > budget_s:
            break
    return sum(times) / len(times), min(times), len(times), cores


def reference_arm(args, workload):
    rank, _, world = dist_env()
    if rank != 0:
        return 0
    mean_s, best_s, done, cores = time_eager_cpu(workload, args.steps, max(1, min(args.warmup, 3)), budget_s=150)
    gbps = workload.algorithmic_bytes / mean_s / 1e9
    line = {
        "impl": "reference", "metric": "achieved_hbm_gbps", "value": round(gbps, 3), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": done, "warmup": args.warmup, "ms_per_step": round(mean_s * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": workload.dtype,
        "data": "synthetic",
        "config": {"workload": workload.name, "description": workload.description,
                   "device": "host CPU", "threads": cores},
        "cpu_baseline": {"value": round(gbps, 3), "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"full {workload.name} workload per step, eager aten graph of the region, {done} steps"},
        "e2e": {"value": round(gbps, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def build_input_sets(workload, device, min_total_bytes):
    """Enough seeded input sets that their tensors together exceed ``min_total_bytes``."""
    import torch
    first = workload.make_inputs(device, 1)
    per_set = sum(t.numel() * t.element_size() for t in first if isinstance(t, torch.Tensor))
    count = max(2, int(min_total_bytes // max(per_set, 1)) + 1)
    sets = [first]
    for s in range(1, count):
        sets.append(workload.make_inputs(device, 1 + s))
    return sets, per_set


REPLAYS = 21  # timed replays of the K-step graph (median reported)


def time_steps(workload, input_sets, steps, warmup, barrier, replays=REPLAYS,
               min_output_bytes=4 * L2_BYTES_ASSUMED):
    """Times `steps` steps, `replays` times. Returns {"ms": median, "ms_min", "ms_max", "replays",
    "launches": kernels this library launched per replay}.

    The K steps are captured into one CUDA graph (step i uses input set i mod n) and a timed
    region is one replay of that graph between two events: the kernels are 20-100 us long, and a
    Python loop cannot issue them fast enough to keep the GPU busy. While capturing, the outputs of
    the most recent steps are kept alive until they add up to `min_output_bytes`, so the allocator
    hands every step a block that has not been written for at least that many bytes: a step's
    results are evicted to DRAM like in real use instead of being overwritten in L2 by the next
    step. The launch count is what the library launched while the graph was being captured.
    """
    import collections

    import torch
    from better_benchmark_b200 import native
    lib = native.load()
    n = len(input_sets)
    for i in range(warmup):
        workload.oracle_forward(input_sets[i % n])
    torch.cuda.synchronize()
    input_ptrs = {t.data_ptr() for s in input_sets for t in s if isinstance(t, torch.Tensor)}
    graph = torch.cuda.CUDAGraph()
    launches0 = lib.b200_launch_count()
    with torch.cuda.graph(graph):
        window, held = collections.deque(), 0
        for i in range(steps):
            outs = workload.oracle_forward(input_sets[i % n])
            outs = [outs] if isinstance(outs, torch.Tensor) else list(outs)
            nbytes = sum(o.numel() * o.element_size() for o in outs
                         if isinstance(o, torch.Tensor) and o.data_ptr() not in input_ptrs)
            window.append((outs, nbytes))
            held += nbytes
            while len(window) > 1 and held - window[0][1] >= min_output_bytes:
                held -= window.popleft()[1]
            del outs
        window.clear()
    launches = lib.b200_launch_count() - launches0
    torch.cuda.synchronize()
    graph.replay()  # untimed: instantiates everything the first replay touches
    torch.cuda.synchronize()
    times = []
    for _ in range(max(1, replays)):
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end))
    barrier()
    check_device_waits()
    return {"ms": statistics.median(times), "ms_min": min(times), "ms_max": max(times),
            "replays": len(times), "launches": int(launches)}


def check_device_waits():
    """Raise if a bounded device-side wait ran out during what was just timed: such a kernel skips
    its remaining work, and a region that timed skipped work must not be reported."""
    from better_benchmark_b200 import kernels, native
    lib = native.load()
    kernels.check_scratch_status()
    gave_up = {name: int(getattr(lib, name)()) for name in
               ("b200_norm_fwd_wait_timeouts", "b200_norm_bwd_wait_timeouts", "b200_batch_norm_wait_timeouts")}
    if any(gave_up.values()):
        raise RuntimeError(f"device-side waits ran out during the timed region: {gave_up}")


def time_cold(workload, inputs):
    """Microseconds of ONE launch of the region from a flushed L2, graph launch included, as the
    reference's bench_oracle times it (min over its repetitions; no comparison arm, no gate)."""
    import torch
    from better_benchmark_b200 import harness
    with torch.no_grad():
        for _ in range(3):
            workload.oracle_forward(inputs)
        torch.cuda.synchronize()
    graph, _ = harness._capture_graph_checked(lambda: workload.oracle_forward(inputs))
    best = min(harness._time_graph(graph, warmup=10, rep=60) for _ in range(2))
    del graph
    return best


def time_e2e(workload, device, steps, warmup):
    """Milliseconds per step with host buffers: H2D of every input from pinned memory, the oracle,
    D2H of every output into pinned memory, every step. The three legs run on three streams with two
    sets of device buffers, so that the upload of step i+1 and the download of step i-1 overlap the
    kernel of step i (PCIe is full duplex); events order them. Returns (ms_per_step, h2d, d2h)."""
    import torch
    host_inputs = [t.pin_memory() if isinstance(t, torch.Tensor) else t for t in workload.make_inputs("cpu", 1)]
    NBUF = 2
    dev_inputs = [[torch.empty_like(t, device=device) if isinstance(t, torch.Tensor) else t for t in host_inputs]
                  for _ in range(NBUF)]
    for h, d in zip(host_inputs, dev_inputs[0]):  # channels-last and other dense layouts keep their strides
        if isinstance(h, torch.Tensor):
            assert h.stride() == d.stride()
    h2d = sum(t.numel() * t.element_size() for t in host_inputs if isinstance(t, torch.Tensor))
    host_outputs = [None] * NBUF
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    s_comp = torch.cuda.current_stream(device)
    in_ready = [torch.cuda.Event() for _ in range(NBUF)]
    comp_done = [torch.cuda.Event() for _ in range(NBUF)]
    out_done = [torch.cuda.Event() for _ in range(NBUF)]
    used = [False] * NBUF
    keep = [None] * NBUF  # the outputs of the step that used buffer set b, alive until their download ran

    def step(i):
        b = i % NBUF
        with torch.cuda.stream(s_in):
            if used[b]:
                s_in.wait_event(comp_done[b])  # the kernel of step i-2 has read this buffer set
            for h, d in zip(host_inputs, dev_inputs[b]):
                if isinstance(h, torch.Tensor):
                    d.copy_(h, non_blocking=True)
            in_ready[b].record(s_in)
        s_comp.wait_event(in_ready[b])
        if used[b]:
            # the download of step i-2 has read its outputs: only now may their memory return to the
            # allocator (which hands it out again on this stream, in stream order)
            s_comp.wait_event(out_done[b])
        keep[b] = None
        outs = workload.oracle_forward(dev_inputs[b])
        outs = [outs] if isinstance(outs, torch.Tensor) else list(outs)
        keep[b] = outs
        comp_done[b].record(s_comp)
        if host_outputs[b] is None:
            host_outputs[b] = [torch.empty_strided(o.shape, o.stride(), dtype=o.dtype).pin_memory() for o in outs]
        with torch.cuda.stream(s_out):
            s_out.wait_event(comp_done[b])
            if used[b]:
                s_out.wait_event(out_done[b])
            for o, h in zip(outs, host_outputs[b]):
                h.copy_(o, non_blocking=True)
            out_done[b].record(s_out)
        used[b] = True

    for i in range(max(2, warmup)):
        step(i)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(s_in)
    for i in range(steps):
        step(i)
    s_out.wait_stream(s_comp)
    s_out.wait_stream(s_in)
    end.record(s_out)
    torch.cuda.synchronize()
    d2h = sum(t.numel() * t.element_size() for t in host_outputs[0])
    return start.elapsed_time(end) / steps, h2d, d2h


def gpu_arm(args, workload):
    import torch
    from better_benchmark_b200.workloads import WORKLOADS
    rank, local_rank, world = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this backend has no CPU path "
                         "(use --impl reference for the host baseline)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    from better_benchmark_b200.replicas import ReplicaGroup
    group = ReplicaGroup(device=device)  # NCCL when world > 1; barrier + max-over-ranks only
    barrier = group.barrier

    peak, peak_source = measured_peak()
    sets, per_set = build_input_sets(workload, device, 4 * L2_BYTES_ASSUMED)
    n_sets = len(sets)
    sampler = ClockSampler(os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",")[local_rank]
                           if os.environ.get("CUDA_VISIBLE_DEVICES") else local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    timing = time_steps(workload, sets, args.steps, args.warmup, barrier)
    launches = timing["launches"]
    total_ms = group.max_over_ranks(timing["ms"])
    ms_per_step = total_ms / args.steps
    # keep the GPU under the same load a little longer so that the clock sampler sees it
    load_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(load_graph):
        for i in range(len(sets)):
            workload.oracle_forward(sets[i])
    t_end = time.time() + 1.0
    while time.time() < t_end:
        for _ in range(20):
            load_graph.replay()
        torch.cuda.synchronize()
    del load_graph
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["window"] = (f"sampled every 100 ms from before the {timing['replays']} timed replays to the end of "
                            "a 1 s continuation under the same load")
    gbps_one = workload.algorithmic_bytes / (ms_per_step * 1e-3) / 1e9
    value = gbps_one * world

    e2e_ms, h2d, d2h = time_e2e(workload, device, max(3, min(args.steps, 20)), 2)
    e2e_ms = group.max_over_ranks(e2e_ms)
    e2e_value = workload.algorithmic_bytes / (e2e_ms * 1e-3) / 1e9 * world

    def entry(wl, t, k):
        per = t["ms"] / k
        return {"us": round(per * 1e3, 2), "frac": round(wl.algorithmic_bytes / (per * 1e-3) / 1e9 / peak, 4),
                "us_min": round(t["ms_min"] / k * 1e3, 2), "us_max": round(t["ms_max"] / k * 1e3, 2),
                "launches": round(t["launches"] / k, 2), "bytes": wl.algorithmic_bytes}

    per_config = {}
    families = {}
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.only_headline:
        per_config[workload.name] = entry(workload, timing, args.steps)
        cold = time_cold(workload, sets[0])
        per_config[workload.name].update(cold_us=round(cold, 2),
                                         cold_frac=round(workload.algorithmic_bytes / (cold * 1e-6) / 1e9 / peak, 4))
        del sets
        torch.cuda.empty_cache()
        for name, wl in WORKLOADS.items():
            if name == workload.name:
                continue
            s, _ = build_input_sets(wl, device, 4 * L2_BYTES_ASSUMED)
            per_config[name] = entry(wl, time_steps(wl, s, args.steps, args.warmup, lambda: None), args.steps)
            cold = time_cold(wl, s[0])
            per_config[name].update(cold_us=round(cold, 2),
                                    cold_frac=round(wl.algorithmic_bytes / (cold * 1e-6) / 1e9 / peak, 4))
            del s
            torch.cuda.empty_cache()
        from better_benchmark_b200.family_cases import FAMILY_CASES
        for name, wl in FAMILY_CASES.items():
            s, _ = build_input_sets(wl, device, 4 * L2_BYTES_ASSUMED)
            k = min(args.steps, 50)
            families[name] = entry(wl, time_steps(wl, s, k, args.warmup, lambda: None, replays=7), k)
            del s
            torch.cuda.empty_cache()
        mean_s, best_s, done, cores = time_eager_cpu(workload, 20, 2, budget_s=20)
        cpu_gbps = workload.algorithmic_bytes / mean_s / 1e9
        cpu_baseline = {"value": round(cpu_gbps, 3), "unit": "GB/s", "cores": cores, "kind": "port",
                        "sample": f"full {workload.name} workload per call, eager aten graph of the region, "
                                  f"{done} calls, mean {mean_s * 1e3:.1f} ms"}
    group.close()
    if rank != 0:
        return 0
    roofline = {"bound": "hbm", "achieved": round(gbps_one, 1), "peak": peak, "unit": "GB/s",
                "frac": round(gbps_one / peak, 4), "traffic": None,
                "peak_source": peak_source, "algorithmic_bytes_per_launch": workload.algorithmic_bytes,
                "launches_per_step": launches / args.steps}
    roofline.update(recorded_traffic(workload.name))
    if per_config:
        roofline["per_config"] = per_config
    line = {
        "metric": "achieved_hbm_gbps", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 6),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": workload.dtype,
        "data": "synthetic",
        "config": {"workload": workload.name, "description": workload.description,
                   "replicas": world,
                   "l2": f"inputs rotate over {n_sets} resident buffer sets "
                         f"({per_set / 1e6:.0f} MB each) and outputs over as many bytes, each more than 4x the 126 MB L2",
                   "timing": f"median of {timing['replays']} replays of the {args.steps}-step graph"},
        "ms_per_step_min": round(timing["ms_min"] / args.steps, 6),
        "ms_per_step_max": round(timing["ms_max"] / args.steps, 6),
        "clocks": clocks,
        "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h), "ms_per_step": round(e2e_ms, 4)},
        "gpu_launches": launches,
        "roofline": roofline,
    }
    if cpu_baseline is not None:
        line["cpu_baseline"] = cpu_baseline
    if families:
        line["families"] = families
    print(json.dumps(line))
    return 0


def sweep_arm(args):
    """Aggregate wall time of the corpus sweep (check + bench of every shape point through persistent
    worker processes, sharded over the first N visible GPUs) on the five benchmark directories."""
    import shutil
    import tempfile
    from better_benchmark_b200 import sweep
    from better_benchmark_b200.workloads import WORKLOADS
    peak, _ = measured_peak()
    root = tempfile.mkdtemp(prefix="b200_sweep_")
    try:
        for wl in WORKLOADS.values():
            dest = os.path.join(root, "repros", "canonical", wl.canonical_id)
            os.makedirs(dest)
            for src in (os.path.join(ROOT, "better-benchmark_b200", "canonical", wl.canonical_id),
                        os.path.join(ROOT, "oracle", "canonical", wl.canonical_id)):  # the eager module is the checker
                for f in os.listdir(src):
                    if os.path.isfile(os.path.join(src, f)):
                        shutil.copy(os.path.join(src, f), os.path.join(dest, f))
        dirs = sweep.find_oracle_dirs([root])
        tasks = sweep.expand_shape_tasks(dirs)
        visible = [d for d in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",") if d.strip()]
        gpus = (visible or [str(i) for i in range(args.gpus)])[:args.gpus]
        out = os.path.join(root, "timings.json")
        results, failures, summary = sweep.run_sweep(
            tasks, gpus, options=dict(warmup=5, rep=50, task_timeout=900, peak_gbps=peak, workers_per_gpu=2),
            output=out, log=lambda *a: print(*a, file=sys.stderr))
        timed = sweep.write_oracle_timings(out, results, failures, sweep.sweep_metadata(summary))
        points = {k: {"oracle_us": v["oracle_us"], **{kk: vv for kk, vv in next(iter(v["points"].values())).items()
                                                       if kk in ("oracle_gbps", "sol_frac", "status")}}
                  for k, v in timed.items() if k not in sweep.RESERVED_KEYS}
        print(json.dumps({"metric": "sweep_wall_s", "value": summary["wall_s"], "unit": "s", "n_gpus": len(gpus),
                          "higher_is_better": False, "points": len(tasks), "failed": len(failures),
                          "workers": summary["n_workers"], "per_dir": points}))
        return 0 if not failures else 1
    finally:
        shutil.rmtree(root, ignore_errors=True)


def main(argv=None):
    from better_benchmark_b200.workloads import HEADLINE, WORKLOADS
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=HEADLINE, choices=sorted(WORKLOADS))
    ap.add_argument("--only-headline", action="store_true", help="skip the other configurations and the CPU baseline")
    ap.add_argument("--sweep", action="store_true",
                    help="run the corpus sweep over the five directories on --gpus GPUs and report its wall time")
    args = ap.parse_args(argv)
    if args.warmup < 3:
        args.warmup = 3
    workload = WORKLOADS[args.workload]
    if args.sweep:
        return sweep_arm(args)
    if args.impl == "reference":
        return reference_arm(args, workload)
    return gpu_arm(args, workload)


if __name__ == "__main__":
    sys.exit(main())
