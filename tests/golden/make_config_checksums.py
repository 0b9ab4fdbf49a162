"""Checksums of the eager ground truth at the five benchmark configurations, full size.

    python tests/golden/make_config_checksums.py

For every configuration the seeded inputs (seed 1) go through the eager module of
oracle/canonical/<id>/repro.py on the CPU, once as they are (the fp32 graph) and once with every
floating tensor widened to fp64. Per output the file keeps shape, dtype, the fp64 sum and absolute
sum, and 64 elements at fixed positions. The numbers pin the ground truth across sessions and torch
versions (a drift shows up as a test failure here, before any kernel is blamed), and give the GPU
tests full-size values to compare the kernels with, without running the eager module there.
"""
import json
import os
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
OUT = Path(__file__).resolve().parent / "config_checksums.json"
SAMPLES = 64


def sample_positions(numel: int, salt: int):
    g = torch.Generator().manual_seed(1000 + salt)
    return torch.randint(0, max(numel, 1), (SAMPLES,), generator=g).tolist() if numel else []


def summarize(outputs):
    out = []
    for k, t in enumerate(outputs):
        flat = t.detach().reshape(-1)
        pos = sample_positions(flat.numel(), k)
        d = flat.double()
        out.append({"shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", ""),
                    "sum": float(d.sum()), "abs_sum": float(d.abs().sum()),
                    "positions": pos, "values": [float(d[p]) for p in pos]})
    return out


def run_config(name):
    from better_benchmark_b200.harness import _normalize_outputs, load_repro_module
    from better_benchmark_b200.workloads import WORKLOADS
    wl = WORKLOADS[name]
    module = load_repro_module(ROOT / "oracle" / "canonical" / wl.canonical_id).Repro()
    result = {}
    for tag, widen in (("fp32_graph", False), ("fp64_graph", True)):
        inputs = wl.make_inputs("cpu", 1)
        if widen:
            inputs = [i.double() if isinstance(i, torch.Tensor) and i.is_floating_point() else i for i in inputs]
        with torch.no_grad():
            outs = _normalize_outputs(module(*inputs))
        result[tag] = summarize(outs)
    return result


def main():
    from better_benchmark_b200.workloads import WORKLOADS
    torch.set_num_threads(max(1, (os.cpu_count() or 2) // 2))
    data = {"torch": torch.__version__, "seed": 1, "configs": {}}
    for name in WORKLOADS:
        data["configs"][name] = run_config(name)
        print(name, [(o["shape"], o["dtype"]) for o in data["configs"][name]["fp32_graph"]])
    OUT.write_text(json.dumps(data, indent=1))
    print("wrote", OUT, OUT.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
