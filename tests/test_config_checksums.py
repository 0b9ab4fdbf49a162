"""Full-size pins of the five benchmark configurations (tests/golden/config_checksums.json, made by
tests/golden/make_config_checksums.py from the eager modules on the CPU, seed 1).

CPU: the eager ground truth still produces the stored numbers (drift between torch versions shows
up here). GPU: the kernels, on the same seeded inputs at full size, reproduce the stored samples
within the acceptance tolerance and the stored sums within a bound scaled by the absolute sum.
"""
import json
from pathlib import Path

import pytest
import torch

from conftest import TOL

DATA = json.loads((Path(__file__).resolve().parent / "golden" / "config_checksums.json").read_text())
ROOT = Path(__file__).resolve().parents[1]


def _flat_outputs(out):
    from better_benchmark_b200.harness import _normalize_outputs
    return _normalize_outputs(out)


@pytest.mark.parametrize("name", ["c1_row_mean", "c2_layer_norm_fwd", "c3_masked_softmax"])
def test_eager_ground_truth_reproduces_the_stored_checksums(name):
    from better_benchmark_b200.harness import load_repro_module
    from better_benchmark_b200.workloads import WORKLOADS
    wl = WORKLOADS[name]
    module = load_repro_module(ROOT / "oracle" / "canonical" / wl.canonical_id).Repro()
    with torch.no_grad():
        outs = _flat_outputs(module(*wl.make_inputs("cpu", 1)))
    stored = DATA["configs"][name]["fp32_graph"]
    assert len(outs) == len(stored)
    for t, ref in zip(outs, stored):
        assert list(t.shape) == ref["shape"] and str(t.dtype) == "torch." + ref["dtype"]
        flat = t.reshape(-1).double()
        got = torch.tensor([float(flat[p]) for p in ref["positions"]], dtype=torch.float64)
        want = torch.tensor(ref["values"], dtype=torch.float64)
        # same ops, same seed: identical unless the torch build reorders a CPU reduction
        assert torch.allclose(got, want, rtol=1e-5, atol=1e-6, equal_nan=True)
        assert abs(float(flat.sum()) - ref["sum"]) <= 1e-6 * max(ref["abs_sum"], 1.0)


def test_every_configuration_is_pinned_in_both_precisions():
    from better_benchmark_b200.workloads import WORKLOADS
    assert set(DATA["configs"]) == set(WORKLOADS) and DATA["seed"] == 1
    for entry in DATA["configs"].values():
        assert len(entry["fp32_graph"]) == len(entry["fp64_graph"]) > 0
        for a, b in zip(entry["fp32_graph"], entry["fp64_graph"]):
            assert a["shape"] == b["shape"] and a["positions"] == b["positions"] and len(a["values"]) == 64


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(DATA["configs"]))
def test_kernels_reproduce_the_stored_full_size_checksums(name):
    from better_benchmark_b200.workloads import WORKLOADS
    wl = WORKLOADS[name]
    outs = _flat_outputs(wl.oracle_forward(wl.make_inputs("cuda", 1)))
    torch.cuda.synchronize()
    fp32, fp64 = DATA["configs"][name]["fp32_graph"], DATA["configs"][name]["fp64_graph"]
    assert len(outs) == len(fp32)
    for k, (t, ref, anchor) in enumerate(zip(outs, fp32, fp64)):
        assert list(t.shape) == ref["shape"] and str(t.dtype) == "torch." + ref["dtype"], f"{name} output {k}"
        flat = t.reshape(-1)
        idx = torch.tensor(ref["positions"], device=flat.device)
        got = flat[idx].double().cpu()
        want = torch.tensor(ref["values"], dtype=torch.float64)
        exact = torch.tensor(anchor["values"], dtype=torch.float64)
        tol = TOL[ref["dtype"]]
        close = torch.isclose(got, want, rtol=tol["rtol"], atol=tol["atol"], equal_nan=True)
        if ref["dtype"] == "float32":
            # long fp32 sums: also fine when at least as close to the fp64 graph as eager fp32 is
            err_k, err_e = (got - exact).abs(), (want - exact).abs()
            close = close | (err_k <= 2 * err_e + 2.4e-7 * exact.abs().clamp(min=1.0))
        assert bool(close.all()), f"{name} output {k}: {got[~close][:4]} vs {want[~close][:4]}"
        total = float(flat.double().sum())
        bound = (2e-3 if ref["dtype"] != "float32" else 2e-6) * max(anchor["abs_sum"], 1.0)
        assert abs(total - anchor["sum"]) <= bound, f"{name} output {k}: sum {total} vs fp64 {anchor['sum']}"
