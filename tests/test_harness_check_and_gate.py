"""check_oracle, output comparison, stochastic detection, the fp64-anchored numerics gate and the
reviewed opt-out (CPU). Cases follow the reference's tests/test_oracle_harness_hardening.py:242-366,
:426-671 and tests/test_canonical_invariants.py:1509-1535."""
import json

import pytest
import torch

from better_benchmark_b200 import harness


class Scale(torch.nn.Module):
    def forward(self, x, k):
        return (x * 2.0, (x > 0).to(torch.int64) * k)


def test_check_oracle_accepts_matching_and_rejects_wrong_outputs():
    x = torch.randn(16, 8)
    good = lambda inp: (inp[0] * 2.0, (inp[0] > 0).to(torch.int64) * inp[1])
    bad_value = lambda inp: (inp[0] * 2.1, (inp[0] > 0).to(torch.int64) * inp[1])
    bad_int = lambda inp: (inp[0] * 2.0, (inp[0] > 0).to(torch.int64) * inp[1] + 1)
    bad_count = lambda inp: inp[0] * 2.0
    bad_shape = lambda inp: ((inp[0] * 2.0)[:8], (inp[0] > 0).to(torch.int64) * inp[1])
    assert harness.check_oracle(good, Scale(), [x, 3]) is True
    assert harness.check_oracle(bad_value, Scale(), [x, 3]) is False
    assert harness.check_oracle(bad_int, Scale(), [x, 3]) is False
    assert harness.check_oracle(bad_count, Scale(), [x, 3]) is False
    assert harness.check_oracle(bad_shape, Scale(), [x, 3]) is False


def test_nan_in_the_same_place_counts_as_equal():
    class M(torch.nn.Module):
        def forward(self, x):
            return torch.log(x)
    x = torch.tensor([1.0, -1.0, 2.0])
    assert harness.check_oracle(lambda inp: torch.log(inp[0]), M(), [x]) is True
    assert harness.check_oracle(lambda inp: torch.nan_to_num(torch.log(inp[0])), M(), [x]) is False


def test_stochastic_outputs_are_detected_and_skipped():
    class Drop(torch.nn.Module):
        def forward(self, x):
            return (torch.nn.functional.dropout(x, 0.5, True), x + 1)
    x = torch.ones(64, 64)
    assert harness.detect_stochastic_outputs(Drop(), [x]) == {0}
    assert harness.check_oracle(lambda inp: (torch.zeros_like(inp[0]), inp[0] + 1), Drop(), [x]) is True


def test_gate_passes_identical_and_small_errors():
    ref = [torch.tensor([1.0, 2.0, 3.0], dtype=torch.float64)]
    same = [torch.tensor([1.0, 2.0, 3.0])]
    assert harness._anchored_numerics_gate(same, same, ref, set())["pass"] is True
    compiled = [torch.tensor([1.0 + 1e-7, 2.0 + 1e-7, 3.0 + 1e-7])]
    oracle = [torch.tensor([1.0 + 2e-7, 2.0 + 2e-7, 3.0 + 2e-7])]
    assert harness._anchored_numerics_gate(oracle, compiled, ref, set())["pass"] is True


def test_gate_fails_an_oracle_much_worse_than_the_comparison_arm():
    ref = [torch.tensor([1.0, 2.0], dtype=torch.float64), torch.tensor([10.0, 20.0], dtype=torch.float64)]
    compiled = [torch.tensor([1.0, 2.0]), torch.tensor([10.0, 20.0])]
    oracle = [torch.tensor([1.0, 2.0]), torch.tensor([10.5, 20.5])]
    res = harness._anchored_numerics_gate(oracle, compiled, ref, set())
    assert res["pass"] is False and res["worst_output_idx"] == 1
    assert res["per_output"][0]["pass"] is True and res["per_output"][1]["pass"] is False


def test_gate_threshold_scales_with_reference_magnitude_and_skips():
    ref = [torch.tensor([1e6, 2e6], dtype=torch.float64)]
    res = harness._anchored_numerics_gate([torch.tensor([1e6 + 5.0, 2e6 + 5.0])], [torch.tensor([1e6, 2e6])], ref, set())
    assert res["pass"] is True                                  # 5 < 1e-5 * 2e6
    res = harness._anchored_numerics_gate([torch.tensor([0.0])], [torch.tensor([1.0])], [torch.tensor([1.0])], {0})
    assert res["pass"] is True and res["per_output"][0]["skip"] == "stochastic"
    ints = [torch.tensor([1, 2])]
    assert harness._anchored_numerics_gate(ints, ints, ints, set())["per_output"][0]["skip"] == "non_float"


def test_gate_sees_a_base_two_exponential_substitution():
    x = torch.randn(1000, generator=torch.Generator().manual_seed(0)) * 3.0
    ref = [torch.exp(x.double())]
    res = harness._anchored_numerics_gate([torch.exp2(x * 1.4426950408889634)], [torch.exp(x)], ref, set())
    assert res["per_output"][0]["err_oracle"] > res["per_output"][0]["err_compiled"]


def test_optout_accepts_plausible_drift_and_refuses_large_or_nonfinite():
    failing = {"pass": False, "per_output": [{"idx": 0, "pass": False, "err_oracle": 2e-3, "ref_absmax": 4.0}]}
    optout = {"verified": True, "reason": "bf16 accumulation order"}
    assert harness.numerics_optout_applies(failing, optout)["accept"] is True
    assert harness.numerics_optout_applies(failing, None)["accept"] is False
    huge = {"pass": False, "per_output": [{"idx": 0, "pass": False, "err_oracle": 3.0, "ref_absmax": 4.0}]}
    assert harness.numerics_optout_applies(huge, optout)["accept"] is False
    nan = {"pass": False, "per_output": [{"idx": 0, "pass": False, "err_oracle": float("nan"), "ref_absmax": 4.0}]}
    assert harness.numerics_optout_applies(nan, optout)["accept"] is False
    assert harness.numerics_optout_applies(None, optout)["accept"] is False


def test_optout_annotation_loading(tmp_path):
    assert harness.load_numerics_optout(tmp_path) is None
    (tmp_path / "meta.json").write_text(json.dumps({"numerics_optout": {"verified": True, "reason": " "}}))
    assert harness.load_numerics_optout(tmp_path) is None          # empty reason: refused
    (tmp_path / "meta.json").write_text(json.dumps({"numerics_optout": {"verified": True, "reason": "reviewed"}}))
    assert harness.load_numerics_optout(tmp_path)["reason"] == "reviewed"
    (tmp_path / "meta.json").write_text("{not json")
    assert harness.load_numerics_optout(tmp_path) is None


def test_cuda_graph_warning_pattern():
    pat = harness._CUDAGRAPH_WARNING
    assert pat.search("CUDAGraph capture is slow") and pat.search("during stream capture") and pat.search("cuda graph")
    assert not pat.search("UserWarning: something unrelated about tensors")


def test_check_all_shapes_uses_separate_input_copies_on_cpu(tmp_path):
    """A repro that mutates its inputs: eager and oracle each get their own seeded copy."""
    from conftest import assemble_canonical_dir
    from better_benchmark_b200.workloads import WORKLOADS
    wl = WORKLOADS["c4_batch_norm_relu"]
    d = assemble_canonical_dir(wl.canonical_id, tmp_path)
    # shrink the point so that the eager module runs in milliseconds
    data = json.loads((d / "shapes.json").read_text())
    data["points"][0]["inputs"][0] = [[4, 64, 6, 6], "bf16", {"st": [2304, 1, 384, 64]}]
    (d / "shapes.json").write_text(json.dumps(data))
    instance_mod = harness.load_repro_module(d)

    def cpu_oracle(inputs):           # stands in for the CUDA oracle on a CPU-only machine
        return instance_mod.Repro()(*inputs)
    results = harness.check_oracle_all_shapes(cpu_oracle, d, d.name, device="cpu")
    assert list(results.values()) == [True]


def test_bench_oracle_refuses_cpu_inputs():
    with pytest.raises(RuntimeError):
        harness.bench_oracle(lambda inp: inp[0], torch.nn.Identity(), [torch.zeros(4)], "x")
