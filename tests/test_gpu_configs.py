"""GPU parity at the five benchmark configurations, full size, through the drop-in boundary.

Each configuration is assembled as a canonical repro directory (repro.py + shapes.json +
oracle.py), loaded the way the harness loads one, and checked three ways:
  * ``check_oracle_all_shapes`` - the reference's own procedure: eager module on the GPU vs the
    oracle on separately seeded randn inputs of the shapes.json point;
  * the configuration's own seeded inputs (value distributions of the benchmark) against the
    eager module on the CPU, at the acceptance tolerance of each output's dtype;
  * output strides, dtypes, aliasing and size-independent properties (softmax rows sum to one,
    the permuted dx equals the plain dx, repeated launches are bit-identical).
"""
import pytest
import torch

from conftest import assemble_canonical_dir, assert_close, assert_sum_close

pytestmark = pytest.mark.gpu


def _load(tmp_path, name):
    from better_benchmark_b200 import harness
    from better_benchmark_b200.workloads import WORKLOADS
    wl = WORKLOADS[name]
    d = assemble_canonical_dir(wl.canonical_id, tmp_path)
    harness.reset_oracle_registry()
    harness.get_gpu_kind._cached = "B200"
    _, fn, d = harness._load_oracle_module(d)
    return wl, d, fn, harness


CONFIGS = ["c1_row_mean", "c2_layer_norm_fwd", "c3_masked_softmax", "c4_batch_norm_relu", "c5_rms_norm_bwd"]


@pytest.mark.parametrize("name", CONFIGS)
def test_config_passes_the_harness_check(tmp_path, name):
    wl, d, fn, harness = _load(tmp_path, name)
    results = harness.check_oracle_all_shapes(fn, d, d.name, atol=1e-2, rtol=1.6e-2)
    assert results and all(results.values()), results
    reg = harness.get_module_registry(fn.__module__)
    assert reg.last_dispatch_info["matched"] == "hardware+shape"


@pytest.mark.parametrize("name", CONFIGS)
def test_config_matches_cpu_eager_on_seeded_inputs(tmp_path, name):
    wl, d, fn, harness = _load(tmp_path, name)
    instance = harness.get_repro_instance(d)
    cpu_inputs = wl.make_inputs("cpu", 1)
    gpu_inputs = wl.make_inputs("cuda", 1)
    with torch.no_grad():
        want = harness._normalize_outputs(instance(*cpu_inputs))
    selected, info = harness.resolve_oracle(fn, gpu_inputs)
    got = harness._normalize_outputs(selected(gpu_inputs))
    assert len(got) == len(want)
    for i, (g, w) in enumerate(zip(got, want)):
        assert g.stride() == w.stride(), f"{name} output {i}: stride {g.stride()} vs eager {w.stride()}"
        if name == "c5_rms_norm_bwd" and i == 1:
            # dweight: an fp32 sum over 16384 rows (see conftest.assert_sum_close)
            import copy
            with torch.no_grad():
                anchor = harness._normalize_outputs(copy.deepcopy(instance).double()(
                    *[t.double() if t.is_floating_point() else t for t in wl.make_inputs("cpu", 1)]))
            assert_sum_close(g, w, anchor[i], f"{name} output {i}")
        else:
            assert_close(g, w, f"{name} output {i}")
    if wl.mutates_inputs:  # running statistics are updated in place and returned as the same tensors
        assert got[3].data_ptr() == gpu_inputs[1].data_ptr() and got[4].data_ptr() == gpu_inputs[2].data_ptr()
        assert_close(gpu_inputs[1], cpu_inputs[1], "running_mean in place")
        assert_close(gpu_inputs[2], cpu_inputs[2], "running_var in place")


def test_softmax_rows_sum_to_one_and_masked_keys_vanish():
    from better_benchmark_b200.workloads import WORKLOADS
    wl = WORKLOADS["c3_masked_softmax"]
    scores, mask = wl.make_inputs("cuda", 3)
    out = wl.oracle_forward([scores, mask]).float()
    sums = out.sum(-1)
    assert torch.allclose(sums, torch.ones_like(sums), atol=2e-3)
    masked = (mask.float() < -1).expand_as(out)
    assert out[masked].abs().max().item() == 0.0


def test_head_major_dx_is_a_permutation_of_plain_dx():
    import better_benchmark_b200.kernels as k
    from better_benchmark_b200.workloads import WORKLOADS
    x, dy, w, rstd = WORKLOADS["c5_rms_norm_bwd"].make_inputs("cuda", 2)
    b, s, h, d = x.shape
    dx_perm, dw_perm, _ = k.norm_bwd(x, dy, w, rstd, rms=True, heads=h)
    dx_plain, dw_plain, _ = k.norm_bwd(x.view(b * s, h * d), dy.view(b * s, h * d), w, rstd, rms=True)
    assert torch.equal(dx_perm, dx_plain.view(b, s, h, d).permute(0, 2, 1, 3).contiguous())
    assert torch.equal(dw_perm, dw_plain)
    k.check_scratch_status()


@pytest.mark.parametrize("name", CONFIGS)
def test_config_is_bit_reproducible_and_graph_capturable(name):
    from better_benchmark_b200 import harness
    from better_benchmark_b200.workloads import WORKLOADS
    wl = WORKLOADS[name]
    inputs = wl.make_inputs("cuda", 5)
    first = [o.clone() for o in harness._normalize_outputs(wl.oracle_forward(inputs))]
    if wl.mutates_inputs:
        inputs = wl.make_inputs("cuda", 5)
    for _ in range(3):
        wl.oracle_forward(inputs)
    torch.cuda.synchronize()
    inputs = wl.make_inputs("cuda", 5)
    graph, warns = harness._capture_graph_checked(lambda: wl.oracle_forward(inputs))
    assert warns == []
    inputs2 = wl.make_inputs("cuda", 5)
    again = harness._normalize_outputs(wl.oracle_forward(inputs2))
    for a, b in zip(first, again):
        assert torch.equal(a, b)
    graph.replay()
    torch.cuda.synchronize()
