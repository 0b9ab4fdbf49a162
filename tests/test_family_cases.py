"""The per-family measurement cases: every case names a kernel family, states its bytes as
"every input once + every output once", and the bench script accepts the sweep mode."""
import re

import torch


def test_family_cases_cover_the_kernel_families_and_state_their_bytes():
    from better_benchmark_b200.family_cases import FAMILY_CASES
    names = set(FAMILY_CASES)
    for needed in ("col_sum_f32", "spatial_mean_cl_bf16", "row_amax_bf16", "row_var_mean_f32", "log_softmax_bf16_f32",
                   "rms_norm_fwd_bf16", "layer_norm_bwd_bf16", "batch_norm_bwd_cl_bf16", "head_split_bf16",
                   "transpose_bf16", "cast_bf16_f32"):
        assert needed in names
    size = {"f32": 4, "bf16": 2}
    # cases kept small on purpose: they measure the dependent chain of a launch, not bandwidth
    latency_cases = {"batch_norm_relu_nchw_small_bf16", "batch_norm_relu_cl_c92_bf16"}
    for case in FAMILY_CASES.values():
        if case.name in latency_cases:
            continue
        assert case.algorithmic_bytes > 64 * 2**20, f"{case.name}: too small to say anything about DRAM (the bench rotates sets over 4x L2)"
        assert case.dtype in size and case.description
    # spot checks of the byte statements against the shapes in the descriptions
    c = FAMILY_CASES["transpose_bf16"]
    assert c.algorithmic_bytes == 2 * 64 * 1024 * 768 * 2
    c = FAMILY_CASES["cast_bf16_f32"]
    assert c.algorithmic_bytes == (64 << 20) * (2 + 4)
    c = FAMILY_CASES["col_sum_f32"]
    assert c.algorithmic_bytes == 16384 * 4096 * 4 + 4096 * 4


def test_bench_script_has_the_sweep_and_reference_modes():
    import bench
    src = open(bench.__file__).read()
    assert re.search(r'"--sweep"', src) and re.search(r'"--impl"', src)
    assert callable(bench.sweep_arm) and callable(bench.reference_arm) and callable(bench.gpu_arm)
